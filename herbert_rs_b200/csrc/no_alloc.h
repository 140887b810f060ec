// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists for hosts of this library that
// cannot call cudaMalloc when they need attention - a serving loop that has handed every free byte
// of the device to its own pool, a real-time caller that cannot afford the device-wide
// synchronisation an allocation may bring, or code that runs while allocation is forbidden.  The
// ordinary entry point (hb_attention_decode_bf16) asks its caller for scratch memory for the
// partial results of the key splits; this one brings its own, a fixed array in the library's
// device image, so the caller passes only inputs and outputs.
//
// Limits and rules:
//  * the scratch array holds HB_NOALLOC_SCRATCH_FLOATS floats (8 MiB); every GPU that loads the
//    library keeps that much reserved until the process exits.  A call that would need more
//    (n_seqs * nh * nsplit * (hd + 2) floats) is refused with a message, nothing is launched;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress) with
//    that device current; make that first call outside any stream capture;
//  * the array's address is looked up and kept per device under the device that is current at the
//    call: the stream must belong to the current device, and first calls on a device that come
//    from several host threads at once must be serialised by the caller (later calls only read);
//  * no cudaMalloc, cudaFree or other allocating routine is called, here or in what it launches;
//  * all calls share the one array, which keeps whatever the previous call left.  Nothing in it
//    has to start at zero: the kernels write every partial result they later read.  Two calls
//    whose kernels may overlap on the GPU (different streams) race on it: keep them on one stream
//    or order them with events.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define HB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Same arguments and result as hb_attention_decode_bf16 without the scratch pointer.
int hb_attention_decode_bf16_noalloc(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                     const void* vcache, const int* seq_len, const int* seq_pages,
                                     int pages_stride, int n_seqs, int nh, int nkv, int hd, int page_size,
                                     int nsplit, float scale, int window, void* stream);

#ifdef __cplusplus
}
#endif
