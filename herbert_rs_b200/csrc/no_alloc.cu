// See no_alloc.h: decode attention with scratch memory that lives in the library itself.
#include "no_alloc.h"

#include "api.h"
#include "common.cuh"

extern "C" long long hb_attention_decode_scratch_floats(int n_seqs, int nh, int hd, int nsplit);
extern "C" int hb_attention_decode_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                        const void* vcache, const int* seq_len, const int* seq_pages,
                                        int pages_stride, float* scratch, int n_seqs, int nh, int nkv, int hd,
                                        int page_size, int nsplit, float scale, int window, void* stream);

// The partial (m, l, o) results of the key splits.  In host code this name is only a handle for
// the runtime's symbol calls, never a pointer a kernel could use; its device address is looked up
// once per device below.
static __device__ __align__(256) float g_noalloc_scratch[HB_NOALLOC_SCRATCH_FLOATS];

#define HB_MAX_DEVICES 64
static float* g_scratch_addr[HB_MAX_DEVICES];   // device address of the array, per device; null until looked up

extern "C" int hb_attention_decode_bf16_noalloc(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                                const void* vcache, const int* seq_len, const int* seq_pages,
                                                int pages_stride, int n_seqs, int nh, int nkv, int hd,
                                                int page_size, int nsplit, float scale, int window, void* stream) {
  HB_REQUIRE(n_seqs > 0 && nh > 0 && hd > 0 && nsplit > 0, "attention_decode_noalloc: sizes must be positive");
  const long long need = hb_attention_decode_scratch_floats(n_seqs, nh, hd, nsplit);
  HB_REQUIRE(need <= (long long)HB_NOALLOC_SCRATCH_FLOATS,
             "attention_decode_noalloc: %lld floats of scratch needed (n_seqs %d x heads %d x splits %d x (head size %d + 2)), "
             "the built-in array holds %d; use fewer splits or sequences, or the entry point that takes scratch",
             need, n_seqs, nh, nsplit, hd, HB_NOALLOC_SCRATCH_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  HB_REQUIRE(e == cudaSuccess, "attention_decode_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
  HB_REQUIRE(device >= 0 && device < HB_MAX_DEVICES, "attention_decode_noalloc: device index %d is out of range", device);
  if (g_scratch_addr[device] == nullptr) {
    // set-up, once per device, with that device current (it is: we just asked which one is)
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    HB_REQUIRE(e == cudaSuccess && p != nullptr, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_addr[device] = p;
  }
  return hb_attention_decode_bf16(q, ldq, out, ldo, kcache, vcache, seq_len, seq_pages, pages_stride,
                                  g_scratch_addr[device], n_seqs, nh, nkv, hd, page_size, nsplit, scale, window, stream);
}
