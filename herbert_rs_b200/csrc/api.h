// C interface of libherbert_b200: every launcher the library exports (the allocation-free entry
// point has its own header, no_alloc.h).  All pointers are device pointers; `stream` is a
// cudaStream_t.  A launcher returns 0 when it has launched; otherwise hb_last_error() holds the
// reason and nothing was launched.  The Python side (ops/__init__.py) keeps a ctypes signature per
// launcher; a test compares those with the declarations below.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// dtype codes used where one entry point serves both paths
#define HB_F32 0
#define HB_BF16 1

// epilogues of the matrix products
#define HB_EPI_STORE 0      // C (activation dtype) = A W^T
#define HB_EPI_STORE_F32 1  // C (float)            = A W^T
#define HB_EPI_RESIDUAL 2   // C (float)           += A W^T
#define HB_EPI_SWIGLU 3     // C (activation dtype) = silu(gate) * up, W rows in groups of 8 gate, 8 up


// attention_decode.cu: decode attention over the paged cache (one query per sequence, keys cut into splits)
long long hb_attention_decode_scratch_floats(int n_seqs, int nh, int hd, int nsplit);
int hb_attention_decode_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache, const void*
    vcache, const int* seq_len, const int* seq_pages, int pages_stride, float* scratch, int n_seqs, int nh,
    int nkv, int hd, int page_size, int nsplit, float scale, int window, void* stream);
int hb_attention_decode_fused_bf16(const void* qkv, int ld, void* out, int ldo, void* kcache, void* vcache,
    const float* qw, const float* kw, float eps, const float* cos_tab, const float* sin_tab, int table_rows,
    int write_cache, const int* seq_len, const int* seq_pages, int pages_stride, float* scratch, int*
    counters, int n_seqs, int nh, int nkv, int page_size, int nsplit, float scale, int window, void* stream);

// attention_prefill.cu: prefill attention, mma.sync flash form, head sizes in steps of 16 up to 256
int hb_attention_prefill_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache, const void*
    vcache, const int* seq_start, const int* seq_pos0, const int* seq_pages, int pages_stride, int n_seqs, int
    max_q_len, int nh, int nkv, int hd, int page_size, float scale, int window, void* stream);

// attention_prefill_tc.cu: prefill attention on tcgen05 tensor cores, head sizes 64 and 128
int hb_attention_prefill_tc_bf16(const void* q, int ldq, int n_tokens, void* out, int ldo, const void* kcache,
    const void* vcache, int n_pages, const int* seq_start, const int* seq_pos0, const int* seq_pages, int
    pages_stride, int n_seqs, int max_q_len, int nh, int nkv, int hd, int page_size, float scale, int window,
    int* error_flag, int* work_counter, void* stream);

// attention_simt.cu: attention of any shape on the CUDA cores (the 32-bit path)
int hb_attention_simt(int dtype, const void* q, int ldq, void* out, int ldo, const void* kcache, const void*
    vcache, const int* tok_seq, const int* tok_pos, const int* seq_pages, int pages_stride, int n_tokens, int
    nh, int nkv, int hd, int page_size, float scale, int window, void* stream);

// elementwise.cu: embedding, RMSNorm, SwiGLU, head norm + rotation + cache write, residual sum, shared-norm finish
int hb_embed(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab,
    void* stream);
int hb_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows, int dim,
    float eps, void* stream);
int hb_swiglu(int dtype, const void* gu, int ld, void* out, int ldo, int n_tokens, int inter, int interleave,
    void* stream);
int hb_qk_norm_rope_cache(int dtype, void* qkv, int ld, const float* qw, const float* kw, float eps, const
    float* cos_tab, const float* sin_tab, int rot, int table_rows, const int* tok_seq, const int* tok_pos,
    const int* seq_pages, int pages_stride, void* kcache, void* vcache, int n_tokens, int nh, int nkv, int hd,
    int page_size, int write_cache, void* stream);
int hb_add_residual(int dtype, float* res, const void* y, int ld, int n_tokens, int dim, void* stream);
int hb_finish_norm(const void* xw, int ld, const float* sumsq, int parts, int stride, float eps, void* out,
    int ldo, int n_rows, int dim, void* stream);

// errors.cu: error text, ABI version, programmatic dependent launch mode
const char* hb_last_error(void);
int hb_abi_version(void);
void hb_set_pdl(int mode);
int hb_get_pdl(void);

// fill.cu: load-time kernels: counter-based normal fill, constant fill, dtype casts
int hb_rng_normal(int dtype, void* out, long long n, unsigned long long key, float mean, float stdev, void*
    stream);
int hb_fill(int dtype, void* out, long long n, float value, void* stream);
int hb_cast(int src, const void* in, int dst, void* out, long long n, int round_bf16, void* stream);

// gemm_simt.cu: matrix product of any shape on the CUDA cores (the 32-bit path)
int hb_gemm_simt(int dtype, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, void* stream);

// gemm_skinny.cu: decode product (at most 64 activation rows), mma.sync, optional shared norm
int hb_gemm_skinny_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
    int epi, void* stream);
int hb_gemm_skinny_norm_parts(int M, int N);
int hb_gemm_skinny_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, const float* in_sumsq, int in_parts, float in_eps, const float* out_w, void* out_xw, int
    out_ld, float* out_sumsq, void* stream);

// gemm_stream.cu: decode product, TMA + tcgen05, K slices (the output head)
long long hb_gemm_stream_scratch_floats(int M, int N, int K);
int hb_gemm_stream_counters(int N);
int hb_gemm_stream_bf16(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
    int epi, float* scratch, long long scratch_floats, int* counters, int n_counters, int* error_flag, void*
    stream);

// gemm_tcgen05.cu: prefill product, TMA + tcgen05, persistent; optional shared norm
int hb_gemm_tcgen05_set_pairs(int on);
int hb_gemm_tcgen05_set_ksplit(int on);
long long hb_gemm_tcgen05_workspace_floats(int ctas);
int hb_gemm_tcgen05_set_workspace(float* floats, int* counters, int ctas);
int hb_gemm_tcgen05_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int
    K, int epi, int* error_flag, void* stream);
int hb_gemm_tcgen05_qkv_ok(int M, int N);
int hb_gemm_tcgen05_qkv_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, const float* in_sumsq, int in_parts, int in_stride, float in_eps, const float* qw, const float* kw,
    float eps, const float* cos_tab, const float* sin_tab, int table_rows, const int* tok_seq, const int*
    tok_pos, const int* seq_pages, int pages_stride, void* kcache, void* vcache, int nh, int nkv, int
    page_size, int write_cache, int* error_flag, void* stream);
int hb_gemm_tcgen05_norm_parts(int M, int N);
int hb_gemm_tcgen05_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
    int K, int epi, const float* in_sumsq, int in_parts, int in_stride, float in_eps, const float* out_w,
    void* out_xw, int out_ld, float* out_sumsq, int out_stride, int* error_flag, void* stream);

// sampling.cu: argmax and temperature / top-k / top-p sampling
int hb_argmax(const float* logits, int ld, int n_rows, int vocab, int* out, void* scratch, long long
    scratch_words, void* stream);
int hb_sample(const float* logits, int ld, int n_rows, int vocab, float temperature, int top_k, float top_p,
    const float* uniforms, int* out, int* overflow, void* stream);

#ifdef __cplusplus
}
#endif
