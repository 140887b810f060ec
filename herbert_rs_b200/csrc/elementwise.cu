// Embedding gather, RMSNorm, SwiGLU and the fused per-head norm + rotation + cache write.
//
// Formulas (reference, CPU path):
//   embedding   x[t,:] = float(E[id_t,:])                      generic_model.rs:104-111
//   RMSNorm     r = 1/sqrt(sum(x^2)/dim + eps); y = (x*r)*w    kernels.rs:54-64
//   SwiGLU      silu(g) = g/(1+exp(-g)); a = silu(g)*u         kernels.rs:677-687
//   head norm   RMSNorm over head_dim, one weight for all heads generic_attention/mod.rs:62-76
//   rotation    pairs (j, j+rot/2): x0*c - x1*s, x0*s + x1*c   kernels.rs:739-759
//   cache write k after norm and rotation, v as projected      generic_attention/prefill/mod.rs:115-232
// All arithmetic is float; T is only the storage type.
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {  // the host validates ids; an invalid one yields zeros, never a stray read
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

template <typename T>
static int embed_launch(const void* table, const int* ids, float* out, int n_tokens, int hidden,
                        int vocab, void* stream) {
  HB_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embed: sizes must be positive");
  int threads = hidden >= 1024 ? 256 : 128;
  hb_launch(embed_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (const T*)table, ids, out, hidden, vocab);
  HB_CHECK_LAUNCH("embed");
  return 0;
}

extern "C" int hb_embed(int dtype, const void* table, const int* ids, float* out, int n_tokens,
                        int hidden, int vocab, void* stream) {
  return dtype == HB_F32 ? embed_launch<float>(table, ids, out, n_tokens, hidden, vocab, stream)
                         : embed_launch<bf16>(table, ids, out, n_tokens, hidden, vocab, stream);
}

// ---------------------------------------------------------------------------------------------
// One block per output row.  rows == nullptr: row r of x; else row rows[r] of x (gather).
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               T* __restrict__ out, const int* __restrict__ rows, int dim, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float s = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    s += v * v;
  }
  s = block_sum(s, red);
  const float inv = 1.0f / sqrtf(s / (float)dim + eps);
  T* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<T>((xr[i] * inv) * w[i]);
}

extern "C" int hb_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows,
                          int n_rows, int dim, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0, "rmsnorm: sizes must be positive");
  int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  if (dtype == HB_F32)
    hb_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x, w, (float*)out, rows, dim, eps);
  else
    hb_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x, w, (bf16*)out, rows, dim, eps);
  HB_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// gu: [n_tokens, 2*inter] with leading dimension ld.  interleave == 0: gate columns [0, inter),
// up columns [inter, 2*inter).  interleave == 8: blocks of 16 columns, 8 gate then 8 up.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int ldo,
                              int inter, int interleave) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const T* row = gu + (size_t)t * ld;
  int gi, ui;
  if (interleave == 0) {
    gi = i;
    ui = inter + i;
  } else {
    gi = (i / interleave) * (2 * interleave) + (i % interleave);
    ui = gi + interleave;
  }
  const float g = to_f32(row[gi]), u = to_f32(row[ui]);
  const float a = (g / (1.0f + expf(-g))) * u;
  out[(size_t)t * ldo + i] = from_f32<T>(a);
}

extern "C" int hb_swiglu(int dtype, const void* gu, int ld, void* out, int ldo, int n_tokens,
                         int inter, int interleave, void* stream) {
  HB_REQUIRE(n_tokens > 0 && inter > 0, "swiglu: sizes must be positive");
  HB_REQUIRE(interleave == 0 || (interleave > 0 && inter % interleave == 0),
             "swiglu: intermediate size %d is no multiple of the interleave %d", inter, interleave);
  HB_REQUIRE(n_tokens <= 65535, "swiglu: at most 65535 tokens per call, got %d", n_tokens);
  dim3 grid(ceil_div(inter, 256), n_tokens);
  if (dtype == HB_F32)
    hb_launch(swiglu_kernel<float>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const float*)gu, ld, (float*)out, ldo, inter, interleave);
  else
    hb_launch(swiglu_kernel<bf16>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const bf16*)gu, ld, (bf16*)out, ldo, inter, interleave);
  HB_CHECK_LAUNCH("swiglu");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// qkv: [n_tokens, ld] rows holding nh query heads, then nkv key heads, then nkv value heads,
// each head_dim wide.  One warp per (token, head).  Query heads are normed and rotated in
// place; key heads are normed, rotated and stored in the cache; value heads are copied to the
// cache.  qw/kw == nullptr: no head norm.  cos_tab == nullptr: no rotation.
// Cache entry layout: [n_pages][nkv][page_size][head_dim]; the page of position p of sequence b
// is seq_pages[b * pages_stride + p / page_size].
struct QkvCacheArgs {
  void* qkv;
  int ld;
  const float* qw;
  const float* kw;
  float eps;
  const float* cos_tab;
  const float* sin_tab;
  int rot;
  int table_rows;
  const int* tok_seq;
  const int* tok_pos;
  const int* seq_pages;
  int pages_stride;
  void* kcache;
  void* vcache;
  int n_tokens, nh, nkv, hd, page_size;
  int write_cache;
};

template <typename T>
__global__ void qk_norm_rope_cache_kernel(QkvCacheArgs a) {
  pdl_wait();
  pdl_launch();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads_total = a.nh + 2 * a.nkv;
  const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (unit >= (long long)a.n_tokens * heads_total) return;
  const int t = (int)(unit / heads_total);
  const int h = (int)(unit % heads_total);
  T* x = (T*)a.qkv + (size_t)t * a.ld + (size_t)h * a.hd;
  const int pos = a.tok_pos[t];
  const int b = a.tok_seq[t];

  // where this head goes in the cache (key and value heads only)
  T* dst = nullptr;
  const bool is_q = h < a.nh;
  const bool is_v = h >= a.nh + a.nkv;
  if (!is_q) {
    if (!a.write_cache) return;
    const int kvh = is_v ? h - a.nh - a.nkv : h - a.nh;
    const int page = a.seq_pages[(size_t)b * a.pages_stride + pos / a.page_size];
    T* base = (T*)(is_v ? a.vcache : a.kcache);
    dst = base + (((size_t)page * a.nkv + kvh) * a.page_size + (pos % a.page_size)) * a.hd;
  }
  if (is_v) {
    for (int d = lane; d < a.hd; d += 32) dst[d] = x[d];
    return;
  }
  const float* w = is_q ? a.qw : a.kw;
  float inv = 1.0f;
  if (w) {
    float s = 0.0f;
    for (int d = lane; d < a.hd; d += 32) {
      float v = to_f32(x[d]);
      s += v * v;
    }
    s = warp_sum(s);
    inv = 1.0f / sqrtf(s / (float)a.hd + a.eps);
  }
  T* o = is_q ? x : dst;
  const int rot = a.cos_tab ? a.rot : 0;
  const int half = rot >> 1;
  const int trow = pos < a.table_rows ? pos : a.table_rows - 1;  // the host refuses pos >= table_rows
  const float* c = a.cos_tab ? a.cos_tab + (size_t)trow * half : nullptr;
  const float* s_ = a.sin_tab ? a.sin_tab + (size_t)trow * half : nullptr;
  for (int j = lane; j < half; j += 32) {
    float x0 = to_f32(x[j]), x1 = to_f32(x[j + half]);
    if (w) {
      x0 = (x0 * inv) * w[j];
      x1 = (x1 * inv) * w[j + half];
    }
    const float cv = c[j], sv = s_[j];
    o[j] = from_f32<T>(x0 * cv - x1 * sv);
    o[j + half] = from_f32<T>(x0 * sv + x1 * cv);
  }
  for (int d = rot + lane; d < a.hd; d += 32) {
    float v = to_f32(x[d]);
    if (w) v = (v * inv) * w[d];
    o[d] = from_f32<T>(v);
  }
}

extern "C" int hb_qk_norm_rope_cache(int dtype, void* qkv, int ld, const float* qw, const float* kw,
                                     float eps, const float* cos_tab, const float* sin_tab, int rot,
                                     int table_rows, const int* tok_seq, const int* tok_pos,
                                     const int* seq_pages, int pages_stride, void* kcache,
                                     void* vcache, int n_tokens, int nh, int nkv, int hd,
                                     int page_size, int write_cache, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && nkv > 0 && hd > 0 && page_size > 0, "qk_norm_rope_cache: sizes must be positive");
  HB_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "qk_norm_rope_cache: rotated width %d must be even and <= head_dim %d", rot, hd);
  HB_REQUIRE((cos_tab == nullptr) == (sin_tab == nullptr), "qk_norm_rope_cache: cos and sin tables come together");
  HB_REQUIRE((qw == nullptr) == (kw == nullptr), "qk_norm_rope_cache: q and k norm weights come together");
  HB_REQUIRE(ld >= (nh + 2 * nkv) * hd, "qk_norm_rope_cache: leading dimension %d < %d", ld, (nh + 2 * nkv) * hd);
  QkvCacheArgs a{qkv, ld, qw, kw, eps, cos_tab, sin_tab, rot, table_rows, tok_seq, tok_pos, seq_pages,
                 pages_stride, kcache, vcache, n_tokens, nh, nkv, hd, page_size, write_cache};
  const long long units = (long long)n_tokens * (nh + 2 * nkv);
  const int wpb = 8;
  const long long blocks = ceil_div_ll(units, wpb);
  HB_REQUIRE(blocks < 2147483647LL, "qk_norm_rope_cache: too many (token, head) pairs");
  if (dtype == HB_F32)
    hb_launch(qk_norm_rope_cache_kernel<float>, dim3((unsigned)blocks), dim3(wpb * 32), 0, (cudaStream_t)stream, a);
  else
    hb_launch(qk_norm_rope_cache_kernel<bf16>, dim3((unsigned)blocks), dim3(wpb * 32), 0, (cudaStream_t)stream, a);
  HB_CHECK_LAUNCH("qk_norm_rope_cache");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// residual[t, :] += y[t, :] (for parts that cannot fuse the sum into their last product)
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ res, const T* __restrict__ y, int ld, int dim) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < dim) res[(size_t)t * dim + i] += to_f32(y[(size_t)t * ld + i]);
}

extern "C" int hb_add_residual(int dtype, float* res, const void* y, int ld, int n_tokens, int dim, void* stream) {
  HB_REQUIRE(n_tokens > 0 && dim > 0 && n_tokens <= 65535, "add_residual: bad sizes");
  dim3 grid(ceil_div(dim, 256), n_tokens);
  if (dtype == HB_F32)
    hb_launch(add_residual_kernel<float>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, res, (const float*)y, ld, dim);
  else
    hb_launch(add_residual_kernel<bf16>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, res, (const bf16*)y, ld, dim);
  HB_CHECK_LAUNCH("add_residual");
  return 0;
}
