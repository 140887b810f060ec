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
#include "qk_norm.cuh"

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

// The same with the row held in registers between the two passes and 16-byte loads: for rows of
// at most 4 * RN_VEC * blockDim.x floats whose length is a multiple of 4.
#define RN_VEC 4
__device__ __forceinline__ void store4(float* o, float4 v) { *reinterpret_cast<float4*>(o) = v; }
__device__ __forceinline__ void store4(bf16* o, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&a);
  u.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(o) = u;
}
template <typename T>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, int dim, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const float4* wv = reinterpret_cast<const float4*>(w);
  const int nvec = dim >> 2;
  float4 v[RN_VEC];
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int k = threadIdx.x + i * blockDim.x;
    v[i] = k < nvec ? xr[k] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  s = block_sum(s, red);
  const float inv = 1.0f / sqrtf(s / (float)dim + eps);
  T* o = out + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int k = threadIdx.x + i * blockDim.x;
    if (k < nvec) {
      const float4 ww = wv[k];
      store4(o + 4 * k, make_float4((v[i].x * inv) * ww.x, (v[i].y * inv) * ww.y, (v[i].z * inv) * ww.z, (v[i].w * inv) * ww.w));
    }
  }
}

extern "C" int hb_rmsnorm(int dtype, const float* x, const float* w, void* out, const int* rows,
                          int n_rows, int dim, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0, "rmsnorm: sizes must be positive");
  int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
  if (dim % 4 == 0 && dim <= 4 * RN_VEC * threads && aligned) {
    if (dtype == HB_F32)
      hb_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x, w, (float*)out, rows, dim, eps);
    else
      hb_launch(rmsnorm_vec_kernel<bf16>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x, w, (bf16*)out, rows, dim, eps);
    HB_CHECK_LAUNCH("rmsnorm");
    return 0;
  }
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

// The common case made cheap: every head is rotated over its whole width (or not at all is not
// handled here), head size a multiple of 4 up to 256.  One block per token; its 8 warps walk the
// token's heads, so the position, the page, the cos/sin values and the norm weights a lane needs
// are fetched once per token instead of once per head, and loads and stores move 2 elements.
__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ld2(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void st2(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_cache_fast_kernel(QkvCacheArgs a) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd = a.hd, half = hd >> 1;
  const int pos = a.tok_pos[t], b = a.tok_seq[t];
  const int trow = pos < a.table_rows ? pos : a.table_rows - 1;
  const int page = a.write_cache ? a.seq_pages[(size_t)b * a.pages_stride + pos / a.page_size] : 0;
  const int j[2] = {2 * lane, 2 * lane + 64};
  float2 c[2], sn[2], qlo[2], qhi[2], klo[2], khi[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (j[i] < half) {
      c[i] = ld2(a.cos_tab + (size_t)trow * half + j[i]);
      sn[i] = ld2(a.sin_tab + (size_t)trow * half + j[i]);
      if (a.qw) {
        qlo[i] = ld2(a.qw + j[i]); qhi[i] = ld2(a.qw + j[i] + half);
        klo[i] = ld2(a.kw + j[i]); khi[i] = ld2(a.kw + j[i] + half);
      }
    }
  }
  T* row = (T*)a.qkv + (size_t)t * a.ld;
  const int heads_total = a.nh + 2 * a.nkv;
  for (int h = warp; h < heads_total; h += 8) {
    T* x = row + (size_t)h * hd;
    const bool is_q = h < a.nh, is_v = h >= a.nh + a.nkv;
    T* dst = x;
    if (!is_q) {
      if (!a.write_cache) continue;
      const int kvh = is_v ? h - a.nh - a.nkv : h - a.nh;
      T* basep = (T*)(is_v ? a.vcache : a.kcache);
      dst = basep + (((size_t)page * a.nkv + kvh) * a.page_size + (pos % a.page_size)) * hd;
    }
    if (is_v) {
      for (int d = 2 * lane; d < hd; d += 64) {
        const float2 v = ld2(x + d);
        st2(dst + d, v.x, v.y);
      }
      continue;
    }
    float2 lo[2], hi[2];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (j[i] < half) {
        lo[i] = ld2(x + j[i]);
        hi[i] = ld2(x + j[i] + half);
        ss += lo[i].x * lo[i].x + lo[i].y * lo[i].y + hi[i].x * hi[i].x + hi[i].y * hi[i].y;
      }
    }
    if (a.qw) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (j[i] < half) {
          const float2 wl = is_q ? qlo[i] : klo[i], wh = is_q ? qhi[i] : khi[i];
          lo[i].x = (lo[i].x * inv) * wl.x; lo[i].y = (lo[i].y * inv) * wl.y;
          hi[i].x = (hi[i].x * inv) * wh.x; hi[i].y = (hi[i].y * inv) * wh.y;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (j[i] < half) {
        st2(dst + j[i], lo[i].x * c[i].x - hi[i].x * sn[i].x, lo[i].y * c[i].y - hi[i].y * sn[i].y);
        st2(dst + j[i] + half, lo[i].x * sn[i].x + hi[i].x * c[i].x, lo[i].y * sn[i].y + hi[i].y * c[i].y);
      }
    }
  }
}

// Head size 128 rotated over its whole width: a head per half-warp, 8- or 16-byte loads and stores
// (the arithmetic lives in qk_norm.cuh).  One block per token; its 16 half-warps walk the heads.
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_cache_128_kernel(QkvCacheArgs a) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, hw = threadIdx.x >> 4, l = threadIdx.x & 15;
  const int pos = a.tok_pos[t], b = a.tok_seq[t];
  const int trow = pos < a.table_rows ? pos : a.table_rows - 1;
  const float* cos_row = a.cos_tab + (size_t)trow * 64;
  const float* sin_row = a.sin_tab + (size_t)trow * 64;
  const int page = a.write_cache ? a.seq_pages[(size_t)b * a.pages_stride + pos / a.page_size] : 0;
  T* row = (T*)a.qkv + (size_t)t * a.ld;
  const int n_qk = a.nh + a.nkv, heads_total = a.nh + 2 * a.nkv;
  for (int h0 = 0; h0 < heads_total; h0 += 16) {          // uniform trip count: the shuffles inside need whole warps
    const int h = h0 + hw;
    const bool is_q = h < a.nh, is_k = !is_q && h < n_qk, is_v = h >= n_qk && h < heads_total;
    const size_t slot = is_q ? 0 : (((size_t)page * a.nkv + (is_k ? h - a.nh : h - n_qk)) * a.page_size + (pos % a.page_size)) * 128;
    const T* x = row + (size_t)(h < heads_total ? h : 0) * 128;
    T* dst = is_q ? row + (size_t)h * 128 : (T*)(is_k ? a.kcache : a.vcache) + slot;
    norm_rotate_head128<T>(is_q || (is_k && a.write_cache), x, dst, is_q ? a.qw : a.kw, a.eps, cos_row, sin_row, l);
    if (is_v && a.write_cache) {
      float v[4];
      Vec4<T>::load(x + 4 * l, v);
      Vec4<T>::store(dst + 4 * l, v);
      Vec4<T>::load(x + 64 + 4 * l, v);
      Vec4<T>::store(dst + 64 + 4 * l, v);
    }
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
  const int esz = dtype == HB_F32 ? 4 : 2;
  const bool fast = cos_tab != nullptr && rot == hd && hd % 4 == 0 && hd <= 256 && ld % 2 == 0 &&
                    ((uintptr_t)qkv % (2 * esz)) == 0 && ((uintptr_t)kcache % (2 * esz)) == 0 &&
                    ((uintptr_t)vcache % (2 * esz)) == 0 && ((uintptr_t)cos_tab & 7) == 0 && ((uintptr_t)sin_tab & 7) == 0 &&
                    (qw == nullptr || (((uintptr_t)qw & 7) == 0 && ((uintptr_t)kw & 7) == 0));
  const int vec = 4 * esz;     // bytes of four elements
  const bool fast128 = fast && hd == 128 && ld % 4 == 0 && ((uintptr_t)qkv % vec) == 0 && ((uintptr_t)kcache % vec) == 0 &&
                       ((uintptr_t)vcache % vec) == 0 && ((uintptr_t)cos_tab & 15) == 0 && ((uintptr_t)sin_tab & 15) == 0 &&
                       (qw == nullptr || (((uintptr_t)qw & 15) == 0 && ((uintptr_t)kw & 15) == 0));
  if (fast128) {
    if (dtype == HB_F32)
      hb_launch(qk_norm_rope_cache_128_kernel<float>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
    else
      hb_launch(qk_norm_rope_cache_128_kernel<bf16>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
    HB_CHECK_LAUNCH("qk_norm_rope_cache");
    return 0;
  }
  if (fast) {
    if (dtype == HB_F32)
      hb_launch(qk_norm_rope_cache_fast_kernel<float>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
    else
      hb_launch(qk_norm_rope_cache_fast_kernel<bf16>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, a);
    HB_CHECK_LAUNCH("qk_norm_rope_cache");
    return 0;
  }
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

// Finishes a norm that a product left half done: out = xw / rms, with rms^2 = sum of the row's
// partial sums / dim + eps (xw = x * w in bfloat16, sumsq [parts][stride]).  For consumers that
// cannot apply the row factor themselves.
__global__ void finish_norm_kernel(const bf16* __restrict__ xw, int ld, const float* __restrict__ sumsq, int parts,
                                   int stride, float eps, bf16* __restrict__ out, int ldo, int dim) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int m = blockIdx.x;
  float s = 0.0f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) s += sumsq[(size_t)i * stride + m];
  s = block_sum(s, red);
  const float inv = rsqrtf(s / (float)dim + eps);
  for (int k = threadIdx.x; k < dim; k += blockDim.x)
    out[(size_t)m * ldo + k] = __float2bfloat16_rn(__bfloat162float(xw[(size_t)m * ld + k]) * inv);
}

extern "C" int hb_finish_norm(const void* xw, int ld, const float* sumsq, int parts, int stride, float eps, void* out,
                              int ldo, int n_rows, int dim, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0 && parts > 0 && stride >= n_rows, "finish_norm: positive sizes, row stride >= rows");
  hb_launch(finish_norm_kernel, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (const bf16*)xw, ld, sumsq, parts, stride,
            eps, (bf16*)out, ldo, dim);
  HB_CHECK_LAUNCH("finish_norm");
  return 0;
}
