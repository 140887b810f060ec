// Grouped-query softmax attention over the paged cache, CUDA cores only, any head size up to
// 256 and any number of heads and groups.  One warp per (token, query head).
//
// This is the attention of the true 32-bit path (prefill and decode alike) and the any-shape
// fallback of the bfloat16 path.  It follows the reference's online-softmax form
// (generic_attention/prefill/kernel_f32.rs:61-111): for every key j in the query's range,
//   s_j = (q . k_j) * scale;  m' = max(m, s_j);  l = l*exp(m-m') + exp(s_j-m');
//   o = o*exp(m-m') + exp(s_j-m') * v_j;   result o / l,
// here taken 32 keys at a time.  Range of the query at position p: keys lo..p with
// lo = max(0, p - window + 1) when window > 0, else 0 (causal; decode.rs:126-295 scans 0..=pos).
// Query head h reads key/value head h / (nh/nkv) (loader_common.rs:1003-1005).
#include "api.h"
#include "common.cuh"

#define ATT_MAX_HD 256
#define ATT_WARPS 4

struct AttnArgs {
  const void* q;
  int ldq;
  void* out;
  int ldo;
  const void* kcache;
  const void* vcache;
  const int* tok_seq;
  const int* tok_pos;
  const int* seq_pages;
  int pages_stride;
  int n_tokens, nh, nkv, hd, page_size;
  float scale;
  int window;
};

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_simt_kernel(AttnArgs a) {
  __shared__ float qs[ATT_WARPS][ATT_MAX_HD];
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * ATT_WARPS + warp;
  if (unit >= (long long)a.n_tokens * a.nh) return;
  const int t = (int)(unit / a.nh), h = (int)(unit % a.nh);
  const int kvh = h / (a.nh / a.nkv);
  const int p = a.tok_pos[t], b = a.tok_seq[t];
  const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
  const T* qp = (const T*)a.q + (size_t)t * a.ldq + (size_t)h * a.hd;
  for (int d = lane; d < a.hd; d += 32) qs[warp][d] = to_f32(qp[d]);
  __syncwarp();
  const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
  const size_t head_stride = (size_t)a.page_size * a.hd;

  float m = -INFINITY, l = 0.0f;
  float o[ATT_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) o[i] = 0.0f;

  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j <= p) {
      const int page = pages[j / a.page_size];
      const T* kr = (const T*)a.kcache + ((size_t)page * a.nkv + kvh) * head_stride + (size_t)(j % a.page_size) * a.hd;
      float dot = 0.0f;
      for (int d = 0; d < a.hd; ++d) dot = fmaf(qs[warp][d], to_f32(kr[d]), dot);
      s = dot * a.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf on the first chunk: exp(-inf) = 0
    const float pj = (j <= p) ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / 32; ++i) o[i] *= corr;
    const int nk = (p - j0 + 1 < 32) ? p - j0 + 1 : 32;
    for (int k = 0; k < nk; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pj, k);
      const int jk = j0 + k;
      const int page = pages[jk / a.page_size];
      const T* vr = (const T*)a.vcache + ((size_t)page * a.nkv + kvh) * head_stride + (size_t)(jk % a.page_size) * a.hd;
#pragma unroll
      for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.hd) o[i] = fmaf(pk, to_f32(vr[d]), o[i]);
      }
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  T* op = (T*)a.out + (size_t)t * a.ldo + (size_t)h * a.hd;
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < a.hd) op[d] = from_f32<T>(o[i] * inv);
  }
}

extern "C" int hb_attention_simt(int dtype, const void* q, int ldq, void* out, int ldo, const void* kcache,
                                 const void* vcache, const int* tok_seq, const int* tok_pos,
                                 const int* seq_pages, int pages_stride, int n_tokens, int nh, int nkv,
                                 int hd, int page_size, float scale, int window, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && nkv > 0 && hd > 0 && page_size > 0, "attention: sizes must be positive");
  HB_REQUIRE(nh % nkv == 0, "attention: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  HB_REQUIRE(hd <= ATT_MAX_HD, "attention: head size %d exceeds the supported maximum %d", hd, ATT_MAX_HD);
  HB_REQUIRE(window >= 0, "attention: window must be >= 0");
  AttnArgs a{q, ldq, out, ldo, kcache, vcache, tok_seq, tok_pos, seq_pages, pages_stride,
             n_tokens, nh, nkv, hd, page_size, scale, window};
  const long long blocks = ceil_div_ll((long long)n_tokens * nh, ATT_WARPS);
  HB_REQUIRE(blocks < 2147483647LL, "attention: too many (token, head) pairs");
  if (dtype == HB_F32)
    hb_launch(attention_simt_kernel<float>, dim3((unsigned)blocks), dim3(ATT_WARPS * 32), 0, (cudaStream_t)stream, a);
  else
    hb_launch(attention_simt_kernel<bf16>, dim3((unsigned)blocks), dim3(ATT_WARPS * 32), 0, (cudaStream_t)stream, a);
  HB_CHECK_LAUNCH("attention_simt");
  return 0;
}
