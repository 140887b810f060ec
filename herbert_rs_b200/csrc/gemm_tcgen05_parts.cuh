// What the tcgen05 product kernels share: tile constants, the norm shared between two products,
// the epilogues of a row's columns, and the cluster and CTA-pair instructions.
#pragma once

#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

#define TG_BM 128
#define TG_THREADS 320      // TMA warp, MMA warp, eight epilogue warps
#define TG_EPI_WARPS 8      // two per tensor-memory lane quadrant, each half of a tile's columns

__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// A norm shared between two products (see gemm_skinny.cu): RMSNorm y = x * w / rms(x) between "add
// into the residual stream x" and "the next product".  The residual epilogue also writes x * w in
// bfloat16 and, per tile of BN output columns, each row's sum of x^2; the product that reads x * w
// multiplies its results by 1 / rms, summed from those partial sums in the order of the tiles.
struct TgNorm {
  const float* in_sumsq;   // consumer: [in_parts][in_stride] partial sums of the activation rows, or null
  int in_parts, in_stride;
  float in_eps;
  const float* out_w;      // producer (residual epilogue): the next norm's weight [N], or null
  bf16* out_xw;            // [M, out_ld]
  int out_ld;
  float* out_sumsq;        // [2 * ceil(N / BN)][out_stride]: one row per half tile of columns
  int out_stride;
};

// The q/k/v product whose epilogue also does what follows it in an attention layer with heads of
// 128 (crates/backends/backend_common/src/generic_attention/prefill/mod.rs:115-232): per-head RMSNorm
// of q and k (one weight vector each, or none), rotation of the pairs (j, j + 64) at the token's
// position, q (bfloat16) into the output, k and v into the paged cache.  A half tile of 128 columns
// is one head, so an epilogue thread (one row, one half tile) holds a whole head of one token.
// The epilogue of 32 consecutive output columns (n ..) of row m, whose float results are in r:
// scale by 1/rms, then store / store as float / add into the residual stream (and begin the next
// norm: x * w in bfloat16, sum of x^2 into sq) / SwiGLU.  Rows beyond M and columns beyond N are skipped.
template <int EPI, bool NORM>
__device__ __forceinline__ void tg_epilogue32(unsigned (&r)[32], int m, int n, int M, int N, void* Cv, int ldc, const TgNorm& nm,
                                              float inv_rms, float& sq) {
  if (m < M) {
    if (NORM) {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * inv_rms);
    }
    if (EPI == HB_EPI_SWIGLU) {
      // columns: [8 gate | 8 up] x 2 -> 16 outputs; output column = n/2 + ...
      bf16* out = (bf16*)Cv + (size_t)m * ldc + (n >> 1);
      float y[16];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gate = __uint_as_float(r[blk * 16 + j]), up = __uint_as_float(r[blk * 16 + 8 + j]);
          // silu(g) * u; fast exponential and division: the result is rounded to bfloat16 next
          y[blk * 8 + j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
        }
      if (n + 32 <= N && ((((size_t)m * ldc + (n >> 1)) & 7) == 0)) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          uint4 v;
          v.x = pack2(y[j], y[j + 1]); v.y = pack2(y[j + 2], y[j + 3]);
          v.z = pack2(y[j + 4], y[j + 5]); v.w = pack2(y[j + 6], y[j + 7]);
          *reinterpret_cast<uint4*>(out + j) = v;
        }
      } else {
#pragma unroll
        for (int blk = 0; blk < 2; ++blk)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (n + blk * 16 + 8 + j < N) out[blk * 8 + j] = __float2bfloat16_rn(y[blk * 8 + j]);
      }
    } else if (EPI == HB_EPI_STORE) {
      bf16* out = (bf16*)Cv + (size_t)m * ldc + n;
      if (n + 32 <= N && ((((size_t)m * ldc + n) & 7) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          v.x = pack2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
          v.y = pack2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          v.z = pack2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
          v.w = pack2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
          *reinterpret_cast<uint4*>(out + j) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (n + j < N) out[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
    } else {
      float* out = (float*)Cv + (size_t)m * ldc + n;
      const bool begin_norm = NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr;
      bf16* xw = begin_norm ? nm.out_xw + (size_t)m * nm.out_ld + n : nullptr;
      if (n + 32 <= N && ((((size_t)m * ldc + n) & 3) == 0) && (!begin_norm || ((((size_t)m * nm.out_ld + n) & 7) == 0))) {
        // every load first, then the arithmetic, then every store: the compiler cannot tell that the
        // three arrays do not overlap and would otherwise wait for each store before the next load
        float4 old4[8], w4[8];
        if (EPI == HB_EPI_RESIDUAL) {
#pragma unroll
          for (int q = 0; q < 8; ++q) old4[q] = *reinterpret_cast<const float4*>(out + 4 * q);
        }
        if (begin_norm) {
#pragma unroll
          for (int q = 0; q < 8; ++q) w4[q] = *reinterpret_cast<const float4*>(nm.out_w + n + 4 * q);
        }
        float v[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          v[4 * q] = __uint_as_float(r[4 * q]); v[4 * q + 1] = __uint_as_float(r[4 * q + 1]);
          v[4 * q + 2] = __uint_as_float(r[4 * q + 2]); v[4 * q + 3] = __uint_as_float(r[4 * q + 3]);
          if (EPI == HB_EPI_RESIDUAL) {
            v[4 * q] += old4[q].x; v[4 * q + 1] += old4[q].y; v[4 * q + 2] += old4[q].z; v[4 * q + 3] += old4[q].w;
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(out + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if (begin_norm) {
#pragma unroll
          for (int j = 0; j < 32; ++j) sq += v[j] * v[j];
#pragma unroll
          for (int q = 0; q < 8; q += 2) {
            uint4 pk;
            pk.x = pack2(v[4 * q] * w4[q].x, v[4 * q + 1] * w4[q].y);
            pk.y = pack2(v[4 * q + 2] * w4[q].z, v[4 * q + 3] * w4[q].w);
            pk.z = pack2(v[4 * q + 4] * w4[q + 1].x, v[4 * q + 5] * w4[q + 1].y);
            pk.w = pack2(v[4 * q + 6] * w4[q + 1].z, v[4 * q + 7] * w4[q + 1].w);
            *reinterpret_cast<uint4*>(xw + 4 * q) = pk;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (n + j < N) {
            float v = __uint_as_float(r[j]);
            if (EPI == HB_EPI_RESIDUAL) v += out[j];
            out[j] = v;
            if (begin_norm) {
              xw[j] = __float2bfloat16_rn(v * nm.out_w[n + j]);
              sq += v * v;
            }
          }
      }
    }
  }
}

// The same for 8 consecutive output columns whose float results are in v (store, store as float, add
// into the residual stream and begin the next norm; SwiGLU needs its groups of 16 and goes by 32).
template <int EPI, bool NORM>
__device__ __forceinline__ void tg_epilogue8(float (&v)[8], int m, int n, int M, int N, void* Cv, int ldc, const TgNorm& nm,
                                             float inv_rms, float& sq) {
  static_assert(EPI != HB_EPI_SWIGLU, "SwiGLU goes by chunks of 32 columns");
  if (m >= M || n >= N) return;
  if (NORM) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= inv_rms;
  }
  const bool whole = n + 8 <= N;
  if (EPI == HB_EPI_STORE) {
    bf16* out = (bf16*)Cv + (size_t)m * ldc + n;
    if (whole && ((((size_t)m * ldc + n) & 7) == 0)) {
      uint4 pk;
      pk.x = pack2(v[0], v[1]); pk.y = pack2(v[2], v[3]); pk.z = pack2(v[4], v[5]); pk.w = pack2(v[6], v[7]);
      *reinterpret_cast<uint4*>(out) = pk;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (n + j < N) out[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* out = (float*)Cv + (size_t)m * ldc + n;
    const bool begin_norm = NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr;
    bf16* xw = begin_norm ? nm.out_xw + (size_t)m * nm.out_ld + n : nullptr;
    if (whole && ((((size_t)m * ldc + n) & 3) == 0) && (!begin_norm || ((((size_t)m * nm.out_ld + n) & 7) == 0))) {
      if (EPI == HB_EPI_RESIDUAL) {
        const float4 o0 = *reinterpret_cast<const float4*>(out), o1 = *reinterpret_cast<const float4*>(out + 4);
        v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
        v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
      }
      *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(out + 4) = make_float4(v[4], v[5], v[6], v[7]);
      if (begin_norm) {
        const float4 w0 = *reinterpret_cast<const float4*>(nm.out_w + n), w1 = *reinterpret_cast<const float4*>(nm.out_w + n + 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) sq += v[j] * v[j];
        uint4 pk;
        pk.x = pack2(v[0] * w0.x, v[1] * w0.y); pk.y = pack2(v[2] * w0.z, v[3] * w0.w);
        pk.z = pack2(v[4] * w1.x, v[5] * w1.y); pk.w = pack2(v[6] * w1.z, v[7] * w1.w);
        *reinterpret_cast<uint4*>(xw) = pk;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (n + j < N) {
          float x = v[j];
          if (EPI == HB_EPI_RESIDUAL) x += out[j];
          out[j] = x;
          if (begin_norm) {
            xw[j] = __float2bfloat16_rn(x * nm.out_w[n + j]);
            sq += x * x;
          }
        }
    }
  }
}

// ---- thread-block clusters and pairs of CTAs (tcgen05 with cta_group::2) ---------------------------
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_id_x() {
  unsigned r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned n_clusters_x() {
  unsigned r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned mapa_shared(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(unsigned bar, unsigned parity) {      // arrivals may come from the peer CTA
  unsigned long long start = 0;
  for (unsigned i = 0;; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((i & 255u) == 255u) {
      const unsigned long long now = global_ns();
      if (start == 0) start = now;
      else if (now - start > TG_WAIT_NS) return false;
    }
  }
}
// A TMA tile load into this CTA's shared memory that signals an mbarrier given by its cluster address.
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar_cluster) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void tc_commit_pair(unsigned bar) {      // arrives at this barrier in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void tc_commit_pair_local(unsigned bar) {      // arrives at this CTA's barrier only
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                                 unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ unsigned cluster_nctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(unsigned cluster_addr, float x, float y, float z, float w) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(cluster_addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// ---- shared between the files of the product (host side) -------------------------------------------
int tg_sm_count();
int tg_tile_cols(int M, int N);      // output columns per tile of the kernels that walk whole tiles: 128 or 256
int tg_pairs_enabled();
int tg_cluster_enabled();
// Products that cut K over a thread-block cluster (gemm_tcgen05_cluster.cu).  1: the product went
// that way; 0: it does not apply; negative: an error (its code negated).
int tg_try_ksplit(bool norm, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                  cudaStream_t s, const TgNorm& nm);
int tg_try_pairk(bool norm, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                 cudaStream_t s, const TgNorm& nm);
