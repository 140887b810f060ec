// Skinny matrix product for decoding: few activation rows against a whole weight matrix.
//   C[M,N] (op)= A[M,K] * W[N,K]^T,  M <= 64, bfloat16 operands, float accumulation.
//
// A decode step reads every weight once and is bound by that stream, so the kernel is laid out
// around the weight bytes (the reference's matvec has the same premise: one pass over W per
// token, backends/backend_bf16_avx512/src/avx512_bf16_matvec.S:1-60).  The weight rows are the
// M operand of the tensor-core instruction ("swapped" roles): one CTA owns 16 weight rows, its 8
// warps share K, and every lane fetches 16 contiguous bytes of a weight row straight from global
// memory into the registers mma.sync.m16n8k16 wants.  The k index inside one instruction is
// permuted the same way for both operands (a lane's 8 consecutive elements serve k-slots
// {2t,2t+1,2t+8,2t+9} of two instructions), which leaves the dot products unchanged.
// The activation rows (at most 64 x K) come through L1/L2.  Partial sums of the 8 warps meet in
// shared memory; the epilogue stores, adds into the float residual stream, or applies SwiGLU to
// rows stored as 8 gate rows followed by the 8 up rows of the same channels.
#include <stdlib.h>

#include "api.h"
#include "common.cuh"

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define SK_NORM_ROWS 16

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16816(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A norm shared between two products.  RMSNorm is y = x * w / rms(x): the product that last adds
// into the residual stream x can also write x * w (bfloat16) and, per group of its output columns,
// the sum of x^2; the product that reads y takes x * w as its activation and multiplies its results
// by 1 / rms, which it gets from those partial sums.  No kernel between the two, no pass over x.
struct SkinnyNorm {
  const float* in_sumsq;   // consumer: [in_parts][SK_NORM_ROWS] partial sums of x^2 of the activation rows, or null
  int in_parts;
  float in_eps;            // 1/rms = rsqrt(sum / K + eps)
  const float* out_w;      // producer (residual epilogue): the next norm's weight [N], or null
  bf16* out_xw;            // [M, out_ld] = residual * out_w
  int out_ld;
  float* out_sumsq;        // [units][SK_NORM_ROWS]
};

// NT: 8-token tiles (M <= 8 * NT).  RG: groups of 16 weight rows per CTA; a warp multiplies each
// activation fragment it loads with RG weight fragments, so the activation traffic per weight byte
// falls with RG (with 16 rows per CTA and 8 tokens it is half the weight traffic).  UNROLL: k steps
// of 32 per batch of loads; two batches are in flight.
template <int NT, int RG, int UNROLL, int EPI, bool NORM>
__global__ void __launch_bounds__(SK_THREADS, (NT * RG <= 2) ? 3 : 2)
gemm_skinny_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw, void* Cv, int ldc,
                   int M, int N, int K, int units_per_cta, SkinnyNorm nm) {
  // A unit is 16 * RG weight rows.  A CTA walks units_per_cta consecutive units, so that the grid is
  // no larger than what the GPU holds at once (no partly filled last wave) and every CTA streams
  // the same number of bytes; the first weight loads of the next unit are issued before the
  // current unit's partial sums are combined.
  __shared__ float red[SK_WARPS][16 * RG][NT * 8 + 1];
  __shared__ float inv_rms[NORM ? SK_NORM_ROWS : 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_units = (N + 16 * RG - 1) / (16 * RG);
  int unit = blockIdx.x * units_per_cta;
  const bf16* w_lo[RG];
  const bf16* w_hi[RG];
  bool lo_ok[RG], hi_ok[RG];
  auto set_rows = [&](int u) {
#pragma unroll
    for (int rg = 0; rg < RG; ++rg) {
      const int r_lo = (u * RG + rg) * 16 + g, r_hi = r_lo + 8;
      lo_ok[rg] = r_lo < N;
      hi_ok[rg] = r_hi < N;
      w_lo[rg] = W + (size_t)(lo_ok[rg] ? r_lo : 0) * ldw;
      w_hi[rg] = W + (size_t)(hi_ok[rg] ? r_hi : 0) * ldw;
    }
  };
  const int ksteps = (K + 31) >> 5;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // Weights never depend on the previous kernel: the first batch of loads is issued before the
  // wait on it, and every later batch is issued before the batch in hand is multiplied.
  uint4 wa[RG][UNROLL], wb[RG][UNROLL], na[RG][UNROLL], nb[RG][UNROLL];
  auto load_w = [&](int ks0, uint4 (*ra)[UNROLL], uint4 (*rb)[UNROLL]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (ks0 + u * SK_WARPS) * 32 + 8 * t;
      const bool ok = k < K;  // K is a multiple of 8: a lane's 8 elements are all inside or all outside
#pragma unroll
      for (int rg = 0; rg < RG; ++rg) {
        ra[rg][u] = (ok && lo_ok[rg]) ? ld_stream16(w_lo[rg] + k) : zero;
        rb[rg][u] = (ok && hi_ok[rg]) ? ld_stream16(w_hi[rg] + k) : zero;
      }
    }
  };
  set_rows(unit);
  load_w(warp, wa, wb);
  pdl_wait();
  if (NORM) {
    // 1 / rms of the activation rows from the producer's partial sums: warp w sums rows w and w + 8
    // in a fixed order; the first __syncthreads() before an epilogue publishes them
    for (int m = warp; m < NT * 8; m += SK_WARPS) {
      float sum = 0.0f;
      if (nm.in_sumsq != nullptr && m < M)
        for (int i = lane; i < nm.in_parts; i += 32) sum += nm.in_sumsq[(size_t)i * SK_NORM_ROWS + m];
      sum = warp_sum(sum);
      if (lane == 0) inv_rms[m] = nm.in_sumsq != nullptr ? rsqrtf(sum / (float)K + nm.in_eps) : 1.0f;
    }
  }
  for (int iu = 0; iu < units_per_cta && unit < n_units; ++iu, ++unit) {
    const int row0 = unit * 16 * RG;
    float acc[RG][NT][4];
#pragma unroll
    for (int rg = 0; rg < RG; ++rg)
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[rg][i][j] = 0.0f;

    for (int ks0 = warp; ks0 < ksteps; ks0 += SK_WARPS * UNROLL) {
      load_w(ks0 + SK_WARPS * UNROLL, na, nb);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = (ks0 + u * SK_WARPS) * 32 + 8 * t;
        const bool ok = k < K;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int m = nt * 8 + g;
          uint4 x = zero;
          if (ok && m < M) x = __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k));
#pragma unroll
          for (int rg = 0; rg < RG; ++rg) {
            mma_bf16_16816(acc[rg][nt], wa[rg][u].x, wb[rg][u].x, wa[rg][u].y, wb[rg][u].y, x.x, x.y);
            mma_bf16_16816(acc[rg][nt], wa[rg][u].z, wb[rg][u].z, wa[rg][u].w, wb[rg][u].w, x.z, x.w);
          }
        }
      }
#pragma unroll
      for (int rg = 0; rg < RG; ++rg)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          wa[rg][u] = na[rg][u];
          wb[rg][u] = nb[rg][u];
        }
    }
    if (iu + 1 < units_per_cta && unit + 1 < n_units) {   // the next unit's first batch, under this unit's reduction
      set_rows(unit + 1);
      load_w(warp, wa, wb);
    } else {
      // this CTA's last weights are in: the next kernel's CTAs may take the places that free up and
      // fetch their own first weights while the partial sums here are combined.  Not earlier: CTAs
      // that wait on an SM take issue slots from the ones that still work there.
      pdl_launch();
    }
    // accumulator layout: acc[..][nt][0..1] = (weight row g, tokens nt*8 + 2t, 2t+1); [2..3] = row g+8
#pragma unroll
    for (int rg = 0; rg < RG; ++rg)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[warp][rg * 16 + g][nt * 8 + 2 * t] = acc[rg][nt][0];
        red[warp][rg * 16 + g][nt * 8 + 2 * t + 1] = acc[rg][nt][1];
        red[warp][rg * 16 + g + 8][nt * 8 + 2 * t] = acc[rg][nt][2];
        red[warp][rg * 16 + g + 8][nt * 8 + 2 * t + 1] = acc[rg][nt][3];
      }
    __syncthreads();
    if (EPI == HB_EPI_SWIGLU) {
      // per group of 16 rows: 8 channels x (NT*8) tokens; output column = (row group) * 8 + channel
      for (int idx = threadIdx.x; idx < RG * 8 * NT * 8; idx += SK_THREADS) {
        const int ch = idx & 7, rg = (idx >> 3) % RG, m = idx / (8 * RG);
        if (m >= M) continue;
        float gate = 0.0f, up = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
          gate += red[w][rg * 16 + ch][m];
          up += red[w][rg * 16 + ch + 8][m];
        }
        if (NORM) {
          gate *= inv_rms[m];
          up *= inv_rms[m];
        }
        const int col = (unit * RG + rg) * 8 + ch;
        if (row0 + rg * 16 + ch + 8 < N) ((bf16*)Cv)[(size_t)m * ldc + col] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
      }
    } else {
      // 16 * RG * NT * 8 is a multiple of 128: whole warps enter an iteration, and the 16 * RG
      // consecutive lanes that share a token row can sum over their columns with shuffles
      for (int idx = threadIdx.x; idx < 16 * RG * NT * 8; idx += SK_THREADS) {
        const int r = idx % (16 * RG), m = idx / (16 * RG);
        const int n = row0 + r;
        const bool ok = m < M && n < N;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) s += red[w][r][m];
        if (NORM) s *= inv_rms[m];
        const size_t o = (size_t)m * ldc + n;
        float sq = 0.0f;
        if (ok) {
          if (EPI == HB_EPI_STORE) ((bf16*)Cv)[o] = __float2bfloat16_rn(s);
          else if (EPI == HB_EPI_STORE_F32) ((float*)Cv)[o] = s;
          else {
            const float v = ((float*)Cv)[o] + s;
            ((float*)Cv)[o] = v;
            if (NORM && nm.out_w != nullptr) {
              nm.out_xw[(size_t)m * nm.out_ld + n] = __float2bfloat16_rn(v * nm.out_w[n]);
              sq = v * v;
            }
          }
        }
        if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr) {
#pragma unroll
          for (int d = 1; d < 16 * RG; d <<= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
          if (r == 0 && m < SK_NORM_ROWS) nm.out_sumsq[(size_t)unit * SK_NORM_ROWS + m] = sq;
        }
      }
    }
    __syncthreads();   // the partial sums are read: the next unit may overwrite them
  }
}

template <int NT, int RG, int UNROLL, bool NORM = false>
static int skinny_launch(const bf16* A, int lda, const bf16* W, int ldw, void* C, int ldc, int M, int N, int K,
                         int epi, cudaStream_t s, SkinnyNorm nm = SkinnyNorm{}) {
  // as many CTAs as the GPU holds at once (asked of the runtime for this instantiation), each with
  // an equal run of units
  static int slots = 0;
  if (slots == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_skinny_kernel<NT, RG, UNROLL, HB_EPI_STORE, NORM>, SK_THREADS, 0) != cudaSuccess || per_sm <= 0) per_sm = 2;
    slots = per_sm * sms;
  }
  const int n_units = ceil_div(N, 16 * RG);
  // fewer than one and a half waves: one unit per CTA keeps more loads in flight than halving the grid
  const int upc = (2 * n_units > 3 * slots) ? ceil_div(n_units, slots) : 1;
  const unsigned grid = (unsigned)ceil_div(n_units, upc);
  switch (epi) {
    case HB_EPI_STORE: hb_launch_pdl(gemm_skinny_kernel<NT, RG, UNROLL, HB_EPI_STORE, NORM>, dim3(grid), dim3(SK_THREADS), 0, s, A, lda, W, ldw, C, ldc, M, N, K, upc, nm); break;
    case HB_EPI_STORE_F32: hb_launch_pdl(gemm_skinny_kernel<NT, RG, UNROLL, HB_EPI_STORE_F32, NORM>, dim3(grid), dim3(SK_THREADS), 0, s, A, lda, W, ldw, C, ldc, M, N, K, upc, nm); break;
    case HB_EPI_RESIDUAL: hb_launch_pdl(gemm_skinny_kernel<NT, RG, UNROLL, HB_EPI_RESIDUAL, NORM>, dim3(grid), dim3(SK_THREADS), 0, s, A, lda, W, ldw, C, ldc, M, N, K, upc, nm); break;
    case HB_EPI_SWIGLU: hb_launch_pdl(gemm_skinny_kernel<NT, RG, UNROLL, HB_EPI_SWIGLU, NORM>, dim3(grid), dim3(SK_THREADS), 0, s, A, lda, W, ldw, C, ldc, M, N, K, upc, nm); break;
    default: HB_FAIL(2, "gemm_skinny: unknown epilogue %d", epi);
  }
  HB_CHECK_LAUNCH("gemm_skinny");
  return 0;
}

// epi HB_EPI_SWIGLU: W holds 2I rows in groups of 16 (8 gate, 8 up); C is [M, I] bfloat16.
// Two row groups per CTA halve the activation traffic and double the loads a CTA has in flight;
// worth it where there are enough rows that the grid still fills the GPU (gate/up at one row:
// 38.7 -> 34.3 us).
static bool skinny_two_groups(int M, int N) { return M <= 16 && N >= 8192; }

extern "C" int hb_gemm_skinny_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
                                   int K, int epi, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_skinny: sizes must be positive");
  HB_REQUIRE(M <= 64, "gemm_skinny: at most 64 activation rows, got %d", M);
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_skinny: K (%d) and the leading dimensions (%d, %d) must be multiples of 8", K, lda, ldw);
  HB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_skinny: operands must be 16-byte aligned");
  HB_REQUIRE(epi != HB_EPI_SWIGLU || N % 16 == 0, "gemm_skinny: SwiGLU rows come in groups of 16, N=%d", N);
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* a = (const bf16*)A;
  const bf16* w = (const bf16*)W;
  const bool two = skinny_two_groups(M, N);
  if (M <= 8) return two ? skinny_launch<1, 2, 2>(a, lda, w, ldw, C, ldc, M, N, K, epi, s)
                         : skinny_launch<1, 1, 4>(a, lda, w, ldw, C, ldc, M, N, K, epi, s);
  if (M <= 16) return two ? skinny_launch<2, 2, 2>(a, lda, w, ldw, C, ldc, M, N, K, epi, s)
                          : skinny_launch<2, 1, 4>(a, lda, w, ldw, C, ldc, M, N, K, epi, s);
  if (M <= 32) return skinny_launch<4, 1, 2>(a, lda, w, ldw, C, ldc, M, N, K, epi, s);
  return skinny_launch<8, 1, 2>(a, lda, w, ldw, C, ldc, M, N, K, epi, s);
}

// How many groups of output columns the product of an [M, K] activation with an [N, K] matrix
// writes partial sums for (the first dimension of out_sumsq).
extern "C" int hb_gemm_skinny_norm_parts(int M, int N) {
  return ceil_div(N, skinny_two_groups(M, N) ? 32 : 16);
}

// The same product with a shared norm on either side (M <= 16):
//   in_sumsq != null: A holds x * w of a norm over K; results are multiplied by 1 / rms of the rows,
//     rms^2 = sum over in_parts partial sums / K + in_eps;
//   out_w != null (epi HB_EPI_RESIDUAL): besides C += ..., out_xw = C * out_w (bfloat16) and
//     out_sumsq[hb_gemm_skinny_norm_parts(M, N)][16] = partial sums of C^2.
extern "C" int hb_gemm_skinny_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M,
                                        int N, int K, int epi, const float* in_sumsq, int in_parts, float in_eps,
                                        const float* out_w, void* out_xw, int out_ld, float* out_sumsq,
                                        void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_skinny_norm: sizes must be positive");
  HB_REQUIRE(M <= SK_NORM_ROWS, "gemm_skinny_norm: at most %d activation rows, got %d", SK_NORM_ROWS, M);
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_skinny_norm: K (%d) and the leading dimensions (%d, %d) must be multiples of 8", K, lda, ldw);
  HB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_skinny_norm: operands must be 16-byte aligned");
  HB_REQUIRE(epi != HB_EPI_SWIGLU || N % 16 == 0, "gemm_skinny_norm: SwiGLU rows come in groups of 16, N=%d", N);
  HB_REQUIRE(in_sumsq == nullptr || in_parts > 0, "gemm_skinny_norm: partial sums without a count");
  HB_REQUIRE(out_w == nullptr || (epi == HB_EPI_RESIDUAL && out_xw != nullptr && out_sumsq != nullptr),
             "gemm_skinny_norm: the next norm's input is written by the residual epilogue and needs both outputs");
  SkinnyNorm nm{in_sumsq, in_parts, in_eps, out_w, (bf16*)out_xw, out_ld, out_sumsq};
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* a = (const bf16*)A;
  const bf16* w = (const bf16*)W;
  const bool two = skinny_two_groups(M, N);
  if (M <= 8) return two ? skinny_launch<1, 2, 2, true>(a, lda, w, ldw, C, ldc, M, N, K, epi, s, nm)
                         : skinny_launch<1, 1, 4, true>(a, lda, w, ldw, C, ldc, M, N, K, epi, s, nm);
  return two ? skinny_launch<2, 2, 2, true>(a, lda, w, ldw, C, ldc, M, N, K, epi, s, nm)
             : skinny_launch<2, 1, 4, true>(a, lda, w, ldw, C, ldc, M, N, K, epi, s, nm);
}
