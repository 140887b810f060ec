// Plain tiled matrix product on the CUDA cores, any sizes:  C[M,N] (op)= A[M,K] * W[N,K]^T.
//
// This is the product of the true 32-bit path (float operands, float FMA, no tensor cores and
// no reduced-precision mode), and the any-shape fallback of the bfloat16 path (bf16 operands
// widened exactly, float accumulation).  The reference's scalar product has the same contract:
// C[m,n] = sum_k A[m,k] * W[n,k] with f32 accumulation (backend_bf16/src/kernels.rs:95-143).
//
// 64x64 output tile, 16-wide k slab, 256 threads, 4x4 outputs per thread.  Edges are guarded
// element by element, so M, N and K need not be multiples of anything.
#include "api.h"
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw, void* Cv, int ldc,
                 int M, int N, int K) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[TK][TN + 4];
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = tid & 15, ty = tid >> 4;  // outputs: rows ty*4.., cols tx*4..
  const int lrow = tid >> 2, lk = (tid & 3) * 4;  // loads: 64 rows x 4 groups of 4 k
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += TK) {
    {
      const int m = m0 + lrow;
      const T* p = A + (size_t)m * lda + k0 + lk;
#pragma unroll
      for (int q = 0; q < 4; ++q) As[lk + q][lrow] = (m < M && k0 + lk + q < K) ? to_f32(p[q]) : 0.0f;
      const int n = n0 + lrow;
      const T* pw = W + (size_t)n * ldw + k0 + lk;
#pragma unroll
      for (int q = 0; q < 4; ++q) Ws[lk + q][lrow] = (n < N && k0 + lk + q < K) ? to_f32(pw[q]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const size_t o = (size_t)m * ldc + n;
      if (EPI == HB_EPI_STORE) ((T*)Cv)[o] = from_f32<T>(acc[i][j]);
      else if (EPI == HB_EPI_STORE_F32) ((float*)Cv)[o] = acc[i][j];
      else ((float*)Cv)[o] += acc[i][j];
    }
  }
}

template <typename T>
static int gemm_simt_launch(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
                            int K, int epi, void* stream) {
  dim3 grid(ceil_div(N, TN), ceil_div(M, TM));
  HB_REQUIRE(grid.y <= 65535, "gemm: too many rows (%d)", M);
  cudaStream_t s = (cudaStream_t)stream;
  switch (epi) {
    case HB_EPI_STORE:
      hb_launch(gemm_simt_kernel<T, HB_EPI_STORE>, dim3(grid), dim3(256), 0, s, (const T*)A, lda, (const T*)W, ldw, C, ldc, M, N, K);
      break;
    case HB_EPI_STORE_F32:
      hb_launch(gemm_simt_kernel<T, HB_EPI_STORE_F32>, dim3(grid), dim3(256), 0, s, (const T*)A, lda, (const T*)W, ldw, C, ldc, M, N, K);
      break;
    case HB_EPI_RESIDUAL:
      hb_launch(gemm_simt_kernel<T, HB_EPI_RESIDUAL>, dim3(grid), dim3(256), 0, s, (const T*)A, lda, (const T*)W, ldw, C, ldc, M, N, K);
      break;
    default:
      HB_FAIL(2, "gemm: unknown epilogue %d", epi);
  }
  HB_CHECK_LAUNCH("gemm_simt");
  return 0;
}

extern "C" int hb_gemm_simt(int dtype, const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                            int M, int N, int K, int epi, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: sizes must be positive (M=%d N=%d K=%d)", M, N, K);
  HB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: leading dimensions too small");
  return dtype == HB_F32 ? gemm_simt_launch<float>(A, lda, W, ldw, C, ldc, M, N, K, epi, stream)
                         : gemm_simt_launch<bf16>(A, lda, W, ldw, C, ldc, M, N, K, epi, stream);
}
