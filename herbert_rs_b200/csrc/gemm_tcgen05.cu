// Prefill matrix product on the 5th-generation tensor cores:  C[M,N] (op)= A[M,K] * W[N,K]^T,
// bfloat16 operands (both K-major, as activations and checkpoint weights are stored), float
// accumulation in tensor memory.  It replaces the reference's one-workgroup-per-output-element
// shader (backends/backend_vulkan bf16_matmul.comp) and its AVX-512 tile kernel
// (backends/backend_bf16_avx512/src/avx512_bf16_matvec.S: avx512_bf16_matmul_tile).
//
// One CTA computes one 128 x BN tile of C (BN = 128 or 256):
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a 128 x 64 slab
//            of A and a BN x 64 slab of W per pipeline stage, signalling an mbarrier per stage;
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=16) four times
//            per stage and commits the stage's "empty" barrier, then the "accumulator ready" one;
//   warps 2-5  read the accumulator with tcgen05.ld (each warp its 32 lanes = 32 rows of C) and
//            apply the epilogue: store, store as float, add into the float residual stream, or
//            SwiGLU over column groups of 8 gate + 8 up.
// No thread-block clusters and no multicast are used.  Rows/columns beyond M, N, K are
// zero-filled by TMA on load and skipped on store.  Every wait on an mbarrier is bounded; a wait
// that runs out sets *error_flag and the CTA winds down (tensor memory is always released).
#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

#define TG_BM 128
#define TG_THREADS 192
#define HB_EPI_SWIGLU 3

template <int BN>
struct TgSmem {
  static constexpr int kStageBytes = (TG_BM + BN) * TG_BK * 2;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* Cv,
                    int ldc, int M, int N, int K, int* error_flag) {
  constexpr int STAGES = TgSmem<BN>::kStages;
  constexpr int STAGE_BYTES = TgSmem<BN>::kStageBytes;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // swizzled tiles want 1024-byte alignment
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bars = base + STAGES * STAGE_BYTES;                  // full[STAGES], empty[STAGES], acc, tmem slot
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8);
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
  const unsigned acc_bar = bars + 2 * STAGES * 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TG_BM, n0 = blockIdx.y * BN;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const unsigned tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(empty_bar(s), ((kb / STAGES) - 1) & 1)) {
          atomicExch(error_flag, 1);
          break;
        }
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        const unsigned a_dst = base + s * STAGE_BYTES;
        tma_load_2d(a_dst, &map_a, kb * TG_BK, m0, full_bar(s));
        tma_load_2d(a_dst + TG_BM * TG_BK * 2, &map_w, kb * TG_BK, n0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D float, A and B bfloat16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TG_BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(full_bar(s), (kb / STAGES) & 1)) {
          atomicExch(error_flag, 2);
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned a_addr = base + s * STAGE_BYTES;
        const unsigned w_addr = a_addr + TG_BM * TG_BK * 2;
#pragma unroll
        for (int k = 0; k < TG_BK / 16; ++k) {
          tc_mma_bf16(tmem_acc, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(w_addr + k * 32), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(empty_bar(s));     // arrives when these MMAs have finished reading the stage
      }
      tc_commit(acc_bar);            // arrives when every MMA issued so far is complete
    }
  } else {
    // epilogue warps: TMEM lane quadrant = warp index modulo 4
    const int quad = warp & 3;
    const bool ready = mbar_wait(acc_bar, 0);
    if (!ready && lane == 0) atomicExch(error_flag, 3);
    tc_fence_after();
    const int m = m0 + quad * 32 + lane;
    if (ready) {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        unsigned r[32];
        tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
        const int n = n0 + c * 32;
        if (m < M) {
          if (EPI == HB_EPI_SWIGLU) {
            // columns: [8 gate | 8 up] x 2 -> 16 outputs; output column = n/2 + ...
            bf16* out = (bf16*)Cv + (size_t)m * ldc + (n >> 1);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (n + blk * 16 + 8 + j < N) {
                  const float gate = __uint_as_float(r[blk * 16 + j]), up = __uint_as_float(r[blk * 16 + 8 + j]);
                  out[blk * 8 + j] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
                }
              }
          } else if (EPI == HB_EPI_STORE) {
            bf16* out = (bf16*)Cv + (size_t)m * ldc + n;
            if (n + 32 <= N && ((((size_t)m * ldc + n) & 7) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
                v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
                *reinterpret_cast<uint4*>(out + j) = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n + j < N) out[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* out = (float*)Cv + (size_t)m * ldc + n;
            if (n + 32 <= N && ((((size_t)m * ldc + n) & 3) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                float4* o4 = reinterpret_cast<float4*>(out + j);
                if (EPI == HB_EPI_RESIDUAL) {
                  const float4 old = *o4;
                  v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *o4 = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n + j < N) {
                  if (EPI == HB_EPI_RESIDUAL) out[j] += __uint_as_float(r[j]);
                  else out[j] = __uint_as_float(r[j]);
                }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(BN) : "memory");
  }
}

template <int BN, int EPI>
static int tg_launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int* err,
                     cudaStream_t s) {
  const int smem = TgSmem<BN>::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(ceil_div(M, TG_BM), ceil_div(N, BN));
  hb_launch(gemm_tcgen05_kernel<BN, EPI>, dim3(grid), dim3(TG_THREADS), smem, s, ma, mw, C, ldc, M, N, K, err);
  HB_CHECK_LAUNCH("gemm_tcgen05");
  return 0;
}

template <int BN>
static int tg_dispatch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int epi,
                       int* err, cudaStream_t s) {
  switch (epi) {
    case HB_EPI_STORE: return tg_launch<BN, HB_EPI_STORE>(ma, mw, C, ldc, M, N, K, err, s);
    case HB_EPI_STORE_F32: return tg_launch<BN, HB_EPI_STORE_F32>(ma, mw, C, ldc, M, N, K, err, s);
    case HB_EPI_RESIDUAL: return tg_launch<BN, HB_EPI_RESIDUAL>(ma, mw, C, ldc, M, N, K, err, s);
    case HB_EPI_SWIGLU: return tg_launch<BN, HB_EPI_SWIGLU>(ma, mw, C, ldc, M, N, K, err, s);
  }
  HB_FAIL(2, "gemm_tcgen05: unknown epilogue %d", epi);
}

// error_flag: one int in device memory, zero before the call; non-zero afterwards means a bounded
// wait ran out inside the kernel (1 producer, 2 MMA issuer, 3 epilogue) and C is not valid.
extern "C" int hb_gemm_tcgen05_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
                                    int K, int epi, int* error_flag, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: sizes must be positive");
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05: K (%d) and the leading dimensions (%d, %d) must be multiples of 8 (16-byte rows for TMA)", K, lda, ldw);
  HB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
  HB_REQUIRE(epi != HB_EPI_SWIGLU || N % 16 == 0, "gemm_tcgen05: SwiGLU columns come in groups of 16, N=%d", N);
  HB_REQUIRE(error_flag != nullptr, "gemm_tcgen05: an error flag is required");
  CUtensorMap ma, mw;
  const int BN = N > 128 ? 256 : 128;
  int rc = make_map(&ma, A, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, BN);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  return BN == 256 ? tg_dispatch<256>(ma, mw, C, ldc, M, N, K, epi, error_flag, s)
                   : tg_dispatch<128>(ma, mw, C, ldc, M, N, K, epi, error_flag, s);
}
