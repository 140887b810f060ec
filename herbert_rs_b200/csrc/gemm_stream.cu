// Weight-streaming matrix product for decode steps on the 5th-generation tensor cores:
//   C[M,N] (op)= X[M,K] * W[N,K]^T   for M <= 64 rows of activations (one per sequence).
//
// A decode step reads every weight exactly once, so this kernel is built around that stream (the
// reference's matvec kernels have the same premise: backends/backend_vulkan bf16_matvec.comp, one
// pass over W per token; backends/backend_bf16_avx512/src/avx512_bf16_matvec.S).  The roles of
// the operands are swapped: 128 weight rows are the M side of tcgen05.mma, the few activation
// rows (padded to 16, 32, 48 or 64) are its N side, so the tensor cores stay busy however small
// the batch is, and the accumulator (128 lanes x <= 64 columns) sits in tensor memory.
//
// Grid = (tiles of 128 weight rows) x (slices of K).  K is cut into slices so that about as many
// CTAs as the GPU can hold stream at once; TMA keeps a ring of 4-6 stages (16 KiB of weights each)
// in flight per CTA.  The slices of one tile are combined without waiting on one another: every
// CTA writes its partial tile to scratch memory and bumps the tile's counter; the CTA that arrives
// last sums all partials in slice order (so the result does not depend on arrival order), applies
// the epilogue and resets the counter.  Epilogues: store, store as float, add into the float
// residual stream, SwiGLU over rows stored as 8 gate rows + 8 up rows.
#include <stdlib.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

#define GS_BM 128
#define GS_THREADS 192
#define GS_W_BYTES (GS_BM * TG_BK * 2)
#define GS_MAX_NP 64

__device__ __forceinline__ void tc_ld16(unsigned taddr, float* r) {
  unsigned u[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}

struct StreamArgs {
  void* C;
  int ldc;
  int M, N, K;
  int NP;         // activation rows padded to a multiple of 16
  int stages;
  int tmem_cols;  // 32 or 64
  float* partials;  // [tiles][slices][NP][128]
  int* counters;    // [tiles], zero between launches
  int* error_flag;
};

template <int EPI>
__global__ void __launch_bounds__(GS_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, StreamArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const int STAGES = a.stages;
  const int stage_bytes = GS_W_BYTES + a.NP * TG_BK * 2;
  const unsigned bars = base + STAGES * stage_bytes;
  volatile unsigned* slots = reinterpret_cast<volatile unsigned*>(gen + STAGES * stage_bytes + (2 * STAGES + 1) * 8);
  // slots[0]: tensor memory address; slots[1]: "this CTA is the last of its tile"
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
  const unsigned acc_bar = bars + 2 * STAGES * 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, slice = blockIdx.y, S = gridDim.y;
  const int n0 = tile * GS_BM;
  const int num_kb = (a.K + TG_BK - 1) / TG_BK;
  const int kb0 = (int)(((long long)num_kb * slice) / S), kb1 = (int)(((long long)num_kb * (slice + 1)) / S);
  const int my_kb = kb1 - kb0;     // >= 1 because S <= num_kb

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)slots)), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const unsigned tmem_acc = slots[0];

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !mbar_wait(empty_bar(s), ((i / STAGES) - 1) & 1)) {
          atomicExch(a.error_flag, 11);
          break;
        }
        mbar_expect_tx(full_bar(s), stage_bytes);
        const unsigned dst = base + s * stage_bytes;
        tma_load_2d(dst, &map_w, (kb0 + i) * TG_BK, n0, full_bar(s));
        tma_load_2d(dst + GS_W_BYTES, &map_x, (kb0 + i) * TG_BK, 0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(a.NP >> 3) << 17) | ((unsigned)(GS_BM >> 4) << 24);
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(full_bar(s), (i / STAGES) & 1)) {
          atomicExch(a.error_flag, 12);
          break;
        }
        tc_fence_after();
        const unsigned w_addr = base + s * stage_bytes;
        const unsigned x_addr = w_addr + GS_W_BYTES;
#pragma unroll
        for (int k = 0; k < TG_BK / 16; ++k)
          tc_mma_bf16(tmem_acc, umma_desc_sw128(w_addr + k * 32), umma_desc_sw128(x_addr + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty_bar(s));
      }
      tc_commit(acc_bar);
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;       // row of the tile = weight row n0 + r = output column
    const int n = n0 + r;
    const bool ready = mbar_wait(acc_bar, 0);
    if (!ready && lane == 0) atomicExch(a.error_flag, 13);
    tc_fence_after();
    float acc[GS_MAX_NP];
#pragma unroll
    for (int c = 0; c < GS_MAX_NP / 16; ++c) {
      if (c * 16 < a.NP) {
        if (ready) tc_ld16(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 16), acc + c * 16);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = 0.0f;
        }
      }
    }
    bool finish = true;
    if (S > 1) {
      float* mine = a.partials + ((size_t)tile * S + slice) * a.NP * GS_BM;
#pragma unroll
      for (int c = 0; c < GS_MAX_NP; ++c)
        if (c < a.NP) mine[(size_t)c * GS_BM + r] = acc[c];
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const int old = atomicAdd(a.counters + tile, 1);
        const unsigned last = (old == S - 1) ? 1u : 0u;
        if (last) a.counters[tile] = 0;      // every slice has arrived: ready for the next launch
        slots[1] = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      finish = slots[1] != 0u;
      if (finish) {
        __threadfence();
        const float* all = a.partials + (size_t)tile * S * a.NP * GS_BM + r;
#pragma unroll
        for (int c = 0; c < GS_MAX_NP; ++c) acc[c] = 0.0f;
        // one slice at a time, in slice order; within a slice every load is independent of the others
        for (int sl = 0; sl < S; ++sl) {
          const float* p = all + (size_t)sl * a.NP * GS_BM;
#pragma unroll
          for (int c0 = 0; c0 < GS_MAX_NP; c0 += 16) {
            if (c0 < a.NP) {
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __ldcg(p + (size_t)(c0 + j) * GS_BM);
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[c0 + j] += v[j];
            }
          }
        }
      }
    }
    if (finish) {
      if (EPI == HB_EPI_SWIGLU) {
        const int col = (n >> 4) * 8 + (lane & 7);
#pragma unroll
        for (int m = 0; m < GS_MAX_NP; ++m) {
          if (m < a.NP) {
            const float up = __shfl_down_sync(0xffffffffu, acc[m], 8);
            if ((lane & 8) == 0 && m < a.M && n + 8 < a.N) {
              const float gate = acc[m];
              ((bf16*)a.C)[(size_t)m * a.ldc + col] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
            }
          }
        }
      } else if (n < a.N) {
#pragma unroll
        for (int m = 0; m < GS_MAX_NP; ++m) {
          if (m < a.M) {
            const size_t o = (size_t)m * a.ldc + n;
            if (EPI == HB_EPI_STORE) ((bf16*)a.C)[o] = __float2bfloat16_rn(acc[m]);
            else if (EPI == HB_EPI_STORE_F32) ((float*)a.C)[o] = acc[m];
            else ((float*)a.C)[o] += acc[m];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(a.tmem_cols) : "memory");
  }
}

static int stream_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

struct StreamPlan {
  int NP, stages, smem, tiles, slices, tmem_cols;
};

static StreamPlan stream_plan(int M, int N, int K) {
  StreamPlan p;
  p.NP = ((M + 15) / 16) * 16;
  const int stage_bytes = GS_W_BYTES + p.NP * TG_BK * 2;
  p.stages = (110 * 1024) / stage_bytes;          // two CTAs per SM
  if (p.stages > 8) p.stages = 8;
  p.smem = p.stages * stage_bytes + 1024 + 256;
  p.tiles = ceil_div(N, GS_BM);
  const int num_kb = ceil_div(K, TG_BK);
  const int slots = stream_sm_count() * 2;
  const int max_slices = 2;        // measured: more slices cost more in the ordered reduction than they gain
  int s = slots / p.tiles;
  if (s > max_slices) s = max_slices;
  if (s > num_kb / 2) s = num_kb / 2;             // at least two k blocks per slice
  if (s < 1) s = 1;
  p.slices = s;
  p.tmem_cols = p.NP <= 32 ? 32 : 64;
  return p;
}

// Floats of scratch and number of counters a call needs (0 floats when K is not cut).
extern "C" long long hb_gemm_stream_scratch_floats(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || M > GS_MAX_NP) return 0;
  StreamPlan p = stream_plan(M, N, K);
  return p.slices > 1 ? (long long)p.tiles * p.slices * p.NP * GS_BM : 0;
}
extern "C" int hb_gemm_stream_counters(int N) { return ceil_div(N, GS_BM); }

template <int EPI>
static int stream_launch(const CUtensorMap& mw, const CUtensorMap& mx, const StreamArgs& a, const StreamPlan& p, cudaStream_t s) {
  static int configured = 0;
  if (configured < p.smem) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    if (e != cudaSuccess) HB_FAIL(3, "gemm_stream: cannot reserve shared memory: %s", cudaGetErrorString(e));
    configured = 112 * 1024;
  }
  dim3 grid(p.tiles, p.slices);
  hb_launch(gemm_stream_kernel<EPI>, dim3(grid), dim3(GS_THREADS), p.smem, s, mw, mx, a);
  HB_CHECK_LAUNCH("gemm_stream");
  return 0;
}

// counters: hb_gemm_stream_counters(N) ints, zero before the first call (the kernel leaves them zero).
// scratch: hb_gemm_stream_scratch_floats(M, N, K) floats (may be null when that is 0).
extern "C" int hb_gemm_stream_bf16(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                   int epi, float* scratch, long long scratch_floats, int* counters, int n_counters,
                                   int* error_flag, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_stream: sizes must be positive");
  HB_REQUIRE(M <= GS_MAX_NP, "gemm_stream: at most %d activation rows, got %d", GS_MAX_NP, M);
  HB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_stream: K (%d) and the leading dimensions (%d, %d) must be multiples of 8 (16-byte rows for TMA)", K, ldx, ldw);
  HB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_stream: operands must be 16-byte aligned");
  HB_REQUIRE(epi != HB_EPI_SWIGLU || N % 16 == 0, "gemm_stream: SwiGLU rows come in groups of 16, N=%d", N);
  HB_REQUIRE(error_flag != nullptr, "gemm_stream: an error flag is required");
  const StreamPlan p = stream_plan(M, N, K);
  if (p.slices > 1) {
    HB_REQUIRE(scratch != nullptr && scratch_floats >= (long long)p.tiles * p.slices * p.NP * GS_BM,
               "gemm_stream: scratch too small (%lld floats given)", scratch_floats);
    HB_REQUIRE(counters != nullptr && n_counters >= p.tiles, "gemm_stream: %d counters needed, %d given", p.tiles, n_counters);
  }
  CUtensorMap mw, mx;
  int rc = make_map(&mw, W, N, K, ldw, GS_BM);
  if (rc) return rc;
  rc = make_map(&mx, X, M, K, ldx, p.NP);
  if (rc) return rc;
  StreamArgs a{C, ldc, M, N, K, p.NP, p.stages, p.tmem_cols, scratch, counters, error_flag};
  cudaStream_t s = (cudaStream_t)stream;
  switch (epi) {
    case HB_EPI_STORE: return stream_launch<HB_EPI_STORE>(mw, mx, a, p, s);
    case HB_EPI_STORE_F32: return stream_launch<HB_EPI_STORE_F32>(mw, mx, a, p, s);
    case HB_EPI_RESIDUAL: return stream_launch<HB_EPI_RESIDUAL>(mw, mx, a, p, s);
    case HB_EPI_SWIGLU: return stream_launch<HB_EPI_SWIGLU>(mw, mx, a, p, s);
  }
  HB_FAIL(2, "gemm_stream: unknown epilogue %d", epi);
}
