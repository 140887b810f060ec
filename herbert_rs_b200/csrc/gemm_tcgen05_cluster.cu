// Products that cut K over a thread-block cluster: few rows, or few tiles (see gemm_tcgen05.cu for
// the kernels that walk whole tiles and for the entry points that choose between them).
#include "gemm_tcgen05_parts.cuh"

// ---------------------------------------------------------------------------------------------
// At most 128 rows (a decode batch, a short prompt) against a matrix with few tiles of output
// columns: the time is the weight stream's, and a tile per CTA would leave most SMs without work.
// Here a thread-block cluster of S CTAs owns a tile and each CTA a range of K.  A CTA streams its
// range through the ring into one accumulator and then sends every row of it, as floats, into the
// shared memory of the CTA that finishes that row (rows are dealt in S blocks; stores through
// distributed shared memory, which nobody waits for).  After one cluster barrier every CTA adds the
// S partial rows it was sent, in the order of their k ranges, and runs the epilogue from its own
// shared memory.  No workspace in global memory, no counters, nobody finishes alone, and no
// multicast: every CTA loads its own slabs.  Up to 64 rows, the activation slab of a stage is 64
// rows; the tensor cores still multiply 128, and what they make of the rows beyond (the weight slab
// behind it) is never stored.
#define TGK_RING_BYTES (225 * 1024)      // per CTA: the ring of stages and, behind it, the rows it is sent
#define TGK_SMEM_BYTES (TGK_RING_BYTES + 1024 + 256)
#define TGK_MAX_STAGES 8

struct TgKsplit {
  int bn;         // output columns per tile: 128, 192 or 256 (whole halves of 128-column tiles: a following norm's partial sums are kept per 64 columns)
  int ways;       // CTAs per tile = size of the cluster; 0: this product does not go that way
  int a_rows;     // rows of the activation slab per stage: 64 or 128
  int stages;
  int rows_per;   // rows each CTA finishes
};

template <int EPI, bool NORM>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_ksplit_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* Cv,
                           int ldc, int M, int N, int K, TgKsplit plan, int* error_flag, TgNorm nm) {
  const int bn = plan.bn, STAGES = plan.stages, rows_per = plan.rows_per;
  const int a_bytes = plan.a_rows * TG_BK * 2, STAGE_BYTES = a_bytes + bn * TG_BK * 2;
  const int row_floats = bn + 4;      // a partial row in shared memory, padded against bank conflicts
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const int recv_off = STAGES * STAGE_BYTES;                 // [S][rows_per][row_floats] floats: what the cluster sends this CTA
  const unsigned bars = base + TGK_RING_BYTES;               // full[8], empty[8], acc_full; then the tensor-memory slot
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + TGK_RING_BYTES + (2 * TGK_MAX_STAGES + 1) * 8);
  auto full_bar = [&](int st) { return bars + st * 8; };
  auto empty_bar = [&](int st) { return bars + (TGK_MAX_STAGES + st) * 8; };
  const unsigned acc_full = bars + 2 * TGK_MAX_STAGES * 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank(), S = (int)cluster_nctarank();
  const int n0 = (int)cluster_id_x() * bn;
  const int num_kb = (K + TG_BK - 1) / TG_BK;
  const int kb0 = (int)(((long long)num_kb * rank) / S), kb1 = (int)(((long long)num_kb * (rank + 1)) / S);
  const unsigned tmem_cols = bn <= 128 ? 128u : 256u;
  float first_inv_rms = 1.0f;

  if (threadIdx.x == 0) {
    for (int st = 0; st < STAGES; ++st) {
      mbar_init(full_bar(st), 1);
      mbar_init(empty_bar(st), 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_arrive();                 // "this CTA runs": waited for before anything is sent to it
  pdl_wait();
  const unsigned tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0, st = it % STAGES;
        if (it >= STAGES && !mbar_wait(empty_bar(st), ((it / STAGES) - 1) & 1)) {
          atomicExch(error_flag, 21);
          break;
        }
        mbar_expect_tx(full_bar(st), STAGE_BYTES);
        const unsigned a_dst = base + st * STAGE_BYTES;
        tma_load_2d(a_dst, &map_a, kb * TG_BK, 0, full_bar(st));
        tma_load_2d(a_dst + a_bytes, &map_w, kb * TG_BK, n0, full_bar(st));
      }
    }
    __syncwarp();
    cluster_wait();
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(TG_BM >> 4) << 24);
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0, st = it % STAGES;
        if (!mbar_wait(full_bar(st), (it / STAGES) & 1)) {
          atomicExch(error_flag, 22);
          break;
        }
        tc_fence_after();
        const unsigned a_addr = base + st * STAGE_BYTES;
        const unsigned w_addr = a_addr + a_bytes;
#pragma unroll
        for (int k = 0; k < TG_BK / 16; ++k)
          tc_mma_bf16(tmem_acc, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(w_addr + k * 32), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        tc_commit(empty_bar(st));
      }
      tc_commit(acc_full);          // arrives when every MMA is complete
    }
    __syncwarp();
    cluster_wait();
  } else {
    // row m of this CTA's partial tile goes to the CTA that finishes it: slot [this rank][m - first row of that CTA]
    const int quad = warp & 3, m = quad * 32 + lane;
    const int chunks = bn >> 5, first = (chunks + 1) >> 1;
    const int c_lo = warp < 6 ? 0 : first, c_hi = warp < 6 ? first : chunks;
    // While the tensor cores work: what the first piece of a row this thread finishes will need from
    // global memory (1 / rms of the row; the residual and the next norm's weights into L1).
    if (S == 1) {
      if (NORM && nm.in_sumsq != nullptr && m < M) {
        float sum = 0.0f;
        for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
        first_inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
      }
    } else {
      const int per_row = EPI == HB_EPI_SWIGLU ? chunks : bn >> 3, cols = EPI == HB_EPI_SWIGLU ? 32 : 8;
      const int item = (int)threadIdx.x - 64, frl = item / per_row, fm = rank * rows_per + frl;
      if (frl < rows_per && fm < M) {
        if (NORM && nm.in_sumsq != nullptr) {
          float sum = 0.0f;
          for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + fm];
          first_inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
        }
        const int fn = n0 + (item % per_row) * cols;
        if (fn < N) {
          if (EPI == HB_EPI_RESIDUAL) prefetch_l1((const float*)Cv + (size_t)fm * ldc + fn);
          if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr) prefetch_l1(nm.out_w + fn);
        }
      }
    }
    const bool ready = mbar_wait(acc_full, 0);
    if (!ready && lane == 0) atomicExch(error_flag, 23);
    __syncwarp();
    cluster_wait();
    if (ready && S == 1) {
      // the tile is whole: straight from tensor memory (store and SwiGLU epilogues only: the launcher sees to it)
      tc_fence_after();
      float sq = 0.0f;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        unsigned r[32];
        tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
        tg_epilogue32<EPI, NORM>(r, m, n0 + c * 32, M, N, Cv, ldc, nm, first_inv_rms, sq);
      }
    } else if (ready) {
      tc_fence_after();
      const int owner = m / rows_per;
      const unsigned slot = mapa_shared(base + (unsigned)recv_off + (unsigned)(((rank * rows_per + (m - owner * rows_per)) * row_floats) * 4),
                                        (unsigned)(owner < S ? owner : 0));
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        unsigned r[32];
        tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
        if (m < M) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            st_cluster_f4(slot + (unsigned)((c * 32 + j) * 4), __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
    }
  }
  pdl_launch();                     // this CTA's loads are done: the next kernel's CTAs may take the places that free up
  tc_fence_before();
  cluster_arrive();                 // every row is where it is finished
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(tmem_cols) : "memory");
  } else if (warp >= 2 && S > 1) {
    // rows rank * rows_per ... of the tile; a thread takes 8 columns of a row (32 for SwiGLU), consecutive lanes consecutive columns
    const int idx = (int)threadIdx.x - 64;
    const float* recv = reinterpret_cast<const float*>(gen + recv_off);
    if constexpr (EPI == HB_EPI_SWIGLU) {
      const int chunks = bn >> 5;
      for (int item0 = 0; item0 < rows_per * chunks; item0 += TG_EPI_WARPS * 32) {
        const int item = item0 + idx;
        const int c = item % chunks, rl = item / chunks, m = rank * rows_per + rl;
        if (rl >= rows_per || m >= M) continue;
        float inv_rms = first_inv_rms, sq = 0.0f;
        if (NORM && nm.in_sumsq != nullptr && item0 > 0) {
          float sum = 0.0f;
          for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
          inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
        }
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
        for (int q = 0; q < S; ++q) {           // in the order of the k ranges
          const float4* src = reinterpret_cast<const float4*>(recv + (size_t)(q * rows_per + rl) * row_floats + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = src[j];
            acc[4 * j] += v.x; acc[4 * j + 1] += v.y; acc[4 * j + 2] += v.z; acc[4 * j + 3] += v.w;
          }
        }
        unsigned r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(acc[j]);
        tg_epilogue32<EPI, NORM>(r, m, n0 + c * 32, M, N, Cv, ldc, nm, inv_rms, sq);
      }
    } else {
      const int groups = bn >> 3;                      // a multiple of 8: the 8 lanes of 64 columns sit side by side
      const int n_end = ((N + 127) / 128) * 128;       // the partial sums of a following norm cover whole 128-column tiles
      for (int item0 = 0; item0 < rows_per * groups; item0 += TG_EPI_WARPS * 32) {
        const int item = item0 + idx;
        const int g8 = item % groups, rl = item / groups, m = rank * rows_per + rl;
        const bool active = rl < rows_per && m < M;
        float sq = 0.0f;
        if (active) {
          float inv_rms = first_inv_rms;
          if (NORM && nm.in_sumsq != nullptr && item0 > 0) {
            float sum = 0.0f;
            for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
            inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
          }
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = 0.0f;
          for (int q = 0; q < S; ++q) {         // in the order of the k ranges
            const float4* src = reinterpret_cast<const float4*>(recv + (size_t)(q * rows_per + rl) * row_floats + g8 * 8);
            const float4 x = src[0], y = src[1];
            v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
            v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
          }
          tg_epilogue8<EPI, NORM>(v, m, n0 + g8 * 8, M, N, Cv, ldc, nm, inv_rms, sq);
        }
        if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr) {
          // one sum per row and 64 columns
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          if (active && (g8 & 7) == 0 && n0 + g8 * 8 < n_end) nm.out_sumsq[(size_t)((n0 + g8 * 8) >> 6) * nm.out_stride + m] = sq;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// 129 to about 512 rows against a matrix with few tiles: too few 256 x 256 tiles for the pairs of CTAs,
// and what an SM takes in from L2 per k block bounds every smaller tile.  Here a cluster of 2 S CTAs
// owns a 256 x 256 tile: S pairs, each pair a range of K (tcgen05 with cta_group::2 inside a pair, as
// in the pair kernel above).  When all of them are through (first cluster barrier: every ring is
// free) each CTA sends the rows of its accumulator, as floats, into the ring of the CTA that
// finishes them (the CTAs with the same half of the tile's rows, rows dealt in S blocks); after the
// second cluster barrier every CTA adds the S partial rows it holds in k order and runs the epilogue,
// 8 columns per thread.  No workspace, no counters, no multicast loads.
#define TGQ_STAGES 6
#define TGQ_STAGE_BYTES (2 * TG_BM * TG_BK * 2)
#define TGQ_SMEM_BYTES (TGQ_STAGES * TGQ_STAGE_BYTES + 1024 + 256)
#define TGQ_BN 256
#define TGQ_ROW_FLOATS (TGQ_BN + 4)

__device__ __forceinline__ void tc_commit_pair_of(unsigned bar, unsigned leader) {      // arrives at this barrier in both CTAs of the pair that starts at rank `leader`
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)(3u << leader))
               : "memory");
}

template <int EPI, bool NORM>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_pair_ksplit_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* Cv,
                                int ldc, int M, int N, int K, int rows_per, int part_cols, int* error_flag, TgNorm nm) {
  static_assert(EPI != HB_EPI_SWIGLU, "store and residual epilogues only");
  static_assert((TG_BM + 8) * TGQ_ROW_FLOATS * 4 <= TGQ_STAGES * TGQ_STAGE_BYTES, "the rows a CTA is sent must fit into its ring");
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bars = base + TGQ_STAGES * TGQ_STAGE_BYTES;       // full[STAGES], empty[STAGES], acc_full; then the tensor-memory slot
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + TGQ_STAGES * TGQ_STAGE_BYTES + (2 * TGQ_STAGES + 1) * 8);
  auto full_bar = [&](int st) { return bars + st * 8; };
  auto empty_bar = [&](int st) { return bars + (TGQ_STAGES + st) * 8; };
  const unsigned acc_full = bars + 2 * TGQ_STAGES * 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank(), leader = rank & ~1u, half = rank & 1u;
  const int S = (int)(cluster_nctarank() >> 1), pair = (int)(rank >> 1);
  const int tiles_m = (M + 2 * TG_BM - 1) / (2 * TG_BM);
  const int tile = (int)cluster_id_x();
  const int m0 = (tile % tiles_m) * 2 * TG_BM + (int)half * TG_BM;      // this CTA's 128 rows of the tile
  const int n0 = (tile / tiles_m) * TGQ_BN;
  const int num_kb = (K + TG_BK - 1) / TG_BK;
  const int kb0 = (int)(((long long)num_kb * pair) / S), kb1 = (int)(((long long)num_kb * (pair + 1)) / S);

  if (threadIdx.x == 0) {
    for (int st = 0; st < TGQ_STAGES; ++st) {
      mbar_init(full_bar(st), 1);     // the pair's first CTA arms it with both CTAs' bytes
      mbar_init(empty_bar(st), 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TGQ_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();               // every CTA's barriers are initialised before its peer signals them
  tc_fence_after();
  pdl_wait();
  const unsigned tmem_acc = *tmem_slot;
  const bool tmem_ok = tmem_acc == 0u;        // the pair's two CTAs must hold their accumulators at one address: the first allocation of an empty SM
  if (!tmem_ok && threadIdx.x == 0) atomicExch(error_flag, 35);
  float first_inv_rms = 1.0f;
  bool ready = false;

  if (!tmem_ok) {
    // nothing is issued; the barriers below are still passed
  } else if (warp == 0) {
    if (lane == 0) {
      const int w_row0 = n0 + (int)half * TG_BM;                     // this CTA's half of the tile's rows of W
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0, st = it % TGQ_STAGES;
        if (it >= TGQ_STAGES && !mbar_wait_cluster(empty_bar(st), ((it / TGQ_STAGES) - 1) & 1)) {
          atomicExch(error_flag, 31);
          break;
        }
        const unsigned full0 = mapa_shared(full_bar(st), leader);
        if (half == 0) mbar_expect_tx(full_bar(st), 2 * TGQ_STAGE_BYTES);
        const unsigned a_dst = base + st * TGQ_STAGE_BYTES;
        tma_load_2d_pair(a_dst, &map_a, kb * TG_BK, m0, full0);
        tma_load_2d_pair(a_dst + TG_BM * TG_BK * 2, &map_w, kb * TG_BK, w_row0, full0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && half == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TGQ_BN >> 3) << 17) | ((unsigned)((2 * TG_BM) >> 4) << 24);
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0, st = it % TGQ_STAGES;
        if (!mbar_wait_cluster(full_bar(st), (it / TGQ_STAGES) & 1)) {
          atomicExch(error_flag, 32);
          break;
        }
        tc_fence_after();
        const unsigned a_addr = base + st * TGQ_STAGE_BYTES;
        const unsigned long long da = umma_desc_sw128(a_addr), dw = umma_desc_sw128(a_addr + TG_BM * TG_BK * 2);
#pragma unroll
        for (int k = 0; k < TG_BK / 16; ++k)
          tc_mma_bf16_pair(tmem_acc, da + (unsigned)(k * 32 >> 4), dw + (unsigned)(k * 32 >> 4), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        tc_commit_pair_of(empty_bar(st), leader);     // both CTAs' stages are free when these MMAs have read them
      }
      tc_commit_pair_of(acc_full, leader);            // both CTAs' accumulators are complete
    }
  } else {
    // while the tensor cores work: 1 / rms of the first row this thread finishes, its residual and norm weights into L1
    const int item = (int)threadIdx.x - 64, frl = item / (TGQ_BN / 8), fm = m0 + pair * rows_per + frl;
    if (frl < rows_per && pair * rows_per + frl < TG_BM && fm < M) {
      if (NORM && nm.in_sumsq != nullptr) {
        float sum = 0.0f;
        for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + fm];
        first_inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
      }
      const int fn = n0 + (item % (TGQ_BN / 8)) * 8;
      if (fn < N) {
        if (EPI == HB_EPI_RESIDUAL) prefetch_l1((const float*)Cv + (size_t)fm * ldc + fn);
        if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr) prefetch_l1(nm.out_w + fn);
      }
    }
    ready = mbar_wait_cluster(acc_full, 0);
    if (!ready && lane == 0) atomicExch(error_flag, 33);
  }
  pdl_launch();                     // this CTA's loads are done
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();               // every pair is through with its ring: rows may be sent into it
  if (warp >= 2 && ready) {
    // row l of this CTA's accumulator goes to the CTA with the same half whose block of rows holds l: slot [this pair][l - its first row]
    tc_fence_after();
    const int quad = warp & 3, l = quad * 32 + lane;
    const int c_lo = warp < 6 ? 0 : TGQ_BN / 64, c_hi = c_lo + TGQ_BN / 64;
    const int owner = l / rows_per;
    const unsigned slot = mapa_shared(base + (unsigned)(((pair * rows_per + (l - owner * rows_per)) * TGQ_ROW_FLOATS) * 4),
                                      (unsigned)(owner < S ? 2 * owner : 0) + half);
#pragma unroll 1
    for (int c = c_lo; c < c_hi; ++c) {
      unsigned r[32];
      tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
      if (m0 + l < M) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st_cluster_f4(slot + (unsigned)((c * 32 + j) * 4), __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    }
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();               // every row is where it is finished
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TGQ_BN) : "memory");
  } else if (warp >= 2) {
    // rows pair * rows_per ... of this CTA's 128; a thread takes 8 columns of a row, consecutive lanes consecutive columns
    constexpr int GROUPS = TGQ_BN / 8;
    const int idx = (int)threadIdx.x - 64;
    const int part_lanes = part_cols >> 3;                                         // 8 or 16 lanes share a partial sum of a following norm
    const int n_end = ((N + 2 * part_cols - 1) / (2 * part_cols)) * 2 * part_cols;   // ... which cover whole tiles of twice that width
    const float* recv = reinterpret_cast<const float*>(gen);
    for (int item0 = 0; item0 < rows_per * GROUPS; item0 += TG_EPI_WARPS * 32) {
      const int item = item0 + idx;
      const int g8 = item % GROUPS, rl = item / GROUPS, l = pair * rows_per + rl, m = m0 + l;
      const bool active = rl < rows_per && l < TG_BM && m < M;
      float sq = 0.0f;
      if (active) {
        float inv_rms = first_inv_rms;
        if (NORM && nm.in_sumsq != nullptr && item0 > 0) {
          float sum = 0.0f;
          for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
          inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
        }
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        for (int q = 0; q < S; ++q) {           // in the order of the k ranges
          const float4* src = reinterpret_cast<const float4*>(recv + (size_t)(q * rows_per + rl) * TGQ_ROW_FLOATS + g8 * 8);
          const float4 x = src[0], y = src[1];
          v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
          v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
        }
        tg_epilogue8<EPI, NORM>(v, m, n0 + g8 * 8, M, N, Cv, ldc, nm, inv_rms, sq);
      }
      if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr) {
        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
        if (part_lanes == 16) sq += __shfl_xor_sync(0xffffffffu, sq, 8);
        if (active && (g8 & (part_lanes - 1)) == 0 && n0 + g8 * 8 < n_end)
          nm.out_sumsq[(size_t)((n0 + g8 * 8) / part_cols) * nm.out_stride + m] = sq;
      }
    }
  }
}


// Clusters of `ways` CTAs of this kernel that the GPU holds at once (asked once per size).
template <int EPI, bool NORM>
static int tg_ksplit_resident(int ways) {
  static int resident[9] = {0};
  if (resident[ways] == 0) {
    resident[ways] = -1;
    if (cudaFuncSetAttribute(gemm_tcgen05_ksplit_kernel<EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, TGK_SMEM_BYTES) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(ways);
      cfg.blockDim = dim3(TG_THREADS);
      cfg.dynamicSmemBytes = TGK_SMEM_BYTES;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = ways;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_ksplit_kernel<EPI, NORM>, &cfg) == cudaSuccess && n > 0) resident[ways] = n;
    }
    cudaGetLastError();
  }
  return resident[ways];
}

// The tile width and cluster size that put the most CTAs to work in one wave: every cluster resident
// at once, K ranges of at least four blocks, at least four stages beside the rows a CTA is sent;
// nothing below three quarters of the SMs.
template <int EPI, bool NORM>
static TgKsplit tg_ksplit_plan(int M, int N, int K) {
  TgKsplit best{0, 0, 0, 0, 0};
  if (!tg_cluster_enabled() || M > TG_BM || N < 256 || tg_tile_cols(M, N) != 128) return best;
  const int num_kb = ceil_div(K, TG_BK), sms = tg_sm_count(), a_rows = M <= 64 ? 64 : TG_BM;
  int best_ctas = 0;
  for (int bn = 128; bn <= 256; bn += 64) {
    const int tiles = ceil_div(N, bn), stage_bytes = (a_rows + bn) * TG_BK * 2;
    for (int ways = 8; ways >= 2; --ways) {
      const int rows_per = ceil_div(M, ways);
      int stages = (TGK_RING_BYTES - ways * rows_per * (bn + 4) * 4) / stage_bytes;
      if (stages > TGK_MAX_STAGES) stages = TGK_MAX_STAGES;
      if (ways > num_kb / 4 || tiles * ways > sms || stages < 3 || tg_ksplit_resident<EPI, NORM>(ways) < tiles) continue;
      const int ctas = (int)((long long)ways * N / bn);       // columns beyond N in the last tile are work without a result
      if (ctas > best_ctas) {
        best_ctas = ctas;
        best = TgKsplit{bn, ways, a_rows, stages, rows_per};
      }
      break;
    }
  }
  if (4 * best_ctas < 3 * sms) best.ways = 0;
  return best;
}

// A matrix wide enough for a tile per SM without cutting K: the narrowest tiles (a multiple of 32
// columns) that still make one wave, every stage of the ring for loads.  Store and SwiGLU epilogues.
template <int EPI, bool NORM>
static TgKsplit tg_whole_plan(int M, int N, int K) {
  TgKsplit none{0, 0, 0, 0, 0};
  if (!tg_cluster_enabled() || EPI == HB_EPI_RESIDUAL || M > TG_BM) return none;
  const int sms = tg_sm_count(), a_rows = M <= 64 ? 64 : TG_BM;
  const int bn = ceil_div(ceil_div(N, sms), 32) * 32;
  if (bn < 64 || bn > 256) return none;
  const int tiles = ceil_div(N, bn);
  int stages = TGK_RING_BYTES / ((a_rows + bn) * TG_BK * 2);
  if (stages > TGK_MAX_STAGES) stages = TGK_MAX_STAGES;
  if (4 * tiles < 3 * sms || stages < 4 || ceil_div(K, TG_BK) < 8 || tg_ksplit_resident<EPI, NORM>(1) < tiles) return none;
  return TgKsplit{bn, 1, a_rows, stages, M};
}

template <int EPI, bool NORM>
static int tg_launch_ksplit(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, const TgKsplit& plan,
                            int* err, cudaStream_t s, const TgNorm& nm) {
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, plan.a_rows);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, plan.bn);
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ceil_div(N, plan.bn) * plan.ways);
  cfg.blockDim = dim3(TG_THREADS);
  cfg.dynamicSmemBytes = TGK_SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = plan.ways;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hb_pdl_enabled() == 1 ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_ksplit_kernel<EPI, NORM>, ma, mw, C, ldc, M, N, K, plan, err, nm);
  HB_CHECK_LAUNCH("gemm_tcgen05 (K ranges in a cluster)");
  return 0;
}

// 1: the product went that way; 0: it does not apply; negative: an error.
template <bool NORM>
static int tg_try_ksplit_t(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                         cudaStream_t s, const TgNorm& nm) {
  TgKsplit plan{0, 0, 0, 0, 0};
  int rc = 0;
  switch (epi) {
    case HB_EPI_STORE:
      if ((plan = tg_ksplit_plan<HB_EPI_STORE, NORM>(M, N, K)).ways > 0 || (plan = tg_whole_plan<HB_EPI_STORE, NORM>(M, N, K)).ways > 0) rc = tg_launch_ksplit<HB_EPI_STORE, NORM>(A, lda, W, ldw, C, ldc, M, N, K, plan, err, s, nm);
      break;
    case HB_EPI_STORE_F32:
      if ((plan = tg_ksplit_plan<HB_EPI_STORE_F32, NORM>(M, N, K)).ways > 0 || (plan = tg_whole_plan<HB_EPI_STORE_F32, NORM>(M, N, K)).ways > 0) rc = tg_launch_ksplit<HB_EPI_STORE_F32, NORM>(A, lda, W, ldw, C, ldc, M, N, K, plan, err, s, nm);
      break;
    case HB_EPI_RESIDUAL:
      if ((plan = tg_ksplit_plan<HB_EPI_RESIDUAL, NORM>(M, N, K)).ways > 0) rc = tg_launch_ksplit<HB_EPI_RESIDUAL, NORM>(A, lda, W, ldw, C, ldc, M, N, K, plan, err, s, nm);
      break;
    case HB_EPI_SWIGLU:
      if ((plan = tg_ksplit_plan<HB_EPI_SWIGLU, NORM>(M, N, K)).ways > 0 || (plan = tg_whole_plan<HB_EPI_SWIGLU, NORM>(M, N, K)).ways > 0) rc = tg_launch_ksplit<HB_EPI_SWIGLU, NORM>(A, lda, W, ldw, C, ldc, M, N, K, plan, err, s, nm);
      break;
  }
  if (rc) return -rc;
  return plan.ways > 0 ? 1 : 0;
}

// Pairs of CTAs per 256 x 256 tile (0: this product does not go that way): the most that make one wave
// with K ranges of at least four blocks, and nothing below three fifths of the SMs.
template <int EPI, bool NORM>
static int tg_pairk_ways(int M, int N, int K) {
  if (!tg_cluster_enabled() || !tg_pairs_enabled() || M <= TG_BM || N < TGQ_BN) return 0;
  const int tiles = ceil_div(M, 2 * TG_BM) * ceil_div(N, TGQ_BN), num_kb = ceil_div(K, TG_BK), sms = tg_sm_count();
  static int resident[5] = {0};       // clusters of 2 * ways CTAs that the GPU holds at once, asked once per size
  for (int ways = 4; ways >= 2; --ways) {
    if (ways > num_kb / 4 || tiles * 2 * ways > sms) continue;
    if (resident[ways] == 0) {
      resident[ways] = -1;
      if (cudaFuncSetAttribute(gemm_tcgen05_pair_ksplit_kernel<EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, TGQ_SMEM_BYTES) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * ways);
        cfg.blockDim = dim3(TG_THREADS);
        cfg.dynamicSmemBytes = TGQ_SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2 * ways;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_ksplit_kernel<EPI, NORM>, &cfg) == cudaSuccess && n > 0) resident[ways] = n;
      }
      cudaGetLastError();
    }
    if (resident[ways] < tiles) continue;
    return 5 * tiles * 2 * ways >= 3 * sms ? ways : 0;
  }
  return 0;
}

template <int EPI, bool NORM>
static int tg_launch_pairk(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int ways, int* err,
                           cudaStream_t s, const TgNorm& nm) {
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, TG_BM);
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ceil_div(M, 2 * TG_BM) * ceil_div(N, TGQ_BN) * 2 * ways);
  cfg.blockDim = dim3(TG_THREADS);
  cfg.dynamicSmemBytes = TGQ_SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2 * ways;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hb_pdl_enabled() == 1 ? 2 : 1;
  const int part_cols = tg_tile_cols(M, N) / 2;        // a following norm's partial sums are kept per half of the other kernels' tiles
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_ksplit_kernel<EPI, NORM>, ma, mw, C, ldc, M, N, K, ceil_div(TG_BM, ways), part_cols, err, nm);
  HB_CHECK_LAUNCH("gemm_tcgen05 (pairs with K ranges in a cluster)");
  return 0;
}

// 1: the product went that way; 0: it does not apply; negative: an error.
template <bool NORM>
static int tg_try_pairk_t(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                        cudaStream_t s, const TgNorm& nm) {
  int ways = 0, rc = 0;
  switch (epi) {
    case HB_EPI_STORE:
      if ((ways = tg_pairk_ways<HB_EPI_STORE, NORM>(M, N, K)) > 0) rc = tg_launch_pairk<HB_EPI_STORE, NORM>(A, lda, W, ldw, C, ldc, M, N, K, ways, err, s, nm);
      break;
    case HB_EPI_STORE_F32:
      if ((ways = tg_pairk_ways<HB_EPI_STORE_F32, NORM>(M, N, K)) > 0) rc = tg_launch_pairk<HB_EPI_STORE_F32, NORM>(A, lda, W, ldw, C, ldc, M, N, K, ways, err, s, nm);
      break;
    case HB_EPI_RESIDUAL:
      if ((ways = tg_pairk_ways<HB_EPI_RESIDUAL, NORM>(M, N, K)) > 0) rc = tg_launch_pairk<HB_EPI_RESIDUAL, NORM>(A, lda, W, ldw, C, ldc, M, N, K, ways, err, s, nm);
      break;
  }
  if (rc) return -rc;
  return ways > 0 ? 1 : 0;
}


int tg_try_ksplit(bool norm, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                  cudaStream_t s, const TgNorm& nm) {
  return norm ? tg_try_ksplit_t<true>(A, lda, W, ldw, C, ldc, M, N, K, epi, err, s, nm)
              : tg_try_ksplit_t<false>(A, lda, W, ldw, C, ldc, M, N, K, epi, err, s, nm);
}
int tg_try_pairk(bool norm, const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi, int* err,
                 cudaStream_t s, const TgNorm& nm) {
  return norm ? tg_try_pairk_t<true>(A, lda, W, ldw, C, ldc, M, N, K, epi, err, s, nm)
              : tg_try_pairk_t<false>(A, lda, W, ldw, C, ldc, M, N, K, epi, err, s, nm);
}
