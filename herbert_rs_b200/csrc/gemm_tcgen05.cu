// Prefill matrix product on the 5th-generation tensor cores:  C[M,N] (op)= A[M,K] * W[N,K]^T,
// bfloat16 operands (both K-major, as activations and checkpoint weights are stored), float
// accumulation in tensor memory.  It replaces the reference's one-workgroup-per-output-element
// shader (backends/backend_vulkan bf16_matmul.comp) and its AVX-512 tile kernel
// (backends/backend_bf16_avx512/src/avx512_bf16_matvec.S: avx512_bf16_matmul_tile).
//
// A persistent grid (one CTA per SM) walks the 128 x BN tiles of C (BN = 128 or 256):
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a 128 x 64 slab
//            of A and a BN x 64 slab of W per pipeline stage, signalling an mbarrier per stage;
//   warp 1   allocates tensor memory (two accumulators of BN columns); one lane issues tcgen05.mma
//            (M=128, N=BN, K=16) four times per stage, commits the stage's "empty" barrier and, at
//            the end of a tile, that accumulator's "full" barrier;
//   warps 2-9  read a finished accumulator with tcgen05.ld (each warp its 32 lanes = 32 rows of
//            C and half of the tile's columns), hand it back ("empty" barrier) and apply the epilogue: store, store as float, add
//            into the float residual stream, or SwiGLU over column groups of 8 gate + 8 up.
// With two accumulators the epilogue of tile i runs while the tensor cores work on tile i+1.
// This kernel uses no thread-block clusters; no kernel of the product uses multicast loads.  Below it: the
// same product by pairs of CTAs (long prompts), and the entry points, which choose between these
// two and the kernels of gemm_tcgen05_cluster.cu (few rows or few tiles: K cut over a cluster).
// What they share is in gemm_tcgen05_parts.cuh.  Rows/columns beyond M, N, K are
// zero-filled by TMA on load and skipped on store.  Every wait on an mbarrier is bounded; a wait
// that runs out sets *error_flag and the CTA winds down (tensor memory is always released).
#include "gemm_tcgen05_parts.cuh"

template <int BN>
struct TgSmem {
  static constexpr int kStageBytes = (TG_BM + BN) * TG_BK * 2;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

#define HB_EPI_QKV 4
struct TgQkv {
  const float* qw;         // norm weights [128], both or neither
  const float* kw;
  float eps;
  const float* cos_tab;    // [table_rows, 64]
  const float* sin_tab;
  int table_rows;
  const int* tok_seq;      // per row of A: sequence of the step, position in it
  const int* tok_pos;
  const int* seq_pages;    // [sequences, pages_stride]
  int pages_stride;
  bf16* kcache;            // [pages, nkv, page_size, 128]
  bf16* vcache;
  int nh, nkv, page_size, write_cache;
};

// How the tiles are dealt to the CTAs.  Whole rounds of G tiles run one tile per CTA and round.  The
// tiles left over (fewer than G) would keep only some SMs busy for a whole tile's time; instead
// their k blocks are laid end to end ("units") and cut into G equal runs, so every CTA gets the
// same amount of work: at most the tail of one tile and the head of the next.  A tile shared by
// several CTAs is finished by whichever of them arrives last at the tile's counter: every piece is
// written to the workspace as float, and the last one adds the pieces in the order of their k
// ranges (so the sum does not depend on who is last) and runs the epilogue.  Nobody waits for
// anybody.
struct TgSched {
  int full_rounds;   // rounds of one whole tile per CTA (the last may be ragged when sk_tiles == 0)
  int sk_tiles;      // tiles cut into runs of k blocks, starting at tile sk_first
  int sk_first;
  int per;           // k blocks per CTA in that part (< k blocks of a tile: a CTA touches at most two tiles)
  float* ws;         // [G][2] pieces of 128 x BN floats, each stored as [BN / 4][128][4]
  int* counters;     // [sk_tiles], zero between launches
};

struct TgSegments {
  int b, G, num_tiles, num_kb, r, u, u1;
  TgSched sc;
  __device__ TgSegments(const TgSched& s, int num_tiles_, int num_kb_)
      : b((int)blockIdx.x), G((int)gridDim.x), num_tiles(num_tiles_), num_kb(num_kb_), r(0), sc(s) {
    u = b * sc.per;
    const int total = sc.sk_tiles * num_kb;
    u1 = u + sc.per < total ? u + sc.per : total;
  }
  // The shared tiles come first: their pieces meet early, and whoever finishes one does so while
  // the tensor cores are already at work on its next (whole) tile.
  __device__ bool next(int& tile, int& kb0, int& kb1) {
    if (u < u1) {
      const int t = u / num_kb;
      kb0 = u - t * num_kb;
      kb1 = kb0 + (u1 - u) < num_kb ? kb0 + (u1 - u) : num_kb;
      tile = sc.sk_first + t;
      u += kb1 - kb0;
      return true;
    }
    while (r < sc.full_rounds) {
      tile = b + r * G;
      ++r;
      if (tile < num_tiles) {
        kb0 = 0;
        kb1 = num_kb;
        return true;
      }
    }
    return false;
  }
};

template <int BN, int EPI, bool NORM>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* Cv,
                    int ldc, int M, int N, int K, int* error_flag, TgNorm nm, TgSched sc) {
  constexpr int STAGES = TgSmem<BN>::kStages;
  constexpr int STAGE_BYTES = TgSmem<BN>::kStageBytes;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // swizzled tiles want 1024-byte alignment
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the tensor-memory slot
  const unsigned bars = base + STAGES * STAGE_BYTES;
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8);
  volatile int* sk_last = reinterpret_cast<volatile int*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 8);
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
  auto acc_full = [&](int b) { return bars + (2 * STAGES + b) * 8; };
  auto acc_empty = [&](int b) { return bars + (2 * STAGES + 2 + b) * 8; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TG_BM - 1) / TG_BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), TG_EPI_WARPS);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const unsigned tmem_base = *tmem_slot;

  // Tiles in the order m fastest: CTAs that run side by side share the same slab of W in L2.
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;        // k blocks issued so far, over all tiles of this CTA
      bool ok = true;
      TgSegments segs(sc, num_tiles, num_kb);
      int tile, kb0, kb1;
      while (ok && segs.next(tile, kb0, kb1)) {
        const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty_bar(s), ((it / STAGES) - 1) & 1)) {
            atomicExch(error_flag, 1);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const unsigned a_dst = base + s * STAGE_BYTES;
          tma_load_2d(a_dst, &map_a, kb * TG_BK, m0, full_bar(s));
          tma_load_2d(a_dst + TG_BM * TG_BK * 2, &map_w, kb * TG_BK, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D float, A and B bfloat16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TG_BM >> 4) << 24);
      int it = 0, local = 0;
      bool ok = true;
      TgSegments segs(sc, num_tiles, num_kb);
      int tile, kb0, kb1;
      for (; ok && segs.next(tile, kb0, kb1); ++local) {
        const int buf = local & 1;
        // the epilogue must have drained this accumulator (its previous use was tile local - 2)
        if (local >= 2 && !mbar_wait(acc_empty(buf), ((local >> 1) - 1) & 1)) {
          atomicExch(error_flag, 4);
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1)) {
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
                        (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(s));     // arrives when these MMAs have finished reading the stage
        }
        tc_commit(acc_full(buf));      // arrives when every MMA of this tile is complete
      }
    }
  } else {
    // epilogue warps: TMEM lane quadrant = warp index modulo 4; warps 2-5 take the first half of a
    // tile's columns, warps 6-9 the second
    const int quad = warp & 3;
    const int c_lo = ((warp - 2) >> 2) * (BN / 64), c_hi = c_lo + BN / 64;
    int local = 0;
    bool ok = true;
    TgSegments segs(sc, num_tiles, num_kb);
    int tile, kb0, kb1;
    for (; ok && segs.next(tile, kb0, kb1); ++local) {
      const int buf = local & 1;
      const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN;
      const int m = m0 + quad * 32 + lane;
      float inv_rms = 1.0f, sq = 0.0f;
      if (NORM && nm.in_sumsq != nullptr && m < M) {         // while the tensor cores still work on this tile
        float sum = 0.0f;
        for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
        inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
      }
      if (!mbar_wait(acc_full(buf), (local >> 1) & 1)) {
        if (lane == 0) atomicExch(error_flag, 3);
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
      const bool whole = kb0 == 0 && kb1 == num_kb;
      // pieces of a shared tile: CTA first_cta + j holds the j-th k range; its slot in the workspace
      // is 2 * cta + (index of the tile among the at most two that CTA touches)
      const int tsk = tile - sc.sk_first;
      int first_cta = 0, n_pieces = 1;
      bool finish = true;
      if (!whole) {
        first_cta = (tsk * num_kb) / sc.per;
        n_pieces = ((tsk + 1) * num_kb - 1) / sc.per - first_cta + 1;
        // a piece is stored as [group of 4 columns][row][4]: the 32 lanes (rows) of a warp write 512 contiguous bytes
        float* mine = sc.ws + (size_t)(2 * blockIdx.x + (tsk - ((int)blockIdx.x * sc.per) / num_kb)) * TG_BM * BN + (quad * 32 + lane) * 4;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
          unsigned r[32];
          tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
          if (m < M) {            // rows beyond M are never read back
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(mine + (size_t)(c * 8 + (j >> 2)) * TG_BM * 4) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(buf));
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");          // the eight epilogue warps
        if (threadIdx.x == 64) {
          const int old = atomicAdd(sc.counters + tsk, 1);
          *sk_last = old == n_pieces - 1;
          if (*sk_last) sc.counters[tsk] = 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        finish = *sk_last != 0;
        asm volatile("bar.sync 1, 256;" ::: "memory");          // everyone has read the flag before it is written again
        if (finish) __threadfence();
      }
      if (!finish) continue;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        unsigned r[32];
        if (whole) {
          tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
          if (c == c_hi - 1) {
            // everything of this accumulator is in registers: the tensor cores may have it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
          }
        } else {
          // the pieces in the order of their k ranges, four pieces' loads in flight at a time
          float acc[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
          for (int p0 = 0; p0 < n_pieces && m < M; p0 += 4) {
            float4 v[4][8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int cta = first_cta + (p0 + q < n_pieces ? p0 + q : p0);
              const float* src = sc.ws + (size_t)(2 * cta + (tsk - (cta * sc.per) / num_kb)) * TG_BM * BN + (quad * 32 + lane) * 4 + (size_t)c * 8 * TG_BM * 4;
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q][j] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)j * TG_BM * 4));
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (p0 + q < n_pieces) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  acc[4 * j] += v[q][j].x; acc[4 * j + 1] += v[q][j].y; acc[4 * j + 2] += v[q][j].z; acc[4 * j + 3] += v[q][j].w;
                }
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(acc[j]);
        }
        tg_epilogue32<EPI, NORM>(r, m, n0 + c * 32, M, N, Cv, ldc, nm, inv_rms, sq);
      }
      if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr && m < M)
        nm.out_sumsq[(size_t)(2 * (tile / tiles_m) + (c_lo > 0)) * nm.out_stride + m] = sq;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// The same product by pairs of CTAs (a thread-block cluster of two, tcgen05 with cta_group::2).
//
// A pair owns a 256 x 256 tile of C.  Each CTA loads its own 128 rows of A and 128 of the tile's 256
// rows of W per stage; one lane of the pair's first CTA issues tcgen05.mma (M=256, N=256, K=16),
// which reads both CTAs' shared memory and accumulates each CTA's 128 rows in that CTA's tensor
// memory.  Per CTA and k block that is 32 KB written by TMA and 32 KB read by the tensor cores, where
// a single CTA's 128 x 256 tile needs 48 KB of each: the single-CTA kernel is bound by shared-memory
// bandwidth (about 190 bytes a cycle wanted, 128 there), the pair is not.
//   full[s]   lives in the first CTA: armed there with both CTAs' bytes; both CTAs' TMA loads signal it
//             (cp.async.bulk.tensor with cta_group::2 may signal the peer's mbarrier; no multicast);
//   empty[s], acc_full[b]   in both CTAs: tcgen05.commit arrives at both (multicast::cluster on the
//             commit, which carries no data);
//   acc_empty[b]  in the first CTA: the sixteen epilogue warps of the pair arrive there.
// Whole tiles only (no tiles shared between pairs); pairs walk the tiles m fastest.
// One head (128 columns starting at tensor-memory address taddr) of row m.  Every lane of the warp
// runs the tensor-memory loads; rows beyond M store nothing.
__device__ __forceinline__ void tg_epilogue_qkv(unsigned taddr, int m, int head, int M, void* Cv, int ldc, float inv_rms,
                                                const TgQkv& q) {
  const int heads_total = q.nh + 2 * q.nkv;
  if (head >= heads_total) return;                                  // uniform over the warp
  const bool is_q = head < q.nh, is_k = !is_q && head < q.nh + q.nkv;
  const bool live = m < M;
  int pos = 0, seq = 0;
  if (live) {
    pos = q.tok_pos[m];
    seq = q.tok_seq[m];
  }
  bf16* dst = nullptr;
  if (live) {
    if (is_q) dst = (bf16*)Cv + (size_t)m * ldc + (size_t)head * 128;
    else if (q.write_cache) {
      const int page = q.seq_pages[(size_t)seq * q.pages_stride + pos / q.page_size];
      const int kvh = is_k ? head - q.nh : head - q.nh - q.nkv;
      dst = (is_k ? q.kcache : q.vcache) + (((size_t)page * q.nkv + kvh) * q.page_size + (pos % q.page_size)) * 128;
    }
  }
  auto store32 = [&](bf16* out, const float* v) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 u;
      u.x = pack2(v[j], v[j + 1]); u.y = pack2(v[j + 2], v[j + 3]);
      u.z = pack2(v[j + 4], v[j + 5]); u.w = pack2(v[j + 6], v[j + 7]);
      *reinterpret_cast<uint4*>(out + j) = u;
    }
  };
  if (!is_q && !is_k) {                                             // v: as projected
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float t[32];
      tc_ld32f(taddr + c * 32, t);
#pragma unroll
      for (int j = 0; j < 32; ++j) t[j] *= inv_rms;
      if (dst != nullptr) store32(dst + c * 32, t);
    }
    return;
  }
  const float* w = is_q ? q.qw : q.kw;
  float inv = 1.0f;
  if (w != nullptr) {                                               // r = 1/sqrt(sum(x^2)/128 + eps), x the projected values
    float ss = 0.0f;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float t[32];
      tc_ld32f(taddr + c * 32, t);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = t[j] * inv_rms;
        ss += x * x;
      }
    }
    inv = 1.0f / sqrtf(ss / 128.0f + q.eps);
  }
  const int trow = pos < q.table_rows ? pos : q.table_rows - 1;
  const float* cos_row = q.cos_tab + (size_t)trow * 64;
  const float* sin_row = q.sin_tab + (size_t)trow * 64;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {                                     // columns 32c.. pair with columns 64 + 32c..
    float lo[32], hi[32];
    tc_ld32f(taddr + c * 32, lo);
    tc_ld32f(taddr + 64 + c * 32, hi);
    if (live) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 c4 = *reinterpret_cast<const float4*>(cos_row + c * 32 + j), s4 = *reinterpret_cast<const float4*>(sin_row + c * 32 + j);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
        float wl[4] = {1.f, 1.f, 1.f, 1.f}, wh[4] = {1.f, 1.f, 1.f, 1.f};
        if (w != nullptr) {
          const float4 a4 = *reinterpret_cast<const float4*>(w + c * 32 + j), b4 = *reinterpret_cast<const float4*>(w + 64 + c * 32 + j);
          wl[0] = a4.x; wl[1] = a4.y; wl[2] = a4.z; wl[3] = a4.w;
          wh[0] = b4.x; wh[1] = b4.y; wh[2] = b4.z; wh[3] = b4.w;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = ((lo[j + i] * inv_rms) * inv) * wl[i], x1 = ((hi[j + i] * inv_rms) * inv) * wh[i];
          lo[j + i] = x0 * cs[i] - x1 * sn[i];
          hi[j + i] = x0 * sn[i] + x1 * cs[i];
        }
      }
      if (dst != nullptr) {
        store32(dst + c * 32, lo);
        store32(dst + 64 + c * 32, hi);
      }
    }
  }
}

#define TGP_STAGES 6
#define TGP_STAGE_BYTES ((TG_BM + 128) * TG_BK * 2)      // 128 rows of A and 128 rows of W, 64 columns each
#define TGP_SMEM_BYTES (TGP_STAGES * TGP_STAGE_BYTES + 1024 + 256)

template <int EPI, bool NORM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* Cv,
                         int ldc, int M, int N, int K, int* error_flag, TgNorm nm, TgQkv qk) {
  constexpr int BN = 256;
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned bars = base + TGP_STAGES * TGP_STAGE_BYTES;
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + TGP_STAGES * TGP_STAGE_BYTES + (2 * TGP_STAGES + 4) * 8);
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (TGP_STAGES + s) * 8; };
  auto acc_full = [&](int b) { return bars + (2 * TGP_STAGES + b) * 8; };
  auto acc_empty = [&](int b) { return bars + (2 * TGP_STAGES + 2 + b) * 8; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();
  const int pair = (int)cluster_id_x(), n_pairs = (int)n_clusters_x();
  const int tiles_m = (M + 2 * TG_BM - 1) / (2 * TG_BM), tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TGP_STAGES; ++s) {
      mbar_init(full_bar(s), 1);      // the first CTA's producer arms it with both CTAs' bytes
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 2 * TG_EPI_WARPS);     // one arrival per epilogue warp of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Each CTA allocates all of its own tensor memory (one CTA per SM: both get column 0), so the
  // pair's product finds each CTA's half of the accumulator at the same address.
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();               // both CTAs' barriers are initialised before either signals the other's
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const unsigned tmem_base = *tmem_slot;
  const bool tmem_ok = tmem_base == 0u;       // everything was asked for: anything else means the SM was not empty
  if (!tmem_ok && threadIdx.x == 0) atomicExch(error_flag, 15);

  if (!tmem_ok) {
    // nothing is issued; fall through to the common end
  } else if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += n_pairs) {
        const int m0 = (tile % tiles_m) * 2 * TG_BM + (int)rank * TG_BM, n0 = (tile / tiles_m) * BN + (int)rank * 128;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % TGP_STAGES;
          if (it >= TGP_STAGES && !mbar_wait_cluster(empty_bar(s), ((it / TGP_STAGES) - 1) & 1)) {
            atomicExch(error_flag, 11);
            ok = false;
            break;
          }
          const unsigned full0 = mapa_shared(full_bar(s), 0);      // the first CTA's barrier
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * TGP_STAGE_BYTES);
          const unsigned a_dst = base + s * TGP_STAGE_BYTES;
          tma_load_2d_pair(a_dst, &map_a, kb * TG_BK, m0, full0);
          tma_load_2d_pair(a_dst + TG_BM * TG_BK * 2, &map_w, kb * TG_BK, n0, full0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // D float, A and B bfloat16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24 (M counts both CTAs' rows)
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)((2 * TG_BM) >> 4) << 24);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, ++local) {
        const int buf = local & 1;
        if (local >= 2 && !mbar_wait_cluster(acc_empty(buf), ((local >> 1) - 1) & 1)) {
          atomicExch(error_flag, 14);
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % TGP_STAGES;
          if (!mbar_wait_cluster(full_bar(s), (it / TGP_STAGES) & 1)) {
            atomicExch(error_flag, 12);
            ok = false;
            break;
          }
          tc_fence_after();
          const unsigned a_addr = base + s * TGP_STAGE_BYTES;
          const unsigned long long da = umma_desc_sw128(a_addr), dw = umma_desc_sw128(a_addr + TG_BM * TG_BK * 2);
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k)
            tc_mma_bf16_pair(tmem_acc, da + (unsigned)(k * 32 >> 4), dw + (unsigned)(k * 32 >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(empty_bar(s));     // both CTAs' stages are free when these MMAs have read them
        }
        tc_commit_pair(acc_full(buf));      // both CTAs' accumulators are complete
      }
    }
  } else {
    const int quad = warp & 3;
    const int c_lo = ((warp - 2) >> 2) * (BN / 64), c_hi = c_lo + BN / 64;
    int local = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % tiles_m) * 2 * TG_BM + (int)rank * TG_BM, n0 = (tile / tiles_m) * BN;
      const int m = m0 + quad * 32 + lane;
      float inv_rms = 1.0f, sq = 0.0f;
      if (NORM && nm.in_sumsq != nullptr && m < M) {
        float sum = 0.0f;
        for (int i = 0; i < nm.in_parts; ++i) sum += nm.in_sumsq[(size_t)i * nm.in_stride + m];
        inv_rms = rsqrtf(sum / (float)K + nm.in_eps);
      }
      if (!mbar_wait_cluster(acc_full(buf), (local >> 1) & 1)) {
        if (lane == 0) atomicExch(error_flag, 13);
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
      const unsigned acc_empty0 = mapa_shared(acc_empty(buf), 0);
      if constexpr (EPI == HB_EPI_QKV) {
        tg_epilogue_qkv(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c_lo * 32), m, (n0 + c_lo * 32) / 128, M, Cv, ldc, inv_rms, qk);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty0);
      } else {
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
          unsigned r[32];
          tc_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), r);
          if (c == c_hi - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty0);
          }
          tg_epilogue32<EPI, NORM>(r, m, n0 + c * 32, M, N, Cv, ldc, nm, inv_rms, sq);
        }
      }
      if (NORM && EPI == HB_EPI_RESIDUAL && nm.out_w != nullptr && m < M)
        nm.out_sumsq[(size_t)(2 * (tile / tiles_m) + (c_lo > 0)) * nm.out_stride + m] = sq;
    }
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();               // neither CTA leaves while the other may still signal its barriers or use its tensor memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// The workspace the launcher may use for shared tiles: floats and counters for a grid of `sms` CTAs.
#define TG_WS_FLOATS_PER_CTA (2 * TG_BM * 256)
static float* g_tg_ws = nullptr;        // set by hb_gemm_tcgen05_set_workspace
static int* g_tg_counters = nullptr;
static int g_tg_ws_ctas = 0;

int tg_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// Whether the leftover tiles of a product are cut into runs of k blocks shared between CTAs.
static bool tg_splits_tiles(int tiles, int num_kb, int sms) {
  const int rem = tiles % sms;
  return g_tg_ws != nullptr && g_tg_ws_ctas >= sms && rem > 0 && rem * 2 <= sms && num_kb >= 8 && (long long)rem * num_kb >= 4LL * sms;
}

// Pairs of CTAs take products of many rows whose tiles are 256 columns wide and all whole.
static int g_tg_pairs = 1;       // hb_gemm_tcgen05_set_pairs(0) switches them off (for measurements)
static int g_tg_cluster = 1;     // hb_gemm_tcgen05_set_ksplit(0): no product cuts K over a cluster
int tg_pairs_enabled() { return g_tg_pairs; }
int tg_cluster_enabled() { return g_tg_cluster; }
static bool tg_use_pairs(int M, int N, int K) {
  (void)K;
  return g_tg_pairs && M >= 512 && N >= 256;
}

template <int EPI, bool NORM>
static int tg_launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int* err,
                          cudaStream_t s, const TgNorm& nm, const TgQkv& qk = TgQkv{}) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, TGP_SMEM_BYTES);
    if (e != cudaSuccess) HB_FAIL(3, "gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", TGP_SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = ceil_div(M, 2 * TG_BM) * ceil_div(N, 256);
  const int pairs = tiles < tg_sm_count() / 2 ? tiles : tg_sm_count() / 2;
  hb_launch(gemm_tcgen05_pair_kernel<EPI, NORM>, dim3(2 * pairs), dim3(TG_THREADS), TGP_SMEM_BYTES, s, ma, mw, C, ldc, M, N, K, err, nm, qk);
  HB_CHECK_LAUNCH("gemm_tcgen05 (pairs)");
  return 0;
}

template <bool NORM>
static int tg_dispatch_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int epi,
                            int* err, cudaStream_t s, const TgNorm& nm) {
  switch (epi) {
    case HB_EPI_STORE: return tg_launch_pair<HB_EPI_STORE, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_STORE_F32: return tg_launch_pair<HB_EPI_STORE_F32, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_RESIDUAL: return tg_launch_pair<HB_EPI_RESIDUAL, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_SWIGLU: return tg_launch_pair<HB_EPI_SWIGLU, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
  }
  HB_FAIL(2, "gemm_tcgen05: unknown epilogue %d", epi);
}

template <int BN, int EPI, bool NORM>
static int tg_launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int* err,
                     cudaStream_t s, const TgNorm& nm) {
  const int smem = TgSmem<BN>::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int tiles = ceil_div(M, TG_BM) * ceil_div(N, BN);
  const int num_kb = ceil_div(K, TG_BK);
  int G = tiles < sms ? tiles : sms;
  TgSched sc{ceil_div(tiles, G), 0, 0, 1, nullptr, nullptr};
  // Leftover tiles are cut into equal runs of k blocks when that pays: a workspace is there, the
  // leftover would leave at least half of the GPU idle, and a run is at least a few k blocks.
  // (Measured at the 8B sizes: with 48 leftover tiles the down projection takes 62 instead of 88 us;
  // with 108 or 128 leftover tiles the products with K = 4096..12288 get slower, because CTAs that
  // start at different k no longer share the weight slabs in L2 in lockstep.)
  const int rem = tiles % sms;
  if (tg_splits_tiles(tiles, num_kb, sms)) {
    G = sms;
    sc.full_rounds = tiles / sms;
    sc.sk_tiles = rem;
    sc.sk_first = sc.full_rounds * sms;
    sc.per = ceil_div(rem * num_kb, sms);
    sc.ws = g_tg_ws;
    sc.counters = g_tg_counters;
  }
  dim3 grid(G);
  hb_launch(gemm_tcgen05_kernel<BN, EPI, NORM>, dim3(grid), dim3(TG_THREADS), smem, s, ma, mw, C, ldc, M, N, K, err, nm, sc);
  HB_CHECK_LAUNCH("gemm_tcgen05");
  return 0;
}

template <int BN, bool NORM>
static int tg_dispatch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int M, int N, int K, int epi,
                       int* err, cudaStream_t s, const TgNorm& nm) {
  switch (epi) {
    case HB_EPI_STORE: return tg_launch<BN, HB_EPI_STORE, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_STORE_F32: return tg_launch<BN, HB_EPI_STORE_F32, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_RESIDUAL: return tg_launch<BN, HB_EPI_RESIDUAL, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
    case HB_EPI_SWIGLU: return tg_launch<BN, HB_EPI_SWIGLU, NORM>(ma, mw, C, ldc, M, N, K, err, s, nm);
  }
  HB_FAIL(2, "gemm_tcgen05: unknown epilogue %d", epi);
}

// Output columns per tile.  Tiles of 256 weight rows feed the tensor cores best; when there are too
// few of them to keep half the SMs busy (decode batches, short prompts, matrices of few rows),
// tiles of 128 give twice the tiles to spread and, where tiles are shared, pieces of half the size.
// Measured at the 8B sizes: 64 rows q/k/v 27.6 -> 18.1 us, down 52.3 -> 33.9; 256 rows o 41.8 ->
// 26.8, down 70 -> 47; 512 rows o 41 -> 30, down 85 -> 67; with more tiles the wide ones win
// (512 rows gate/up 89 against 108).
int tg_tile_cols(int M, int N) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  if (N <= 128) return 128;
  return ceil_div(M, TG_BM) * ceil_div(N, 256) * 2 > sms ? 256 : 128;
}

// Gives the products a workspace for tiles shared between CTAs: `floats` must hold
// hb_gemm_tcgen05_workspace_floats(ctas) floats and `counters` ctas ints, zero, for ctas >= the
// number of SMs.  Without it (null) every tile is computed by one CTA.  Calls that use the same
// workspace must be on one stream.
// 0: every product by single CTAs (for measurements); 1 (default): pairs of CTAs where they apply.
extern "C" int hb_gemm_tcgen05_set_pairs(int on) {
  g_tg_pairs = on ? 1 : 0;
  return 0;
}
// 0: no product cuts K over a cluster (for measurements); 1 (default): products of at most 128 rows do where it applies.
extern "C" int hb_gemm_tcgen05_set_ksplit(int on) {
  g_tg_cluster = on ? 1 : 0;
  return 0;
}
extern "C" long long hb_gemm_tcgen05_workspace_floats(int ctas) { return (long long)ctas * TG_WS_FLOATS_PER_CTA; }
extern "C" int hb_gemm_tcgen05_set_workspace(float* floats, int* counters, int ctas) {
  g_tg_ws = floats;
  g_tg_counters = counters;
  g_tg_ws_ctas = floats != nullptr && counters != nullptr ? ctas : 0;
  return 0;
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
  const int BN = tg_tile_cols(M, N);
  const bool pairs = BN == 256 && tg_use_pairs(M, N, K);
  int rc = make_map(&ma, A, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, pairs ? 128 : BN);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const TgNorm none{};
  if (const int went = tg_try_pairk(false, A, lda, W, ldw, C, ldc, M, N, K, epi, error_flag, s, none)) return went > 0 ? 0 : -went;
  if (pairs) return tg_dispatch_pair<false>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, none);
  if (const int went = tg_try_ksplit(false, A, lda, W, ldw, C, ldc, M, N, K, epi, error_flag, s, none)) return went > 0 ? 0 : -went;
  return BN == 256 ? tg_dispatch<256, false>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, none)
                   : tg_dispatch<128, false>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, none);
}

// The q/k/v product of an attention layer with heads of 128 and full rotation, for steps of 512 rows
// and more (pairs of CTAs): C[:, :nh*128] = normed, rotated q (bfloat16); k (normed, rotated) and v go
// into the paged cache and are not written to C.  in_sumsq as in hb_gemm_tcgen05_norm_bf16 (or null).
// hb_gemm_tcgen05_qkv_ok says whether a product of these sizes can go this way.
extern "C" int hb_gemm_tcgen05_qkv_ok(int M, int N) {
  return g_tg_pairs && M >= 512 && N >= 256 && N % 128 == 0 && tg_tile_cols(M, N) == 256;
}
extern "C" int hb_gemm_tcgen05_qkv_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                        const float* in_sumsq, int in_parts, int in_stride, float in_eps, const float* qw,
                                        const float* kw, float eps, const float* cos_tab, const float* sin_tab,
                                        int table_rows, const int* tok_seq, const int* tok_pos, const int* seq_pages,
                                        int pages_stride, void* kcache, void* vcache, int nh, int nkv, int page_size,
                                        int write_cache, int* error_flag, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05_qkv: sizes must be positive");
  HB_REQUIRE(hb_gemm_tcgen05_qkv_ok(M, N), "gemm_tcgen05_qkv: %d rows by %d columns do not run as pairs of CTAs with whole heads per half tile", M, N);
  HB_REQUIRE(nh > 0 && nkv > 0 && N == (nh + 2 * nkv) * 128, "gemm_tcgen05_qkv: %d columns are not %d + 2 x %d heads of 128", N, nh, nkv);
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldc % 8 == 0, "gemm_tcgen05_qkv: K (%d) and the leading dimensions (%d, %d, %d) must be multiples of 8", K, lda, ldw, ldc);
  HB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)C & 15) == 0, "gemm_tcgen05_qkv: operands must be 16-byte aligned");
  HB_REQUIRE(kcache != nullptr && vcache != nullptr && ((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "gemm_tcgen05_qkv: the cache must be 16-byte aligned");
  HB_REQUIRE((qw == nullptr) == (kw == nullptr), "gemm_tcgen05_qkv: norm weights for both q and k, or for neither");
  HB_REQUIRE(qw == nullptr || ((((uintptr_t)qw | (uintptr_t)kw) & 15) == 0), "gemm_tcgen05_qkv: norm weights must be 16-byte aligned");
  HB_REQUIRE(cos_tab != nullptr && sin_tab != nullptr && table_rows > 0 && ((((uintptr_t)cos_tab | (uintptr_t)sin_tab) & 15) == 0),
             "gemm_tcgen05_qkv: needs rotation tables, 16-byte aligned");
  HB_REQUIRE(tok_seq != nullptr && tok_pos != nullptr && seq_pages != nullptr && page_size > 0, "gemm_tcgen05_qkv: needs the step's token and page arrays");
  HB_REQUIRE(in_sumsq == nullptr || (in_parts > 0 && in_stride >= M), "gemm_tcgen05_qkv: partial sums need a count and a row stride >= M");
  HB_REQUIRE(error_flag != nullptr, "gemm_tcgen05_qkv: an error flag is required");
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, 128);
  if (rc) return rc;
  const TgNorm nm{in_sumsq, in_parts, in_stride, in_eps, nullptr, nullptr, 0, nullptr, 0};
  const TgQkv qk{qw, kw, eps, cos_tab, sin_tab, table_rows, tok_seq, tok_pos, seq_pages, pages_stride, (bf16*)kcache, (bf16*)vcache,
                 nh, nkv, page_size, write_cache};
  return tg_launch_pair<HB_EPI_QKV, true>(ma, mw, C, ldc, M, N, K, error_flag, (cudaStream_t)stream, nm, qk);
}

// Half tiles of output columns (one per epilogue thread of a row), i.e. rows of out_sumsq, of a product with N output columns.
extern "C" int hb_gemm_tcgen05_norm_parts(int M, int N) { return 2 * ceil_div(N, tg_tile_cols(M, N)); }

// The same product with a shared norm on either side (any M):
//   in_sumsq != null: A holds x * w of a norm over K; results are multiplied by 1 / rms of the rows,
//     rms^2 = sum_i in_sumsq[i * in_stride + row] / K + in_eps, i < in_parts;
//   out_w != null (epi HB_EPI_RESIDUAL): besides C += ..., out_xw = C * out_w (bfloat16) and
//     out_sumsq[hb_gemm_tcgen05_norm_parts(M, N)][out_stride] = partial sums of C^2 (out_stride >= M).
extern "C" int hb_gemm_tcgen05_norm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M,
                                         int N, int K, int epi, const float* in_sumsq, int in_parts, int in_stride,
                                         float in_eps, const float* out_w, void* out_xw, int out_ld,
                                         float* out_sumsq, int out_stride, int* error_flag, void* stream) {
  HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05_norm: sizes must be positive");
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05_norm: K (%d) and the leading dimensions (%d, %d) must be multiples of 8 (16-byte rows for TMA)", K, lda, ldw);
  HB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tcgen05_norm: operands must be 16-byte aligned");
  HB_REQUIRE(epi != HB_EPI_SWIGLU || N % 16 == 0, "gemm_tcgen05_norm: SwiGLU columns come in groups of 16, N=%d", N);
  HB_REQUIRE(error_flag != nullptr, "gemm_tcgen05_norm: an error flag is required");
  HB_REQUIRE(in_sumsq == nullptr || (in_parts > 0 && in_stride >= M), "gemm_tcgen05_norm: partial sums need a count and a row stride >= M");
  HB_REQUIRE(out_w == nullptr || (epi == HB_EPI_RESIDUAL && out_xw != nullptr && out_sumsq != nullptr && out_stride >= M),
             "gemm_tcgen05_norm: the next norm's input is written by the residual epilogue and needs both outputs, row stride >= M");
  HB_REQUIRE(out_w == nullptr || (((uintptr_t)out_w & 15) == 0), "gemm_tcgen05_norm: the norm weight must be 16-byte aligned");
  CUtensorMap ma, mw;
  const int BN = tg_tile_cols(M, N);
  const bool pairs = BN == 256 && tg_use_pairs(M, N, K);
  int rc = make_map(&ma, A, M, K, lda, TG_BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, pairs ? 128 : BN);
  if (rc) return rc;
  const TgNorm nm{in_sumsq, in_parts, in_stride, in_eps, out_w, (bf16*)out_xw, out_ld, out_sumsq, out_stride};
  cudaStream_t s = (cudaStream_t)stream;
  if (const int went = tg_try_pairk(true, A, lda, W, ldw, C, ldc, M, N, K, epi, error_flag, s, nm)) return went > 0 ? 0 : -went;
  if (pairs) return tg_dispatch_pair<true>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, nm);
  if (const int went = tg_try_ksplit(true, A, lda, W, ldw, C, ldc, M, N, K, epi, error_flag, s, nm)) return went > 0 ? 0 : -went;
  return BN == 256 ? tg_dispatch<256, true>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, nm)
                   : tg_dispatch<128, true>(ma, mw, C, ldc, M, N, K, epi, error_flag, s, nm);
}
