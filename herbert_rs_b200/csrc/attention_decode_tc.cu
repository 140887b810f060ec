// Decode attention on the 5th-generation tensor cores (tcgen05), bfloat16, head size 128.
//
// One new query per sequence against its cached keys.  With so few query rows the roles are
// turned round so that the tensor cores still see a full tile: the 128 keys of a tile are the M
// side,  S^T = K Q^T  (M=128 keys, N=16 = the query heads of one kv group, padded), and
// O^T = V^T P^T  (M=128 = head size, N=16, K=128 keys) with V read as it lies in the cache
// (MN-major A operand).  S^T and O^T live in tensor memory; O^T is accumulated there across the
// key tiles of the CTA and rescaled in place (tcgen05.ld / st) when a head's maximum moves.
//   warp 0     TMA: the group's query rows once, then K and V tiles (two pages each) into 3-stage rings;
//   warp 1     one lane issues the MMAs; S^T of tile j+1 is computed while tile j is in the softmax;
//   warps 2-5  one thread per key of the tile (and per row of O^T): score from tensor memory, mask,
//              per-head maximum and sum across the 128 threads (shuffles + shared memory), P^T as
//              bfloat16 into shared memory in the swizzled K-major layout.
// Work is split like attention_decode.cu (key range, kv head, sequence); each split writes its
// (m, l, o) to scratch and the same second kernel combines them.  Arithmetic as in the reference
// (decode.rs:126-295: s = q.k * scale over keys lo..p, softmax, o = sum p v), all sums in float.
// Every wait on an mbarrier is bounded and sets *error_flag when it runs out.
#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

#define DT_THREADS 192
#define DT_KEYS 128
#define DT_HD 128
#define DT_STAGES 3
#define DT_SUB (128 * 128)          // one [128 rows][64 columns] swizzled sub-tile
#define DT_TILE (2 * DT_SUB)        // a K or V tile: 128 keys x 128 columns
#define DT_QSUB (16 * 128)          // one [16 rows][64 columns] sub-tile (Q and P^T)

int hb_attention_decode_combine(const float* part_o, const float* part_ml, void* out, int ldo, int n_seqs, int nh, int hd,
                                int nsplit, cudaStream_t s);

struct DecodeTcArgs {
  const int* seq_len;
  const int* seq_pages;
  int pages_stride;
  float* part_o;
  float* part_ml;
  int nh, nkv, page_size, nsplit, q_rows_per_token;
  float scale_log2;
  int window;
  int* error_flag;
};

__global__ void __launch_bounds__(DT_THREADS, 1)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, DecodeTcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned q_s = base, k_s = q_s + 4096, v_s = k_s + DT_STAGES * DT_TILE, p_s = v_s + DT_STAGES * DT_TILE;   // p_s: two P^T buffers
  unsigned char* p_gen = gen + (p_s - base);
  float* red_m = reinterpret_cast<float*>(gen + (p_s - base) + 8192);   // [4][16]
  float* red_l = red_m + 64;                                            // [4][16]
  const unsigned bars = p_s + 8192 + 512;
  // barriers: 0 q_full | 1-3 k_full | 4-6 k_empty | 7-9 v_full | 10-12 v_empty | 13,14 s_full | 15,16 s_empty | 17 p_ready | 18,19 o_done (per P^T buffer)
  auto bar = [&](int i) { return bars + i * 8; };
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + (bars - base) + 20 * 8);

  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.nh / a.nkv;
  const int len = a.seq_len[b], p = len - 1;
  const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
  const int tile_lo = lo / DT_KEYS, tile_hi = (len + DT_KEYS - 1) / DT_KEYS;
  const int per = (tile_hi - tile_lo + a.nsplit - 1) / a.nsplit;
  const int t0 = tile_lo + split * per, t1 = min(tile_hi, t0 + per);
  const int n_tiles = max(0, t1 - t0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 20; ++i) mbar_init(bar(i), (i == 15 || i == 16 || i == 17) ? 4 : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(64) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;
  const unsigned tm_s[2] = {tmem, tmem + 16u};
  const unsigned tm_o = tmem + 32u;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(bar(0), 2 * DT_QSUB);
      const int qrow = b * a.q_rows_per_token + kvh * G;
      tma_load_2d(q_s, &map_q, 0, qrow, bar(0));
      tma_load_2d(q_s + DT_QSUB, &map_q, 64, qrow, bar(0));
      const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % DT_STAGES;
        int rows[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int key0 = (t0 + j) * DT_KEYS + half * 64;
          const int lp = key0 / a.page_size;
          const int page = lp < a.pages_stride ? pages[lp] : 0;     // beyond the sequence: any page, its keys are masked
          rows[half] = (page * a.nkv + kvh) * a.page_size + key0 % a.page_size;
        }
        if (j >= DT_STAGES && !mbar_wait(bar(4 + st), ((j / DT_STAGES) - 1) & 1)) { atomicExch(a.error_flag, 41); break; }
        mbar_expect_tx(bar(1 + st), DT_TILE);
#pragma unroll
        for (int jb = 0; jb < 2; ++jb)
#pragma unroll
          for (int half = 0; half < 2; ++half)
            tma_load_2d(k_s + st * DT_TILE + jb * DT_SUB + half * 8192, &map_k, jb * 64, rows[half], bar(1 + st));
        if (j >= DT_STAGES && !mbar_wait(bar(10 + st), ((j / DT_STAGES) - 1) & 1)) { atomicExch(a.error_flag, 42); break; }
        mbar_expect_tx(bar(7 + st), DT_TILE);
#pragma unroll
        for (int jb = 0; jb < 2; ++jb)
#pragma unroll
          for (int half = 0; half < 2; ++half)
            tma_load_2d(v_s + st * DT_TILE + jb * DT_SUB + half * 8192, &map_v, jb * 64, rows[half], bar(7 + st));
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      // D float, A and B bfloat16, M = 128, N = 16; the second product reads A (= V) MN-major (bit 15)
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
      const unsigned idesc_pv = idesc_qk | (1u << 15);
      bool ok = mbar_wait(bar(0), 0);
      if (!ok) atomicExch(a.error_flag, 43);
      auto issue_qk = [&](int j) -> bool {
        const int st = j % DT_STAGES, sb = j & 1;
        if (j >= 2 && !mbar_wait(bar(15 + sb), ((j >> 1) - 1) & 1)) { atomicExch(a.error_flag, 44); return false; }
        if (!mbar_wait(bar(1 + st), (j / DT_STAGES) & 1)) { atomicExch(a.error_flag, 45); return false; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < DT_HD / 16; ++ks)
          tc_mma_bf16(tm_s[sb], umma_desc_sw128(k_s + st * DT_TILE + (ks >> 2) * DT_SUB + (ks & 3) * 32),
                      umma_desc_sw128(q_s + (ks >> 2) * DT_QSUB + (ks & 3) * 32), idesc_qk, ks > 0 ? 1u : 0u);
        tc_commit(bar(4 + st));
        tc_commit(bar(13 + sb));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % DT_STAGES;
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        if (!mbar_wait(bar(17), j & 1)) { atomicExch(a.error_flag, 46); break; }
        if (!mbar_wait(bar(7 + st), (j / DT_STAGES) & 1)) { atomicExch(a.error_flag, 47); break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < DT_KEYS / 16; ++ks)
          tc_mma_bf16(tm_o, umma_desc_sw128_mn(v_s + st * DT_TILE + ks * 2048, DT_SUB),
                      umma_desc_sw128(p_s + (j & 1) * 4096 + (ks >> 2) * DT_QSUB + (ks & 3) * 32), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        tc_commit(bar(10 + st));
        tc_commit(bar(18 + (j & 1)));
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // key of the tile, and row (head-size index) of O^T
    const unsigned lane_off = (unsigned)(quad * 32) << 16;
    float m_ref[16], l[16];
#pragma unroll
    for (int h = 0; h < 16; ++h) {
      m_ref[h] = -INFINITY;
      l[h] = 0.0f;
    }
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(bar(13 + sb), (j >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 48); ok = false; break; }
      tc_fence_after();
      float s[16];
      tc_ld16f(tm_s[sb] + lane_off, s);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar(15 + sb));
      const int key = (t0 + j) * DT_KEYS + r;
      const bool keep = key <= p && key >= lo;
      // per-head maximum over the tile's 128 keys
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        if (h < G) {
          s[h] = keep ? s[h] * a.scale_log2 : -INFINITY;
          const float w = warp_max(s[h]);
          if (lane == 0) red_m[quad * 16 + h] = w;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float f[16];
      bool moved = false;
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        f[h] = 1.0f;
        if (h < G) {
          const float mt = fmaxf(fmaxf(red_m[h], red_m[16 + h]), fmaxf(red_m[32 + h], red_m[48 + h]));
          const float m_new = fmaxf(m_ref[h], mt);
          if (m_new != m_ref[h]) {
            f[h] = (m_ref[h] == -INFINITY) ? 0.0f : fast_exp2(m_ref[h] - m_new);
            moved = true;
          }
          m_ref[h] = m_new;
        }
      }
      if (j >= 2) {
        // this tile's P^T buffer was last read by the product of tile j-2
        if (!mbar_wait(bar(18 + (j & 1)), ((j >> 1) - 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 49); ok = false; break; }
      }
      if (j > 0 && moved) {       // `moved` is the same for all 128 threads: they hold the same maxima
        // a maximum moved: O^T must be rescaled in place, which needs every earlier product complete
        if (!mbar_wait(bar(18 + ((j - 1) & 1)), ((j - 1) >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 51); ok = false; break; }
        tc_fence_after();
        float o[16];
        tc_ld16f(tm_o + lane_off, o);
#pragma unroll
        for (int h = 0; h < 16; ++h) o[h] *= f[h];
        tc_st16f(tm_o + lane_off, o);
      }
      // P^T (bfloat16, K-major with the 128-byte swizzle: row = head, 64 keys per 128-byte row) and the sums
      unsigned char* prow = p_gen + (j & 1) * 4096 + (r >> 6) * DT_QSUB + (r & 7) * 2;
      const int chunk = (r & 63) >> 3;
#pragma unroll
      for (int h = 0; h < 16; ++h) {
        if (h < G) {
          const float mu = (m_ref[h] == -INFINITY) ? 0.0f : m_ref[h];
          const float pv = keep ? fast_exp2(s[h] - mu) : 0.0f;
          *reinterpret_cast<bf16*>(prow + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16_rn(pv);
          const float w = warp_sum(pv);
          if (lane == 0) red_l[quad * 16 + h] = w;
        }
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
      for (int h = 0; h < 16; ++h)
        if (h < G) l[h] = l[h] * f[h] + (red_l[h] + red_l[16 + h]) + (red_l[32 + h] + red_l[48 + h]);
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar(17));
    }
    // this split's partial result: (m in natural-log units, l, o)
    float o[16];
#pragma unroll
    for (int h = 0; h < 16; ++h) o[h] = 0.0f;
    if (ok && n_tiles > 0) {
      if (mbar_wait(bar(18 + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1)) {
        tc_fence_after();
        tc_ld16f(tm_o + lane_off, o);
      } else if (lane == 0) {
        atomicExch(a.error_flag, 50);
      }
    }
#pragma unroll
    for (int h = 0; h < 16; ++h) {
      if (h < G) {
        const size_t pi = ((size_t)b * a.nh + kvh * G + h) * a.nsplit + split;
        a.part_o[pi * DT_HD + r] = o[h];
        if (r == 0) {
          a.part_ml[pi * 2] = m_ref[h] * 0.6931471805599453f;
          a.part_ml[pi * 2 + 1] = l[h];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64) : "memory");
  }
}

// Same contract as hb_attention_decode_bf16 (scratch of hb_attention_decode_scratch_floats floats);
// head size 128 only; q rows must be a whole number of heads wide (ldq a multiple of 128).
extern "C" int hb_attention_decode_tc_bf16(const void* q, int ldq, int n_tokens, void* out, int ldo, const void* kcache,
                                           const void* vcache, int n_pages, const int* seq_len, const int* seq_pages,
                                           int pages_stride, float* scratch, int n_seqs, int nh, int nkv, int hd,
                                           int page_size, int nsplit, float scale, int window, int* error_flag,
                                           void* stream) {
  HB_REQUIRE(n_seqs > 0 && nh > 0 && nkv > 0 && n_pages > 0 && n_tokens >= n_seqs, "attention_decode_tc: sizes must be positive");
  HB_REQUIRE(hd == DT_HD, "attention_decode_tc: head size %d is not 128", hd);
  HB_REQUIRE(nh % nkv == 0 && nh / nkv <= 16, "attention_decode_tc: at most 16 query heads per key/value head");
  HB_REQUIRE(page_size % 64 == 0, "attention_decode_tc: page size %d must be a multiple of 64", page_size);
  HB_REQUIRE(ldq % DT_HD == 0 && ((uintptr_t)q & 15) == 0, "attention_decode_tc: query rows must be whole heads wide and 16-byte aligned");
  HB_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "attention_decode_tc: cache must be 16-byte aligned");
  HB_REQUIRE(nsplit >= 1 && nsplit <= 65535 && n_seqs <= 65535 && nkv <= 65535, "attention_decode_tc: grid too large");
  HB_REQUIRE(scale > 0.0f && window >= 0 && error_flag != nullptr, "attention_decode_tc: bad arguments");
  CUtensorMap mq, mk, mv;
  const int rows_per_token = ldq / DT_HD;
  int rc = make_map_cols(&mq, q, (long long)n_tokens * rows_per_token, DT_HD, DT_HD, 16);
  if (rc) return rc;
  const long long cache_rows = (long long)n_pages * nkv * page_size;
  rc = make_map_cols(&mk, kcache, cache_rows, DT_HD, DT_HD, 64);
  if (rc) return rc;
  rc = make_map_cols(&mv, vcache, cache_rows, DT_HD, DT_HD, 64);
  if (rc) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)n_seqs * nh * nsplit * DT_HD;
  DecodeTcArgs a{seq_len, seq_pages, pages_stride, part_o, part_ml, nh, nkv, page_size, nsplit, rows_per_token,
                 scale * 1.4426950408889634f, window, error_flag};
  const int smem = 4096 + 2 * DT_STAGES * DT_TILE + 8192 + 512 + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  hb_launch(attention_decode_tc_kernel, dim3(nsplit, nkv, n_seqs), dim3(DT_THREADS), smem, s, mq, mk, mv, a);
  HB_CHECK_LAUNCH("attention_decode_tc");
  return hb_attention_decode_combine(part_o, part_ml, out, ldo, n_seqs, nh, DT_HD, nsplit, s);
}
