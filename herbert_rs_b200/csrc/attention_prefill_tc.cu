// Prefill attention on the 5th-generation tensor cores (tcgen05), bfloat16, head sizes 64 and 128.
//
// The same arithmetic as attention_prefill.cu (causal grouped-query softmax attention in the flash
// form, float softmax; reference: generic_attention/prefill/kernel_f32.rs:61-111), arranged for
// tensor memory: a CTA owns 128 consecutive queries of one head of one sequence and walks the key
// tiles (128 keys = two 64-key pages) of its causal range.
//   warp 0     TMA: the Q tile once, then K and V tiles into two-stage rings (128-byte swizzle);
//   warp 1     one lane issues tcgen05.mma:  S = Q K^T  (M=128, N=128) into one of two S buffers in
//              tensor memory, and  O_j = P V  (M=128, N=head size; V is the MN-major operand as it
//              lies in the cache) into one of two O buffers;
//   warps 2-9  two threads per query row (each half of the tile's keys and of the output columns):
//              read the row of S from tensor memory (no shuffles), mask,
//              running maximum and sum in float, P = 2^(s*c - m) as bfloat16 into shared memory in
//              the swizzled K-major layout the tensor cores read, and o = o * 2^(m_old - m_new) + O_j
//              in registers; finally o / l goes to global memory.
// The tensor cores compute S of tile j+1 while the row threads work on tile j.  Every wait on an
// mbarrier is bounded; a wait that runs out sets *error_flag and the CTA winds down.
#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

// PARTS threads per query row (2, or 4 for head size 128): each takes 128 / PARTS keys of a tile and
// HD / PARTS output columns.  Measured at head size 128: four threads per row are 9 % faster on long
// prompts (8,192 tokens: 774 against 843 us) and slower on short ones (many 128-token prompts: 101
// against 88 us), where the larger block barrier and exchange weigh more than the shorter passes.
#define PT_THREADS(PARTS) (64 + 128 * (PARTS))         // TMA warp, MMA warp, 4 softmax warps per part
#define PT_Q 128        // queries per CTA
#define PT_KEYS 128     // keys per tile
#define PT_SUB (128 * 128)   // bytes of one [128 rows][64 columns] swizzled sub-tile

struct PrefillTcArgs {
  bf16* out;
  int ldo;
  const int* seq_start;
  const int* seq_pos0;
  const int* seq_pages;
  int pages_stride;
  int nh, nkv, page_size;
  float scale_log2;   // scale * log2(e)
  int window;
  int* error_flag;
  int n_seqs, q_tiles;   // items = q_tiles x nh x n_seqs (some without queries when the sequences differ in length)
  int* work_counter;     // next item; zero when the kernel starts
};

// One unit of work: 128 consecutive queries of one head of one sequence.
struct PtItem {
  int b, h, kvh, row0, qlen, pos0, q_first, p_first, p_last, tile_lo, n_tiles;
  bool valid;      // false: the sequence has no queries in this tile (shorter than the longest of the batch)
};
__device__ __forceinline__ PtItem pt_item(const PrefillTcArgs& a, int idx) {
  // the longest key ranges (last query tiles) first; neighbours share a sequence and a kv head
  PtItem it;
  const int per_qt = a.nh * a.n_seqs;
  const int qt = a.q_tiles - 1 - idx / per_qt, rem = idx % per_qt;
  it.b = rem / a.nh;
  it.h = rem % a.nh;
  it.kvh = it.h / (a.nh / a.nkv);
  it.row0 = a.seq_start[it.b];
  it.qlen = a.seq_start[it.b + 1] - it.row0;
  it.pos0 = a.seq_pos0[it.b];
  it.q_first = qt * PT_Q;
  it.valid = it.q_first < it.qlen;
  const int q_last = min(it.qlen, it.q_first + PT_Q) - 1;
  it.p_first = it.pos0 + it.q_first;
  it.p_last = it.pos0 + q_last;
  const int lo_first = (a.window > 0 && it.p_first - a.window + 1 > 0) ? it.p_first - a.window + 1 : 0;
  it.tile_lo = lo_first / PT_KEYS;
  it.n_tiles = it.valid ? it.p_last / PT_KEYS + 1 - it.tile_lo : 0;
  return it;
}

template <int HD, int PARTS>
__global__ void __launch_bounds__(PT_THREADS(PARTS), 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcArgs a) {
  constexpr int NB = HD / 64;                 // 64-column blocks of the head
  constexpr int TILE_BYTES = NB * PT_SUB;     // one Q, K, V tile
  constexpr int ROW_WARPS = 4 * PARTS;
  constexpr int ROW_THREADS = 32 * ROW_WARPS;
  constexpr int KP = PT_KEYS / PARTS;         // keys of a tile per thread (64 or 32)
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned q_s = base, k_s = q_s + TILE_BYTES, v_s = k_s + 2 * TILE_BYTES, p_s = v_s + 2 * TILE_BYTES;
  unsigned char* p_gen = gen + (p_s - base);
  const unsigned bars = p_s + 2 * PT_SUB;
  // barriers: 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 v_full | 7,8 v_empty | 9,10 s_full | 11,12 s_empty
  //           13 p_ready | 14,15 o_full | 16,17 o_empty | 18 q_empty | 19,20 item_full | 21,22 item_empty
  auto bar = [&](int i) { return bars + i * 8; };
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + (bars - base) + 23 * 8);
  volatile int* item_ring = reinterpret_cast<volatile int*>(gen + (bars - base) + 23 * 8 + 8);      // [2]
  float* xch = reinterpret_cast<float*>(gen + (bars - base) + 256);   // [2 tile parities][PARTS][128 rows] maxima, then [PARTS][128] sums
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 23; ++i) {
      const bool from_rows = (i == 11 || i == 12 || i == 13 || i == 16 || i == 17);   // arrived at by the row warps
      const bool from_consumers = (i == 21 || i == 22);                               // the MMA lane and the row warps
      mbar_init(bar(i), from_rows ? ROW_WARPS : (from_consumers ? ROW_WARPS + 1 : 1));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const unsigned tmem = *tmem_slot;
  const unsigned tm_s[2] = {tmem, tmem + 128u};
  const unsigned tm_o[2] = {tmem + 256u, tmem + 256u + (unsigned)HD};
  const int total_items = a.q_tiles * a.nh * a.n_seqs;

  // The CTAs are persistent: each takes the next item from a counter in global memory when it has
  // issued everything for its current one.  The TMA warp fetches the index and hands it to the
  // other warps through a ring of two slots, so it can load the next item's tiles while the
  // current item is still being worked on.  `g` counts this CTA's key tiles over all its items:
  // ring stages and barrier phases carry on from item to item.
  if (warp == 0) {
    if (lane == 0) {
      int g = 0, n_valid = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        if (n >= 2 && !mbar_wait(bar(21 + slot), ((n >> 1) - 1) & 1)) { atomicExch(a.error_flag, 31); break; }
        const int fetched = atomicAdd(a.work_counter, 1);
        const int idx = fetched < total_items ? fetched : -1;
        item_ring[slot] = idx;
        mbar_arrive_cta(bar(19 + slot));
        if (idx < 0) break;
        const PtItem it = pt_item(a, idx);
        if (!it.valid) continue;
        // the Q buffer is free once the previous item's last S product has read it
        if (n_valid >= 1 && !mbar_wait(bar(18), (n_valid - 1) & 1)) { atomicExch(a.error_flag, 32); break; }
        ++n_valid;
        mbar_expect_tx(bar(0), TILE_BYTES);
#pragma unroll
        for (int jb = 0; jb < NB; ++jb) tma_load_2d(q_s + jb * PT_SUB, &map_q, it.h * HD + jb * 64, it.row0 + it.q_first, bar(0));
        const int* pages = a.seq_pages + (size_t)it.b * a.pages_stride;
        for (int j = 0; j < it.n_tiles; ++j, ++g) {
          const int st = g & 1;
          int rows[2];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int key0 = (it.tile_lo + j) * PT_KEYS + half * 64;
            const int lp = key0 / a.page_size;
            const int page = lp < a.pages_stride ? pages[lp] : 0;     // beyond the sequence: any page, its keys are masked
            rows[half] = (page * a.nkv + it.kvh) * a.page_size + key0 % a.page_size;
          }
          if (g >= 2 && !mbar_wait(bar(3 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 21); ok = false; break; }
          mbar_expect_tx(bar(1 + st), TILE_BYTES);
#pragma unroll
          for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int half = 0; half < 2; ++half)
              tma_load_2d(k_s + st * TILE_BYTES + jb * PT_SUB + half * 8192, &map_k, jb * 64, rows[half], bar(1 + st));
          if (g >= 2 && !mbar_wait(bar(7 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 22); ok = false; break; }
          mbar_expect_tx(bar(5 + st), TILE_BYTES);
#pragma unroll
          for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int half = 0; half < 2; ++half)
              tma_load_2d(v_s + st * TILE_BYTES + jb * PT_SUB + half * 8192, &map_v, jb * 64, rows[half], bar(5 + st));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // D float, A and B bfloat16; B of the second product is MN-major (bit 16)
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PT_KEYS >> 3) << 17) | ((unsigned)(PT_Q >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(PT_Q >> 4) << 24);
      int g0 = 0, n_valid = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(bar(19 + slot), (n >> 1) & 1)) { atomicExch(a.error_flag, 33); break; }
        const int idx = item_ring[slot];
        mbar_arrive_cta(bar(21 + slot));
        if (idx < 0) break;
        const PtItem it = pt_item(a, idx);
        if (!it.valid) continue;
        if (!mbar_wait(bar(0), n_valid & 1)) { atomicExch(a.error_flag, 23); break; }
        ++n_valid;
        const int n_tiles = it.n_tiles;
        auto issue_qk = [&](int j) -> bool {
          const int g = g0 + j, st = g & 1;
          if (g >= 2 && !mbar_wait(bar(11 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 24); return false; }   // S buffer drained
          if (!mbar_wait(bar(1 + st), (g >> 1) & 1)) { atomicExch(a.error_flag, 25); return false; }                  // K tile landed
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const unsigned off = (ks >> 2) * PT_SUB + (ks & 3) * 32;
            tc_mma_bf16(tm_s[st], umma_desc_sw128(q_s + off), umma_desc_sw128(k_s + st * TILE_BYTES + off), idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc_commit(bar(3 + st));    // K stage free
          tc_commit(bar(9 + st));    // S ready
          if (j == n_tiles - 1) tc_commit(bar(18));   // Q free for the next item
          return true;
        };
        ok = issue_qk(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
          const int g = g0 + j, st = g & 1;
          if (j + 1 < n_tiles) ok = issue_qk(j + 1);
          if (!ok) break;
          if (!mbar_wait(bar(13), g & 1)) { atomicExch(a.error_flag, 26); ok = false; break; }                                    // P written
          if (!mbar_wait(bar(5 + st), (g >> 1) & 1)) { atomicExch(a.error_flag, 27); ok = false; break; }                         // V tile landed
          if (g >= 2 && !mbar_wait(bar(16 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 28); ok = false; break; }        // O buffer drained
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < PT_KEYS / 16; ++ks) {
            const unsigned p_off = (ks >> 2) * PT_SUB + (ks & 3) * 32;
            tc_mma_bf16(tm_o[st], umma_desc_sw128(p_s + p_off), umma_desc_sw128_mn(v_s + st * TILE_BYTES + ks * 2048, PT_SUB),
                        idesc_pv, ks > 0 ? 1u : 0u);
          }
          tc_commit(bar(7 + st));    // V stage free
          tc_commit(bar(14 + st));   // O_j ready (and P free)
        }
        g0 += n_tiles;
      }
    }
  } else {
    // PARTS threads per query row: warps 2-5 take the first KP keys of a tile and the first HD / PARTS
    // output columns, warps 6-9 the next, and so on; a warp may only touch the 32 tensor memory lanes
    // of its quadrant (warp index modulo 4), so the threads of a row sit in warps w, w+4, w+8, ...
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // which part of the row (0..PARTS-1)
    const int r = quad * 32 + lane;              // row of the tile
    const unsigned lane_off = (unsigned)(quad * 32) << 16;
    constexpr int HH = HD / PARTS;                // output columns per thread
    const unsigned s_col = (unsigned)(half * KP), o_col = (unsigned)(half * HH);
    int g0 = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int slot = n & 1;
      if (!mbar_wait(bar(19 + slot), (n >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 34); break; }
      const int idx = item_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar(21 + slot));
      if (idx < 0) break;
      const PtItem it = pt_item(a, idx);
      if (!it.valid) continue;
      const int n_tiles = it.n_tiles, tile_lo = it.tile_lo, p_first = it.p_first, p_last = it.p_last;
      const int qi = it.q_first + r;
      const bool valid = qi < it.qlen;
      const int p = it.pos0 + qi;
      const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
      const int lo_last = (a.window > 0 && p_last - a.window + 1 > 0) ? p_last - a.window + 1 : 0;
      float m = -INFINITY, l = 0.0f, m_acc = -INFINITY;   // m_acc: the maximum the rows of o are scaled to
      float o[HH];
#pragma unroll
      for (int i = 0; i < HH; ++i) o[i] = 0.0f;
      auto accumulate = [&](int g) -> bool {        // waits for O of tile g
        const int st = g & 1;
        if (!mbar_wait(bar(14 + st), (g >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 29); return false; }
        tc_fence_after();
        return true;
      };
      float m_tile[2] = {-INFINITY, -INFINITY};      // maximum in force when P of a tile was formed, by stage
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = g0 + j, st = g & 1;
        const int key0 = (tile_lo + j) * PT_KEYS + half * KP;     // first key of this thread's share
        if (!mbar_wait(bar(9 + st), (g >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 30); ok = false; break; }
        tc_fence_after();
        const bool need_mask = ((tile_lo + j) * PT_KEYS + PT_KEYS - 1 > p_first) || ((tile_lo + j) * PT_KEYS < lo_last);
        // pass 1: the row's maximum over this thread's half of the tile (raw scores: the scale is positive)
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < KP / 32; ++c) {
          float s[32];
          tc_ld32f(tm_s[st] + lane_off + s_col + c * 32, s);
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c * 32 + i;
              mx = fmaxf(mx, (key <= p && key >= lo) ? s[i] : -INFINITY);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, s[i]);
          }
        }
        mx *= a.scale_log2;
        // the other half of the row: exchange through shared memory (buffers alternate with the tile)
        float* xm = xch + (g & 1) * (PARTS * 128);
        xm[half * 128 + r] = mx;
        asm volatile("bar.sync 1, %0;" ::"n"(ROW_THREADS) : "memory");
#pragma unroll
        for (int q = 0; q < PARTS; ++q) mx = fmaxf(mx, xm[q * 128 + r]);
        const float m_new = fmaxf(m, mx);
        const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
        // the previous tile's P V must be complete before P is overwritten
        if (j > 0) {
          ok = accumulate(g - 1);
          if (!ok) break;
        }
        // pass 2: P = 2^(s*c - m) into shared memory (K-major, 128-byte swizzle), partial row sum in float
        float sum = 0.0f;
#pragma unroll 1
        for (int c = 0; c < KP / 32; ++c) {
          float s[32];
          tc_ld32f(tm_s[st] + lane_off + s_col + c * 32, s);
          unsigned pk[16];
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c * 32 + i;
              s[i] = (key <= p && key >= lo) ? fast_exp2(fmaf(s[i], a.scale_log2, -m_use)) : 0.0f;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = fast_exp2(fmaf(s[i], a.scale_log2, -m_use));
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            sum += s[i] + s[i + 1];
            __nv_bfloat162 v = __floats2bfloat162_rn(s[i], s[i + 1]);
            pk[i >> 1] = *reinterpret_cast<unsigned*>(&v);
          }
          // 32 keys = four 16-byte chunks of this row in the 64-key sub-tile they belong to; chunk index xor row % 8
          const int k_in_tile = half * KP + c * 32;
          unsigned char* rowp = p_gen + (k_in_tile >> 6) * PT_SUB + r * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (((k_in_tile & 63) >> 3) + q4) ^ (r & 7);
            *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
          }
        }
        const float corr = (m == -INFINITY) ? 0.0f : fast_exp2(m - m_use);
        l = l * corr + sum;          // this thread's share of the row sum; the two shares meet at the end
        m = m_new;
        m_tile[st] = m_new;
        // S buffer read, P written: hand both to the tensor cores
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cta(bar(11 + st));
          mbar_arrive_cta(bar(13));
        }
        // the previous tile's result goes into the registers now, while the tensor cores run this tile's P V
        if (j > 0) {
          const int sp = (g - 1) & 1;
          const float mt = m_tile[sp];
          const float f = (mt == -INFINITY) ? 1.0f : fast_exp2(((m_acc == -INFINITY) ? mt : m_acc) - mt);
#pragma unroll
          for (int c = 0; c < HH / 32; ++c) {      // unrolled: o stays in registers
            float t[32];
            tc_ld32f(tm_o[sp] + lane_off + o_col + c * 32, t);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * f + t[i];
          }
          m_acc = mt;
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cta(bar(16 + sp));    // O buffer free
        }
      }
      if (!ok) break;
      // the row sum is the sum of the two threads' shares (both scaled to the same final maximum)
      float* xl = xch + 2 * PARTS * 128;
      xl[half * 128 + r] = l;
      asm volatile("bar.sync 1, %0;" ::"n"(ROW_THREADS) : "memory");
      l = 0.0f;
#pragma unroll
      for (int q = 0; q < PARTS; ++q) l += xl[q * 128 + r];
      {
        const int g = g0 + n_tiles - 1, sp = g & 1;
        ok = accumulate(g);
        if (!ok) break;
        const float mt = m_tile[sp];
        const float f = (mt == -INFINITY) ? 1.0f : fast_exp2(((m_acc == -INFINITY) ? mt : m_acc) - mt);
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        bf16* dst = a.out + (size_t)(it.row0 + qi) * a.ldo + (size_t)it.h * HD + half * HH;
#pragma unroll
        for (int c = 0; c < HH / 32; ++c) {
          float t[32];
          tc_ld32f(tm_o[sp] + lane_off + o_col + c * 32, t);
          if (c == HH / 32 - 1) {
            // the last read of this O buffer: the tensor cores may have it back for the next item
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(bar(16 + sp));
          }
          if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              unsigned w[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float x0 = (o[c * 32 + i + 2 * u] * f + t[i + 2 * u]) * inv;
                const float x1 = (o[c * 32 + i + 2 * u + 1] * f + t[i + 2 * u + 1]) * inv;
                __nv_bfloat162 v = __floats2bfloat162_rn(x0, x1);
                w[u] = *reinterpret_cast<unsigned*>(&v);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      g0 += n_tiles;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// q: [n_tokens, ldq] with the query heads in its first nh*hd columns; the cache holds n_pages pages.
extern "C" int hb_attention_prefill_tc_bf16(const void* q, int ldq, int n_tokens, void* out, int ldo, const void* kcache,
                                            const void* vcache, int n_pages, const int* seq_start, const int* seq_pos0,
                                            const int* seq_pages, int pages_stride, int n_seqs, int max_q_len, int nh,
                                            int nkv, int hd, int page_size, float scale, int window, int* error_flag,
                                            int* work_counter, void* stream) {
  HB_REQUIRE(n_seqs > 0 && max_q_len > 0 && nh > 0 && nkv > 0 && n_tokens > 0 && n_pages > 0, "attention_prefill_tc: sizes must be positive");
  HB_REQUIRE(hd == 64 || hd == 128, "attention_prefill_tc: head size %d is not 64 or 128", hd);
  HB_REQUIRE(nh % nkv == 0, "attention_prefill_tc: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  HB_REQUIRE(page_size % 64 == 0, "attention_prefill_tc: page size %d must be a multiple of 64", page_size);
  HB_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0,
             "attention_prefill_tc: queries and output need 16-byte aligned rows");
  HB_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "attention_prefill_tc: cache must be 16-byte aligned");
  HB_REQUIRE(nh <= 65535 && n_seqs <= 65535 && window >= 0 && error_flag != nullptr && work_counter != nullptr,
             "attention_prefill_tc: bad arguments (an error flag and a work counter, one int each, are required)");
  HB_REQUIRE(scale > 0.0f, "attention_prefill_tc: the score scale must be positive");
  CUtensorMap mq, mk, mv;
  int rc = make_map_cols(&mq, q, n_tokens, nh * hd, ldq, PT_Q);
  if (rc) return rc;
  const long long cache_rows = (long long)n_pages * nkv * page_size;
  rc = make_map_cols(&mk, kcache, cache_rows, hd, hd, 64);
  if (rc) return rc;
  rc = make_map_cols(&mv, vcache, cache_rows, hd, hd, 64);
  if (rc) return rc;
  const int q_tiles = ceil_div(max_q_len, PT_Q);
  PrefillTcArgs a{(bf16*)out, ldo, seq_start, seq_pos0, seq_pages, pages_stride, nh, nkv, page_size,
                  scale * 1.4426950408889634f, window, error_flag, n_seqs, q_tiles, work_counter};
  cudaStream_t s = (cudaStream_t)stream;
  const long long items = (long long)q_tiles * nh * n_seqs;
  HB_REQUIRE(items < 2147483647LL, "attention_prefill_tc: too many query tiles");
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  dim3 grid((unsigned)(items < sms ? items : sms));
  cudaError_t e = cudaMemsetAsync(work_counter, 0, sizeof(int), s);
  if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reset the work counter: %s", cudaGetErrorString(e));
  const int smem = 6 * (hd / 64) * PT_SUB + 2 * PT_SUB - (hd / 64) * PT_SUB + 1024 + 256 + 6144;   // tiles, slack, barriers, exchange
  if (hd == 128 && max_q_len >= 4096) {
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_tc_kernel<128, 4>, grid, dim3(PT_THREADS(4)), smem, s, mq, mk, mv, a);
  } else if (hd == 128) {
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_tc_kernel<128, 2>, grid, dim3(PT_THREADS(2)), smem, s, mq, mk, mv, a);
  } else {
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_tc_kernel<64, 2>, grid, dim3(PT_THREADS(2)), smem, s, mq, mk, mv, a);
  }
  HB_CHECK_LAUNCH("attention_prefill_tc");
  return 0;
}
