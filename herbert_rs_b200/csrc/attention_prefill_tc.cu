// Prefill attention on the 5th-generation tensor cores (tcgen05), bfloat16, head sizes 64 and 128.
//
// The same arithmetic as attention_prefill.cu (causal grouped-query softmax attention in the flash
// form, float softmax; reference: generic_attention/prefill/kernel_f32.rs:61-111), arranged for
// tensor memory.  A CTA works on two query heads of one key/value head at a time (the reference
// walks the query heads of a key/value head together too, kernel_bf16.rs:236-300): 128 consecutive
// queries of each, over the key tiles (128 keys = two 64-key pages) of their common causal range.
// Both heads read the same K and V tiles, so those are fetched once, and while the row threads of
// one head do their softmax the tensor cores run the products of the other ("ping-pong").
//   warp 0     TMA: the two Q tiles, then K and V tiles into two-stage rings (128-byte swizzle);
//   warp 1     one lane issues tcgen05.mma:  S_t = Q_t K^T  (M=128, N=128) into the head's S buffer
//              in tensor memory, and  O_t += P_t V  (M=128, N=head size; V is the MN-major operand
//              as it lies in the cache) into the head's O buffer, which stays in tensor memory over
//              all key tiles;
//   warps 2-5  head 0, warps 6-9 head 1: one thread per query row.  It reads its row of S (128
//              values) from tensor memory into registers, frees S at once, masks, takes the row
//              maximum, forms P = 2^(s*c - m) as bfloat16 and writes it back into tensor memory over
//              the scores it came from (two values per column: the A operand of the second product is
//              read from tensor memory, so P never passes through shared memory, whose bandwidth the
//              tensor cores' operand reads already use up) and keeps the row sum in float.  m is the maximum the row was last scaled to: it is raised, and O and l are
//              rescaled, only when the tile's maximum exceeds it by more than 2^8 (a factor that
//              cancels in O / l), which after the first tiles almost never happens, so O is not
//              touched between products.
// A head pair whose second head does not exist (an odd number of query heads per key/value head)
// runs the first head alone.  CTAs are persistent and take items from a counter, longest first.
// Every wait on an mbarrier is bounded; a wait that runs out sets *error_flag and the CTA winds down.
#include "api.h"
#include "common.cuh"
#include "tcgen05_utils.cuh"

#define PT_THREADS 320       // TMA warp, MMA warp, four softmax warps per head
#define PT_Q 128             // queries per head and item
#define PT_KEYS 128          // keys per tile
#define PT_SUB (128 * 128)   // bytes of one [128 rows][64 columns] swizzled sub-tile
#define PT_RAISE 8.0f        // the reference maximum is raised when a tile exceeds it by this much (log2 units)

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
  int n_seqs, q_tiles;   // items = q_tiles x n_seqs x nkv x head pairs (some without queries when the sequences differ in length)
  int* work_counter;     // next item; zero when the kernel starts, and left at zero by the CTA that fetches last
};

// One unit of work: 128 consecutive queries of two heads (or one) of one key/value head of one sequence.
struct PtItem {
  int b, kvh, h0, streams, row0, qlen, pos0, q_first, p_first, p_last, tile_lo, n_tiles;
  bool valid;      // false: the sequence has no queries in this tile (shorter than the longest of the batch)
};
__device__ __forceinline__ PtItem pt_item(const PrefillTcArgs& a, int idx) {
  // the longest key ranges (last query tiles) first; neighbours share a sequence and a kv head
  PtItem it;
  const int G = a.nh / a.nkv, pairs = (G + 1) >> 1;
  const int per_seq = a.nkv * pairs, per_qt = per_seq * a.n_seqs;
  const int qt = a.q_tiles - 1 - idx / per_qt, rem = idx % per_qt;
  it.b = rem / per_seq;
  const int r2 = rem % per_seq, pair = r2 % pairs;
  it.kvh = r2 / pairs;
  it.h0 = it.kvh * G + 2 * pair;
  it.streams = (2 * pair + 1 < G) ? 2 : 1;
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

__device__ __forceinline__ void tc_ld32_issue(unsigned taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
        "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
        "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
        "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr));
}
// Two floats in one 64-bit register and the packed float instructions of this architecture.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// The product with the A operand in tensor memory (row i of A in lane i, two bfloat16 per column).
__device__ __forceinline__ void tc_mma_bf16_ta(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                               unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const unsigned* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int HD>
__global__ void __launch_bounds__(PT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcArgs a) {
  constexpr int NB = HD / 64;                 // 64-column blocks of the head
  constexpr int TILE_BYTES = NB * PT_SUB;     // one Q, K, V tile
  extern __shared__ unsigned char smem_raw[];
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
  const unsigned q_s = base, k_s = q_s + 2 * TILE_BYTES, v_s = k_s + 2 * TILE_BYTES;
  const unsigned bars = v_s + 2 * TILE_BYTES;
  // barriers: 0 q_full | 1 q_empty | 2,3 k_full | 4,5 k_empty | 6,7 v_full | 8,9 v_empty | 10,11 s_full (per head)
  //           14,15 p_ready | 17,18 o_full | 19,20 o_empty | 21,22 item_full | 23,24 item_empty
  constexpr int N_BARS = 25;
  auto bar = [&](int i) { return bars + i * 8; };
  volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(gen + (bars - base) + N_BARS * 8);
  volatile int* item_ring = reinterpret_cast<volatile int*>(gen + (bars - base) + N_BARS * 8 + 8);      // [2]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) {
      const bool from_rows = (i == 14 || i == 15 || i == 19 || i == 20);   // the four row warps of a head
      const bool from_consumers = (i == 23 || i == 24);                                          // the MMA lane and all row warps
      mbar_init(bar(i), from_rows ? 4 : (from_consumers ? 9 : 1));
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
  const int G = a.nh / a.nkv;
  const int total_items = a.q_tiles * a.n_seqs * a.nkv * ((G + 1) >> 1);

  // The CTAs are persistent: each takes the next item from a counter in global memory when it has
  // issued everything for its current one.  The TMA warp fetches the index and hands it to the
  // other warps through a ring of two slots, so it can load the next item's tiles while the
  // current item is still being worked on.  Counters of key tiles, of a head's tiles and of the P
  // buffer's uses run on from item to item: ring stages and barrier phases carry over.
  if (warp == 0) {
    if (lane == 0) {
      int g = 0, n_valid = 0;
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        if (n >= 2 && !mbar_wait(bar(23 + slot), ((n >> 1) - 1) & 1)) { atomicExch(a.error_flag, 31); break; }
        const int fetched = atomicAdd(a.work_counter, 1);
        // every CTA stops at its first index beyond the items, so the fetch that returns items + CTAs - 1
        // is the last of the launch: it leaves the counter at zero for the next one
        if (fetched == total_items + (int)gridDim.x - 1) atomicExch(a.work_counter, 0);
        const int idx = fetched < total_items ? fetched : -1;
        item_ring[slot] = idx;
        mbar_arrive_cta(bar(21 + slot));
        if (idx < 0) break;
        const PtItem it = pt_item(a, idx);
        if (!it.valid) continue;
        // the Q buffers are free once the previous item's last S products have read them
        if (n_valid >= 1 && !mbar_wait(bar(1), (n_valid - 1) & 1)) { atomicExch(a.error_flag, 32); break; }
        ++n_valid;
        mbar_expect_tx(bar(0), it.streams * TILE_BYTES);
        for (int t = 0; t < it.streams; ++t)
#pragma unroll
          for (int jb = 0; jb < NB; ++jb)
            tma_load_2d(q_s + t * TILE_BYTES + jb * PT_SUB, &map_q, (it.h0 + t) * HD + jb * 64, it.row0 + it.q_first, bar(0));
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
          if (g >= 2 && !mbar_wait(bar(4 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 21); ok = false; break; }
          mbar_expect_tx(bar(2 + st), TILE_BYTES);
#pragma unroll
          for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int half = 0; half < 2; ++half)
              tma_load_2d(k_s + st * TILE_BYTES + jb * PT_SUB + half * 8192, &map_k, jb * 64, rows[half], bar(2 + st));
          if (g >= 2 && !mbar_wait(bar(8 + st), ((g >> 1) - 1) & 1)) { atomicExch(a.error_flag, 22); ok = false; break; }
          mbar_expect_tx(bar(6 + st), TILE_BYTES);
#pragma unroll
          for (int jb = 0; jb < NB; ++jb)
#pragma unroll
            for (int half = 0; half < 2; ++half)
              tma_load_2d(v_s + st * TILE_BYTES + jb * PT_SUB + half * 8192, &map_v, jb * 64, rows[half], bar(6 + st));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // D float, A and B bfloat16; B of the second product is MN-major (bit 16)
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PT_KEYS >> 3) << 17) | ((unsigned)(PT_Q >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(PT_Q >> 4) << 24);
      const unsigned long long desc_q[2] = {umma_desc_sw128(q_s), umma_desc_sw128(q_s + TILE_BYTES)};
      const unsigned long long desc_k[2] = {umma_desc_sw128(k_s), umma_desc_sw128(k_s + TILE_BYTES)};
      const unsigned long long desc_v[2] = {umma_desc_sw128_mn(v_s, PT_SUB), umma_desc_sw128_mn(v_s + TILE_BYTES, PT_SUB)};
      int g0 = 0, n_valid = 0;
      int c[2] = {0, 0}, items_done[2] = {0, 0};     // per head: key tiles and items so far
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(bar(21 + slot), (n >> 1) & 1)) { atomicExch(a.error_flag, 33); break; }
        const int idx = item_ring[slot];
        mbar_arrive_cta(bar(23 + slot));
        if (idx < 0) break;
        const PtItem it = pt_item(a, idx);
        if (!it.valid) continue;
        if (!mbar_wait(bar(0), n_valid & 1)) { atomicExch(a.error_flag, 23); break; }
        ++n_valid;
        const int n_tiles = it.n_tiles, streams = it.streams;
        auto issue_qk = [&](int t, int j) -> bool {
          // The scores overwrite the head's previous P.  Its rows have read the previous scores (they
          // wrote P after that), and the product that reads P was issued before this one: tcgen05.mma
          // instructions of a CTA execute in the order of their issue.
          const int g = g0 + j, st = g & 1;
          if (!mbar_wait(bar(2 + st), (g >> 1) & 1)) { atomicExch(a.error_flag, 25); return false; }             // K tile landed
          tc_fence_after();
          // descriptors differ in their address field only (16-byte units, the low bits of the word)
          const unsigned long long dq = desc_q[t], dk = desc_k[st];
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const unsigned off16 = ((ks >> 2) * PT_SUB + (ks & 3) * 32) >> 4;
            tc_mma_bf16(tm_s[t], dq + off16, dk + off16, idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc_commit(bar(10 + t));    // S ready
          if (t == streams - 1) {
            tc_commit(bar(4 + st));                      // K stage free
            if (j == n_tiles - 1) tc_commit(bar(1));     // Q free for the next item
          }
          return true;
        };
        auto issue_pv = [&](int t, int j) -> bool {
          const int g = g0 + j, st = g & 1, ct = c[t] + j;
          if (!mbar_wait(bar(14 + t), ct & 1)) { atomicExch(a.error_flag, 26); return false; }                     // P written (and O rescaled)
          if (!mbar_wait(bar(6 + st), (g >> 1) & 1)) { atomicExch(a.error_flag, 27); return false; }               // V tile landed
          if (j == 0 && items_done[t] >= 1 && !mbar_wait(bar(19 + t), (items_done[t] - 1) & 1)) { atomicExch(a.error_flag, 28); return false; }   // O read out
          tc_fence_after();
          const unsigned long long dv = desc_v[st];
#pragma unroll
          for (int ks = 0; ks < PT_KEYS / 16; ++ks)      // 16 keys of P = 8 columns of tensor memory
            tc_mma_bf16_ta(tm_o[t], tm_s[t] + ks * 8, dv + (unsigned)(ks * 2048 >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(bar(17 + t));    // O holds this tile too
          if (t == streams - 1) tc_commit(bar(8 + st));   // V stage free
          return true;
        };
        // Per head: scores, (rows: softmax), P V, next scores, ...; while one head's rows work, the
        // tensor cores run the other head's two products.
        for (int t = 0; t < streams && ok; ++t) ok = issue_qk(t, 0);
        for (int j = 0; j < n_tiles && ok; ++j)
          for (int t = 0; t < streams && ok; ++t) {
            ok = issue_pv(t, j);
            if (ok && j + 1 < n_tiles) ok = issue_qk(t, j + 1);
          }
        g0 += n_tiles;
        for (int t = 0; t < streams; ++t) {
          c[t] += n_tiles;
          ++items_done[t];
        }
      }
    }
  } else {
    // One thread per query row.  A warp may only touch the 32 tensor memory lanes of its quadrant
    // (warp index modulo 4): warps 2-5 are head 0, warps 6-9 head 1.
    const int t = (warp - 2) >> 2;               // which head of the pair
    const int quad = warp & 3;
    const int r = quad * 32 + lane;              // row of the tile
    const unsigned lane_off = (unsigned)(quad * 32) << 16;
    int c_t = 0;                                 // this head's key tiles so far
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int slot = n & 1;
      if (!mbar_wait(bar(21 + slot), (n >> 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 34); break; }
      const int idx = item_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar(23 + slot));
      if (idx < 0) break;
      const PtItem it = pt_item(a, idx);
      if (!it.valid) continue;
      const int n_tiles = it.n_tiles, streams = it.streams;
      if (t >= streams) continue;  // the pair has one head only: nothing for this group
      const int tile_lo = it.tile_lo, p_first = it.p_first, p_last = it.p_last;
      const int qi = it.q_first + r;
      const bool valid = qi < it.qlen;
      const int p = it.pos0 + qi;
      const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
      const int lo_last = (a.window > 0 && p_last - a.window + 1 > 0) ? p_last - a.window + 1 : 0;
      float m = -INFINITY, l = 0.0f;     // m: the maximum the row's P, l and O are scaled to
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int ct = c_t + j;
        const int key0 = (tile_lo + j) * PT_KEYS;
        if (!mbar_wait(bar(10 + t), ct & 1)) { if (lane == 0) atomicExch(a.error_flag, 30); ok = false; break; }
        tc_fence_after();
        float s[PT_KEYS];
#pragma unroll
        for (int cc = 0; cc < PT_KEYS / 32; ++cc) tc_ld32_issue(tm_s[t] + lane_off + cc * 32, s + cc * 32);
        tc_wait_ld();
        const bool need_mask = (key0 + PT_KEYS - 1 > p_first) || (key0 < lo_last);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < PT_KEYS; ++i) {
            const int key = key0 + i;
            s[i] = (key <= p && key >= lo) ? s[i] : -INFINITY;
          }
        }
        float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: the instruction's latency is hidden
#pragma unroll
        for (int i = 0; i < PT_KEYS; i += 8)
#pragma unroll
          for (int q = 0; q < 4; ++q) mxs[q] = max3(mxs[q], s[i + 2 * q], s[i + 2 * q + 1]);
        float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
        mx *= a.scale_log2;         // the scale is positive: the maximum of the raw scores is the maximum
        const bool raise = mx > m + PT_RAISE || (m == -INFINITY && mx > -INFINITY);
        if (j > 0 && __any_sync(0xffffffffu, raise)) {
          // rescale O to the new maximum (rows that keep theirs: factor 1); the product of the tile before must be complete
          if (!mbar_wait(bar(17 + t), (ct - 1) & 1)) { if (lane == 0) atomicExch(a.error_flag, 29); ok = false; break; }
          tc_fence_after();
          const float f = raise ? ((m == -INFINITY) ? 0.0f : fast_exp2(m - mx)) : 1.0f;
#pragma unroll 1
          for (int cc = 0; cc < HD / 16; ++cc) {
            float o[16];
            tc_ld16f(tm_o[t] + lane_off + cc * 16, o);
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] *= f;
            tc_st16f(tm_o[t] + lane_off + cc * 16, o);
          }
        }
        if (raise) {
          l *= (m == -INFINITY) ? 0.0f : fast_exp2(m - mx);
          m = mx;
        }
        const float m_use = (m == -INFINITY) ? 0.0f : m;
        // P = 2^(s*c - m) as bfloat16 pairs; masked scores are -inf and give 0
        unsigned pk[PT_KEYS / 2];
        const unsigned long long c2 = pack2(a.scale_log2, a.scale_log2), m2 = pack2(-m_use, -m_use);
        unsigned long long sum2 = pack2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < PT_KEYS; i += 2) {
          float x0, x1;
          unpack2(fma2(pack2(s[i], s[i + 1]), c2, m2), x0, x1);      // two scores per instruction
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          sum2 = add2(sum2, pack2(e0, e1));
          __nv_bfloat162 v = __floats2bfloat162_rn(e0, e1);
          pk[i >> 1] = *reinterpret_cast<unsigned*>(&v);
        }
        float sum_a, sum_b;
        unpack2(sum2, sum_a, sum_b);
        const float sum = sum_a + sum_b;
        l += sum;
        // P goes where the row's scores were: 64 columns of two bfloat16 each
        tc_st32(tm_s[t] + lane_off, pk);
        tc_st32(tm_s[t] + lane_off + 32, pk + 32);
        tc_wait_st();
        // P written (and O rescaled): hand them to the tensor cores
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(bar(14 + t));
      }
      if (!ok) break;
      {
        const int ct = c_t + n_tiles - 1;
        if (!mbar_wait(bar(17 + t), ct & 1)) { if (lane == 0) atomicExch(a.error_flag, 36); ok = false; break; }
        tc_fence_after();
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        bf16* dst = a.out + (size_t)(it.row0 + qi) * a.ldo + (size_t)(it.h0 + t) * HD;
#pragma unroll
        for (int cc = 0; cc < HD / 32; ++cc) {
          float o[32];
          tc_ld32_issue(tm_o[t] + lane_off + cc * 32, o);
          tc_wait_ld();
          if (cc == HD / 32 - 1) {
            // the last read of this O buffer: the tensor cores may have it back for the next item
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(bar(19 + t));
          }
          if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              unsigned w[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[i + 2 * u] * inv, o[i + 2 * u + 1] * inv);
                w[u] = *reinterpret_cast<unsigned*>(&v);
              }
              *reinterpret_cast<uint4*>(dst + cc * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
      c_t += n_tiles;
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
  const int pairs = (nh / nkv + 1) / 2;
  const long long items = (long long)q_tiles * n_seqs * nkv * pairs;
  HB_REQUIRE(items < 2147483647LL, "attention_prefill_tc: too many query tiles");
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  dim3 grid((unsigned)(items < sms ? items : sms));
  cudaError_t e;
  // two Q tiles, two stages of K and of V; slack for the 1024-byte alignment; barriers and the item ring
  const int smem = 6 * (hd / 64) * PT_SUB + 1024 + 512;
  if (hd == 128) {
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_tc_kernel<128>, grid, dim3(PT_THREADS), smem, s, mq, mk, mv, a);
  } else {
    e = cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_tc_kernel<64>, grid, dim3(PT_THREADS), smem, s, mq, mk, mv, a);
  }
  HB_CHECK_LAUNCH("attention_prefill_tc");
  return 0;
}
