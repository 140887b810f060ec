// Decode attention over the paged cache: one new query per sequence, bfloat16, tensor cores.
//
// Work is split over (key range, kv head, sequence): a CTA takes a run of 64-key pages of one kv
// head of one sequence and serves all query heads of that kv head's group at once, so a key or
// value is read from memory once for the whole group (the reference pairs the heads of a group
// against each key row the same way: backends/backend_common/src/avx512_attn_dot8_bf16.S, and
// its Metal flash-decoding kernel splits the keys into tiles with partial (m, l, o) results:
// backends/backend_metal attention_decode_flash_v2.metal).  Pages travel global -> shared with
// cp.async in a ring of stages; each of the 4 warps owns 16 keys of every page:
//   S = Q K^T  (mma.sync m16n8k16, query heads padded to 16 rows), s = dot * scale,
//   online softmax in float (running m, l per head),  O += P V  (V through ldmatrix.trans).
// Warps, then splits, are merged with the usual rescaling; every split writes (m, l, O) to
// scratch memory and a second kernel combines them:  out = sum_s e^{m_s - m} O_s / sum_s e^{m_s - m} l_s.
// Keys visible to the query at position p: lo..p, lo = max(0, p - window + 1) if window > 0.
#include <stdlib.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"
#include "qk_norm.cuh"

// exp: the hardware's fast exponential (ex2.approx, about 2 ulp in float).  The probabilities are
// rounded to bfloat16 for the P V product right after, so nothing is lost; sums stay in float.

#define AD_WARPS 4
#define AD_THREADS (AD_WARPS * 32)
#define AD_TILE 64
#define AD_MAX_TILES 1024   // tiles one CTA may be given (65,536 keys); the launcher sizes the splits to that

struct DecodeArgs {
  const bf16* q;       // [B, ldq]: row b holds the query heads of sequence b's new token
  int ldq;
  const bf16* kcache;  // [pages][nkv][page_size][hd]
  const bf16* vcache;
  const int* seq_len;  // length after this step (the new token's key is already stored)
  const int* seq_pages;
  int pages_stride;
  float* part_o;       // [B][nh][nsplit][hd]
  float* part_ml;      // [B][nh][nsplit][2]
  int nh, nkv, hd, page_size, nsplit;
  float scale;
  int window;
  int stages;
};

// What the fused variant of the keys-as-M kernel needs besides: it takes the raw q/k/v row of each
// sequence's new token, applies the per-head RMSNorm and the rotation to the query heads it serves
// (and, in the CTA whose keys include the new position, to the new key, which it stores in the
// cache together with the new value before it reads its pages), and the split that finishes last
// combines all splits' partial results.  Three kernels' work in one launch.
struct DecodeFuse {
  const bf16* qkv;       // [B, ld]: q heads, then k heads, then v heads of the new token, as the projection left them
  int ld;
  const float* qw;       // per-head norm weights [hd] (null: no norm)
  const float* kw;
  float eps;
  const float* cos_tab;  // [table_rows][hd / 2]
  const float* sin_tab;
  int table_rows;
  int write_cache;       // 0: a layer that reads another layer's cache stores nothing
  bf16* kcache_w;        // the same cache, writable
  bf16* vcache_w;
  int* counters;         // [B * nkv], zero between launches
  bf16* out;             // [B, ldo]
  int ldo;
};

// HDM: the largest head size this instantiation holds in registers (hd <= HDM, hd % 16 == 0).
template <int HDM>
__global__ void __launch_bounds__(AD_THREADS) attention_decode_kernel(DecodeArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int hd = a.hd, G = a.nh / a.nkv;
  const int row_bytes = hd * 2 + 16;                 // padded: conflict-free ldmatrix for any hd % 16 == 0
  const int tile_bytes = AD_TILE * row_bytes;
  const int chunks_per_row = hd >> 3;

  const int len = a.seq_len[b];
  const int p = len - 1;
  const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
  const int tile_lo = lo / AD_TILE, tile_hi = (len + AD_TILE - 1) / AD_TILE;   // tiles [tile_lo, tile_hi)
  const int ntiles = tile_hi - tile_lo;
  // tiles dealt evenly: the first ntiles % nsplit splits take one more than the others
  const int per = ntiles / a.nsplit, extra = ntiles % a.nsplit;
  const int t0 = tile_lo + split * per + min(split, extra);
  const int t1 = t0 + per + (split < extra ? 1 : 0);
  const int tiles_per_page = a.page_size / AD_TILE;
  const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
  const size_t head_elems = (size_t)a.page_size * hd;
  // the pages of this CTA's tiles, fetched once (a look-up per tile would put a memory round trip
  // in front of every copy)
  __shared__ int page_ids[AD_MAX_TILES];
  const int first_tile = t0;
  for (int i = threadIdx.x; i < t1 - t0; i += AD_THREADS) page_ids[i] = pages[(t0 + i) / tiles_per_page];
  __syncthreads();

  // The 16-byte chunks of a tile this thread copies: offsets worked out once, so that issuing a
  // tile's copies is one add per chunk.
  constexpr int SLOTS = HDM / 16;            // 64 rows * (hd / 8) chunks / 128 threads, at hd = HDM
  int g_off[SLOTS], s_off[SLOTS];
  {
    int r = threadIdx.x / chunks_per_row, cc = threadIdx.x % chunks_per_row;
    const int step_r = AD_THREADS / chunks_per_row, step_c = AD_THREADS % chunks_per_row;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
      g_off[i] = r * hd + cc * 8;
      s_off[i] = r < AD_TILE ? r * row_bytes + cc * 16 : -1;
      r += step_r;
      cc += step_c;
      if (cc >= chunks_per_row) {
        cc -= chunks_per_row;
        ++r;
      }
    }
  }
  const unsigned smem_u = (unsigned)__cvta_generic_to_shared(smem);
  auto issue = [&](int tile, int stage) {
    const int page = page_ids[tile - first_tile];
    const size_t off = ((size_t)page * a.nkv + kvh) * head_elems + (size_t)(tile % tiles_per_page) * AD_TILE * hd;
    const bf16* kg = a.kcache + off;
    const bf16* vg = a.vcache + off;
    const unsigned ks = smem_u + stage * 2 * tile_bytes;
    const unsigned vs = ks + tile_bytes;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
      if (s_off[i] >= 0) {
        cp_async16_s(ks + s_off[i], kg + g_off[i]);
        cp_async16_s(vs + s_off[i], vg + g_off[i]);
      }
    }
  };
  // ldmatrix addresses of this lane inside a tile (the k or d step adds a constant)
  const int lm = lane >> 3;
  const unsigned k_lane = (unsigned)((warp * 16 + (lm >> 1) * 8 + (lane & 7)) * row_bytes + (lm & 1) * 16);
  const unsigned v_lane = (unsigned)((warp * 16 + (lm & 1) * 8 + (lane & 7)) * row_bytes + (lm >> 1) * 16);

  // query fragments: rows = heads of the group (g and g + 8), zero beyond G
  unsigned qf[HDM / 16][4];
  {
    const bf16* qb = a.q + (size_t)b * a.ldq + (size_t)kvh * G * hd;
#pragma unroll
    for (int ks = 0; ks < HDM / 16; ++ks) {
      qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
      if (ks * 16 < hd) {
        const int d = ks * 16 + 2 * t;
        if (g < G) {
          qf[ks][0] = *reinterpret_cast<const unsigned*>(qb + (size_t)g * hd + d);
          qf[ks][2] = *reinterpret_cast<const unsigned*>(qb + (size_t)g * hd + d + 8);
        }
        if (g + 8 < G) {
          qf[ks][1] = *reinterpret_cast<const unsigned*>(qb + (size_t)(g + 8) * hd + d);
          qf[ks][3] = *reinterpret_cast<const unsigned*>(qb + (size_t)(g + 8) * hd + d + 8);
        }
      }
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};   // heads g and g + 8
  float o[HDM / 8][4];
#pragma unroll
  for (int i = 0; i < HDM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  const int S = a.stages;
  for (int i = 0; i < S - 1; ++i) {
    if (t0 + i < t1) issue(t0 + i, i);
    cp_async_commit();
  }
  for (int tile = t0; tile < t1; ++tile) {
    const int it = tile - t0;
    if (tile + S - 1 < t1) issue(tile + S - 1, (it + S - 1) % S);
    cp_async_commit();
    // groups committed so far: S - 1 + it + 1; the group of `tile` is done when at most S - 1 are pending
    if (S == 2) cp_async_wait<1>(); else if (S == 3) cp_async_wait<2>(); else cp_async_wait<3>();
    __syncthreads();
    const unsigned ks = smem_u + (unsigned)(it % S) * 2 * tile_bytes;
    const unsigned vs = ks + tile_bytes;
    const int key0 = tile * AD_TILE + warp * 16;
    if (key0 <= p && key0 + 15 >= lo) {
      // ---- S = Q K^T for this warp's 16 keys -------------------------------------------------
      float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
      for (int kk = 0; kk < HDM / 16; ++kk) {
        if (kk * 16 < hd) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_s(b0, b1, b2, b3, ks + k_lane + kk * 32);
          mma16816(s[0], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
          mma16816(s[1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
        }
      }
      // ---- mask, online softmax ---------------------------------------------------------------
      float mx[2] = {-INFINITY, -INFINITY};
      const bool edge = key0 + 15 > p || key0 < lo;      // only the first and last tiles of the range need the mask
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = s[nt][j] * a.scale;
          if (edge) {
            const int key = key0 + nt * 8 + 2 * t + (j & 1);
            if (!(key <= p && key >= lo)) v = -INFINITY;
          }
          s[nt][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        corr[r] = (m_new == -INFINITY) ? 1.0f : __expf(m[r] - m_new);
        m[r] = m_new;
      }
      float ps[2] = {0.0f, 0.0f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float pv = (s[nt][j] == -INFINITY) ? 0.0f : __expf(s[nt][j] - m[j >> 1]);
          s[nt][j] = pv;
          ps[j >> 1] += pv;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 1);
        ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 2);
        l[r] = l[r] * corr[r] + ps[r];
      }
      const unsigned pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
      const unsigned pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
      // ---- O = O * corr + P V (the rescale is skipped while no maximum of the warp's rows moved) ---
      const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f);
#pragma unroll
      for (int nd = 0; nd < HDM / 16; ++nd) {
        if (nd * 16 < hd) {
          if (rescale) {
            o[2 * nd][0] *= corr[0]; o[2 * nd][1] *= corr[0]; o[2 * nd][2] *= corr[1]; o[2 * nd][3] *= corr[1];
            o[2 * nd + 1][0] *= corr[0]; o[2 * nd + 1][1] *= corr[0]; o[2 * nd + 1][2] *= corr[1]; o[2 * nd + 1][3] *= corr[1];
          }
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans_s(b0, b1, b2, b3, vs + v_lane + nd * 32);
          mma16816(o[2 * nd], pa0, pa1, pa2, pa3, b0, b1);
          mma16816(o[2 * nd + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
    }
    __syncthreads();   // every warp is done with this stage before it is refilled
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the 4 warps through shared memory ---------------------------------------------------
  float* sm_m = reinterpret_cast<float*>(smem);            // [4][16]
  float* sm_l = sm_m + AD_WARPS * 16;                      // [4][16]
  float* sm_o = sm_l + AD_WARPS * 16;                      // [4][16][hd]
  if (t == 0) {
    sm_m[warp * 16 + g] = m[0]; sm_m[warp * 16 + g + 8] = m[1];
    sm_l[warp * 16 + g] = l[0]; sm_l[warp * 16 + g + 8] = l[1];
  }
#pragma unroll
  for (int nd = 0; nd < HDM / 8; ++nd) {
    if (nd * 8 < hd) {
      const int d = nd * 8 + 2 * t;
      float* r0 = sm_o + ((size_t)warp * 16 + g) * hd + d;
      float* r1 = sm_o + ((size_t)warp * 16 + g + 8) * hd + d;
      r0[0] = o[nd][0]; r0[1] = o[nd][1];
      r1[0] = o[nd][2]; r1[1] = o[nd][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * hd; idx += AD_THREADS) {
    const int r = idx / hd, d = idx % hd;
    if (r >= 16) break;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w) mm = fmaxf(mm, sm_m[w * 16 + r]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w) {
      const float mw = sm_m[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.0f : __expf(mw - mm);
      acc += f * sm_o[((size_t)w * 16 + r) * hd + d];
      ll += f * sm_l[w * 16 + r];
    }
    const int h = kvh * G + r;
    const size_t pi = ((size_t)b * a.nh + h) * a.nsplit + split;
    a.part_o[pi * hd + d] = acc;
    if (d == 0) {
      a.part_ml[pi * 2] = mm;
      a.part_ml[pi * 2 + 1] = ll;
    }
  }
}

// The same work with the roles of the tensor-core operands turned round, for head size 128: the
// 16 keys of a warp's slab are the M side, the (up to 8 * NH) query heads of the group the N side:
//   S^T[16 keys x 8 heads] = K_slab Q^T,   O^T[128 x 8 heads] += V_slab^T P^T.
// Half the MMAs of the kernel above (no rows of padding), half the accumulator registers, and a
// thread owns two heads outright, so the running maximum needs three shuffles per slab and the
// running sum none until the end.  P^T changes from accumulator to B-operand layout with movmatrix.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
  unsigned r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void mma16816_ab(float* d, const unsigned* a4, unsigned b0, unsigned b1) {
  mma16816(d, a4[0], a4[1], a4[2], a4[3], b0, b1);
}

__device__ __forceinline__ void st_bf2(bf16* p, float x, float y) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}

template <int NH, bool FUSED>
__global__ void __launch_bounds__(AD_THREADS) attention_decode_km_kernel(DecodeArgs a, DecodeFuse f) {
  constexpr int HD = 128;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ __align__(16) bf16 sm_q[FUSED ? 8 * NH * HD : 8];
  __shared__ int s_last;
  // Before the wait on the kernel before: only what the host wrote ahead of the step (lengths, page
  // tables) and what earlier steps left in the cache.
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int G = a.nh / a.nkv;
  constexpr int row_bytes = HD * 2 + 16;
  constexpr int tile_bytes = AD_TILE * row_bytes;
  constexpr int chunks_per_row = HD >> 3;

  const int len = a.seq_len[b];
  const int p = len - 1;
  const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
  const int tile_lo = lo / AD_TILE, tile_hi = (len + AD_TILE - 1) / AD_TILE;
  const int ntiles = tile_hi - tile_lo;
  // tiles dealt evenly: the first ntiles % nsplit splits take one more than the others
  const int per = ntiles / a.nsplit, extra = ntiles % a.nsplit;
  const int t0 = tile_lo + split * per + min(split, extra);
  const int t1 = t0 + per + (split < extra ? 1 : 0);
  const int tiles_per_page = a.page_size / AD_TILE;
  const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
  const size_t head_elems = (size_t)a.page_size * HD;
  __shared__ int page_ids[AD_MAX_TILES];
  for (int i = threadIdx.x; i < t1 - t0; i += AD_THREADS) page_ids[i] = pages[(t0 + i) / tiles_per_page];
  const bool writer = FUSED && f.write_cache && t0 < t1 && t1 == tile_hi;   // this CTA's keys end with the new position
  __syncthreads();

  constexpr int SLOTS = HD / 16;
  int g_off[SLOTS], s_off[SLOTS];
#pragma unroll
  for (int i = 0; i < SLOTS; ++i) {
    const int c = threadIdx.x + i * AD_THREADS;
    const int r = c / chunks_per_row, cc = c % chunks_per_row;
    g_off[i] = r * HD + cc * 8;
    s_off[i] = r * row_bytes + cc * 16;
  }
  const unsigned smem_u = (unsigned)__cvta_generic_to_shared(smem);
  auto issue = [&](int tile, int stage) {
    const int page = page_ids[tile - t0];
    const size_t off = ((size_t)page * a.nkv + kvh) * head_elems + (size_t)(tile % tiles_per_page) * AD_TILE * HD;
    const bf16* kg = a.kcache + off;
    const bf16* vg = a.vcache + off;
    const unsigned ks = smem_u + stage * 2 * tile_bytes;
    const unsigned vs = ks + tile_bytes;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
      cp_async16_s(ks + s_off[i], kg + g_off[i]);
      cp_async16_s(vs + s_off[i], vg + g_off[i]);
    }
  };
  const int S = a.stages;
  auto first_tiles = [&]() {
    for (int i = 0; i < S - 1; ++i) {
      if (t0 + i < t1) issue(t0 + i, i);
      cp_async_commit();
    }
  };
  // The tile with the new position is written in this step (here, or by a kernel before this one):
  // a CTA whose first loads would reach it starts them after the new key and value are stored.
  const bool early = !(t0 < t1 && t1 == tile_hi && t1 - t0 <= S - 1);
  pdl_wait();
  // This step's q (and, in the CTA that stores them, k and v) are asked for before the tiles: behind
  // the tiles' bulk loads these few bytes would wait for all of them.
  const int trow = p < f.table_rows ? p : f.table_rows - 1;
  const bf16* row = FUSED ? f.qkv + (size_t)b * f.ld : nullptr;
  const int qh = 2 * warp + (lane >> 4), qhc = qh < G ? qh : 0;     // a head per half-warp (the first 2 * AD_WARPS heads)
  NormRotateLoads q_regs, k_regs;
  uint2 v_regs = make_uint2(0u, 0u);
  if (FUSED) q_regs = norm_rotate_load<bf16>(qh < G, row + (size_t)(kvh * G + qhc) * HD, f.qw, f.cos_tab + (size_t)trow * 64,
                                             f.sin_tab + (size_t)trow * 64, lane & 15);
  if (writer) {
    if (warp == 0) k_regs = norm_rotate_load<bf16>(lane < 16, row + (size_t)(a.nh + kvh) * HD, f.kw, f.cos_tab + (size_t)trow * 64,
                                                   f.sin_tab + (size_t)trow * 64, lane & 15);
    else if (warp == 1) v_regs = *reinterpret_cast<const uint2*>(row + (size_t)(a.nh + a.nkv + kvh) * HD + 4 * lane);
  }
  if (early) first_tiles();
  if (writer) {
    // store the new token's key (normed, rotated) and value before their page is read
    const size_t dst = (((size_t)pages[p / a.page_size] * a.nkv + kvh) * a.page_size + (p % a.page_size)) * HD;
    if (warp == 0) norm_rotate_finish<bf16>(k_regs, lane < 16, f.kcache_w + dst, f.kw != nullptr, f.eps, lane & 15);
    else if (warp == 1) *reinterpret_cast<uint2*>(f.vcache_w + dst + 4 * lane) = v_regs;
  }
  if (!early) {
    __syncthreads();        // the new key and value are stored before their tile is fetched
    first_tiles();
  }
  // A-operand fragments come from shared memory: K rows as they lie, V transposed
  const int lm = lane >> 3;
  const unsigned k_lane = (unsigned)((warp * 16 + (lm & 1) * 8 + (lane & 7)) * row_bytes + (lm >> 1) * 16);
  const unsigned v_lane = (unsigned)((warp * 16 + (lm >> 1) * 8 + (lane & 7)) * row_bytes + (lm & 1) * 16);

  // per thread: heads n*8 + 2t and n*8 + 2t + 1
  float m[NH][2], l[NH][2], o[NH][HD / 16][4];
#pragma unroll
  for (int n = 0; n < NH; ++n) {
    m[n][0] = m[n][1] = -INFINITY;
    l[n][0] = l[n][1] = 0.0f;
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[n][i][0] = o[n][i][1] = o[n][i][2] = o[n][i][3] = 0.0f;
  }

  if (FUSED) {
    // the query heads of this group, normed and rotated, while the first pages are on their way
    norm_rotate_finish<bf16>(q_regs, qh < G, sm_q + qhc * HD, f.qw != nullptr, f.eps, lane & 15);
    for (int h0 = 2 * AD_WARPS; h0 < G; h0 += 2 * AD_WARPS) {           // more heads than half-warps
      const int h = h0 + 2 * warp + (lane >> 4);
      const int hc = h < G ? h : 0;
      norm_rotate_head128<bf16>(h < G, row + (size_t)(kvh * G + hc) * HD, sm_q + hc * HD, f.qw, f.eps,
                                f.cos_tab + (size_t)trow * 64, f.sin_tab + (size_t)trow * 64, lane & 15);
    }
    __syncthreads();
  }
  // B operand of the first product: Q^T, head g of each 8-head tile, d pairs (2t, 2t+1) and (2t+8, 2t+9)
  unsigned qf[NH][HD / 16][2];
  {
    const bf16* qb = FUSED ? sm_q : a.q + (size_t)b * a.ldq + (size_t)kvh * G * HD;
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      const int h = n * 8 + g;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        qf[n][ks][0] = qf[n][ks][1] = 0u;
        if (h < G) {
          qf[n][ks][0] = *reinterpret_cast<const unsigned*>(qb + (size_t)h * HD + ks * 16 + 2 * t);
          qf[n][ks][1] = *reinterpret_cast<const unsigned*>(qb + (size_t)h * HD + ks * 16 + 2 * t + 8);
        }
      }
    }
  }
  for (int tile = t0; tile < t1; ++tile) {
    const int it = tile - t0;
    if (tile + S - 1 < t1) issue(tile + S - 1, (it + S - 1) % S);
    cp_async_commit();
    if (S == 2) cp_async_wait<1>(); else if (S == 3) cp_async_wait<2>(); else cp_async_wait<3>();
    __syncthreads();
    const unsigned ks = smem_u + (unsigned)(it % S) * 2 * tile_bytes;
    const unsigned vs = ks + tile_bytes;
    const int key0 = tile * AD_TILE + warp * 16;
    if (key0 <= p && key0 + 15 >= lo) {
      // ---- S^T = K Q^T: rows = this warp's 16 keys, columns = heads ------------------------------
      float s[NH][4];
#pragma unroll
      for (int n = 0; n < NH; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        unsigned af[4];
        ldmatrix_x4_s(af[0], af[1], af[2], af[3], ks + k_lane + kk * 32);
#pragma unroll
        for (int n = 0; n < NH; ++n) mma16816_ab(s[n], af, qf[n][kk][0], qf[n][kk][1]);
      }
      // s[n][0], s[n][1]: key g, heads 2t, 2t+1;  s[n][2], s[n][3]: key g + 8, the same heads
      const bool edge = key0 + 15 > p || key0 < lo;
      const bool k0_ok = !edge || (key0 + g <= p && key0 + g >= lo);
      const bool k1_ok = !edge || (key0 + g + 8 <= p && key0 + g + 8 >= lo);
      bool rescale = false;
      float corr[NH][2];
      unsigned pb[NH][2];
#pragma unroll
      for (int n = 0; n < NH; ++n) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float v0 = k0_ok ? s[n][j] * a.scale : -INFINITY;
          float v1 = k1_ok ? s[n][2 + j] * a.scale : -INFINITY;
          float mx = fmaxf(v0, v1);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m[n][j], mx);
          const float mu = (m_new == -INFINITY) ? 0.0f : m_new;
          corr[n][j] = (m_new == m[n][j]) ? 1.0f : __expf(m[n][j] - m_new);     // m = -inf before: exp(-inf) = 0
          rescale |= corr[n][j] != 1.0f;
          m[n][j] = m_new;
          v0 = k0_ok ? __expf(v0 - mu) : 0.0f;
          v1 = k1_ok ? __expf(v1 - mu) : 0.0f;
          l[n][j] = l[n][j] * corr[n][j] + (v0 + v1);          // this thread's keys only; the lanes' shares meet at the end
          s[n][j] = v0;
          s[n][2 + j] = v1;
        }
        // P^T from accumulator layout (key g; heads 2t, 2t+1) to B-operand layout (head g; keys 2t, 2t+1)
        pb[n][0] = movmatrix_trans(pack_bf16(s[n][0], s[n][1]));
        pb[n][1] = movmatrix_trans(pack_bf16(s[n][2], s[n][3]));
      }
      rescale = __any_sync(0xffffffffu, rescale);
      // ---- O^T += V^T P^T: rows = 16 values of the head size per step, columns = heads -------------
#pragma unroll
      for (int md = 0; md < HD / 16; ++md) {
        unsigned af[4];
        ldmatrix_x4_trans_s(af[0], af[1], af[2], af[3], vs + v_lane + md * 32);
#pragma unroll
        for (int n = 0; n < NH; ++n) {
          if (rescale) {
            o[n][md][0] *= corr[n][0]; o[n][md][1] *= corr[n][1];
            o[n][md][2] *= corr[n][0]; o[n][md][3] *= corr[n][1];
          }
          mma16816_ab(o[n][md], af, pb[n][0], pb[n][1]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  pdl_launch();     // the keys are read: the next kernel's CTAs may come in while the partial results meet

  // ---- merge the 4 warps through shared memory ---------------------------------------------------
  constexpr int HP = 8 * NH;                               // heads, padded
  float* sm_m = reinterpret_cast<float*>(smem);            // [4][HP]
  float* sm_l = sm_m + AD_WARPS * HP;                      // [4][HP]
  float* sm_o = sm_l + AD_WARPS * HP;                      // [4][HP][HD]
#pragma unroll
  for (int n = 0; n < NH; ++n) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float ll = l[n][j];                                  // sum over the 8 lanes that share these heads
      ll += __shfl_xor_sync(0xffffffffu, ll, 4);
      ll += __shfl_xor_sync(0xffffffffu, ll, 8);
      ll += __shfl_xor_sync(0xffffffffu, ll, 16);
      if (g == 0) {
        sm_m[warp * HP + n * 8 + 2 * t + j] = m[n][j];
        sm_l[warp * HP + n * 8 + 2 * t + j] = ll;
      }
    }
#pragma unroll
    for (int md = 0; md < HD / 16; ++md) {
      float* c0 = sm_o + ((size_t)warp * HP + n * 8 + 2 * t) * HD + md * 16 + g;
      c0[0] = o[n][md][0];            // head 2t,   d = md*16 + g
      c0[HD] = o[n][md][1];           // head 2t+1, d = md*16 + g
      c0[8] = o[n][md][2];            // head 2t,   d = md*16 + g + 8
      c0[HD + 8] = o[n][md][3];       // head 2t+1, d = md*16 + g + 8
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += AD_THREADS) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w) mm = fmaxf(mm, sm_m[w * HP + r]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w) {
      const float mw = sm_m[w * HP + r];
      const float f = (mw == -INFINITY) ? 0.0f : __expf(mw - mm);
      acc += f * sm_o[((size_t)w * HP + r) * HD + d];
      ll += f * sm_l[w * HP + r];
    }
    const int h = kvh * G + r;
    if (FUSED && a.nsplit == 1) {                            // nothing to combine with: the result itself
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
      f.out[(size_t)b * f.ldo + (size_t)h * HD + d] = __float2bfloat16_rn(acc * inv);
      continue;
    }
    const size_t pi = ((size_t)b * a.nh + h) * a.nsplit + split;
    a.part_o[pi * HD + d] = acc;
    if (d == 0) {
      a.part_ml[pi * 2] = mm;
      a.part_ml[pi * 2 + 1] = ll;
    }
  }
  if (FUSED && a.nsplit > 1) {
    // The split that arrives last at this (sequence, kv head)'s counter combines all of them, in
    // the order of the splits whoever it is, with the arithmetic of the combine kernel below.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      int* ctr = f.counters + (size_t)b * a.nkv + kvh;
      const int old = atomicAdd(ctr, 1);
      s_last = old == a.nsplit - 1;
      if (s_last) *ctr = 0;                                  // every split has arrived: ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int ns = a.nsplit;
    float* sm_ms = reinterpret_cast<float*>(smem);           // [G][ns] maxima, then [G][ns] sums (the pipeline's memory is free)
    float* sm_ls = sm_ms + G * ns;
    for (int idx = threadIdx.x; idx < G * ns; idx += AD_THREADS) {
      const size_t e = ((size_t)b * a.nh + kvh * G) * ns + idx;   // heads of the group and their splits are contiguous
      sm_ms[idx] = __ldcg(a.part_ml + e * 2);
      sm_ls[idx] = __ldcg(a.part_ml + e * 2 + 1);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * (HD / 4); idx += AD_THREADS) {       // four values of one head per thread
      const int r = idx / (HD / 4), d = (idx % (HD / 4)) * 4, h = kvh * G + r;
      const float* po = a.part_o + ((size_t)b * a.nh + h) * ns * HD + d;
      float mm = -INFINITY;
      for (int sp = 0; sp < ns; ++sp) mm = fmaxf(mm, sm_ms[r * ns + sp]);
      float ll = 0.0f;
      for (int sp = 0; sp < ns; ++sp) {
        const float ms = sm_ms[r * ns + sp];
        if (ms != -INFINITY) ll += __expf(ms - mm) * sm_ls[r * ns + sp];
      }
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int sp0 = 0; sp0 < ns; sp0 += 8) {
        float4 o8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o8[j] = sp0 + j < ns ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)(sp0 + j) * HD)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (sp0 + j < ns) {
            const float ms = sm_ms[r * ns + sp0 + j];
            if (ms != -INFINITY) {
              const float e = __expf(ms - mm);
              acc.x += e * o8[j].x; acc.y += e * o8[j].y; acc.z += e * o8[j].z; acc.w += e * o8[j].w;
            }
          }
        }
      }
      bf16* dst = f.out + (size_t)b * f.ldo + (size_t)h * HD + d;
      st_bf2(dst, acc.x * inv, acc.y * inv);
      st_bf2(dst + 2, acc.z * inv, acc.w * inv);
    }
  }
}

// out[b][h][:] = sum_s e^{m_s - m} O_s / sum_s e^{m_s - m} l_s
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                bf16* __restrict__ out, int ldo, int nh, int hd, int nsplit) {
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x, b = blockIdx.y;
  const size_t base = ((size_t)b * nh + h) * nsplit;
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.0f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) ll += __expf(ms - mm) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) acc += __expf(ms - mm) * part_o[(base + s) * hd + d];
    }
    out[(size_t)b * ldo + (size_t)h * hd + d] = __float2bfloat16_rn(acc * inv);
  }
}

static int decode_smem_bytes(int hd, int stages) {
  const int pipeline = stages * 2 * AD_TILE * (hd * 2 + 16);
  const int merge = (2 * AD_WARPS * 16 + AD_WARPS * 16 * hd) * 4;
  return pipeline > merge ? pipeline : merge;
}

// Three stages of key/value tiles where two CTAs of that size still share an SM, else two.
static int decode_stages(int hd) { return decode_smem_bytes(hd, 3) > 110 * 1024 ? 2 : 3; }

extern "C" long long hb_attention_decode_scratch_floats(int n_seqs, int nh, int hd, int nsplit) {
  return (long long)n_seqs * nh * nsplit * (hd + 2);
}

// scratch: hb_attention_decode_scratch_floats(...) floats; the kernel writes every element it later reads.
extern "C" int hb_attention_decode_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                        const void* vcache, const int* seq_len, const int* seq_pages,
                                        int pages_stride, float* scratch, int n_seqs, int nh, int nkv, int hd,
                                        int page_size, int nsplit, float scale, int window, void* stream) {
  HB_REQUIRE(n_seqs > 0 && nh > 0 && nkv > 0 && hd > 0, "attention_decode: sizes must be positive");
  HB_REQUIRE(nh % nkv == 0, "attention_decode: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  HB_REQUIRE(nh / nkv <= 16, "attention_decode: at most 16 query heads per key/value head, got %d", nh / nkv);
  HB_REQUIRE(hd % 16 == 0 && hd <= 256, "attention_decode: head size %d must be a multiple of 16, at most 256", hd);
  HB_REQUIRE(page_size % AD_TILE == 0, "attention_decode: page size %d must be a multiple of %d", page_size, AD_TILE);
  HB_REQUIRE(nsplit >= 1 && nsplit <= 65535 && n_seqs <= 65535 && nkv <= 65535, "attention_decode: grid too large");
  HB_REQUIRE(ldq % 2 == 0 && ((uintptr_t)q & 3) == 0, "attention_decode: queries must be 4-byte aligned");
  HB_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "attention_decode: cache must be 16-byte aligned");
  HB_REQUIRE(window >= 0, "attention_decode: window must be >= 0");
  HB_REQUIRE((long long)pages_stride * (page_size / AD_TILE) <= (long long)AD_MAX_TILES * nsplit,
             "attention_decode: %d pages per sequence in %d splits exceed %d tiles per CTA", pages_stride, nsplit, AD_MAX_TILES);
  cudaStream_t s = (cudaStream_t)stream;
  const int stages = decode_stages(hd);
  const int smem = decode_smem_bytes(hd, stages);
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)n_seqs * nh * nsplit * hd;
  DecodeArgs a{(const bf16*)q, ldq, (const bf16*)kcache, (const bf16*)vcache, seq_len, seq_pages, pages_stride,
               part_o, part_ml, nh, nkv, hd, page_size, nsplit, scale, window, stages};
  dim3 grid(nsplit, nkv, n_seqs);
  cudaError_t e;
  if (hd <= 64) {
    e = cudaFuncSetAttribute(attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_decode_kernel<64>, dim3(grid), dim3(AD_THREADS), smem, s, a);
  } else if (hd == 128) {
    if (nh / nkv <= 8) {
      e = cudaFuncSetAttribute(attention_decode_km_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) HB_FAIL(3, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      hb_launch(attention_decode_km_kernel<1, false>, dim3(grid), dim3(AD_THREADS), smem, s, a, DecodeFuse{});
    } else {
      e = cudaFuncSetAttribute(attention_decode_km_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) HB_FAIL(3, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      hb_launch(attention_decode_km_kernel<2, false>, dim3(grid), dim3(AD_THREADS), smem, s, a, DecodeFuse{});
    }
  } else if (hd < 128) {
    e = cudaFuncSetAttribute(attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_decode_kernel<128>, dim3(grid), dim3(AD_THREADS), smem, s, a);
  } else {
    e = cudaFuncSetAttribute(attention_decode_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_decode_kernel<256>, dim3(grid), dim3(AD_THREADS), smem, s, a);
  }
  HB_CHECK_LAUNCH("attention_decode");
  dim3 cgrid(nh, n_seqs);
  hb_launch(attention_decode_combine_kernel, dim3(cgrid), dim3(hd >= 128 ? 128 : 64), 0, s, part_o, part_ml, (bf16*)out, ldo, nh, hd, nsplit);
  HB_CHECK_LAUNCH("attention_decode_combine");
  return 0;
}

// Head size 128, one launch: per-head norm and rotation of the new token's q and k, the cache
// write, attention over the cache, and the combination of the key splits.
//   qkv [n_seqs, ld]: raw rows (q heads | k heads | v heads); qw/kw: norm weights [128] or both null;
//   cos_tab/sin_tab [table_rows, 64]: the rotation covers the whole head;
//   counters: n_seqs * nkv ints, zero before the first launch (the kernel leaves them zero);
//   scratch as for hb_attention_decode_bf16.  seq_len counts the new token; its position is seq_len - 1.
extern "C" int hb_attention_decode_fused_bf16(const void* qkv, int ld, void* out, int ldo, void* kcache, void* vcache,
                                              const float* qw, const float* kw, float eps, const float* cos_tab,
                                              const float* sin_tab, int table_rows, int write_cache,
                                              const int* seq_len, const int* seq_pages, int pages_stride,
                                              float* scratch, int* counters, int n_seqs, int nh, int nkv,
                                              int page_size, int nsplit, float scale, int window, void* stream) {
  const int hd = 128;
  HB_REQUIRE(n_seqs > 0 && nh > 0 && nkv > 0, "attention_decode_fused: sizes must be positive");
  HB_REQUIRE(nh % nkv == 0, "attention_decode_fused: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  HB_REQUIRE(nh / nkv <= 16, "attention_decode_fused: at most 16 query heads per key/value head, got %d", nh / nkv);
  HB_REQUIRE(page_size % AD_TILE == 0, "attention_decode_fused: page size %d must be a multiple of %d", page_size, AD_TILE);
  HB_REQUIRE(nsplit >= 1 && nsplit <= 65535 && n_seqs <= 65535 && nkv <= 65535, "attention_decode_fused: grid too large");
  HB_REQUIRE(ld % 4 == 0 && ((uintptr_t)qkv & 7) == 0, "attention_decode_fused: q/k/v rows must be 8-byte aligned");
  HB_REQUIRE(ldo % 2 == 0 && ((uintptr_t)out & 3) == 0, "attention_decode_fused: output rows must be 4-byte aligned");
  HB_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "attention_decode_fused: cache must be 16-byte aligned");
  HB_REQUIRE((qw == nullptr) == (kw == nullptr), "attention_decode_fused: norm weights for both q and k, or for neither");
  HB_REQUIRE(qw == nullptr || ((((uintptr_t)qw | (uintptr_t)kw) & 15) == 0), "attention_decode_fused: norm weights must be 16-byte aligned");
  HB_REQUIRE(cos_tab != nullptr && sin_tab != nullptr && table_rows > 0 && ((((uintptr_t)cos_tab | (uintptr_t)sin_tab) & 15) == 0),
             "attention_decode_fused: needs rotation tables, 16-byte aligned");
  HB_REQUIRE(window >= 0, "attention_decode_fused: window must be >= 0");
  HB_REQUIRE(counters != nullptr && scratch != nullptr, "attention_decode_fused: needs counters and scratch");
  HB_REQUIRE((long long)(nh / nkv) * nsplit * 8 <= 64 * 1024, "attention_decode_fused: %d heads per group x %d splits exceed the combine's shared memory", nh / nkv, nsplit);
  HB_REQUIRE((long long)pages_stride * (page_size / AD_TILE) <= (long long)AD_MAX_TILES * nsplit,
             "attention_decode_fused: %d pages per sequence in %d splits exceed %d tiles per CTA", pages_stride, nsplit, AD_MAX_TILES);
  cudaStream_t s = (cudaStream_t)stream;
  const int stages = decode_stages(hd);
  const int smem = decode_smem_bytes(hd, stages);
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)n_seqs * nh * nsplit * hd;
  DecodeArgs a{nullptr, 0, (const bf16*)kcache, (const bf16*)vcache, seq_len, seq_pages, pages_stride,
               part_o, part_ml, nh, nkv, hd, page_size, nsplit, scale, window, stages};
  DecodeFuse f{(const bf16*)qkv, ld, qw, kw, eps, cos_tab, sin_tab, table_rows, write_cache, (bf16*)kcache, (bf16*)vcache,
               counters, (bf16*)out, ldo};
  dim3 grid(nsplit, nkv, n_seqs);
  cudaError_t e;
  if (nh / nkv <= 8) {
    e = cudaFuncSetAttribute(attention_decode_km_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode_fused: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch_pdl(attention_decode_km_kernel<1, true>, dim3(grid), dim3(AD_THREADS), smem, s, a, f);
  } else {
    e = cudaFuncSetAttribute(attention_decode_km_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_decode_fused: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch_pdl(attention_decode_km_kernel<2, true>, dim3(grid), dim3(AD_THREADS), smem, s, a, f);
  }
  HB_CHECK_LAUNCH("attention_decode_fused");
  return 0;
}
