// Prefill attention over the paged cache: many queries per sequence, bfloat16, tensor cores.
//
// Causal grouped-query attention in the flash form: scores never leave the chip, so memory is
// O(T) where the reference's shader keeps a [T, heads, cached] score buffer
// (backends/backend_vulkan attention_prefill.comp) and its CPU kernel walks one key at a time
// (backends/backend_common/src/generic_attention/prefill/kernel_f32.rs:61-111).  Same arithmetic:
// s = (q . k) * scale, keys j <= p (and j > p - window if the layer has a window), running maximum
// m and sum l per query, o = o * e^{m - m'} + e^{s - m'} v, result o / l; all in float.
//
// A CTA serves 64 consecutive queries of one query head of one sequence: 4 warps x 16 rows.  Keys
// and values are read from the cache (the step's own keys were stored before this kernel runs), so
// a prompt that continues a cached prefix works the same way.  64-key tiles (one page, or a part
// of one) go global -> shared with cp.async in a ring; S = Q K^T and O += P V run on mma.sync
// m16n8k16 with K through ldmatrix and V through ldmatrix.trans.
#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

// exp: the hardware's fast exponential (ex2.approx, about 2 ulp in float).  The probabilities are
// rounded to bfloat16 for the P V product right after, so nothing is lost; sums stay in float.

#define AP_WARPS 4
#define AP_THREADS (AP_WARPS * 32)
#define AP_TILE 64
#define AP_QTILE 64
#define AP_PAGE_IDS 1024     // tiles whose pages one CTA keeps in shared memory (65,536 keys)

struct PrefillArgs {
  const bf16* q;   // [T, ldq]; row t holds the query heads of token t
  int ldq;
  bf16* out;       // [T, ldo]
  int ldo;
  const bf16* kcache;
  const bf16* vcache;
  const int* seq_start;  // [B + 1] first row of each sequence in this step
  const int* seq_pos0;   // [B] cached length before this step = position of the sequence's first row
  const int* seq_pages;
  int pages_stride;
  int nh, nkv, hd, page_size;
  float scale;
  int window;
  int stages;
};

template <int HDM>
__global__ void __launch_bounds__(AP_THREADS) attention_prefill_kernel(PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch();
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int row0 = a.seq_start[b], qlen = a.seq_start[b + 1] - row0;
  if (qt * AP_QTILE >= qlen) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int hd = a.hd, kvh = h / (a.nh / a.nkv);
  const int row_bytes = hd * 2 + 16;
  const int tile_bytes = AP_TILE * row_bytes;
  const int chunks_per_row = hd >> 3;
  const int pos0 = a.seq_pos0[b];

  const int q_first = qt * AP_QTILE;                                  // index within the sequence's rows
  const int q_last = min(qlen, q_first + AP_QTILE) - 1;
  const int p_first = pos0 + q_first, p_last = pos0 + q_last;          // positions of the CTA's queries
  const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
  const int tile_lo = lo_first / AP_TILE, tile_hi = p_last / AP_TILE + 1;
  const int tiles_per_page = a.page_size / AP_TILE;
  const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
  const size_t head_elems = (size_t)a.page_size * hd;
  // pages of the tiles this CTA walks, fetched in blocks of AP_PAGE_IDS ahead of their copies
  __shared__ int page_ids[AP_PAGE_IDS];
  int first_tile = tile_lo;
  auto fetch_pages = [&](int from) {
    first_tile = from;
    for (int i = threadIdx.x; i < AP_PAGE_IDS && from + i < tile_hi; i += AP_THREADS) page_ids[i] = pages[(from + i) / tiles_per_page];
  };
  fetch_pages(tile_lo);
  __syncthreads();

  // This thread's first 16-byte chunk of a tile and the step to its next one (no division in the loop).
  const int chunk_r0 = threadIdx.x / chunks_per_row, chunk_c0 = threadIdx.x % chunks_per_row;
  const int step_r = AP_THREADS / chunks_per_row, step_c = AP_THREADS % chunks_per_row;
  auto issue = [&](int tile, int stage) {
    const int page = page_ids[tile - first_tile];
    const size_t off = ((size_t)page * a.nkv + kvh) * head_elems + (size_t)(tile % tiles_per_page) * AP_TILE * hd;
    const bf16* kg = a.kcache + off;
    const bf16* vg = a.vcache + off;
    unsigned char* ks = smem + (size_t)stage * 2 * tile_bytes;
    unsigned char* vs = ks + tile_bytes;
    int r = chunk_r0, cc = chunk_c0;
    while (r < AP_TILE) {
      cp_async16(ks + r * row_bytes + cc * 16, kg + (size_t)r * hd + cc * 8);
      cp_async16(vs + r * row_bytes + cc * 16, vg + (size_t)r * hd + cc * 8);
      r += step_r;
      cc += step_c;
      if (cc >= chunks_per_row) {
        cc -= chunks_per_row;
        ++r;
      }
    }
  };

  // this warp's 16 queries: rows g and g + 8
  const int qi0 = q_first + warp * 16 + g, qi1 = qi0 + 8;
  const bool v0 = qi0 < qlen, v1 = qi1 < qlen;
  const int p0 = pos0 + qi0, p1 = pos0 + qi1;
  const int lo0 = (a.window > 0 && p0 - a.window + 1 > 0) ? p0 - a.window + 1 : 0;
  const int lo1 = (a.window > 0 && p1 - a.window + 1 > 0) ? p1 - a.window + 1 : 0;
  const int wp_first = pos0 + q_first + warp * 16;                     // the warp's first and last query position
  const int wp_last = min(p_last, wp_first + 15);
  const int wlo = (a.window > 0 && wp_first - a.window + 1 > 0) ? wp_first - a.window + 1 : 0;
  const bool warp_active = q_first + warp * 16 < qlen;

  unsigned qf[HDM / 16][4];
  {
    const bf16* q0 = a.q + (size_t)(row0 + qi0) * a.ldq + (size_t)h * hd;
    const bf16* q1 = a.q + (size_t)(row0 + qi1) * a.ldq + (size_t)h * hd;
#pragma unroll
    for (int ks = 0; ks < HDM / 16; ++ks) {
      qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
      if (ks * 16 < hd) {
        const int d = ks * 16 + 2 * t;
        if (v0) {
          qf[ks][0] = *reinterpret_cast<const unsigned*>(q0 + d);
          qf[ks][2] = *reinterpret_cast<const unsigned*>(q0 + d + 8);
        }
        if (v1) {
          qf[ks][1] = *reinterpret_cast<const unsigned*>(q1 + d);
          qf[ks][3] = *reinterpret_cast<const unsigned*>(q1 + d + 8);
        }
      }
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[HDM / 8][4];
#pragma unroll
  for (int i = 0; i < HDM / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  const int S = a.stages;
  for (int i = 0; i < S - 1; ++i) {
    if (tile_lo + i < tile_hi) issue(tile_lo + i, i);
    cp_async_commit();
  }
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int it = tile - tile_lo;
    if (tile + S - 1 < tile_hi) issue(tile + S - 1, (it + S - 1) % S);
    cp_async_commit();
    if (S == 2) cp_async_wait<1>(); else cp_async_wait<2>();
    __syncthreads();
    const unsigned char* ks = smem + (size_t)(it % S) * 2 * tile_bytes;
    const unsigned char* vs = ks + tile_bytes;
    const int key0 = tile * AP_TILE;
    if (warp_active && key0 <= wp_last && key0 + AP_TILE - 1 >= wlo) {
      // ---- S = Q K^T : 16 queries x 64 keys ---------------------------------------------------------
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HDM / 16; ++kk) {
        if (kk * 16 < hd) {
          const int mi = lane >> 3;
#pragma unroll
          for (int np = 0; np < 4; ++np) {      // pairs of 8-key tiles
            const int key = np * 16 + (mi >> 1) * 8 + (lane & 7);
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, ks + key * row_bytes + (kk * 16 + (mi & 1) * 8) * 2);
            mma16816(s[2 * np], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
            mma16816(s[2 * np + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
          }
        }
      }
      // ---- scale, mask, online softmax --------------------------------------------------------------
      const bool need_mask = (key0 + AP_TILE - 1 > wp_first) || (a.window > 0 && key0 < wp_last - a.window + 1);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = s[nt][j] * a.scale;
          if (need_mask) {
            const int key = key0 + nt * 8 + 2 * t + (j & 1);
            const bool ok = (j < 2) ? (v0 && key <= p0 && key >= lo0) : (v1 && key <= p1 && key >= lo1);
            if (!ok) v = -INFINITY;
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
      for (int nt = 0; nt < 8; ++nt)
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
#pragma unroll
      for (int nd = 0; nd < HDM / 8; ++nd) {
        o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
      }
      // ---- O += P V : four 16-key slices -----------------------------------------------------------------
#pragma unroll
      for (int kc = 0; kc < 4; ++kc) {
        const unsigned pa0 = pack_bf16(s[2 * kc][0], s[2 * kc][1]), pa1 = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
        const unsigned pa2 = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]), pa3 = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
#pragma unroll
        for (int nd = 0; nd < HDM / 16; ++nd) {
          if (nd * 16 < hd) {
            const int mi = lane >> 3;
            const int key = kc * 16 + (mi & 1) * 8 + (lane & 7);
            unsigned b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, vs + key * row_bytes + (nd * 16 + (mi >> 1) * 8) * 2);
            mma16816(o[2 * nd], pa0, pa1, pa2, pa3, b0, b1);
            mma16816(o[2 * nd + 1], pa0, pa1, pa2, pa3, b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
  bf16* o0 = a.out + (size_t)(row0 + qi0) * a.ldo + (size_t)h * hd;
  bf16* o1 = a.out + (size_t)(row0 + qi1) * a.ldo + (size_t)h * hd;
#pragma unroll
  for (int nd = 0; nd < HDM / 8; ++nd) {
    if (nd * 8 < hd) {
      const int d = nd * 8 + 2 * t;
      if (v0) *reinterpret_cast<unsigned*>(o0 + d) = pack_bf16(o[nd][0] * inv0, o[nd][1] * inv0);
      if (v1) *reinterpret_cast<unsigned*>(o1 + d) = pack_bf16(o[nd][2] * inv1, o[nd][3] * inv1);
    }
  }
}

extern "C" int hb_attention_prefill_bf16(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                         const void* vcache, const int* seq_start, const int* seq_pos0,
                                         const int* seq_pages, int pages_stride, int n_seqs, int max_q_len,
                                         int nh, int nkv, int hd, int page_size, float scale, int window,
                                         void* stream) {
  HB_REQUIRE(n_seqs > 0 && max_q_len > 0 && nh > 0 && nkv > 0 && hd > 0, "attention_prefill: sizes must be positive");
  HB_REQUIRE(nh % nkv == 0, "attention_prefill: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  HB_REQUIRE(hd % 16 == 0 && hd <= 256, "attention_prefill: head size %d must be a multiple of 16, at most 256", hd);
  HB_REQUIRE(page_size % AP_TILE == 0, "attention_prefill: page size %d must be a multiple of %d", page_size, AP_TILE);
  HB_REQUIRE(ldq % 2 == 0 && ldo % 2 == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0,
             "attention_prefill: queries and output must be 4-byte aligned");
  HB_REQUIRE(((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0, "attention_prefill: cache must be 16-byte aligned");
  HB_REQUIRE(nh <= 65535 && n_seqs <= 65535, "attention_prefill: grid too large");
  HB_REQUIRE(window >= 0, "attention_prefill: window must be >= 0");
  HB_REQUIRE((long long)pages_stride * (page_size / AP_TILE) <= AP_PAGE_IDS, "attention_prefill: sequences of more than %d keys are not supported", AP_PAGE_IDS * AP_TILE);
  int stages = 3;
  int smem = stages * 2 * AP_TILE * (hd * 2 + 16);
  if (smem > 110 * 1024) {
    stages = 2;
    smem = stages * 2 * AP_TILE * (hd * 2 + 16);
  }
  PrefillArgs a{(const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kcache, (const bf16*)vcache, seq_start, seq_pos0,
                seq_pages, pages_stride, nh, nkv, hd, page_size, scale, window, stages};
  dim3 grid(ceil_div(max_q_len, AP_QTILE), nh, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (hd <= 64) {
    e = cudaFuncSetAttribute(attention_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_kernel<64>, dim3(grid), dim3(AP_THREADS), smem, s, a);
  } else if (hd <= 128) {
    e = cudaFuncSetAttribute(attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_kernel<128>, dim3(grid), dim3(AP_THREADS), smem, s, a);
  } else {
    e = cudaFuncSetAttribute(attention_prefill_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL(3, "attention_prefill: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    hb_launch(attention_prefill_kernel<256>, dim3(grid), dim3(AP_THREADS), smem, s, a);
  }
  HB_CHECK_LAUNCH("attention_prefill");
  return 0;
}
