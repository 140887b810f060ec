// Token choice on the device: greedy argmax, and temperature / top-k / top-p sampling.
//
// Reference semantics (crates/core/src/sampler.rs:72-145, 244-254):
//   temperature == 0  -> argmax, the first maximum wins;
//   otherwise s_i = logit_i / temperature; keep the top_k largest (0 = off); softmax over the
//   survivors; if top_p < 1 keep the shortest prefix, in descending probability, whose
//   cumulative probability reaches top_p, and renormalise; draw with one uniform r in [0,1):
//   the first survivor whose cumulative probability exceeds r, else the last one.
// Here the survivor sets are found by value thresholds (radix descent on an order-preserving
// integer key), so elements exactly equal to a threshold all survive, and the cumulative
// draw runs in index order.  The distribution is the reference's; which token a given r maps
// to is this library's own (stated) convention, shared with the host twin in
// herbert_rs_b200/sampling/sampler.py.
#include "api.h"
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned int order_key(float v) {
  unsigned int u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned int k) {       // the inverse of order_key
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_launch();
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best) {  // strictly greater: the lowest index of equal values stays
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    // every value -inf or NaN: the reference's argmax returns 0 (sampler.rs:244-254)
    if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

// Two stages for large vocabularies: every row is cut into ARGMAX_CHUNKS pieces that separate
// blocks scan (so a batch of 8 rows keeps far more than 8 SMs busy), then one warp per row picks
// the best piece; ties go to the lower index at both stages.
#define ARGMAX_CHUNKS 64

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int ld, int vocab, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_wait();
  pdl_launch();
  const int chunk = blockIdx.x, row = blockIdx.y;
  const int per = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
  const int beg = chunk * per, end = min(vocab, beg + per);
  const float* r = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
    const float v = r[i];
    if (v > best) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    pv[(size_t)row * ARGMAX_CHUNKS + chunk] = best;
    pi[(size_t)row * ARGMAX_CHUNKS + chunk] = bi;
  }
}

__global__ void __launch_bounds__(32)
argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int* __restrict__ out) {
  pdl_wait();
  pdl_launch();
  const int row = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < ARGMAX_CHUNKS; c += 32) {
    const float v = pv[(size_t)row * ARGMAX_CHUNKS + c];
    const int i = pi[(size_t)row * ARGMAX_CHUNKS + c];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

// scratch (optional): 2 * ARGMAX_CHUNKS * n_rows 4-byte words; with it, large vocabularies take two stages.
extern "C" int hb_argmax(const float* logits, int ld, int n_rows, int vocab, int* out, void* scratch,
                         long long scratch_words, void* stream) {
  HB_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "argmax: bad sizes");
  if (scratch != nullptr && vocab >= 8192 && scratch_words >= 2LL * ARGMAX_CHUNKS * n_rows && n_rows <= 65535) {
    float* pv = (float*)scratch;
    int* pi = (int*)scratch + (size_t)ARGMAX_CHUNKS * n_rows;
    hb_launch(argmax_partial_kernel, dim3(ARGMAX_CHUNKS, n_rows), dim3(256), 0, (cudaStream_t)stream, logits, ld, vocab, pv, pi);
    HB_CHECK_LAUNCH("argmax_partial");
    hb_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, (cudaStream_t)stream, (const float*)pv, (const int*)pi, out);
    HB_CHECK_LAUNCH("argmax_final");
    return 0;
  }
  hb_launch(argmax_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, out);
  HB_CHECK_LAUNCH("argmax");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Scans done by one warp instead of one thread (a thread's serial walk over hundreds of bins in
// shared memory costs tens of microseconds).  Bins are walked from the highest down.
//   count form: the bin b with  sum(hist[b+1..]) < want <= sum(hist[b..]);  returns b and the sum above it.
__device__ __forceinline__ void warp_find_count_bin(const unsigned int* hist, int nbins, int want, int lane, int* bin_out, int* above_out) {
  const int per = nbins / 32;                       // nbins is a multiple of 32
  const int hi = nbins - 1 - lane * per;            // this lane's bins: hi, hi-1, ..., hi-per+1
  int mine = 0;
  for (int j = 0; j < per; ++j) mine += (int)hist[hi - j];
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const int excl = incl - mine;                      // count in all bins above this lane's
  const unsigned int owners = __ballot_sync(0xffffffffu, excl < want && incl >= want);
  const int owner = owners ? __ffs(owners) - 1 : 31; // nobody: fewer elements than wanted, the lowest bin
  if (lane == owner) {
    int cum = excl, b = hi;
    for (int j = 0; j < per; ++j, --b) {
      if (cum + (int)hist[b] >= want || j == per - 1) break;
      cum += (int)hist[b];
    }
    *bin_out = b;
    *above_out = cum;
  }
}
//   mass form (nucleus): among bins with entries, the highest b with  above + sum(mass[b..]) >= target;
//   if rounding leaves the total below the target, the lowest bin with entries.  Returns b and the mass above it.
__device__ __forceinline__ void warp_find_mass_bin(const unsigned int* hist, const float* mass, int nbins, float above, float target,
                                                   int lane, int* bin_out, float* above_out) {
  const int per = nbins / 32;                       // nbins is a multiple of 32
  const int hi = nbins - 1 - lane * per;
  float mine = 0.0f;
  for (int j = 0; j < per; ++j) mine += mass[hi - j];
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const float excl = above + (incl - mine);
  // walk this lane's bins exactly as a single thread would, starting from the mass above them
  int found_b = -1, lowest = -1;
  float cum = excl, found_cum = 0.0f;
  for (int j = 0; j < per; ++j) {
    const int b = hi - j;
    if (hist[b] == 0) continue;
    lowest = b;
    if (found_b < 0 && cum + mass[b] >= target) {
      found_b = b;
      found_cum = cum;
    }
    cum += mass[b];
  }
  const unsigned int finders = __ballot_sync(0xffffffffu, found_b >= 0);
  const unsigned int havers = __ballot_sync(0xffffffffu, lowest >= 0);
  if (finders) {
    if (lane == __ffs(finders) - 1) {
      *bin_out = found_b;
      *above_out = found_cum;
    }
  } else if (havers) {
    const int owner = 31 - __clz(havers);            // the lane with the lowest bins that has entries
    if (lane == owner) {
      *bin_out = lowest;
      *above_out = cum - mass[lowest];
    }
  }
}


struct SampleShared {
  unsigned int hist[256];
  float mass[256];
  float red[32];
  float scan[SAMPLE_THREADS];
  unsigned int prefix;
  int remaining;
  float mass_above;
  int chosen_thread;
  int result;
  int last_survivor;
  int last_of_warp[32];
  int bin;
  float target;
  unsigned int hist12[4096];   // the nucleus search's first level: 12 bits
  float mass12[4096];
};

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature, int top_k,
              float top_p, const float* __restrict__ uniforms, int* __restrict__ out, const int* __restrict__ only_rows) {
  __shared__ SampleShared sh;
  pdl_wait();
  pdl_launch();
  if (only_rows != nullptr && only_rows[blockIdx.x] == 0) return;      // the list kernel has chosen for this row
  const int tid = threadIdx.x;
  const float* row = logits + (size_t)blockIdx.x * ld;

  // ---- A: key of the top_k-th largest scaled logit (0 = keep all) ---------------------------
  unsigned int kth_key = 0;
  if (top_k > 0 && top_k < vocab) {
    if (tid == 0) {
      sh.prefix = 0;
      sh.remaining = top_k;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = tid; i < 256; i += blockDim.x) sh.hist[i] = 0;
      __syncthreads();
      const unsigned int prefix = sh.prefix;
      const unsigned int himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < vocab; i += blockDim.x) {
        const unsigned int key = order_key(row[i]);
        if ((key & himask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, b = 255;
        for (; b > 0; --b) {
          if (cum + (int)sh.hist[b] >= sh.remaining) break;
          cum += (int)sh.hist[b];
        }
        sh.remaining -= cum;
        sh.prefix = prefix | ((unsigned int)b << shift);
      }
      __syncthreads();
    }
    // the descent ran on the raw logits (dividing by a positive temperature keeps the order): the
    // threshold among the scaled values is the scaled top_k-th raw value, ties included
    kth_key = order_key(key_value(sh.prefix) / temperature);
  }

  // ---- B: maximum (the nucleus search sums the survivors' softmax mass itself) -------------------------
  float mx = -INFINITY;
  {
    const bool vec4 = (ld & 3) == 0 && (((uintptr_t)logits) & 15) == 0;
    const int nvec = vec4 ? vocab >> 2 : 0;
    for (int v0 = tid; v0 < nvec; v0 += 2 * SAMPLE_THREADS) {
      const float4 a = reinterpret_cast<const float4*>(row)[v0];
      const float4 b = v0 + SAMPLE_THREADS < nvec ? reinterpret_cast<const float4*>(row)[v0 + SAMPLE_THREADS] : a;
      mx = fmaxf(fmaxf(fmaxf(mx, a.x), fmaxf(a.y, a.z)), fmaxf(fmaxf(a.w, b.x), fmaxf(fmaxf(b.y, b.z), b.w)));
    }
    for (int i = 4 * nvec + tid; i < vocab; i += SAMPLE_THREADS) mx = fmaxf(mx, row[i]);
  }
  mx = block_max(mx, sh.red) / temperature;          // max(x / t) = max(x) / t

  // ---- C: nucleus threshold key: radix descent over 12, 8, 8 and 4 bits of the keys ------------------
  // The first level meets every surviving element; with 4,096 bins the lanes of a warp seldom add
  // to the same bin at once (float atomics in shared memory take turns), the later levels meet only
  // the elements of one bin.
  unsigned int final_key = kth_key;
  if (top_p < 1.0f) {
    const int lane_c = tid & 31;
    const bool vec4 = (ld & 3) == 0 && (((uintptr_t)logits) & 15) == 0;
    const int nvec = vec4 ? vocab >> 2 : 0;
    if (tid == 0) {
      sh.prefix = 0;
      sh.mass_above = 0.0f;
    }
    for (int level = 0; level < 4; ++level) {
      const int bits = level == 0 ? 12 : (level == 3 ? 4 : 8);
      const int shift = level == 0 ? 20 : (level == 1 ? 12 : (level == 2 ? 4 : 0));
      unsigned int* hist = level == 0 ? sh.hist12 : sh.hist;
      float* mass = level == 0 ? sh.mass12 : sh.mass;
      const int nbins = level == 0 ? 4096 : 256;
      for (int i = tid; i < nbins; i += SAMPLE_THREADS) {
        mass[i] = 0.0f;
        hist[i] = 0;
      }
      __syncthreads();
      const unsigned int prefix = sh.prefix;
      const unsigned int himask = level == 0 ? 0u : (0xffffffffu << (shift + bits));
      const unsigned int binmask = (1u << bits) - 1u;
      auto count = [&](float x) {
        const float sv = x / temperature;
        const unsigned int key = order_key(sv);
        if (key >= kth_key && (key & himask) == prefix) {
          atomicAdd(&mass[(key >> shift) & binmask], expf(sv - mx));
          atomicAdd(&hist[(key >> shift) & binmask], 1u);
        }
      };
      for (int v0 = tid; v0 < nvec; v0 += 2 * SAMPLE_THREADS) {
        const float4 a = reinterpret_cast<const float4*>(row)[v0];
        const bool two = v0 + SAMPLE_THREADS < nvec;
        const float4 b = two ? reinterpret_cast<const float4*>(row)[v0 + SAMPLE_THREADS] : a;
        count(a.x); count(a.y); count(a.z); count(a.w);
        if (two) {
          count(b.x); count(b.y); count(b.z); count(b.w);
        }
      }
      for (int i = 4 * nvec + tid; i < vocab; i += SAMPLE_THREADS) count(row[i]);
      __syncthreads();
      if (tid < 32) {
        if (level == 0) {
          // the survivors' whole mass is the sum of the first level's bins, added in a fixed order
          float total = 0.0f;
          for (int i = lane_c; i < nbins; i += 32) total += mass[i];
          total = warp_sum(total);
          if (lane_c == 0) sh.target = top_p * total;
          __syncwarp();
        }
        const float above = sh.mass_above, target = sh.target;
        __syncwarp();
        warp_find_mass_bin(hist, mass, nbins, above, target, lane_c, &sh.bin, &sh.mass_above);
        __syncwarp();
        if (lane_c == 0) sh.prefix = prefix | ((unsigned int)sh.bin << shift);
      }
      __syncthreads();
    }
    if (sh.prefix > final_key) final_key = sh.prefix;
  }

  // ---- D/E: draw in index order.  Every warp owns a contiguous run of the row and reads it 128
  // consecutive elements at a time; the warps' masses are scanned; the run that holds the target is
  // cut into 32 sub-runs, one per warp, whose masses are scanned in turn; the warp of the sub-run
  // that holds the target finds the element with warp scans over the values it kept in registers.
  const int warp = tid >> 5, lane = tid & 31;        // the block has SAMPLE_THREADS threads: 32 warps
  const int run = ((vocab + 31) / 32 + 127) & ~127;
  const int beg = min(vocab, warp * run), end = min(vocab, beg + run);
  const bool vec = (ld & 3) == 0 && (((uintptr_t)logits) & 15) == 0;
  float lane_mass = 0.0f;
  int last = -1;
  for (int i0 = beg + 4 * lane; i0 < end; i0 += 256) {
    float x[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = i0 + 128 * u;
      if (vec && i + 3 < end) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        x[u][0] = v.x; x[u][1] = v.y; x[u][2] = v.z; x[u][3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[u][j] = i + j < end ? row[i + j] : 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + 128 * u + j;
        const float sv = x[u][j] / temperature;
        if (i < end && order_key(sv) >= final_key) {
          lane_mass += expf(sv - mx);
          last = i;
        }
      }
  }
  lane_mass = warp_sum(lane_mass);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
  if (tid == 0) {
    sh.result = -1;
    sh.last_survivor = -1;
  }
  __syncthreads();
  if (lane == 0) {
    sh.scan[warp] = lane_mass;
    sh.last_of_warp[warp] = last;
    if (last >= 0) atomicMax(&sh.last_survivor, last);
  }
  __syncthreads();
  // inclusive scan of 32 masses by warp 0, a fixed tree; the first part whose running sum passes the
  // target is chosen (0x7fffffff: none, rounding); sh.mass[w] = mass before part w
  auto choose_part = [&](float before, bool first) {
    float w = sh.scan[lane];
    const float own = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    if (first && lane == 31) sh.mass_above = uniforms[blockIdx.x] * w;      // the target: uniform x total mass
    __syncwarp();
    const float target = sh.mass_above;
    const unsigned int hit = __ballot_sync(0xffffffffu, own > 0.0f && target < before + w);
    if (lane == 0) sh.chosen_thread = hit ? __ffs(hit) - 1 : 0x7fffffff;
    sh.mass[lane] = before + (w - own);
  };
  if (warp == 0) choose_part(0.0f, true);
  __syncthreads();
  const int chosen_run = sh.chosen_thread;
  const float target = sh.mass_above;
  const float before_run = chosen_run != 0x7fffffff ? sh.mass[chosen_run] : 0.0f;
  __syncthreads();                                   // everyone has read them before they are written again
  if (chosen_run != 0x7fffffff) {
    constexpr int GROUPS = 8;                        // 32 warps x 8 groups x 32 elements: runs up to 8,192 elements
    const int rb = min(vocab, chosen_run * run), re = min(vocab, rb + run);
    const int sub = ((re - rb + 31) / 32 + 31) & ~31;
    if (sub <= 32 * GROUPS) {
      const int sb = min(re, rb + warp * sub), se = min(re, sb + sub);
      float e[GROUPS];
      float m = 0.0f;
#pragma unroll
      for (int gi = 0; gi < GROUPS; ++gi) {
        const int i = sb + gi * 32 + lane;
        e[gi] = 0.0f;
        if (i < se) {
          const float sv = row[i] / temperature;
          if (order_key(sv) >= final_key) e[gi] = expf(sv - mx);
        }
        m += e[gi];
      }
      m = warp_sum(m);
      if (lane == 0) sh.scan[warp] = m;
      __syncthreads();
      if (warp == 0) choose_part(before_run, false);
      __syncthreads();
      if (sh.chosen_thread == warp) {
        float c = sh.mass[warp];
        int pick = -1;
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi) {
          float incl = e[gi];
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
          }
          const unsigned int hit = __ballot_sync(0xffffffffu, e[gi] > 0.0f && target < c + incl);
          if (hit && pick < 0) pick = sb + gi * 32 + __ffs(hit) - 1;
          c += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) sh.result = pick;
      }
    } else if (warp == chosen_run) {
      // a run too long for the registers: this warp walks it, 32 elements at a time
      float c = before_run;
      int pick = -1;
      for (int i0 = rb; i0 < re && pick < 0; i0 += 32) {
        const int i = i0 + lane;
        float e = 0.0f;
        if (i < re) {
          const float sv = row[i] / temperature;
          if (order_key(sv) >= final_key) e = expf(sv - mx);
        }
        float incl = e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const unsigned int hit = __ballot_sync(0xffffffffu, e > 0.0f && target < c + incl);
        if (hit) pick = i0 + __ffs(hit) - 1;
        c += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) sh.result = pick;
    }
  }
  __syncthreads();
  // rounding may leave the target just beyond the sums that were formed again: the last survivor of the chosen run, or of the row
  if (tid == 0)
    out[blockIdx.x] = sh.result >= 0 ? sh.result
                                     : (chosen_run != 0x7fffffff ? sh.last_of_warp[chosen_run] : max(sh.last_survivor, 0));
}

// ---------------------------------------------------------------------------------------------
// The same choice when top_k is small against a large vocabulary (the usual case: 40 of 151,936).
// The kernel above walks the whole row a dozen times with one CTA; here the row is read twice:
//   pass 1  histogram of the top 12 bits of the raw logits' keys (sign, exponent, 3 bits of the
//           fraction: an eighth of an octave per bin) -> the bin b that holds the top_k-th largest value;
//   pass 2  every element whose top 12 bits are >= b goes into a list in shared memory (value /
//           temperature and index, in any order); that list holds all top_k survivors and ties.
// Everything else (the exact top_k threshold, maximum, softmax mass, the nucleus threshold and the
// draw in index order) then runs over the list with the arithmetic of the kernel above.  A row with
// more candidates than the list holds (flat logits) is left to the kernel above.  Without top_k
// (top_p alone) the list takes as many whole bins from the top as it holds, pass 2 also sums the
// row's softmax mass, and a row whose nucleus reaches below the list is left to the kernel above.
#define SAMPLE_LIST 2048
#define SAMPLE_BINS 4096       // 12 bits

struct SampleListShared {
  float val[SAMPLE_LIST];
  int idx[SAMPLE_LIST];
  unsigned int hist[SAMPLE_BINS];  // pass 1: 12-bit bins; then its first 256 entries serve the radix passes;
                                   // at the end the whole array holds the survivors (values, then indices)
  unsigned long long mass64[256];  // masses as integers (x 2^40): sums that do not depend on the order of the adds
  unsigned long long acc64;
  float mass[256];
  float red[32];
  float scan[SAMPLE_THREADS];
  unsigned int prefix;
  int remaining;
  float mass_above;
  int chosen_thread;
  int result;
  int bin, n, above;
};

__device__ __forceinline__ unsigned long long mass_fixed(float e) { return __float2ull_rn(e * 0x1p40f); }

// Sum of the threads' integers over the block; every thread gets it.
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* acc) {
  __syncthreads();
  if (threadIdx.x == 0) *acc = 0ull;
  __syncthreads();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0 && v != 0ull) atomicAdd(acc, v);
  __syncthreads();
  return *acc;
}

__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_topk_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature, int top_k,
                   float top_p, const float* __restrict__ uniforms, int* __restrict__ out, int* __restrict__ overflow) {
  __shared__ SampleListShared sh;
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)blockIdx.x * ld;
  const bool vec = (ld & 3) == 0 && (((uintptr_t)logits) & 15) == 0;
  const int nvec = vec ? vocab >> 2 : 0;                    // float4 groups; the rest one by one

  // ---- pass 1: histogram of the keys' top 12 bits, and the row's maximum ----------------------------
  for (int i = tid; i < SAMPLE_BINS; i += SAMPLE_THREADS) sh.hist[i] = 0;
  __syncthreads();
  // Bins and the maximum are taken on the raw logits: dividing by the temperature (> 0) keeps the
  // order, so the bin of the top_k-th raw value bounds the same candidates, and max(x / t) = max(x) / t.
  float mx = -INFINITY;
  for (int v0 = tid; v0 < nvec; v0 += 2 * SAMPLE_THREADS) {
    float4 x[2];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (v0 + u * SAMPLE_THREADS < nvec) x[u] = reinterpret_cast<const float4*>(row)[v0 + u * SAMPLE_THREADS];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (v0 + u * SAMPLE_THREADS < nvec) {
        const float xv[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mx = fmaxf(mx, xv[j]);
          atomicAdd(&sh.hist[order_key(xv[j]) >> 20], 1u);
        }
      }
  }
  for (int i = 4 * nvec + tid; i < vocab; i += SAMPLE_THREADS) {
    mx = fmaxf(mx, row[i]);
    atomicAdd(&sh.hist[order_key(row[i]) >> 20], 1u);
  }
  mx = mx / temperature;
  mx = block_max(mx, sh.red);                       // its barriers also close the histogram
  if (warp == 0) {
    if (top_k > 0) {
      // the bin of the top_k-th largest value: the list takes that bin and every bin above it
      warp_find_count_bin(sh.hist, SAMPLE_BINS, top_k, lane, &sh.bin, &sh.above);
      __syncwarp();
      if (lane == 0) sh.n = sh.above + (int)sh.hist[sh.bin];
    } else {
      // no top_k: as many whole bins from the top as the list holds
      warp_find_count_bin(sh.hist, SAMPLE_BINS, SAMPLE_LIST + 1, lane, &sh.bin, &sh.above);
      __syncwarp();
      if (lane == 0) {
        sh.bin += 1;
        sh.n = sh.above;
      }
    }
  }
  __syncthreads();
  const unsigned int bin = (unsigned int)sh.bin;
  const int n = sh.n;
  if (n > SAMPLE_LIST || n == 0) {                // the list cannot hold the candidates: the general kernel takes the row
    if (tid == 0) {
      overflow[blockIdx.x] = 1;
      out[blockIdx.x] = 0;
    }
    return;
  }
  if (tid == 0) overflow[blockIdx.x] = 0;

  // ---- pass 2: the candidates into the list, in any order; without top_k also the row's softmax mass
  if (tid == 0) sh.remaining = 0;                  // the list's fill count
  __syncthreads();
  const bool whole_mass = top_k <= 0;
  float row_mass = 0.0f;                           // per thread over a fixed set of elements in a fixed order
  for (int v0 = tid; v0 < nvec; v0 += 2 * SAMPLE_THREADS) {
    float4 x[2];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (v0 + u * SAMPLE_THREADS < nvec) x[u] = reinterpret_cast<const float4*>(row)[v0 + u * SAMPLE_THREADS];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (v0 + u * SAMPLE_THREADS < nvec) {
        const float xv[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (whole_mass) row_mass += expf(xv[j] / temperature - mx);
          if ((order_key(xv[j]) >> 20) >= bin) {
            const int pos = atomicAdd(&sh.remaining, 1);     // < n <= SAMPLE_LIST: the histogram counted the same elements
            sh.val[pos] = xv[j] / temperature;
            sh.idx[pos] = 4 * (v0 + u * SAMPLE_THREADS) + j;
          }
        }
      }
  }
  for (int i = 4 * nvec + tid; i < vocab; i += SAMPLE_THREADS) {
    const float xv = row[i];
    if (whole_mass) row_mass += expf(xv / temperature - mx);
    if ((order_key(xv) >> 20) >= bin) {
      const int pos = atomicAdd(&sh.remaining, 1);
      sh.val[pos] = xv / temperature;
      sh.idx[pos] = i;
    }
  }
  __syncthreads();

  // ---- A: key of the top_k-th largest value, exactly (radix descent over the list) -----------------
  unsigned int kth_key = 0;
  if (top_k > 0 && top_k < n) {
    if (tid == 0) {
      sh.prefix = 0;
      sh.remaining = top_k;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) sh.hist[tid] = 0;
      __syncthreads();
      const unsigned int prefix = sh.prefix;
      const unsigned int himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < n; i += SAMPLE_THREADS) {
        const unsigned int key = order_key(sh.val[i]);
        if ((key & himask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (warp == 0) {
        const int want = sh.remaining;
        __syncwarp();
        warp_find_count_bin(sh.hist, 256, want, lane, &sh.bin, &sh.above);
        __syncwarp();
        if (lane == 0) {
          sh.remaining = want - sh.above;
          sh.prefix = prefix | ((unsigned int)sh.bin << shift);
        }
      }
      __syncthreads();
    }
    kth_key = sh.prefix;
  }

  // ---- B: softmax mass of the survivors (the list is in no fixed order: integer sums) ----------------
  unsigned long long part = 0ull;
  for (int i = tid; i < n; i += SAMPLE_THREADS)
    if (order_key(sh.val[i]) >= kth_key) part += mass_fixed(expf(sh.val[i] - mx));
  const float list_mass = (float)block_sum_u64(part, &sh.acc64) * 0x1p-40f;
  float sum_e = list_mass;
  if (whole_mass) {
    sum_e = block_sum(row_mass, sh.red);
    if (list_mass < top_p * sum_e) {               // the nucleus reaches below the list: the general kernel takes the row
      if (tid == 0) {
        overflow[blockIdx.x] = 1;
        out[blockIdx.x] = 0;
      }
      return;
    }
  }

  // ---- C: nucleus threshold key ------------------------------------------------------------------
  unsigned int final_key = kth_key;
  if (top_p < 1.0f) {
    const float target = top_p * sum_e;
    if (tid == 0) {
      sh.prefix = 0;
      sh.mass_above = 0.0f;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) {
        sh.mass64[tid] = 0ull;
        sh.hist[tid] = 0;
      }
      __syncthreads();
      const unsigned int prefix = sh.prefix;
      const unsigned int himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < n; i += SAMPLE_THREADS) {
        const float sval = sh.val[i];
        const unsigned int key = order_key(sval);
        if (key >= kth_key && (key & himask) == prefix) {
          atomicAdd(&sh.mass64[(key >> shift) & 255u], mass_fixed(expf(sval - mx)));
          atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
        }
      }
      __syncthreads();
      if (tid < 256) sh.mass[tid] = (float)sh.mass64[tid] * 0x1p-40f;
      __syncthreads();
      if (warp == 0) {
        const float above = sh.mass_above;
        __syncwarp();
        warp_find_mass_bin(sh.hist, sh.mass, 256, above, target, lane, &sh.bin, &sh.mass_above);
        __syncwarp();
        if (lane == 0) sh.prefix = prefix | ((unsigned int)sh.bin << shift);
      }
      __syncthreads();
    }
    if (sh.prefix > final_key) final_key = sh.prefix;
  }

  // ---- the survivors, put in index order -----------------------------------------------------------
  float* sval = reinterpret_cast<float*>(sh.hist);
  int* sidx = reinterpret_cast<int*>(sh.hist + SAMPLE_LIST);
  if (tid == 0) sh.remaining = 0;
  __syncthreads();
  for (int i = tid; i < n; i += SAMPLE_THREADS)
    if (order_key(sh.val[i]) >= final_key) {
      const int pos = atomicAdd(&sh.remaining, 1);
      sval[pos] = sh.val[i];
      sidx[pos] = sh.idx[i];
    }
  __syncthreads();
  const int ns = sh.remaining;
  {
    // rank of a survivor = survivors with a smaller index; every thread holds its (at most two)
    // survivors in registers over the barrier and stores them at their ranks
    float my_val[SAMPLE_LIST / SAMPLE_THREADS];
    int my_idx[SAMPLE_LIST / SAMPLE_THREADS], my_rank[SAMPLE_LIST / SAMPLE_THREADS];
#pragma unroll
    for (int e = 0; e < SAMPLE_LIST / SAMPLE_THREADS; ++e) {
      const int i = tid + e * SAMPLE_THREADS;
      my_rank[e] = -1;
      if (i < ns) {
        my_val[e] = sval[i];
        my_idx[e] = sidx[i];
        int r = 0;
        for (int j = 0; j < ns; ++j) r += sidx[j] < my_idx[e] ? 1 : 0;
        my_rank[e] = r;
      }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < SAMPLE_LIST / SAMPLE_THREADS; ++e)
      if (my_rank[e] >= 0) {
        sval[my_rank[e]] = my_val[e];
        sidx[my_rank[e]] = my_idx[e];
      }
    __syncthreads();
  }

  // ---- D/E: draw in index order over contiguous segments of the survivors ----------------------------
  const int seg = (ns + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int beg = min(ns, tid * seg), end = min(ns, beg + seg);
  float segmass = 0.0f;
  for (int i = beg; i < end; ++i) segmass += expf(sval[i] - mx);
  if (tid == 0) {
    sh.chosen_thread = 0x7fffffff;
    sh.result = -1;
  }
  // inclusive scan of the segments' masses over the block, as a fixed tree: within a warp, then over the warps
  float run = segmass;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, run, o);
    if (lane >= o) run += t;
  }
  if (lane == 31) sh.red[warp] = run;
  __syncthreads();
  if (warp == 0) {
    float w = sh.red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    sh.red[lane] = w;                                // inclusive over the warps
  }
  __syncthreads();
  sh.scan[tid] = run + (warp > 0 ? sh.red[warp - 1] : 0.0f);
  __syncthreads();
  const float total = sh.scan[SAMPLE_THREADS - 1];
  const float target = uniforms[blockIdx.x] * total;
  const float incl = sh.scan[tid];
  const float excl = tid == 0 ? 0.0f : sh.scan[tid - 1];
  if (segmass > 0.0f && target < incl) atomicMin(&sh.chosen_thread, tid);
  __syncthreads();
  if (sh.chosen_thread == tid) {
    float c = excl;
    int pick = sidx[end - 1];
    for (int i = beg; i < end; ++i) {
      c += expf(sval[i] - mx);
      if (target < c) {
        pick = sidx[i];
        break;
      }
    }
    sh.result = pick;
  }
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = sh.result >= 0 ? sh.result : (ns > 0 ? sidx[ns - 1] : 0);
}

// overflow (optional): n_rows ints of scratch; with it, a small top_k (or top_p alone) against a large
// vocabulary takes the two-pass list kernel, and the general kernel only runs for rows the list could not hold.
extern "C" int hb_sample(const float* logits, int ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, const float* uniforms, int* out, int* overflow, void* stream) {
  HB_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes");
  HB_REQUIRE(temperature > 0.0f, "sample: temperature must be > 0 (0 is greedy: use argmax)");
  HB_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
  HB_REQUIRE(top_p > 0.0f, "sample: top_p must be > 0");
  const bool small_k = top_k > 0 && top_k <= SAMPLE_LIST / 4, nucleus_only = top_k == 0 && top_p < 1.0f;
  if (overflow != nullptr && (small_k || nucleus_only) && vocab >= 4 * SAMPLE_LIST) {
    hb_launch(sample_topk_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, temperature,
              top_k, top_p, uniforms, out, overflow);
    HB_CHECK_LAUNCH("sample_topk");
    // the general kernel returns at once for every row that is done (all of them, unless logits are flat)
    hb_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, temperature, top_k,
              top_p, uniforms, out, (const int*)overflow);
    HB_CHECK_LAUNCH("sample");
    return 0;
  }
  hb_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, temperature, top_k,
            top_p, uniforms, out, (const int*)nullptr);
  HB_CHECK_LAUNCH("sample");
  return 0;
}
