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
              float top_p, const float* __restrict__ uniforms, int* __restrict__ out) {
  __shared__ SampleShared sh;
  pdl_wait();
  pdl_launch();
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
        const unsigned int key = order_key(row[i] / temperature);
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
    kth_key = sh.prefix;
  }

  // ---- B: maximum and softmax mass of the survivors ---------------------------------------------
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i] / temperature);
  mx = block_max(mx, sh.red);
  float part = 0.0f;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float s = row[i] / temperature;
    if (order_key(s) >= kth_key) part += expf(s - mx);
  }
  const float sum_e = block_sum(part, sh.red);

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
      for (int i = tid; i < 256; i += blockDim.x) {
        sh.mass[i] = 0.0f;
        sh.hist[i] = 0;
      }
      __syncthreads();
      const unsigned int prefix = sh.prefix;
      const unsigned int himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float s = row[i] / temperature;
        const unsigned int key = order_key(s);
        if (key >= kth_key && (key & himask) == prefix) {
          atomicAdd(&sh.mass[(key >> shift) & 255u], expf(s - mx));
          atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
        }
      }
      __syncthreads();
      if (tid == 0) {
        float cum = sh.mass_above;
        int b = 255, lowest = 255;
        bool found = false;
        for (; b >= 0; --b) {
          if (sh.hist[b] == 0) continue;
          lowest = b;
          if (cum + sh.mass[b] >= target) {
            found = true;
            break;
          }
          cum += sh.mass[b];
        }
        if (!found) {  // rounding left the total just below the target: keep everything
          b = lowest;
          cum -= sh.mass[b];
        }
        sh.mass_above = cum;
        sh.prefix = prefix | ((unsigned int)b << shift);
      }
      __syncthreads();
    }
    if (sh.prefix > final_key) final_key = sh.prefix;
  }

  // ---- D/E: draw in index order over contiguous segments ----------------------------------------
  const int seg = (vocab + blockDim.x - 1) / blockDim.x;
  const int beg = tid * seg, end = min(vocab, beg + seg);
  float segmass = 0.0f;
  int last = -1;
  for (int i = beg; i < end; ++i) {
    const float s = row[i] / temperature;
    if (order_key(s) >= final_key) {
      segmass += expf(s - mx);
      last = i;
    }
  }
  sh.scan[tid] = segmass;
  if (tid == 0) {
    sh.chosen_thread = 0x7fffffff;
    sh.result = -1;
    sh.last_survivor = -1;
  }
  __syncthreads();
  if (tid == 0) {  // serial inclusive scan: 1024 adds, in a fixed order
    float c = 0.0f;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      c += sh.scan[i];
      sh.scan[i] = c;
    }
  }
  if (last >= 0) atomicMax(&sh.last_survivor, last);
  __syncthreads();
  const float total = sh.scan[blockDim.x - 1];
  const float target = uniforms[blockIdx.x] * total;
  const float incl = sh.scan[tid];
  const float excl = tid == 0 ? 0.0f : sh.scan[tid - 1];
  if (segmass > 0.0f && target < incl) atomicMin(&sh.chosen_thread, tid);
  __syncthreads();
  if (sh.chosen_thread == tid) {
    float c = excl;
    int pick = last;
    for (int i = beg; i < end; ++i) {
      const float s = row[i] / temperature;
      if (order_key(s) >= final_key) {
        c += expf(s - mx);
        if (target < c) {
          pick = i;
          break;
        }
      }
    }
    sh.result = pick;
  }
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = sh.result >= 0 ? sh.result : max(sh.last_survivor, 0);
}

extern "C" int hb_sample(const float* logits, int ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, const float* uniforms, int* out, void* stream) {
  HB_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes");
  HB_REQUIRE(temperature > 0.0f, "sample: temperature must be > 0 (0 is greedy: use argmax)");
  HB_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
  HB_REQUIRE(top_p > 0.0f, "sample: top_p must be > 0");
  hb_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, temperature, top_k,
                                                                    top_p, uniforms, out);
  HB_CHECK_LAUNCH("sample");
  return 0;
}
