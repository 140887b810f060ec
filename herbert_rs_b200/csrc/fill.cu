// Load-time kernels: counter-based normal random fill, constant fill, dtype casts.
//
// The reference has no random-weights mode and converts dtypes on the CPU while loading
// (backends/backend_common/src/loader_common.rs:33-54: F32 -> BF16 round to nearest even,
// core/src/tensor.rs:46-56).  Here the casts run on the device, and random weights come from a
// generator addressed by (key, element index), so that the same (seed, tensor name) gives the
// same bytes whether a tensor is made here or by the host twin (weights/counter_rng.py).
//
// Bit-for-bit agreement with the host twin needs arithmetic that both sides round alike: 64-bit
// integer mixing, exact integer -> float conversions, and float add / mul / div / sqrt each
// rounded to nearest on its own (never contracted into a fused multiply-add: the __f*_rn
// intrinsics are exempt from contraction).  Logarithm, sine and cosine are polynomials built from
// those operations, not library calls, whose last bit differs between CPU and GPU.
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

// splitmix64 finaliser over key + (index + 1) * golden ratio
__device__ __forceinline__ unsigned long long rng_mix(unsigned long long key, unsigned long long idx) {
  unsigned long long z = key + (idx + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

#define RN_MUL(a, b) __fmul_rn((a), (b))
#define RN_ADD(a, b) __fadd_rn((a), (b))

// One standard normal from 64 random bits (Box-Muller, cosine branch).
//   u = (2a + 1) / 2^24 with a of 23 bits: never 0, never 1
//   angle = 2 pi t / 2^25 with t of 25 bits: quadrant = t >> 23, the rest folded into [0, pi/4]
__device__ __forceinline__ float rng_normal_from_bits(unsigned long long z) {
  // ---- radius = sqrt(-2 ln u) --------------------------------------------------------------
  const unsigned n = 2u * (unsigned)(z >> 41) + 1u;             // odd, < 2^24: exact as a float
  const unsigned nb = __float_as_uint(__uint2float_rn(n));
  int e = (int)(nb >> 23) - 127;
  float m = __uint_as_float((nb & 0x7FFFFFu) | 0x3F800000u);      // in [1, 2)
  if (m > __uint_as_float(0x3FB504F3u)) { m = RN_MUL(m, 0.5f); e += 1; }           // in (0.7071, 1.4143]
  const float s = __fdiv_rn(RN_ADD(m, -1.0f), RN_ADD(m, 1.0f));   // ln m = 2 atanh(s)
  const float s2 = RN_MUL(s, s);
  float p = RN_ADD(RN_MUL(s2, __uint_as_float(0x3DE38E39u)), __uint_as_float(0x3E124925u));
  p = RN_ADD(RN_MUL(s2, p), 0.2f);
  p = RN_ADD(RN_MUL(s2, p), __uint_as_float(0x3EAAAAABu));
  p = RN_ADD(RN_MUL(s2, p), 1.0f);
  const float lnm = RN_MUL(RN_MUL(s, 2.0f), p);
  const float lnu = RN_ADD(RN_MUL((float)(e - 24), __uint_as_float(0x3F317218u)), lnm);     // < 0
  const float radius = __fsqrt_rn(RN_MUL(lnu, -2.0f));
  // ---- cos(angle) ---------------------------------------------------------------------------
  const unsigned t = (unsigned)(z >> 16) & 0x1FFFFFFu;
  const unsigned quadrant = t >> 23;
  unsigned g = 2u * (t & 0x7FFFFFu) + 1u;                         // odd, < 2^24: angle in the quadrant = (pi/2) g / 2^24
  const bool fold = g > 0x800000u;                                // beyond pi/4: use the co-function of pi/2 - angle
  if (fold) g = 0x1000000u - g;
  const float x = RN_MUL(__uint2float_rn(g), __uint_as_float(0x33C90FDBu));     // (pi/2) / 2^24
  const float x2 = RN_MUL(x, x);
  float sn = RN_ADD(RN_MUL(x2, __uint_as_float(0x3638EF1Du)), __uint_as_float(0xB9500D01u));
  sn = RN_ADD(RN_MUL(x2, sn), __uint_as_float(0x3C088889u));
  sn = RN_ADD(RN_MUL(x2, sn), __uint_as_float(0xBE2AAAABu));
  sn = RN_ADD(RN_MUL(RN_MUL(x2, x), sn), x);
  float cs = RN_ADD(RN_MUL(x2, __uint_as_float(0xB493F27Eu)), __uint_as_float(0x37D00D01u));
  cs = RN_ADD(RN_MUL(x2, cs), __uint_as_float(0xBAB60B61u));
  cs = RN_ADD(RN_MUL(x2, cs), __uint_as_float(0x3D2AAAABu));
  cs = RN_ADD(RN_MUL(x2, cs), -0.5f);
  cs = RN_ADD(RN_MUL(x2, cs), 1.0f);
  const float c_in = fold ? sn : cs, s_in = fold ? cs : sn;       // cos and sin of the angle inside its quadrant
  const float c = quadrant == 0 ? c_in : quadrant == 1 ? -s_in : quadrant == 2 ? -c_in : s_in;
  return RN_MUL(radius, c);
}

template <typename T>
__global__ void rng_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean, float stdev) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float zn = rng_normal_from_bits(rng_mix(key, (unsigned long long)i));
    out[i] = from_f32<T>(RN_ADD(mean, RN_MUL(stdev, zn)));
  }
}

static int fill_grid(long long n) {
  long long blocks = ceil_div_ll(n, 256);
  return (int)(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

// out[i] = mean + stdev * normal(key, i), i < n; out is float (dtype 0) or bfloat16 (1).
extern "C" int hb_rng_normal(int dtype, void* out, long long n, unsigned long long key, float mean, float stdev,
                             void* stream) {
  HB_REQUIRE(n >= 0, "rng_normal: negative length");
  if (n == 0) return 0;
  if (dtype == HB_F32)
    hb_launch(rng_normal_kernel<float>, dim3(fill_grid(n)), dim3(256), 0, (cudaStream_t)stream, (float*)out, n, key, mean, stdev);
  else
    hb_launch(rng_normal_kernel<bf16>, dim3(fill_grid(n)), dim3(256), 0, (cudaStream_t)stream, (bf16*)out, n, key, mean, stdev);
  HB_CHECK_LAUNCH("rng_normal");
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void fill_kernel(T* __restrict__ out, long long n, float value) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T v = from_f32<T>(value);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = v;
}

__global__ void fill_i32_kernel(int* __restrict__ out, long long n, int value) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}

// dtype 0 float, 1 bfloat16, 2 int32 (value truncated)
extern "C" int hb_fill(int dtype, void* out, long long n, float value, void* stream) {
  HB_REQUIRE(n >= 0, "fill: negative length");
  HB_REQUIRE(dtype >= 0 && dtype <= 2, "fill: dtype code %d is not float (0), bfloat16 (1) or int32 (2)", dtype);
  if (n == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HB_F32) hb_launch(fill_kernel<float>, dim3(fill_grid(n)), dim3(256), 0, st, (float*)out, n, value);
  else if (dtype == HB_BF16) hb_launch(fill_kernel<bf16>, dim3(fill_grid(n)), dim3(256), 0, st, (bf16*)out, n, value);
  else hb_launch(fill_i32_kernel, dim3(fill_grid(n)), dim3(256), 0, st, (int*)out, n, (int)value);
  HB_CHECK_LAUNCH("fill");
  return 0;
}

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float cast_in(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float cast_in(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float cast_in(const __half* p, long long i) { return __half2float(p[i]); }

// round_bf16: the value passes through bfloat16 (round to nearest even) whatever the output type,
// which is what the reference does to every F32 tensor it loads.
template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ in, D* __restrict__ out, long long n, int round_bf16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = cast_in(in, i);
    if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
    out[i] = from_f32<D>(v);
  }
}

template <typename S>
static int cast_from(const void* in, int dst, void* out, long long n, int round_bf16, cudaStream_t st) {
  if (dst == HB_F32)
    hb_launch(cast_kernel<S, float>, dim3(fill_grid(n)), dim3(256), 0, st, (const S*)in, (float*)out, n, round_bf16);
  else
    hb_launch(cast_kernel<S, bf16>, dim3(fill_grid(n)), dim3(256), 0, st, (const S*)in, (bf16*)out, n, round_bf16);
  HB_CHECK_LAUNCH("cast");
  return 0;
}

// out[i] = (dst type) in[i]; src: 0 float, 1 bfloat16, 2 float16; dst: 0 float, 1 bfloat16.
extern "C" int hb_cast(int src, const void* in, int dst, void* out, long long n, int round_bf16, void* stream) {
  HB_REQUIRE(n >= 0, "cast: negative length");
  HB_REQUIRE(src >= 0 && src <= 2, "cast: source dtype code %d is not float (0), bfloat16 (1) or float16 (2)", src);
  HB_REQUIRE(dst == HB_F32 || dst == HB_BF16, "cast: destination dtype code %d is not float (0) or bfloat16 (1)", dst);
  if (n == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (src == 0) return cast_from<float>(in, dst, out, n, round_bf16, st);
  if (src == 1) return cast_from<bf16>(in, dst, out, n, round_bf16, st);
  return cast_from<__half>(in, dst, out, n, round_bf16, st);
}
