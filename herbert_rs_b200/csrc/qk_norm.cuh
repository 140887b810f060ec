// Per-head RMSNorm and rotation of one head of 128 values by half a warp, shared by the
// stand-alone norm/rotation/cache kernel and the fused decode attention so that both give the
// same bits.  Lane l (0..15 of its half-warp) holds x[4l..4l+3] and x[64+4l..64+4l+3]: the two
// halves that the rotation pairs (crates/backends/backend_common/src/kernels.rs: rotate-half
// form, pairs (j, j + rot/2)).
#pragma once

#include "common.cuh"

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* v) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __bfloat162float(a.x); v[1] = __bfloat162float(a.y); v[2] = __bfloat162float(b.x); v[3] = __bfloat162float(b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const unsigned*>(&a);
    t.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

// The loads of one head's values, norm weights and angles, apart from the arithmetic: a caller that
// has bulk loads to issue as well asks for these first, or they queue up behind the bulk.
struct NormRotateLoads {
  float lo[4], hi[4];
  float4 wl, wh, c4, s4;
};
template <typename T>
__device__ __forceinline__ NormRotateLoads norm_rotate_load(bool active, const T* x, const float* w, const float* cos_row,
                                                            const float* sin_row, int l) {
  NormRotateLoads r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.lo[i] = r.hi[i] = 0.0f;
  r.wl = r.wh = r.c4 = make_float4(1.f, 1.f, 1.f, 1.f);
  r.s4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (active) {
    Vec4<T>::load(x + 4 * l, r.lo);
    Vec4<T>::load(x + 64 + 4 * l, r.hi);
    if (w != nullptr) {
      r.wl = *reinterpret_cast<const float4*>(w + 4 * l);
      r.wh = *reinterpret_cast<const float4*>(w + 64 + 4 * l);
    }
    r.c4 = *reinterpret_cast<const float4*>(cos_row + 4 * l);
    r.s4 = *reinterpret_cast<const float4*>(sin_row + 4 * l);
  }
  return r;
}

// Every lane of the warp must call this (the sums use full-warp shuffles that stay inside a
// half-warp); a half-warp with nothing to do passes active = false and touches no memory.
template <typename T>
__device__ __forceinline__ void norm_rotate_finish(NormRotateLoads& r, bool active, T* dst, bool normed, float eps, int l) {
  float* lo = r.lo;
  float* hi = r.hi;
  if (normed) {
    float ss = lo[0] * lo[0] + lo[1] * lo[1] + lo[2] * lo[2] + lo[3] * lo[3] + hi[0] * hi[0] + hi[1] * hi[1] + hi[2] * hi[2] + hi[3] * hi[3];
    ss += __shfl_xor_sync(0xffffffffu, ss, 8);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    if (active) {
      const float inv = 1.0f / sqrtf(ss / 128.0f + eps);
      lo[0] = (lo[0] * inv) * r.wl.x; lo[1] = (lo[1] * inv) * r.wl.y; lo[2] = (lo[2] * inv) * r.wl.z; lo[3] = (lo[3] * inv) * r.wl.w;
      hi[0] = (hi[0] * inv) * r.wh.x; hi[1] = (hi[1] * inv) * r.wh.y; hi[2] = (hi[2] * inv) * r.wh.z; hi[3] = (hi[3] * inv) * r.wh.w;
    }
  }
  if (active) {
    const float c[4] = {r.c4.x, r.c4.y, r.c4.z, r.c4.w}, s[4] = {r.s4.x, r.s4.y, r.s4.z, r.s4.w};
    float olo[4], ohi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      olo[i] = lo[i] * c[i] - hi[i] * s[i];
      ohi[i] = lo[i] * s[i] + hi[i] * c[i];
    }
    Vec4<T>::store(dst + 4 * l, olo);
    Vec4<T>::store(dst + 64 + 4 * l, ohi);
  }
}

// Both in one: x, dst: 8-byte (bfloat16) or 16-byte (float) aligned; w: norm weight [128] or null;
// cos_row, sin_row: the 64 angles of the token's position, 16-byte aligned.  Every lane of the warp calls it.
template <typename T>
__device__ __forceinline__ void norm_rotate_head128(bool active, const T* x, T* dst, const float* w, float eps,
                                                    const float* cos_row, const float* sin_row, int l) {
  NormRotateLoads r = norm_rotate_load<T>(active, x, w, cos_row, sin_row, l);
  norm_rotate_finish<T>(r, active, dst, w != nullptr, eps, l);
}
