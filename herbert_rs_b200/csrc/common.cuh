// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions used by every kernel file:
//  * activations and cache entries are of type T = float (32-bit path) or __nv_bfloat16;
//    sums, norms, softmax, rotation and the residual stream are always float;
//  * every launcher is `extern "C"`, takes raw device pointers plus a cudaStream_t (as void*),
//    returns 0 on success and a non-zero code after storing a message for hb_last_error();
//  * a launcher validates sizes on the host and refuses what its kernel cannot do; it never
//    launches a kernel that could give a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// ---- host-side error reporting ------------------------------------------------------------
void hb_set_error(const char* fmt, ...);
#define HB_FAIL(code, ...)            \
  do {                                \
    hb_set_error(__VA_ARGS__);        \
    return (code);                    \
  } while (0)
#define HB_REQUIRE(cond, ...)         \
  do {                                \
    if (!(cond)) HB_FAIL(2, __VA_ARGS__); \
  } while (0)
#define HB_CHECK_LAUNCH(name)                                                   \
  do {                                                                          \
    cudaError_t e__ = cudaGetLastError();                                       \
    if (e__ != cudaSuccess) HB_FAIL(3, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// ---- launching ------------------------------------------------------------------------------
// Every kernel is launched through hb_launch.  With programmatic dependent launch switched on
// (hb_set_pdl(1); off by default) a kernel may be scheduled while its predecessor in the stream is
// still draining; it must then call pdl_wait() before it reads anything the predecessor wrote or
// writes anything the predecessor may still read.  pdl_launch() tells the hardware that the next
// kernel may start its own prologue.  It is called after pdl_wait(), so that at most one kernel
// ahead of the running one sits on the SMs, and in the long decode kernels only when the CTA's own
// loads are done: CTAs that wait beside working ones cost those issue slots (measured: the step
// twice as long with the trigger at the start).  Both are no-ops for a kernel launched without the attribute.
int hb_pdl_enabled(void);   // 0 off, 1 every kernel, 2 only the launches that ask for it (hb_launch_pdl)
template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch_ex(int want_pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const int mode = hb_pdl_enabled();
  cfg.numAttrs = (mode == 1 || (mode == 2 && want_pdl)) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  return hb_launch_ex(0, kernel, grid, block, smem, stream, static_cast<KArgs>(args)...);
}
// For kernels whose prologue is worth starting early (weight loads that do not depend on the predecessor).
template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        Args&&... args) {
  return hb_launch_ex(1, kernel, grid, block, smem, stream, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- conversions ---------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions -----------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over a whole block (any multiple of 32 threads up to 1024); every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? smem32[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }
