// Shared helpers of the infllm_b200 kernels: error reporting, dtype traits, small device utilities.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/infllm_b200.h"

namespace infllm {

// ---- error plumbing: one message per host thread, codes from the public header
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
void count_launch();  // every kernel launch of the library is counted (infllm_launch_count)

#define INFLLM_CUDA_OK(expr)                                                                  \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::infllm::fail(INFLLM_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                            __FILE__, __LINE__);                                              \
  } while (0)

#define INFLLM_LAUNCH_OK(name)                                                                \
  do {                                                                                        \
    cudaError_t _e = cudaGetLastError();                                                      \
    if (_e != cudaSuccess)                                                                    \
      return ::infllm::fail(INFLLM_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    ::infllm::count_launch();                                                                 \
  } while (0)

// ---- programmatic dependent launch for the chain of small kernels behind a decode token.  A kernel of the chain
// waits, before it touches anything, until the grids before it have completed and their writes are visible, and
// then lets the next launch of its stream be scheduled (its CTAs come onto the SMs as this grid's drain).  In this
// order a kernel that is being scheduled knows that everything before its predecessor is complete, so it may do,
// ahead of its own wait, work that depends on nothing its predecessor writes (chain_trigger(), then chain_wait()
// where the predecessor's results are first needed).  The statements do nothing in a kernel that was launched the
// ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_enter() {
  chain_wait();
  chain_trigger();
}
// launch `kern` so that it may start while the kernel before it on the stream winds down (it must call chain_enter())
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

#define INFLLM_TRY(expr)        \
  do {                          \
    int _rc = (expr);           \
    if (_rc != INFLLM_OK) return _rc; \
  } while (0)

// ---- 16-bit activation types
template <typename T>
struct Act;
template <>
struct Act<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 x) { return __bfloat1622float2(x); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) {
    return __floats2bfloat162_rn(a, b);
  }
};
template <>
struct Act<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__half2 x) { return __half22float2(x); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) { return __floats2half2_rn(a, b); }
};

// fp32 as an output type of the log-sum-exp merge (per-rank partials that are merged again)
template <>
struct Act<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};

// dispatch a lambda-like macro on the runtime dtype code
#define INFLLM_DISPATCH_DTYPE(dtype, T, ...)                          \
  do {                                                                \
    if ((dtype) == INFLLM_BF16) {                                     \
      using T = __nv_bfloat16;                                        \
      __VA_ARGS__                                                     \
    } else if ((dtype) == INFLLM_FP16) {                              \
      using T = __half;                                               \
      __VA_ARGS__                                                     \
    } else {                                                          \
      return ::infllm::fail(INFLLM_E_UNSUPPORTED, "dtype code %d", (int)(dtype)); \
    }                                                                 \
  } while (0)

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace infllm
