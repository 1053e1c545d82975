// Shared helpers of the sm_100a kernels: dtype codes of the C interface, 32-bit conversions,
// warp and block reductions, and the error convention (every entry point returns 0 or a
// negative code and leaves a message that tllm_last_error() returns).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define TLLM_F32 0
#define TLLM_BF16 1

#define TLLM_OK 0
#define TLLM_ERR_ARG -1      // a size or dtype the kernel does not take
#define TLLM_ERR_CUDA -2     // the launch failed

namespace tllm {

inline char* error_buffer() {
  static thread_local char buf[512];
  return buf;
}

#define TLLM_FAIL(code, ...)                                   \
  do {                                                         \
    snprintf(::tllm::error_buffer(), 512, __VA_ARGS__);        \
    return (code);                                             \
  } while (0)

#define TLLM_REQUIRE(cond, ...) \
  do {                          \
    if (!(cond)) TLLM_FAIL(TLLM_ERR_ARG, __VA_ARGS__); \
  } while (0)

#define TLLM_CHECK_LAUNCH(name)                                                        \
  do {                                                                                 \
    cudaError_t e_ = cudaGetLastError();                                               \
    if (e_ != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over the block; every thread gets the result.  `scratch` holds at least 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace tllm

// Each shared object exports its own tllm_last_error().
#define TLLM_DEFINE_LAST_ERROR \
  extern "C" const char* tllm_last_error() { return ::tllm::error_buffer(); }
