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

#define TLLM_LAUNCH(name, kernel, grid, block, smem, stream, ...)                                   \
  do {                                                                                              \
    cudaError_t e_ = ::tllm::launch_kernel(kernel, grid, block, smem, stream, __VA_ARGS__);         \
    if (e_ != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e_));        \
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

// ---- programmatic dependent launch
// Every kernel of the step begins with pdl_trigger() (the next kernel of the stream may be placed on
// SMs as they free up) and calls pdl_wait() before it touches anything an earlier kernel wrote or
// still reads.  What a kernel does before pdl_wait() must depend on nothing but constants of the
// model (weights): that part overlaps the tail of its predecessor.  Without the launch attribute
// both instructions do nothing, so the same kernels run in plain stream order too.
//
// With -DTLLM_TRACE (a build for measurements) the first thread of the first CTA of every launch also
// notes the global timer at both points: when the CTA started, and when its wait for the kernel
// before it returned -- which is when that kernel had finished.  The notes of one step, read back
// with tllm_trace_dump(), are the timeline of the step inside its CUDA graph.
#ifdef TLLM_TRACE
struct TraceRec {
  unsigned long long t_enter, t_ready;
  unsigned int gx, gy, gz, bx;
  unsigned long long t_mark[4];   // optional notes of the kernel itself, see trace_mark()
};
__device__ TraceRec g_trace[8192];
__device__ unsigned int g_trace_n;
__shared__ unsigned int s_trace_slot;
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool trace_here() { return (blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x) == 0; }
#endif

// A kernel may note up to four more moments of its first CTA (nothing without -DTLLM_TRACE).
__device__ __forceinline__ void trace_mark(int i) {
#ifdef TLLM_TRACE
  if (trace_here()) g_trace[s_trace_slot].t_mark[i] = trace_now();
#endif
}

// ... and a number of its own in the last of the four slots (which product this launch was).
__device__ __forceinline__ void trace_tag(unsigned long long v) {
#ifdef TLLM_TRACE
  if (trace_here()) g_trace[s_trace_slot].t_mark[3] = v;
#endif
}

__device__ __forceinline__ void pdl_trigger() {
#ifdef TLLM_TRACE
  if (trace_here()) {
    const unsigned int i = atomicAdd(&g_trace_n, 1u) & 8191u;
    s_trace_slot = i;
    g_trace[i].t_enter = trace_now();
    g_trace[i].t_ready = 0;
    g_trace[i].t_mark[0] = g_trace[i].t_mark[1] = g_trace[i].t_mark[2] = g_trace[i].t_mark[3] = 0;
    g_trace[i].gx = gridDim.x; g_trace[i].gy = gridDim.y; g_trace[i].gz = gridDim.z; g_trace[i].bx = blockDim.x;
  }
#endif
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef TLLM_TRACE
  if (trace_here()) g_trace[s_trace_slot].t_ready = trace_now();
#endif
}

inline int& pdl_enabled() {
  static int on = 1;
  return on;
}

// Launches `kernel`, as a programmatic dependent of the stream's previous kernel when enabled.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tllm

// Each shared object exports its own tllm_last_error() and tllm_set_pdl().
#ifdef TLLM_TRACE
#define TLLM_DEFINE_TRACE                                                                                   \
  extern "C" int tllm_trace_dump(void* host, int max_records) {                                              \
    unsigned int n = 0;                                                                                      \
    cudaDeviceSynchronize();                                                                                 \
    cudaMemcpyFromSymbol(&n, ::tllm::g_trace_n, sizeof(n));                                                  \
    if (n > 8192u) n = 8192u;                                                                                \
    if ((int)n > max_records) n = (unsigned int)max_records;                                                 \
    cudaMemcpyFromSymbol(host, ::tllm::g_trace, sizeof(::tllm::TraceRec) * n);                               \
    const unsigned int zero = 0;                                                                             \
    cudaMemcpyToSymbol(::tllm::g_trace_n, &zero, sizeof(zero));                                              \
    return (int)n;                                                                                           \
  }
#else
#define TLLM_DEFINE_TRACE
#endif

#define TLLM_DEFINE_LAST_ERROR                                                  \
  extern "C" const char* tllm_last_error() { return ::tllm::error_buffer(); }  \
  extern "C" void tllm_set_pdl(int on) { ::tllm::pdl_enabled() = on ? 1 : 0; } \
  TLLM_DEFINE_TRACE
