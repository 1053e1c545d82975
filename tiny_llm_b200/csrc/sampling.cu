// Next-token choice on the device, one block per row of 32-bit logits.
//   argmax: first maximum, lowest index on ties (tiny_llm/logit_processors/argmax_processor.cpp:24-31).
//   sample: the reference's chain temperature -> top-k -> top-p -> multinomial
//     (tiny_llm/pipeline/pipeline.cpp:157-161), which it runs on the CPU with sorts
//     (sort_processors.cpp:53-142, sample_processors.cpp:7-54).  Here nothing is sorted: the k-th
//     largest value and the top-p cut are found by a bitwise search over the ordered bit patterns
//     of the values, each probe being one counting pass over the row.
//       top-k keeps exactly k values: those above the k-th largest, and of those equal to it the
//         ones with the lowest token ids.
//       top-p drops the smallest values while their summed probability stays <= 1 - p; values
//         that tie at the cut are kept or dropped together; the maximum always stays.
//       multinomial walks the kept tokens in ascending id and takes the first whose running
//         probability exceeds u, u in [0,1) drawn from (seed, counter) of the row by splitmix64, so a
//         request's draws do not depend on its batch.
//     A row with temperature <= 0 is taken greedily.
// `work` is scratch of n*V floats in global memory: the row's scaled logits, then its weights.
#include <math_constants.h>

#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int ST = 1024;

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct BlockScratch {
  float f[33];
  int i[33];
  unsigned long long u[33];
};

__device__ __forceinline__ float block_max_f(float v, BlockScratch& sc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sc.f[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? sc.f[lane] : -CUDART_INF_F;
    t = warp_max(t);
    if (lane == 0) sc.f[32] = t;
  }
  __syncthreads();
  return sc.f[32];
}

__device__ __forceinline__ float block_sum_f(float v, BlockScratch& sc) { return block_sum(v, sc.f); }

__device__ __forceinline__ int block_sum_i(int v, BlockScratch& sc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sc.i[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int t = lane < (blockDim.x >> 5) ? sc.i[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sc.i[32] = t;
  }
  __syncthreads();
  return sc.i[32];
}

// Exclusive scan of 0/1 flags over the block in thread order; *total gets the block's count.
__device__ __forceinline__ int block_excl_scan_flag(bool flag, int* total, BlockScratch& sc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(ballot & ((1u << lane) - 1u));
  __syncthreads();
  if (lane == 0) sc.i[warp] = __popc(ballot);
  __syncthreads();
  if (warp == 0) {
    const int c = lane < (blockDim.x >> 5) ? sc.i[lane] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    sc.i[lane] = incl - c;
    if (lane == 31) sc.i[32] = incl;
  }
  __syncthreads();
  *total = sc.i[32];
  return sc.i[warp] + in_warp;
}

// Inclusive scan of floats over the block in thread order; *total gets the block's sum.
__device__ __forceinline__ float block_incl_scan_f(float v, float* total, BlockScratch& sc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) sc.f[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const float c = lane < (blockDim.x >> 5) ? sc.f[lane] : 0.f;
    float w = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    sc.f[lane] = w - c;
    if (lane == 31) sc.f[32] = w;
  }
  __syncthreads();
  *total = sc.f[32];
  return sc.f[warp] + incl;
}

__device__ __forceinline__ int block_argmax(const float* __restrict__ row, int v, BlockScratch& sc) {
  float best = -CUDART_INF_F;
  int idx = 0x7fffffff;
  if ((v & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 16-byte loads, two in flight per thread; a thread's elements come in ascending order
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int v4 = v >> 2;
    for (int i = threadIdx.x; i < v4; i += 2 * blockDim.x) {
      const int i2 = i + blockDim.x;
      const float4 a = row4[i];
      const float4 b = i2 < v4 ? row4[i2] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
      const float xa[4] = {a.x, a.y, a.z, a.w}, xb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (idx == 0x7fffffff || xa[e] > best) { best = xa[e]; idx = 4 * i + e; }
      if (i2 < v4) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (xb[e] > best) { best = xb[e]; idx = 4 * i2 + e; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < v; i += blockDim.x) {
      const float x = row[i];
      if (idx == 0x7fffffff || x > best) { best = x; idx = i; }
    }
  }
  // pack (ordered value, inverted index) so that one max picks the value, then the lowest index
  unsigned long long key = idx == 0x7fffffff ? 0ull
      : ((unsigned long long)ordered_key(best) << 32) | (unsigned long long)(0xffffffffu - (unsigned)idx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sc.u[warp] = key;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < (blockDim.x >> 5) ? sc.u[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
      t = other > t ? other : t;
    }
    if (lane == 0) sc.u[32] = t;
  }
  __syncthreads();
  return (int)(0xffffffffu - (unsigned)(sc.u[32] & 0xffffffffull));
}

// `status` (may be null): the device word in which the step's kernels record a bounded wait that
// expired.  Block 0 copies it behind the chosen ids (out[gridDim.x]), so that it reaches the host in
// the copy that carries the ids and a step whose kernel gave up is never mistaken for a result.
__device__ __forceinline__ void forward_status(const int* status, int* out) {
  if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) out[gridDim.x] = *status;
}

__global__ void __launch_bounds__(ST)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int v, const int* __restrict__ status) {
  __shared__ BlockScratch sc;
  pdl_trigger();
  pdl_wait();
  forward_status(status, out);
  const int b = blockIdx.x;
  const int r = block_argmax(logits + (size_t)b * v, v, sc);
  if (threadIdx.x == 0) out[b] = r;
}

__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work, int v,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int* __restrict__ out,
              const int* __restrict__ status) {
  __shared__ BlockScratch sc;
  __shared__ int s_choice, s_last;
  pdl_trigger();
  pdl_wait();
  forward_status(status, out);
  const int b = blockIdx.x;
  const float* row = logits + (size_t)b * v;
  const float temp = temperature[b];
  if (!(temp > 0.f)) {
    const int r = block_argmax(row, v, sc);
    if (threadIdx.x == 0) out[b] = r;
    return;
  }
  float* x = work + (size_t)b * v;
  const int k = top_k[b];
  const float p = top_p[b];

  // scaled logits and their maximum
  float mx = -CUDART_INF_F;
  for (int i = threadIdx.x; i < v; i += ST) {
    const float s = row[i] / temp;
    x[i] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max_f(mx, sc);

  // top-k: tau = ordered key of the k-th largest value
  if (k > 0 && k < v) {
    uint32_t tau = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = tau | (1u << bit);
      int cnt = 0;
      for (int i = threadIdx.x; i < v; i += ST) cnt += ordered_key(x[i]) >= cand;
      if (block_sum_i(cnt, sc) >= k) tau = cand;
    }
    int gt = 0;
    for (int i = threadIdx.x; i < v; i += ST) gt += ordered_key(x[i]) > tau;
    const int need = k - block_sum_i(gt, sc);   // how many of the values equal to tau stay
    int base = 0;
    for (int c0 = 0; c0 < v; c0 += ST) {
      const int i = c0 + threadIdx.x;
      const uint32_t key = i < v ? ordered_key(x[i]) : 0u;
      const bool tie = i < v && key == tau;
      int total;
      const int rank = base + block_excl_scan_flag(tie, &total, sc);
      if (i < v && (key < tau || (tie && rank >= need))) x[i] = -CUDART_INF_F;
      base += total;
    }
  }

  // weights e_i = exp(x_i - max) of the kept tokens, 0 for the dropped ones
  float z = 0.f;
  for (int i = threadIdx.x; i < v; i += ST) {
    const float s = x[i];
    const float e = s == -CUDART_INF_F ? 0.f : expf(s - mx);
    x[i] = e;
    z += e;
  }
  z = block_sum_f(z, sc);

  // top-p: largest cut tau (as float bits, e >= 0) with sum(e_i < tau) <= (1 - p) z; tau <= bits(1.0f) keeps the maximum
  if (p < 1.f) {
    const float budget = (1.f - p) * z;
    const uint32_t one = __float_as_uint(1.0f);
    uint32_t tau = 0;
    for (int bit = 30; bit >= 0; --bit) {
      const uint32_t cand = tau | (1u << bit);
      if (cand > one) continue;
      float mass = 0.f;
      for (int i = threadIdx.x; i < v; i += ST) {
        const float e = x[i];
        mass += __float_as_uint(e) < cand ? e : 0.f;
      }
      if (block_sum_f(mass, sc) <= budget) tau = cand;
    }
    float z2 = 0.f;
    for (int i = threadIdx.x; i < v; i += ST) {
      float e = x[i];
      if (__float_as_uint(e) < tau) { e = 0.f; x[i] = 0.f; }
      z2 += e;
    }
    z = block_sum_f(z2, sc);
  }

  // multinomial: first token id whose running weight exceeds u * z
  const float target = uniform_from(seeds[b], counters[b]) * z;
  if (threadIdx.x == 0) { s_choice = 0x7fffffff; s_last = -1; }
  __syncthreads();
  float base = 0.f;
  for (int c0 = 0; c0 < v; c0 += ST) {
    const int i = c0 + threadIdx.x;
    const float e = i < v ? x[i] : 0.f;
    float total;
    const float incl = base + block_incl_scan_f(e, &total, sc);
    if (e > 0.f) {
      atomicMax(&s_last, i);
      if (incl > target) atomicMin(&s_choice, i);
    }
    base += total;
    __syncthreads();
    if (s_choice != 0x7fffffff) break;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[b] = s_choice != 0x7fffffff ? s_choice : s_last;
}

}  // namespace tllm

using namespace tllm;

// status (both entry points): null, or the device status word of the step's kernels; out then has
// room for n + 1 ints and out[n] receives the word.
extern "C" int tllm_argmax(const float* logits, int* out, int n, int v, const int* status, void* stream) {
  TLLM_REQUIRE(n > 0 && v > 0, "argmax: empty input (%d rows of %d)", n, v);
  TLLM_LAUNCH("argmax", argmax_kernel, n, ST, 0, (cudaStream_t)stream, logits, out, v, status);
  return TLLM_OK;
}

extern "C" int tllm_sample(const float* logits, float* work, int n, int v, const float* temperature, const int* top_k,
                           const float* top_p, const unsigned long long* seeds, const unsigned long long* counters,
                           int* out, const int* status, void* stream) {
  TLLM_REQUIRE(n > 0 && v > 0, "sample: empty input (%d rows of %d)", n, v);
  TLLM_REQUIRE(work != nullptr, "sample: needs n*V floats of scratch");
  TLLM_LAUNCH("sample", sample_kernel, n, ST, 0, (cudaStream_t)stream, logits, work, v, temperature, top_k, top_p, seeds, counters, out, status);
  return TLLM_OK;
}

// ---------------------------------------------------------------- sampling without a caller's scratch
// See sampling_noalloc.h.  The scratch of the sampling kernel lives in this file-scope device array.
// In host code `g_noalloc_scratch` is only a handle for the symbol, not an address the GPU can use:
// its device address is looked up once per device with cudaGetSymbolAddress and kept here.
#include "sampling_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[TLLM_SAMPLE_NOALLOC_MAX_FLOATS];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal
std::mutex g_noalloc_setup;               // two host threads may make their first call at once
}  // namespace

extern "C" int tllm_sample_noalloc(const float* logits, int n, int v, const float* temperature, const int* top_k,
                                   const float* top_p, const unsigned long long* seeds,
                                   const unsigned long long* counters, int* out, void* stream) {
  TLLM_REQUIRE(n > 0 && v > 0, "sample_noalloc: empty input (%d rows of %d)", n, v);
  TLLM_REQUIRE((long long)n * v <= (long long)TLLM_SAMPLE_NOALLOC_MAX_FLOATS,
               "sample_noalloc: %d rows of %d logits need %lld floats of scratch, the built-in array holds %d; "
               "use tllm_sample with scratch of your own", n, v, (long long)n * v, TLLM_SAMPLE_NOALLOC_MAX_FLOATS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "sample_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  TLLM_REQUIRE(dev >= 0 && dev < kMaxDevices, "sample_noalloc: device ordinal %d is out of range", dev);
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> hold(g_noalloc_setup);
    if (g_noalloc_ptr[dev] == nullptr) {
      // set-up, once per device, with that device current: must happen outside of stream capture
      float* p = nullptr;
      e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr)
        TLLM_FAIL(TLLM_ERR_CUDA, "sample_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
  }
  TLLM_LAUNCH("sample_noalloc", sample_kernel, n, ST, 0, (cudaStream_t)stream, logits, scratch, v,
              temperature, top_k, top_p, seeds, counters, out, (const int*)nullptr);
  return TLLM_OK;
}
