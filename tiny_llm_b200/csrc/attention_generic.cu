// Attention of the step's queries over the paged cache, one warp per (token, query head), any
// head size that is a multiple of 16 up to 256, any number of heads and groups, any page size.
// It is the attention of the true 32-bit path and the fallback of the bfloat16 path.
//
// The keys a query at position p sees are j in [max(0, p - window + 1), p].  They are walked in
// tiles of 32 that start at multiples of 32 of the absolute position, with a running softmax
// (m, l, o) in 32-bit, so the order of the sums is a function of p alone: the result does not
// depend on how the request's tokens were cut into steps, on the rest of the batch or on the
// page ids.  Reference counterpart: tiny_llm/ops/cuda/flash_attention.cu:338-442 (64-key tiles,
// one lane per key, P.V by shuffles), whose mask compares a chunk-local query index with the
// absolute key index (:63-66, :402-405).
#include <math_constants.h>

#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T> struct Vec;            // 16-byte vectors of the cache rows
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void load16(const float* p, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float* dst) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    dst[2 * i] = f.x; dst[2 * i + 1] = f.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ kcache,
                               const T* __restrict__ vcache, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ token_request,
                               const int* __restrict__ positions, T* __restrict__ out, int n_tokens,
                               int nq, int nkv, int hd, int page_size, long long page_stride,
                               long long head_stride, float scale, int window) {
  __shared__ __align__(16) float q_s[WARPS][MAX_HD];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long task = (long long)blockIdx.x * WARPS + warp;
  if (task >= (long long)n_tokens * nq) return;
  const int t = (int)(task / nq), h = (int)(task % nq);
  const int kvh = h / (nq / nkv);
  const int req = token_request[t];
  const int p = positions[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* table = block_table + (size_t)req * max_blocks;

  const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(qrow[d]) * scale;
  __syncwarp();

  float m = -CUDART_INF_F, l = 0.f;
  float o[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) o[i] = 0.f;

  for (int j0 = (lo / 32) * 32; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    bool valid = j >= lo && j <= p && j / page_size < max_blocks;
    const int page = valid ? table[j / page_size] : -1;
    valid = valid && page >= 0;   // a table entry that names no page is never followed
    long long row_off = 0;
    float s = -CUDART_INF_F;
    if (valid) {
      row_off = (long long)page * page_stride + (long long)kvh * head_stride + (long long)(j % page_size) * hd;
      const T* krow = kcache + row_off;
      float acc = 0.f;
      for (int d = 0; d < hd; d += Vec<T>::N) {
        float kv[Vec<T>::N];
        load16(krow + d, kv);
#pragma unroll
        for (int e = 0; e < Vec<T>::N; ++e) acc = fmaf(q_s[warp][d + e], kv[e], acc);
      }
      s = acc;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float m_ref = m_new == -CUDART_INF_F ? 0.f : m_new;   // a tile without a visible key changes nothing
    const float pr = valid ? expf(s - m_ref) : 0.f;
    const float corr = expf(m - m_ref);           // 0 on the first tile (m = -inf)
    l = l * corr + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) o[i] *= corr;
    const int last = min(31, p - j0);
    const int first = max(0, lo - j0);
    for (int kk = first; kk <= last; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      if (pk == 0.f) continue;   // uniform across the warp: nothing to add, and the row may name no page
      const long long off = __shfl_sync(0xffffffffu, row_off, kk);
      const T* vrow = vcache + off;
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[i] = fmaf(pk, to_f32(vrow[d]), o[i]);
      }
    }
  }
  T* orow = out + (size_t)t * nq * hd + (size_t)h * hd;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_f32<T>(o[i] * inv);
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_paged_attention_generic(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                            const int* block_table, int max_blocks, const int* token_request,
                                            const int* positions, void* out, int n_tokens, int nq, int nkv, int hd,
                                            int page_size, long long page_stride, long long head_stride,
                                            float scale, int window, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && nq % nkv == 0,
               "attention: %d tokens, %d heads, %d key/value heads (heads must be a multiple of key/value heads)", n_tokens, nq, nkv);
  TLLM_REQUIRE(hd >= 16 && hd <= MAX_HD && hd % 16 == 0,
               "attention: head size %d is not built (multiples of 16 up to %d are)", hd, MAX_HD);
  TLLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attention: page size %d, %d blocks, window %d", page_size, max_blocks, window);
  const int elem = dtype == TLLM_F32 ? 4 : 2;
  TLLM_REQUIRE(((size_t)kcache % 16) == 0 && ((size_t)vcache % 16) == 0 && (page_stride * elem) % 16 == 0 && (head_stride * elem) % 16 == 0,
               "attention: cache rows must be 16-byte aligned");
  const long long tasks = (long long)n_tokens * nq;
  const long long blocks = (tasks + WARPS - 1) / WARPS;
  TLLM_REQUIRE(blocks <= 2147483647LL, "attention: %lld (token, head) pairs exceed the grid", tasks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("paged_attention_generic", paged_attention_generic_kernel<float>, (unsigned)blocks, WARPS * 32, 0, s,
        (const float*)q, q_row_stride, (const float*)kcache, (const float*)vcache, block_table, max_blocks,
        token_request, positions, (float*)out, n_tokens, nq, nkv, hd, page_size, page_stride, head_stride, scale, window);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("paged_attention_generic", paged_attention_generic_kernel<__nv_bfloat16>, (unsigned)blocks, WARPS * 32, 0, s,
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table,
        max_blocks, token_request, positions, (__nv_bfloat16*)out, n_tokens, nq, nkv, hd, page_size, page_stride,
        head_stride, scale, window);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "attention: unknown dtype code %d", dtype);
  return TLLM_OK;
}
