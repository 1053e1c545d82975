// Memory-bound kernels of the step: embedding gather, RMSNorm, SiLU*up, and the fused
// rotate-and-cache kernel (RoPE on queries and keys in 32-bit, keys and values written into
// their pages).  All take float32 or bfloat16 activations; statistics and angles are 32-bit.
// Reference counterparts: tiny_llm/ops/cuda/embedding.cu:10-29, norm.cu:16-49, silu.cu:7-12,
// arithmetic.cu:7-22, rope.cu:26-95, gemm.cu:380-411 (the scatter of K/V rows into pages).
#include <algorithm>
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

// ---------------------------------------------------------------- embedding: out[t,:] = table[tokens[t],:]
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int n_tokens, int hidden) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const T* row = table + (size_t)tokens[t] * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

// ---------------------------------------------------------------- RMSNorm
// y_j = (w_j * x_j) / sqrt(sum_j(x_j^2)/H + eps); one block per row; rows may be gathered.
template <typename T>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                T* __restrict__ out, const int* __restrict__ rows, int n_rows,
                                int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = src[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);   // one division per row; the elements are multiplied
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>((w[i] * src[i]) * inv);
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  uint2 pk;
  *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = pk;
}

// The same for widths that are multiples of 4 and at most 4 * VEC * blockDim: the row is read once,
// with 16-byte loads, and kept in registers between the two passes.
template <typename T, int VEC>
__global__ void rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    T* __restrict__ out, const int* __restrict__ rows, int n_rows,
                                    int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  // the weight is a constant of the model (and `rows` comes with the step's tables): both are read
  // before the wait for the kernel that writes x, so that only x itself is waited for afterwards
  const int r = blockIdx.x;
  const int n4 = hidden / 4;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 g[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    g[i] = idx < n4 ? __ldg(w4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src_row = r < n_rows ? (rows ? rows[r] : r) : 0;
  pdl_wait();
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)src_row * hidden);
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    v[i] = idx < n4 ? src[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);   // one division per row; the elements are multiplied
  T* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4)
      store4(dst + 4 * idx, (g[i].x * v[i].x) * inv, (g[i].y * v[i].y) * inv, (g[i].z * v[i].z) * inv, (g[i].w * v[i].w) * inv);
  }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// `gu` rows hold gate and up interleaved in blocks: [2 g B, 2 g B + B) gate, next B up.  With
// ZERO the source is a float32 accumulation buffer (split-K partial sums land there) that this
// kernel hands back cleared: every element is read once, by the thread that then zeroes it.
template <typename TIn, typename TOut, bool ZERO>
__global__ void silu_mul_kernel(TIn* __restrict__ gu, TOut* __restrict__ out, int m, int inter, int blk) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)m * inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(idx / inter), col = (int)(idx % inter);
    const int g = col / blk, j = col % blk;
    TIn* src = gu + (size_t)row * 2 * inter + (size_t)g * 2 * blk;
    const float gate = to_f32(src[j]), up = to_f32(src[blk + j]);
    if (ZERO) { src[j] = from_f32<TIn>(0.f); src[blk + j] = from_f32<TIn>(0.f); }
    out[idx] = from_f32<TOut>((gate / (1.f + expf(-gate))) * up);
  }
}

// ---------------------------------------------------------------- rotate and cache
// qkv row: [nq*hd queries | nkv*hd keys | nkv*hd values] (keys/values absent when slot_mapping is
// null).  Queries are rotated in place; keys are rotated and written to the key pages, values are
// copied to the value pages, both at slot_mapping[t] = page*page_size + offset.
// Rotation (rotate-half over the whole head; rot_dim is hd or 0): x'_i = c x_i - s x_{i+hd/2},
// x'_{i+hd/2} = s x_i + c x_{i+hd/2}.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, float* __restrict__ src, int src_stride,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     int n_tokens, int nq, int nkv, int hd, int row_stride,
                                     T* __restrict__ kcache, T* __restrict__ vcache,
                                     const int* __restrict__ slot_mapping, int page_size,
                                     long long page_stride, long long head_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride;
  float* srow = src ? src + (size_t)t * src_stride : nullptr;   // float32 source that is handed back zeroed
  const bool write_kv = slot_mapping != nullptr;
  const int heads = write_kv ? nq + nkv : nq;
  const int half_hd = hd / 2;
  long long slot_base = 0;
  if (write_kv) {
    const int slot = slot_mapping[t];
    if (slot < 0) return;   // a token without a slot writes nothing
    slot_base = (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * hd;
  }
  // queries and keys: one thread per (head, i < hd/2) rotates the pair of dims (i, i + hd/2)
  for (int idx = threadIdx.x; idx < heads * half_hd; idx += blockDim.x) {
    const int h = idx / half_hd, i = idx % half_hd;
    const int e = h * hd + i;
    float va, vb;
    if (srow) {
      // the projection's output is a tensor of the model's dtype: its sums are rounded to it before the rotation,
      // as where the projection itself stores them
      va = to_f32(from_f32<T>(srow[e])); vb = to_f32(from_f32<T>(srow[e + half_hd]));
      srow[e] = 0.f; srow[e + half_hd] = 0.f;
    } else {
      va = to_f32(row[e]); vb = to_f32(row[e + half_hd]);
    }
    float oa = va, ob = vb;
    if (cos_t) {
      const float c = cos_t[(size_t)pos * half_hd + i], s = sin_t[(size_t)pos * half_hd + i];
      oa = c * va - s * vb;
      ob = s * va + c * vb;
    }
    T* dst = h < nq ? row + (size_t)h * hd : kcache + slot_base + (long long)(h - nq) * head_stride;
    dst[i] = from_f32<T>(oa);
    dst[i + half_hd] = from_f32<T>(ob);
  }
  if (write_kv) {
    const int v0 = (nq + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
      const int h = idx / hd, i = idx % hd;
      T val;
      if (srow) { val = from_f32<T>(srow[v0 + idx]); srow[v0 + idx] = 0.f; }
      else val = row[v0 + idx];
      vcache[slot_base + (long long)h * head_stride + i] = val;
    }
  }
}

// ---- the same with 16-byte accesses, for head sizes that are multiples of 16 and aligned rows:
// one thread rotates eight consecutive pairs (i, i + hd/2).
__device__ __forceinline__ void load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, float* __restrict__ src, int src_stride,
                                         const int* __restrict__ positions,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         int n_tokens, int nq, int nkv, int hd, int row_stride,
                                         T* __restrict__ kcache, T* __restrict__ vcache,
                                         const int* __restrict__ slot_mapping, int page_size,
                                         long long page_stride, long long head_stride) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride;
  float* srow = src ? src + (size_t)t * src_stride : nullptr;
  const bool write_kv = slot_mapping != nullptr;
  const int heads = write_kv ? nq + nkv : nq;
  const int half_hd = hd / 2, groups = half_hd / 8;   // groups of eight pairs per head
  long long slot_base = 0;
  if (write_kv) {
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    slot_base = (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * hd;
  }
  const float zeros[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  // gridDim.y CTAs share a token's work items
  const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
  for (int idx = first; idx < heads * groups; idx += step) {
    const int h = idx / groups, i = (idx % groups) * 8;
    const int e = h * hd + i;
    float va[8], vb[8], oa[8], ob[8];
    if (srow) {
      load8(srow + e, va); load8(srow + e + half_hd, vb);
      store8(srow + e, zeros); store8(srow + e + half_hd, zeros);
#pragma unroll
      for (int j = 0; j < 8; ++j) { va[j] = to_f32(from_f32<T>(va[j])); vb[j] = to_f32(from_f32<T>(vb[j])); }   // (as above)
    } else {
      load8(row + e, va); load8(row + e + half_hd, vb);
    }
    if (cos_t) {
      float c[8], sn[8];
      load8(cos_t + (size_t)pos * half_hd + i, c);
      load8(sin_t + (size_t)pos * half_hd + i, sn);
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = c[j] * va[j] - sn[j] * vb[j]; ob[j] = sn[j] * va[j] + c[j] * vb[j]; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = va[j]; ob[j] = vb[j]; }
    }
    T* dst = h < nq ? row + (size_t)h * hd : kcache + slot_base + (long long)(h - nq) * head_stride;
    store8(dst + i, oa);
    store8(dst + i + half_hd, ob);
  }
  if (write_kv) {
    const int v0 = (nq + nkv) * hd;
    for (int idx = first; idx < nkv * hd / 8; idx += step) {
      const int h = (idx * 8) / hd, i = (idx * 8) % hd;
      float v[8];
      if (srow) { load8(srow + v0 + idx * 8, v); store8(srow + v0 + idx * 8, zeros); }
      else load8(row + v0 + idx * 8, v);
      store8(vcache + slot_base + (long long)h * head_stride + i, v);
    }
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_embedding(const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                              int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && hidden > 0, "embedding: empty input (%d tokens, width %d)", n_tokens, hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("embedding", embedding_kernel<float>, n_tokens, threads, 0, s, tokens, (const float*)table, out, n_tokens, hidden);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("embedding", embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, tokens, (const __nv_bfloat16*)table, out, n_tokens, hidden);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "embedding: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_rms_norm(const float* x, const float* w, void* out, const int* rows, int n_rows, int hidden,
                             float eps, int out_dtype, void* stream) {
  TLLM_REQUIRE(n_rows > 0 && hidden > 0, "rms_norm: empty input (%d rows, width %d)", n_rows, hidden);
  TLLM_REQUIRE(out_dtype == TLLM_F32 || out_dtype == TLLM_BF16, "rms_norm: unknown dtype code %d", out_dtype);
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = hidden % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0;
  if (aligned && hidden <= 4 * 4 * 256) {
    // 128 or 256 threads, up to four 16-byte loads each
    const int n4 = hidden / 4;
    // Few rows (decode): more threads per row, fewer loads per thread in a row.  Only for bfloat16 output:
    // the 32-bit path promises sums whose order does not depend on what else is in the batch.
    const bool wide = out_dtype == TLLM_BF16 && n_rows <= 64;
    const int threads = wide ? (n4 <= 128 ? 128 : (n4 <= 256 ? 256 : 512)) : (n4 <= 128 * 4 ? 128 : 256);
    const int vec = (n4 + threads - 1) / threads;
#define TLLM_NORM_CASE(V)                                                                                                   \
  if (out_dtype == TLLM_F32)                                                                                               \
    TLLM_LAUNCH("rms_norm", (rms_norm_vec_kernel<float, V>), n_rows, threads, 0, s, x, w, (float*)out, rows, n_rows, hidden, eps); \
  else                                                                                                                     \
    TLLM_LAUNCH("rms_norm", (rms_norm_vec_kernel<__nv_bfloat16, V>), n_rows, threads, 0, s, x, w, (__nv_bfloat16*)out, rows, n_rows, hidden, eps); \
  return TLLM_OK;
    if (vec <= 1) { TLLM_NORM_CASE(1) }
    if (vec == 2) { TLLM_NORM_CASE(2) }
    if (vec == 3) { TLLM_NORM_CASE(3) }
    { TLLM_NORM_CASE(4) }
#undef TLLM_NORM_CASE
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == TLLM_F32)
    TLLM_LAUNCH("rms_norm", rms_norm_kernel<float>, n_rows, threads, 0, s, x, w, (float*)out, rows, n_rows, hidden, eps);
  else
    TLLM_LAUNCH("rms_norm", rms_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, s, x, w, (__nv_bfloat16*)out, rows, n_rows, hidden, eps);
  return TLLM_OK;
}

// in_dtype: dtype of `gu`; out_dtype: dtype of `out`.  zero_src != 0 (float32 `gu` only): `gu` is a
// split-K accumulation buffer and is handed back cleared.
extern "C" int tllm_silu_mul(void* gu, void* out, int m, int inter, int blk, int in_dtype, int out_dtype, int zero_src,
                             void* stream) {
  TLLM_REQUIRE(m > 0 && inter > 0 && blk > 0 && inter % blk == 0,
               "silu_mul: %d rows, width %d, block %d (the block must divide the width)", m, inter, blk);
  const size_t total = (size_t)m * inter;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == TLLM_F32 && out_dtype == TLLM_F32 && !zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, float, false>), blocks, threads, 0, s, (float*)gu, (float*)out, m, inter, blk);
  else if (in_dtype == TLLM_BF16 && out_dtype == TLLM_BF16 && !zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<__nv_bfloat16, __nv_bfloat16, false>), blocks, threads, 0, s, (__nv_bfloat16*)gu, (__nv_bfloat16*)out, m, inter, blk);
  else if (in_dtype == TLLM_F32 && out_dtype == TLLM_BF16 && zero_src)
    TLLM_LAUNCH("silu_mul", (silu_mul_kernel<float, __nv_bfloat16, true>), blocks, threads, 0, s, (float*)gu, (__nv_bfloat16*)out, m, inter, blk);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "silu_mul: dtype codes %d -> %d with zero_src %d are not built", in_dtype, out_dtype, zero_src);
  return TLLM_OK;
}

// `src` (optional): float32 rows of src_stride values to read instead of `qkv`; they are handed back
// zeroed (a split-K accumulation buffer); the rotated queries are written to `qkv` all the same.
extern "C" int tllm_rope_kv_write(void* qkv, float* src, int src_stride, const int* positions, const float* cos_t,
                                  const float* sin_t, int rot_dim, int n_tokens, int nq, int nkv, int hd, int row_stride,
                                  void* kcache, void* vcache, const int* slot_mapping, int page_size,
                                  long long page_stride, long long head_stride, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0, "rope_kv_write: empty input");
  TLLM_REQUIRE(hd > 0 && hd % 2 == 0, "rope_kv_write: head size %d must be even", hd);
  TLLM_REQUIRE(rot_dim == 0 || (cos_t && sin_t), "rope_kv_write: rotary size %d without tables", rot_dim);
  TLLM_REQUIRE(rot_dim == 0 || rot_dim == hd, "rope_kv_write: partial rotary (%d of %d dims) is not built", rot_dim, hd);
  TLLM_REQUIRE(!slot_mapping || (kcache && vcache && page_size > 0), "rope_kv_write: a slot mapping needs cache pointers and a page size");
  const int work = (nq + nkv) * hd / 2;
  const int threads = work >= 512 ? 256 : 128;
  cudaStream_t s = (cudaStream_t)stream;
  const float* c = rot_dim ? cos_t : nullptr;
  const float* sn = rot_dim ? sin_t : nullptr;
  const int esz = dtype == TLLM_F32 ? 4 : 2;
  const bool vec = hd % 16 == 0 && ((uintptr_t)qkv % 16) == 0 && ((long long)row_stride * esz) % 16 == 0 &&
                   (!src || (((uintptr_t)src % 16) == 0 && src_stride % 4 == 0)) &&
                   (!slot_mapping || (((uintptr_t)kcache % 16) == 0 && ((uintptr_t)vcache % 16) == 0 &&
                                      (page_stride * esz) % 16 == 0 && (head_stride * esz) % 16 == 0)) &&
                   (!c || (((uintptr_t)c % 16) == 0 && ((uintptr_t)sn % 16) == 0));
  if (vec) {
    const int items = (nq + nkv) * (hd / 16);
    const int vthreads = items >= 256 ? 256 : 128;
    // few tokens: up to four CTAs per token, so that no thread walks its items one after the other
    const int parts = n_tokens <= 256 ? std::min(4, (items + vthreads - 1) / vthreads) : 1;
    const dim3 vgrid((unsigned)n_tokens, (unsigned)parts);
    if (dtype == TLLM_F32)
      TLLM_LAUNCH("rope_kv_write", rope_kv_write_vec_kernel<float>, vgrid, vthreads, 0, s, (float*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, page_stride, head_stride);
    else if (dtype == TLLM_BF16)
      TLLM_LAUNCH("rope_kv_write", rope_kv_write_vec_kernel<__nv_bfloat16>, vgrid, vthreads, 0, s, (__nv_bfloat16*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, page_stride, head_stride);
    else
      TLLM_FAIL(TLLM_ERR_ARG, "rope_kv_write: unknown dtype code %d", dtype);
    return TLLM_OK;
  }
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("rope_kv_write", rope_kv_write_kernel<float>, n_tokens, threads, 0, s, (float*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (float*)kcache, (float*)vcache, slot_mapping, page_size, page_stride, head_stride);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("rope_kv_write", rope_kv_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (__nv_bfloat16*)qkv, src, src_stride, positions, c, sn, n_tokens, nq, nkv, hd, row_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slot_mapping, page_size, page_stride, head_stride);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "rope_kv_write: unknown dtype code %d", dtype);
  return TLLM_OK;
}
