// C[M,N] = A[M,K] . W[N,K]^T on the CUDA cores with 32-bit accumulation (FFMA only, no tensor-core
// mode): the product of the true 32-bit path, and the fallback of the bfloat16 path for sizes the
// tensor-core kernels refuse.  Any M, N, K.  Every output element is a sum over k in ascending
// order of 16-wide slices, whatever M is, so a row's result does not depend on its batch.
// Reference counterpart: tiny_llm/ops/cuda/gemm.cu:67-106 (64x256 tile, 8x8 outputs per thread).
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

// out modes
constexpr int OUT_SAME = 0;   // store in the input dtype
constexpr int OUT_F32 = 1;    // store float32
constexpr int OUT_ACC = 2;    // out (float32) += product

template <typename T, int MODE>
__global__ void __launch_bounds__(THREADS)
linear_generic_kernel(const T* __restrict__ a, const T* __restrict__ w, void* __restrict__ out,
                      int m, int n, int k, int lda, int ldo) {
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lk = tid % BK, lr = tid / BK;  // loader: k index and first row; rows lr + 16 i
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k; k0 += BK) {
    const int kk = k0 + lk;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = lr + 16 * i;
      const int gm = m0 + r, gn = n0 + r;
      as[lk][r] = (gm < m && kk < k) ? to_f32(a[(size_t)gm * lda + kk]) : 0.f;
      ws[lk][r] = (gn < n && kk < k) ? to_f32(w[(size_t)gn * k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < BK; ++p) {
      const float4 av = *reinterpret_cast<const float4*>(&as[p][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&ws[p][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= n) continue;
      const size_t o = (size_t)gm * ldo + gn;
      if (MODE == OUT_SAME) reinterpret_cast<T*>(out)[o] = from_f32<T>(acc[i][j]);
      else if (MODE == OUT_F32) reinterpret_cast<float*>(out)[o] = acc[i][j];
      else reinterpret_cast<float*>(out)[o] += acc[i][j];
    }
  }
}

template <typename T>
int launch(const void* a, const void* w, void* out, int m, int n, int k, int lda, int ldo, int mode, cudaStream_t s) {
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  if (mode == OUT_SAME)
    TLLM_LAUNCH("linear_generic", (linear_generic_kernel<T, OUT_SAME>), grid, THREADS, 0, s, (const T*)a, (const T*)w, out, m, n, k, lda, ldo);
  else if (mode == OUT_F32)
    TLLM_LAUNCH("linear_generic", (linear_generic_kernel<T, OUT_F32>), grid, THREADS, 0, s, (const T*)a, (const T*)w, out, m, n, k, lda, ldo);
  else if (mode == OUT_ACC)
    TLLM_LAUNCH("linear_generic", (linear_generic_kernel<T, OUT_ACC>), grid, THREADS, 0, s, (const T*)a, (const T*)w, out, m, n, k, lda, ldo);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "linear: unknown output mode %d", mode);
  return TLLM_OK;
}

}  // namespace tllm

extern "C" int tllm_linear_generic(const void* a, const void* w, void* out, int m, int n, int k, int lda, int ldo,
                                   int dtype, int mode, void* stream) {
  TLLM_REQUIRE(m > 0 && n > 0 && k > 0, "linear: empty product %d x %d x %d", m, n, k);
  TLLM_REQUIRE(lda >= k && ldo >= n, "linear: row strides %d, %d are shorter than the rows %d, %d", lda, ldo, k, n);
  TLLM_REQUIRE((m + tllm::BM - 1) / tllm::BM <= 65535, "linear: %d rows exceed the grid", m);
  if (dtype == TLLM_F32) return tllm::launch<float>(a, w, out, m, n, k, lda, ldo, mode, (cudaStream_t)stream);
  if (dtype == TLLM_BF16) return tllm::launch<__nv_bfloat16>(a, w, out, m, n, k, lda, ldo, mode, (cudaStream_t)stream);
  TLLM_FAIL(TLLM_ERR_ARG, "linear: unknown dtype code %d", dtype);
}
