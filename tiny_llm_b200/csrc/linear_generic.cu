// C[M,N] = A[M,K] . W[N,K]^T on the CUDA cores with 32-bit accumulation (FFMA only, no tensor-core
// mode): the product of the true 32-bit path, and the fallback of the bfloat16 path for sizes the
// tensor-core kernels refuse.  Any M, N, K.  Every output element is ONE chain of fmaf over k in
// ascending order starting from zero, whatever M is and whichever of the two kernels below computes it,
// so a row's result does not depend on its batch, to the bit.
//   linear_generic_kernel: 64 x 64 tiles, 4 x 4 outputs per thread (any sizes and both dtypes);
//   linear_large_kernel: float32, 128 x 128 tiles, 8 x 8 outputs per thread (products of at least 128 x 128);
//   linear_skinny_kernel: float32, at most 16 rows (decoded tokens): a CTA takes 8 or 16 weight rows and
//     streams them through shared memory in chunks of 128 k (cp.async, three stages), one thread per
//     output element.  With so few rows the 64-row tile left 32 CTAs to stream a matrix that 148 SMs could
//     pull, each with one load in flight per thread.
// Reference counterpart: tiny_llm/ops/cuda/gemm.cu:67-106 (64x256 tile, 8x8 outputs per thread).
#include <cstdint>

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

// ---------------------------------------------------------------- many rows: 128 x 128 tiles, 8 x 8 outputs per thread
// The same chains of fmaf (k ascending from zero for every output element), with an eighth of the shared-memory reads
// per fmaf of the 64 x 64 kernel: 16-byte global loads of the next 16-wide slice of k into registers while the current
// one is multiplied, shared memory transposed to [k][row] so that a thread's eight rows (and eight columns) are two
// 16-byte reads.  Taken for products of at least 128 x 128 whose rows start on 16 bytes; float32 only.
constexpr int LBM = 128, LBN = 128, LBK = 16, LTHREADS = 256;

template <int MODE>
__global__ void __launch_bounds__(LTHREADS)
linear_large_kernel(const float* __restrict__ a, const float* __restrict__ w, float* __restrict__ out,
                    int m, int n, int k, int lda, int ldo) {
  __shared__ __align__(16) float as[2][LBK][LBM + 4];
  __shared__ __align__(16) float ws[2][LBK][LBN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;          // this thread's columns tx * 4 + {0..3} and 64 + tx * 4 + {0..3}; rows likewise
  const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
  // loader: thread -> (row lr of the tile, k quad lq); two rows per operand (lr and lr + 64)
  const int lr = tid / 4, lq = (tid % 4) * 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  float4 ra[2], rw[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gm = m0 + lr + 64 * h, gn = n0 + lr + 64 * h, kk = k0 + lq;
      ra[h] = (gm < m && kk < k) ? *reinterpret_cast<const float4*>(a + (size_t)gm * lda + kk) : make_float4(0.f, 0.f, 0.f, 0.f);
      rw[h] = (gn < n && kk < k) ? *reinterpret_cast<const float4*>(w + (size_t)gn * k + kk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lr + 64 * h;
      as[buf][lq + 0][r] = ra[h].x; as[buf][lq + 1][r] = ra[h].y; as[buf][lq + 2][r] = ra[h].z; as[buf][lq + 3][r] = ra[h].w;
      ws[buf][lq + 0][r] = rw[h].x; ws[buf][lq + 1][r] = rw[h].y; ws[buf][lq + 2][r] = rw[h].z; ws[buf][lq + 3][r] = rw[h].w;
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < k; k0 += LBK) {
    const bool more = k0 + LBK < k;
    if (more) fetch(k0 + LBK);
#pragma unroll
    for (int p = 0; p < LBK; ++p) {
      const float4 a0 = *reinterpret_cast<const float4*>(&as[buf][p][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&as[buf][p][64 + ty * 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&ws[buf][p][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&ws[buf][p][64 + tx * 4]);
      const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= n) continue;
      const size_t o = (size_t)gm * ldo + gn;
      if (MODE == OUT_ACC) out[o] += acc[i][j];
      else out[o] = acc[i][j];
    }
  }
}

static int launch_large(const float* a, const float* w, float* out, int m, int n, int k, int lda, int ldo, int mode, cudaStream_t s) {
  dim3 grid((n + LBN - 1) / LBN, (m + LBM - 1) / LBM);
  if (mode == OUT_ACC)
    TLLM_LAUNCH("linear_large", linear_large_kernel<OUT_ACC>, grid, LTHREADS, 0, s, a, w, out, m, n, k, lda, ldo);
  else
    TLLM_LAUNCH("linear_large", linear_large_kernel<OUT_F32>, grid, LTHREADS, 0, s, a, w, out, m, n, k, lda, ldo);
  return TLLM_OK;
}

// ---------------------------------------------------------------- at most 16 rows, float32
constexpr int SK_KC = 128, SK_LD = SK_KC + 4, SK_STAGES = 3, SK_THREADS = 128;

__device__ __forceinline__ void sk_cp16(float* dst, const float* src, bool ok) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = ok ? 16 : 0;   // 0: the 16 bytes are filled with zeros, which leave a chain of fmaf as it is
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
template <int R, int MODE>   // R rows of A per CTA (1, 2, 4, 8 or 16); BNS weight rows: R x BNS = at most 128 threads compute
__global__ void __launch_bounds__(SK_THREADS)
linear_skinny_kernel(const float* __restrict__ a, const float* __restrict__ w, float* __restrict__ out,
                     int m, int n, int k, int lda, int ldo) {
  constexpr int BNS = R == 16 ? 8 : 16;
  extern __shared__ __align__(16) uint8_t sk_smem[];
  float (*w_s)[BNS][SK_LD] = reinterpret_cast<float (*)[BNS][SK_LD]>(sk_smem);
  float (*a_s)[R][SK_LD] = reinterpret_cast<float (*)[R][SK_LD]>(sk_smem + sizeof(float) * SK_STAGES * BNS * SK_LD);
  pdl_trigger();
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BNS, m0 = blockIdx.y * R;
  const int chunks = (k + SK_KC - 1) / SK_KC;
  auto load_w = [&](int chunk, int stage) {
    const int k0 = chunk * SK_KC;
    for (int idx = tid; idx < BNS * (SK_KC / 4); idx += SK_THREADS) {
      const int row = idx / (SK_KC / 4), kk = (idx % (SK_KC / 4)) * 4;
      const bool ok = n0 + row < n && k0 + kk < k;   // k is a multiple of 4
      sk_cp16(&w_s[stage][row][kk], ok ? w + (size_t)(n0 + row) * k + k0 + kk : w, ok);
    }
  };
  auto load_a = [&](int chunk, int stage) {
    const int k0 = chunk * SK_KC;
    for (int idx = tid; idx < R * (SK_KC / 4); idx += SK_THREADS) {
      const int row = idx / (SK_KC / 4), kk = (idx % (SK_KC / 4)) * 4;
      const bool ok = m0 + row < m && k0 + kk < k;
      sk_cp16(&a_s[stage][row][kk], ok ? a + (size_t)(m0 + row) * lda + k0 + kk : a, ok);
    }
  };
  // the weights depend on no earlier kernel: their first chunks are on the way before the wait
  for (int st = 0; st < SK_STAGES - 1; ++st)
    if (st < chunks) load_w(st, st);
  pdl_wait();
  for (int st = 0; st < SK_STAGES - 1; ++st) {
    if (st < chunks) load_a(st, st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const bool computes = tid < R * BNS;
  const int r = tid / BNS, c = tid % BNS;
  float acc = 0.f;
  for (int i = 0; i < chunks; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(SK_STAGES - 2) : "memory");
    __syncthreads();   // chunk i has landed for every thread, and everyone has left chunk i - 1, whose stage is refilled now
    const int nxt = i + SK_STAGES - 1;
    if (nxt < chunks) { load_w(nxt, nxt % SK_STAGES); load_a(nxt, nxt % SK_STAGES); }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (computes) {
      const float* ar = a_s[i % SK_STAGES][r];
      const float* wr = w_s[i % SK_STAGES][c];
#pragma unroll 8
      for (int kk = 0; kk < SK_KC; kk += 4) {
        const float4 av = *reinterpret_cast<const float4*>(ar + kk);
        const float4 wv = *reinterpret_cast<const float4*>(wr + kk);
        acc = fmaf(av.x, wv.x, acc);
        acc = fmaf(av.y, wv.y, acc);
        acc = fmaf(av.z, wv.z, acc);
        acc = fmaf(av.w, wv.w, acc);
      }
    }
  }
  const int gm = m0 + r, gn = n0 + c;
  if (computes && gm < m && gn < n) {
    const size_t o = (size_t)gm * ldo + gn;
    if (MODE == OUT_ACC) out[o] += acc;
    else out[o] = acc;
  }
}

template <int R>
int launch_skinny(const float* a, const float* w, float* out, int m, int n, int k, int lda, int ldo, int mode, cudaStream_t s) {
  constexpr int BNS = R == 16 ? 8 : 16;
  constexpr int SMEM = (int)sizeof(float) * SK_STAGES * (BNS + R) * SK_LD;   // at most 38 KB
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<R, OUT_ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_skinny_kernel<R, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "linear_skinny: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((n + BNS - 1) / BNS, (m + R - 1) / R);
  if (mode == OUT_ACC)
    TLLM_LAUNCH("linear_skinny", (linear_skinny_kernel<R, OUT_ACC>), grid, SK_THREADS, SMEM, s, a, w, out, m, n, k, lda, ldo);
  else
    TLLM_LAUNCH("linear_skinny", (linear_skinny_kernel<R, OUT_F32>), grid, SK_THREADS, SMEM, s, a, w, out, m, n, k, lda, ldo);
  return TLLM_OK;
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

// skinny: 0 keeps the 64 x 64 tile kernel for every size (tests compare it with the two others, which must agree with it to the bit)
extern "C" int tllm_linear_generic(const void* a, const void* w, void* out, int m, int n, int k, int lda, int ldo,
                                   int dtype, int mode, int skinny, void* stream) {
  TLLM_REQUIRE(m > 0 && n > 0 && k > 0, "linear: empty product %d x %d x %d", m, n, k);
  TLLM_REQUIRE(lda >= k && ldo >= n, "linear: row strides %d, %d are shorter than the rows %d, %d", lda, ldo, k, n);
  TLLM_REQUIRE((m + tllm::BM - 1) / tllm::BM <= 65535, "linear: %d rows exceed the grid", m);
  if (dtype == TLLM_F32 && m <= 16 && skinny != 0 && k % 4 == 0 && lda % 4 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
      (mode == tllm::OUT_SAME || mode == tllm::OUT_F32 || mode == tllm::OUT_ACC)) {
    const float* af = (const float*)a;
    const float* wf = (const float*)w;
    float* of = (float*)out;
    cudaStream_t s = (cudaStream_t)stream;
    if (m <= 1) return tllm::launch_skinny<1>(af, wf, of, m, n, k, lda, ldo, mode, s);
    if (m <= 2) return tllm::launch_skinny<2>(af, wf, of, m, n, k, lda, ldo, mode, s);
    if (m <= 4) return tllm::launch_skinny<4>(af, wf, of, m, n, k, lda, ldo, mode, s);
    if (m <= 8) return tllm::launch_skinny<8>(af, wf, of, m, n, k, lda, ldo, mode, s);
    return tllm::launch_skinny<16>(af, wf, of, m, n, k, lda, ldo, mode, s);
  }
  if (dtype == TLLM_F32 && skinny != 0 && m >= 128 && n >= 128 && k % 4 == 0 && lda % 4 == 0 && ((uintptr_t)a % 16) == 0 &&
      ((uintptr_t)w % 16) == 0 && (m + tllm::LBM - 1) / tllm::LBM <= 65535)
    return tllm::launch_large((const float*)a, (const float*)w, (float*)out, m, n, k, lda, ldo, mode, (cudaStream_t)stream);
  if (dtype == TLLM_F32) return tllm::launch<float>(a, w, out, m, n, k, lda, ldo, mode, (cudaStream_t)stream);
  if (dtype == TLLM_BF16) return tllm::launch<__nv_bfloat16>(a, w, out, m, n, k, lda, ldo, mode, (cudaStream_t)stream);
  TLLM_FAIL(TLLM_ERR_ARG, "linear: unknown dtype code %d", dtype);
}
