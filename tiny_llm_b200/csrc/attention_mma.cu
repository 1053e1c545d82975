// bfloat16 attention of the step's queries over the paged cache on the tensor cores, for prefill
// portions and decoded tokens alike, compiled for one head size (-DTLLM_HEAD_DIM=...).
//
// A CTA serves one (request, key/value head, slice of keys) and a tile of "rows"; a row is a
// (new token, query head of the group) pair, so the G = heads / kv_heads query heads that share a
// key/value head also share every K/V tile the CTA loads.  Two kernels are built.  For portions of
// prompts, four warps own 16 rows each of a 64-row tile and walk the keys together.  For decoded
// tokens (at most 16 rows per request and key/value head) the four warps share the 16 rows and
// split every 64-key tile between them, 16 keys each, with a running softmax of their own that is
// merged through shared memory at the end: no warp computes for rows that do not exist.  Keys and
// values of a 64-key tile are gathered from their pages into shared memory with cp.async, one page
// lookup per row, several stages deep; S = Q K^T and O += P V run on mma.sync.m16n8k16 (bfloat16 in, 32-bit accumulate); the
// running softmax (max, sum, rescale) is kept in 32-bit registers with exp2 on scores scaled by
// log2(e)/sqrt(hd)-style factors; P is rounded to bfloat16 only as the operand of the P V product.
//
// Visibility is one rule: key j is visible to the row of a token at position p iff j <= p and,
// with a window w, j > p - w.  With `splits` > 1 the keys of a request are cut into slices of whole
// tiles, each CTA writes an unnormalised partial (o, max, sum) per row to scratch, and
// attention_combine merges them; with one split the result is written directly.
//
// Reference counterpart: tiny_llm/ops/cuda/flash_attention.cu:338-442 (32-bit SIMT, one lane per
// key, 64-key tiles, chunk-local causal mask).
#include "attention_tiles.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

template <int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
attention_mma_kernel(const AttnParams p) {
  constexpr int BM = WARPS * 16;   // rows per CTA
  static_assert(WARPS == 4, "the tile loader gives one row of keys or values to each of 128 threads");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* k_s = q_s + BM * LDS;                 // STAGES tiles
  __nv_bfloat16* v_s = k_s + STAGES * BN * LDS;        // STAGES tiles
  pdl_trigger();
  pdl_wait();

  // CTAs start in the order of blockIdx.x.  The tiles of the latest tokens see the most keys, so the
  // order is: the last tile of every request and key/value head, then the tiles before them, and so
  // on; the short ones fill the gaps at the end instead of the long ones trailing behind.
  const int kvh = blockIdx.x % p.nkv;
  const int req = (blockIdx.x / p.nkv) % p.n_requests;
  const int tile = p.tiles_per_req - 1 - blockIdx.x / (p.nkv * p.n_requests);
  const int split = blockIdx.z;
  const int group = p.nq / p.nkv;
  const int tok0 = p.cu_q[req];
  const int q_len = p.cu_q[req + 1] - tok0;
  const int rows_total = q_len * group;
  const int row0 = tile * BM;
  if (row0 >= rows_total) return;
  const int start = p.q_start[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int* table = p.block_table + (size_t)req * p.max_blocks;

  // keys this tile of rows can see at all, then this CTA's slice of them (whole 64-key tiles)
  const int tok_lo = row0 / group;
  const int tok_hi = min(q_len - 1, (row0 + BM - 1) / group);
  const int key_hi = start + tok_hi;
  const int key_lo = p.window > 0 ? max(0, start + tok_lo - p.window + 1) : 0;
  const int first_tile = key_lo / BN, last_tile = key_hi / BN;
  const int n_tiles = last_tile - first_tile + 1;
  const int per_split = (n_tiles + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * per_split;
  const int t_end = min(last_tile + 1, t_begin + per_split);   // exclusive
  int* page_slots = reinterpret_cast<int*>(v_s + STAGES * BN * LDS);
  const PageLookup pages = stage_pages(table, page_slots, t_begin * BN, t_end * BN, p.page_size, p.max_blocks, threadIdx.x, WARPS * 32);
  __syncthreads();

  // ---- Q tile: row r -> token r / group, head kvh * group + r % group
  for (int idx = threadIdx.x; idx < BM * CHUNKS; idx += WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int row = row0 + r;
    const bool ok = row < rows_total;
    const __nv_bfloat16* src = p.q;
    if (ok) src = p.q + (size_t)(tok0 + row / group) * p.q_row_stride + (size_t)(kvh * group + row % group) * HD + c * 8;
    cp_async16(q_s + r * LDS + c * 8, src, ok);
  }
  cp_async_commit();
  // prologue: the first STAGES - 1 tiles are requested; every stage is one commit group, empty or not
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (t_begin + st < t_end)
      load_kv_rows(k_s + st * BN * LDS, v_s + st * BN * LDS, pages, (t_begin + st) * BN, key_lo, key_hi, kvh, p, threadIdx.x);
    cp_async_commit();
  }

  // per-thread rows: g and g + 8 of the warp's 16
  const int r_a = row0 + warp * 16 + g, r_b = r_a + 8;
  const int pos_a = start + r_a / group, pos_b = start + r_b / group;
  const bool live_a = r_a < rows_total, live_b = r_b < rows_total;
  const int lo_a = p.window > 0 ? pos_a - p.window + 1 : 0, lo_b = p.window > 0 ? pos_b - p.window + 1 : 0;
  // what all 16 rows of this warp can see (the same for every lane); rows beyond the request's last
  // hold zero queries and are never stored, so they need no mask of their own
  const int wrow = row0 + warp * 16;
  const int warp_pos_min = start + wrow / group;
  const int warp_lo_max = p.window > 0 ? start + (wrow + 15) / group - p.window + 1 : 0;

  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int tix = t_begin; tix < t_end; ++tix) {
    const int stage = (tix - t_begin) % STAGES;
    const __nv_bfloat16* kt = k_s + stage * BN * LDS;
    const __nv_bfloat16* vt = v_s + stage * BN * LDS;
    cp_async_wait<STAGES - 2>();   // this tile (and the queries) have landed
    __syncthreads();               // ... for every thread, and the stage read last iteration is free
    {
      const int nxt = tix + STAGES - 1;
      if (nxt < t_end) {
        const int ns = (nxt - t_begin) % STAGES;
        load_kv_rows(k_s + ns * BN * LDS, v_s + ns * BN * LDS, pages, nxt * BN, key_lo, key_hi, kvh, p, threadIdx.x);
      }
      cp_async_commit();
    }

    // ---- S = Q K^T for this warp's 16 rows x 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int k0 = 0; k0 < HD; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (warp * 16 + (lane & 15)) * LDS + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n0 = 0; n0 < BN; n0 += 16) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (n0 + (lane & 7) + (lane >> 4) * 8) * LDS + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n0 / 8], a, b[0], b[1]);
        mma_bf16(s[n0 / 8 + 1], a, b[2], b[3]);
      }
    }

    // ---- mask, running softmax in 32-bit.  Scores stay raw; the scale (times log2 e) is folded into
    // the exponent: p = 2^(s * c - m * c).  A tile that every row of the warp sees whole skips the mask.
    const int j_base = tix * BN;
    const float c = p.scale_log2;
    if (!(j_base + BN - 1 <= warp_pos_min && j_base >= warp_lo_max)) {
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j_base + i * 8 + t4 * 2 + e;
          if (!(live_a && j <= pos_a && j >= lo_a)) s[i][e] = -CUDART_INF_F;
          if (!(live_b && j <= pos_b && j >= lo_b)) s[i][2 + e] = -CUDART_INF_F;
        }
      }
    }
    float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      mx_a = fmaxf(mx_a, fmaxf(s[i][0], s[i][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[i][2], s[i][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a * c), mn_b = fmaxf(m_b, mx_b * c);   // running maxima in scaled units
    const float ms_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, ms_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
    const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);   // 0 while nothing was seen
    m_a = mn_a; m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t pfrag[BN / 16][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      const float p0 = ex2(fmaf(s[i][0], c, -ms_a)), p1 = ex2(fmaf(s[i][1], c, -ms_a));
      const float p2 = ex2(fmaf(s[i][2], c, -ms_b)), p3 = ex2(fmaf(s[i][3], c, -ms_b));
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      // accumulator layout of two adjacent 8-key tiles = A-operand layout of one 16-key step
      pfrag[i / 2][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
      pfrag[i / 2][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;   // per-thread partial sums; reduced across the quad at the end
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int d0 = 0; d0 < HD; d0 += 16) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + d0 + (lane >> 4) * 8);
        mma_bf16(o[d0 / 8], pfrag[kk], b[0], b[1]);
        mma_bf16(o[d0 / 8 + 1], pfrag[kk], b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

  // ---- write: rows -> (token, head)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? r_b : r_a;
    if (row >= rows_total) continue;
    const float l = half ? l_b : l_a, m = half ? m_b : m_a;
    const size_t th = (size_t)(tok0 + row / group) * p.nq + (size_t)(kvh * group + row % group);
    if (p.splits == 1) {
      const float inv = 1.f / l;
      __nv_bfloat16* dst = p.out + th * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = pack_bf16(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
    } else {
      float* dst = p.part_o + (th * p.splits + split) * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + t4 * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      if (t4 == 0) {
        p.part_ml[(th * p.splits + split) * 2] = m;
        p.part_ml[(th * p.splits + split) * 2 + 1] = l;
      }
    }
  }
}

// ---------------------------------------------------------------- decoded tokens
template <int STAGES>
__global__ void __launch_bounds__(128)
attention_decode_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  pdl_trigger();
  attention_decode_item<STAGES>(p, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, smem_raw, [] { __syncthreads(); },
                                [] { pdl_wait(); });
}

// A launch whose grid.z CTAs of every (x, y) form one thread-block cluster.
template <typename Kernel>
static cudaError_t launch_z_clusters(Kernel kernel, dim3 grid, int smem, cudaStream_t s, const AttnParams& p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = grid.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// Decoded tokens over short slices (at most four tiles each): one warp per tile.
constexpr int WIDE_SMEM = (16 + 4 * 2 * BN) * LDS * 2 + TABLE_SLOTS * 4;
template <bool CLUSTER>
__global__ void __launch_bounds__(128)
attention_decode_wide_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  pdl_trigger();
  // CLUSTER: launched with clusters of (1, 1, splits) on a grid whose z extent is `splits`: blockIdx.z is the rank
  attention_decode_item_wide<CLUSTER>(p, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, smem_raw, [] { pdl_wait(); });
}

// Merges the slices of every (token, head), one warp each.
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out, int splits, int rows) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row < rows) attention_combine_row(part_o, part_ml, out, splits, (size_t)row, threadIdx.x & 31);
}

}  // namespace tllm


using namespace tllm;

extern "C" int tllm_attention_head_dim() { return HD; }

// 1 if the kernel with one warp per tile can run at this head size: its per-warp buffers must leave room for two
// CTAs on an SM, and the merge buffers must fit them.
extern "C" int tllm_attention_mma_wide_fits() {
  return WIDE_SMEM <= 113 * 1024 && 5 * 16 * (HD + 2) * 4 <= 4 * 2 * BN * LDS * 2;
}

// Bytes of scratch (float32 partials) a call with these sizes needs; 0 when splits == 1.
extern "C" long long tllm_attention_mma_scratch_bytes(int n_tokens, int nq, int splits) {
  return splits <= 1 ? 0 : (long long)n_tokens * nq * splits * (HD + 2) * 4;
}

// Attention of the step's tokens over the paged cache (bfloat16).  `splits` > 1: the keys of decoded tokens in that many
// slices, merged from `scratch` by a kernel behind, unless `wide` has bit 1.  `wide` (decoded tokens only): bit 0 = one warp
// per 64-key tile (slices of at most four tiles, `max_kv_len` the longest context of the step), bit 1 = the 2 to 8 slices
// of a (request, key/value head) form a cluster that merges them itself (no scratch, no merging kernel).
extern "C" int tllm_attention_mma(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                  const int* block_table, int max_blocks, const int* cu_q, const int* q_start,
                                  void* out, int n_tokens, int n_requests, int max_q_len, int nq, int nkv, int hd,
                                  int page_size, long long page_stride, long long head_stride, float scale, int window,
                                  int splits, void* scratch, int wide, int max_kv_len, void* stream) {
  TLLM_REQUIRE(hd == HD, "attention_mma: built for head size %d, called with %d", HD, hd);
  TLLM_REQUIRE(n_tokens > 0 && n_requests > 0 && max_q_len > 0 && nq > 0 && nkv > 0 && nq % nkv == 0,
               "attention_mma: %d tokens, %d requests, %d heads, %d key/value heads", n_tokens, n_requests, nq, nkv);
  TLLM_REQUIRE(scale > 0.f, "attention_mma: the score scale must be positive (got %g)", (double)scale);
  TLLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && splits >= 1, "attention_mma: page size %d, %d blocks, window %d, %d splits", page_size, max_blocks, window, splits);
  TLLM_REQUIRE(((uintptr_t)q % 16) == 0 && (q_row_stride % 8) == 0 && ((uintptr_t)kcache % 16) == 0 && ((uintptr_t)vcache % 16) == 0 &&
               (page_stride % 8) == 0 && (head_stride % 8) == 0, "attention_mma: rows must be 16-byte aligned");
  TLLM_REQUIRE(splits == 1 || (wide & 2) || scratch != nullptr, "attention_mma: %d splits need scratch", splits);
  TLLM_REQUIRE(nkv <= 65535 && splits <= 65535, "attention_mma: grid too large");
  const int group = nq / nkv;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.kcache = (const __nv_bfloat16*)kcache; p.vcache = (const __nv_bfloat16*)vcache;
  p.block_table = block_table; p.cu_q = cu_q; p.q_start = q_start; p.out = (__nv_bfloat16*)out;
  p.part_o = (float*)scratch;
  p.part_ml = splits > 1 ? (float*)scratch + (size_t)n_tokens * nq * splits * HD : nullptr;
  p.page_stride = page_stride; p.head_stride = head_stride; p.q_row_stride = q_row_stride; p.max_blocks = max_blocks;
  p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window; p.splits = splits; p.n_requests = n_requests;
  p.scale_log2 = scale * 1.4426950408889634f;
  // decoded tokens (at most 16 rows per request and key/value head): one-warp CTAs, four stages
  const bool small = (long long)max_q_len * group <= 16;
  p.tiles_per_req = small ? 1 : (int)(((long long)max_q_len * group + 63) / 64);
  const long long gx = (long long)n_requests * p.tiles_per_req;
  TLLM_REQUIRE(gx <= 2147483647LL, "attention_mma: grid too large");
  cudaStream_t s = (cudaStream_t)stream;
  // wide, bit 0 (decoded tokens only): every slice has at most four tiles for the longest context of the step, and one
  // warp takes each (tllm_attention_mma_wide_fits says whether this head size leaves room for two such CTAs on an SM)
  const bool cluster = (wide & 2) != 0;   // bit 1: the slices of a (request, key/value head) merge inside a cluster
  if (cluster) TLLM_REQUIRE((wide & 1) && splits >= 2 && splits <= 8,
                            "attention_mma: a cluster merges the 2 to 8 slices of the kernel with one warp per tile (got %d)", splits);
  if (wide & 1) {
    TLLM_REQUIRE(small && tllm_attention_mma_wide_fits() && max_kv_len > 0 && ((max_kv_len + BN - 1) / BN + splits - 1) / splits <= 4,
                 "attention_mma: one warp per tile needs decoded tokens and slices of at most four tiles (%d keys in %d slices)",
                 max_kv_len, splits);
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_decode_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WIDE_SMEM);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WIDE_SMEM);
      if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_mma: cannot reserve %d bytes of shared memory: %s", WIDE_SMEM, cudaGetErrorString(e));
      configured = true;
    }
    if (cluster) {
      cudaError_t e = launch_z_clusters(attention_decode_wide_kernel<true>, dim3((unsigned)n_requests, nkv, splits), WIDE_SMEM, s, p);
      if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_decode_wide (cluster of %d): %s", splits, cudaGetErrorString(e));
      return TLLM_OK;
    }
    TLLM_LAUNCH("attention_decode_wide", attention_decode_wide_kernel<false>, dim3((unsigned)n_requests, nkv, splits), 128, WIDE_SMEM, s, p);
  } else if (small) {
    constexpr int ST = 3;
    // the merge buffers (4 x 16 x (HD + 2) floats) reuse the tile stages
    static_assert(4 * 16 * (HD + 2) * 4 <= ST * BN * LDS * 2, "merge buffers must fit the key stages");
    const int smem = (16 + 2 * ST * BN) * LDS * 2 + TABLE_SLOTS * 4;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      configured = true;
    }
    TLLM_LAUNCH("attention_decode", attention_decode_kernel<ST>, dim3((unsigned)n_requests, nkv, splits), 128, smem, s, p);
  } else {
    constexpr int ST = 2;
    const int smem = (64 + 2 * ST * BN) * LDS * 2 + TABLE_SLOTS * 4;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<4, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      configured = true;
    }
    TLLM_REQUIRE(gx * nkv <= 2147483647LL, "attention_mma: grid too large");
    TLLM_LAUNCH("attention_mma", (attention_mma_kernel<4, ST>), dim3((unsigned)(gx * nkv), 1, splits), 128, smem, s, p);
  }
  if (splits > 1)
    TLLM_LAUNCH("attention_combine", attention_combine_kernel, (unsigned)(((size_t)n_tokens * nq + 3) / 4), 128, 0, s,
                p.part_o, p.part_ml, p.out, splits, n_tokens * nq);
  return TLLM_OK;
}
