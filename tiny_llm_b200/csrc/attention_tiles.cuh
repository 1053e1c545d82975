// Pieces of the bfloat16 paged attention that more than one kernel uses, compiled for one head size
// (-DTLLM_HEAD_DIM=...): the tile constants, the cp.async / ldmatrix / mma.sync wrappers, the
// gather of a 64-key tile from its pages, the work of one (request, key/value head, slice of keys)
// for decoded tokens as a device function of 128 threads, and the merge of the slices of one
// (token, head).  The stand-alone decode kernel runs the device function as one CTA; the fused decode
// step runs it on teams of four warps of a larger CTA, which is why the barrier is a parameter.
#pragma once
#include <math_constants.h>

#include "common.cuh"

#ifndef TLLM_HEAD_DIM
#error "compile with -DTLLM_HEAD_DIM=<multiple of 16 up to 256>"
#endif

namespace tllm {

constexpr int HD = TLLM_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int BN = 64;            // keys per tile
constexpr int LDS = HD + 8;       // shared-memory row stride in elements: +16 bytes keeps ldmatrix conflict-free
constexpr int CHUNKS = HD / 8;    // 16-byte chunks per row

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;   // 0: the destination is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
// The same copy with an L2 policy (keys and values are read once per step: they should not push the
// step's small, hot tensors out of L2).
__device__ __forceinline__ uint64_t l2_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void cp_async16_hint(void* dst, const void* src, bool pred, uint64_t policy) {
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one instruction; 2^(-inf) = 0
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct AttnParams {
  const __nv_bfloat16* q;        // rows of q_row_stride elements; queries first in each row
  const __nv_bfloat16* kcache;   // [pages, kv_heads, page_size, HD]
  const __nv_bfloat16* vcache;
  const int* block_table;        // [R, max_blocks]
  const int* cu_q;               // [R + 1]
  const int* q_start;            // [R]: position of the request's first token in this step
  __nv_bfloat16* out;            // [T, nq * HD]
  float* part_o;                 // [T * nq, splits, HD]   (splits > 1)
  float* part_ml;                // [T * nq, splits, 2]
  long long page_stride, head_stride;
  int q_row_stride, max_blocks, nq, nkv, page_size, window, tiles_per_req, splits, n_requests;
  float scale_log2;              // scale * log2(e)
};

// A tile is 128 rows, 64 keys then 64 values; warp w gathers rows [32 w, 32 w + 32).  Each lane looks
// up the page of one row; the copies are then issued so that consecutive lanes fetch consecutive
// 16-byte pieces of a row (whole 128-byte lines per instruction), the row's address coming from
// its lane by shuffle.
constexpr int TABLE_SLOTS = 512;   // block-table entries of a CTA's keys that are kept in shared memory

// Where a request's pages are: the entries for the keys a CTA walks are copied to shared memory once
// (they come with the step's tables, so before the wait for the kernel in front), because a lookup in
// global memory in front of every tile's copies is a round trip to L2 that the whole warp waits for.
struct PageLookup {
  const int* table;    // the request's row of the block table
  const int* staged;   // entries [first, first + count) of it, in shared memory
  int first, count, max_blocks;
  __device__ __forceinline__ int operator()(int block) const {
    if (block >= max_blocks) return -1;
    const int i = block - first;
    return i >= 0 && i < count ? staged[i] : table[block];
  }
};
// Copies the entries for keys [j_lo, j_hi) into `slots` (TABLE_SLOTS ints); the caller synchronises the threads.
__device__ __forceinline__ PageLookup stage_pages(const int* table, int* slots, int j_lo, int j_hi, int page_size,
                                                  int max_blocks, int tid, int threads) {
  PageLookup pl;
  pl.table = table; pl.staged = slots; pl.max_blocks = max_blocks;
  pl.first = max(0, j_lo) / page_size;
  const int last = min(max_blocks, (max(0, j_hi) + page_size - 1) / page_size);
  pl.count = max(0, min(TABLE_SLOTS, last - pl.first));
  for (int i = tid; i < pl.count; i += threads) slots[i] = table[pl.first + i];
  return pl;
}

__device__ __forceinline__ void load_kv_rows(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst, const PageLookup& pages, int j0,
                                             int j_begin, int j_end, int kvh, const AttnParams& p, int tid,
                                             bool read_once = false) {
  const int warp = tid >> 5, lane = tid & 31;
  const int row = warp * 32 + lane;            // 0..63 keys, 64..127 values
  const bool is_v = row >= BN;
  const int j = j0 + (row & (BN - 1));
  bool ok = j >= j_begin && j <= j_end;
  const int page = ok ? pages(j / p.page_size) : -1;
  ok = ok && page >= 0;
  const __nv_bfloat16* src = is_v ? p.vcache : p.kcache;
  if (ok) src += (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(j % p.page_size) * HD;
  __nv_bfloat16* dst = (warp < 2 ? k_dst : v_dst) + (warp & 1) * 32 * LDS;   // this warp's 32 rows
  const uint64_t once = l2_evict_first();
#pragma unroll
  for (int idx = lane; idx < 32 * CHUNKS; idx += 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, r);
    const int okr = __shfl_sync(0xffffffffu, (int)ok, r);
    // decoded tokens read every key once per step; the tiles of a prompt portion are shared by its CTAs through L2
    if (read_once) cp_async16_hint(dst + r * LDS + c * 8, reinterpret_cast<const __nv_bfloat16*>(a) + (okr ? c * 8 : 0), okr != 0, once);
    else cp_async16(dst + r * LDS + c * 8, reinterpret_cast<const __nv_bfloat16*>(a) + (okr ? c * 8 : 0), okr != 0);
  }
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// two floats at `ptr` of this CTA's shared memory, read from the CTA of rank `rank` in the cluster
__device__ __forceinline__ float2 ld_cluster_f32x2(const float* ptr, uint32_t rank) {
  uint32_t remote;
  float2 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(ptr)), "r"(rank));
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
  return v;
}


// The end of a decode work item whose key slices are the CTAs of one thread-block cluster (2 to 8 of them, the slice
// index being the rank): each has left its result in its own shared memory (`c_o` [16][HD] unnormalised, `c_ml` [16][2]
// maximum and sum), the cluster meets, and every CTA finishes a share of the output elements from all the peers'
// results over distributed shared memory: no partial results in global memory and no merging kernel after this one.
__device__ __forceinline__ void cluster_merge_and_write(const AttnParams& p, const float* c_o, const float* c_ml, int split,
                                                        int tid, int rows_total, int tok0, int group, int kvh) {
  cluster_sync_all();       // every slice's result lies in its CTA's shared memory
  for (int idx = split * 128 + tid; idx < rows_total * (HD / 2); idx += p.splits * 128) {
    const int r = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
    float2 ml[8], ov[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ml[j] = make_float2(-CUDART_INF_F, 0.f);
      ov[j] = make_float2(0.f, 0.f);
      if (j < p.splits) {
        ml[j] = ld_cluster_f32x2(c_ml + r * 2, (uint32_t)j);
        ov[j] = ld_cluster_f32x2(c_o + r * HD + d, (uint32_t)j);
      }
    }
    float m = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, ml[j].x);
    const float m_ref = m == -CUDART_INF_F ? 0.f : m;
    float l = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = exp2f(ml[j].x - m_ref);    // 0 for a slice that saw no key of the row
      l += f * ml[j].y;
      acc0 += f * ov[j].x;
      acc1 += f * ov[j].y;
    }
    const size_t th = (size_t)(tok0 + r / group) * p.nq + (size_t)(kvh * group + r % group);
    const float inv = 1.f / l;
    *reinterpret_cast<uint32_t*>(p.out + th * HD + d) = pack_bf16(acc0 * inv, acc1 * inv);
  }
  trace_mark(3);
  cluster_sync_all();       // no CTA leaves while a peer still reads its shared memory
}

// Decoded tokens: at most 16 rows (new tokens x query heads of the group) of one request and
// key/value head over one slice of its keys, by 128 threads (`tid` in [0, 128)) that share
// `smem_raw` ((16 + 2 STAGES 64) rows of LDS elements, then TABLE_SLOTS ints) and meet at `sync()`.  The four warps split
// every 64-key tile between them, 16 keys each, keep a running softmax of their own and merge them
// through shared memory at the end.  With p.splits == 1 the rows are normalised and written to
// p.out; else the unnormalised partial (o, max, sum) goes to p.part_o / p.part_ml.  The caller
// synchronises the 128 threads before the shared memory is used again.
//
// `dep()` is called once, before the first read of what the kernel before this one wrote (the step's
// queries, and the keys and values of the step's own tokens).  The request's older keys and values
// and the step's tables are older than that kernel: their tiles are asked for before `dep()`, so that
// under programmatic dependent launch they travel while the projection before attention still runs.
template <int STAGES, typename Sync, typename Dep>
__device__ __forceinline__ void attention_decode_item(const AttnParams& p, int req, int kvh, int split, int tid,
                                                      uint8_t* smem_raw, Sync sync, Dep dep) {
  static_assert(BN == 64, "one thread per key row and per value row of a tile");
  static_assert(4 * 16 * (HD + 2) * 4 <= STAGES * BN * LDS * 2, "merge buffers must fit the key stages");
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // 16 rows
  __nv_bfloat16* k_s = q_s + 16 * LDS;                               // STAGES tiles
  __nv_bfloat16* v_s = k_s + STAGES * BN * LDS;
  const int group = p.nq / p.nkv;
  const int tok0 = p.cu_q[req];
  const int q_len = p.cu_q[req + 1] - tok0;
  const int rows_total = q_len * group;        // <= 16 by the launch condition
  const int start = p.q_start[req];
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int* table = p.block_table + (size_t)req * p.max_blocks;

  const int key_hi = start + q_len - 1;
  const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int first_tile = key_lo / BN, last_tile = key_hi / BN;
  const int n_tiles = last_tile - first_tile + 1;
  const int per_split = (n_tiles + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * per_split;
  const int t_end = min(last_tile + 1, t_begin + per_split);
  int* page_slots = reinterpret_cast<int*>(v_s + STAGES * BN * LDS);
  const PageLookup pages = stage_pages(table, page_slots, t_begin * BN, t_end * BN, p.page_size, p.max_blocks, tid, 128);
  sync();

  // the first STAGES - 1 tiles: those that end before the step's first token are older than the step
  bool early[STAGES - 1];
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    early[st] = t_begin + st < t_end && (t_begin + st + 1) * BN <= start;
    if (early[st])
      load_kv_rows(k_s + st * BN * LDS, v_s + st * BN * LDS, pages, (t_begin + st) * BN, key_lo, key_hi, kvh, p, tid, true);
  }
  dep();
  for (int idx = tid; idx < 16 * CHUNKS; idx += 128) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < rows_total;
    const __nv_bfloat16* src = p.q;
    if (ok) src = p.q + (size_t)(tok0 + r / group) * p.q_row_stride + (size_t)(kvh * group + r % group) * HD + c * 8;
    cp_async16(q_s + r * LDS + c * 8, src, ok);
  }
  cp_async_commit();   // the queries and the early tiles
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (!early[st] && t_begin + st < t_end)
      load_kv_rows(k_s + st * BN * LDS, v_s + st * BN * LDS, pages, (t_begin + st) * BN, key_lo, key_hi, kvh, p, tid, true);
    cp_async_commit();
  }

  const int pos_a = start + g / group, pos_b = start + (g + 8) / group;
  const bool live_a = g < rows_total, live_b = g + 8 < rows_total;
  const int lo_a = p.window > 0 ? pos_a - p.window + 1 : 0, lo_b = p.window > 0 ? pos_b - p.window + 1 : 0;
  // what all rows can see: keys up to the first new token's position, from the last one's window on
  // (rows beyond the request's last hold zero queries and are never stored)
  const int lo_max = p.window > 0 ? start + q_len - 1 - p.window + 1 : 0;
  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  uint32_t qf[HD / 16][4];

  for (int tix = t_begin; tix < t_end; ++tix) {
    const int stage = (tix - t_begin) % STAGES;
    const __nv_bfloat16* kt = k_s + stage * BN * LDS + warp * 16 * LDS;   // this warp's 16 keys of the tile
    const __nv_bfloat16* vt = v_s + stage * BN * LDS + warp * 16 * LDS;
    cp_async_wait<STAGES - 2>();
    sync();
    {
      const int nxt = tix + STAGES - 1;
      if (nxt < t_end) {
        const int ns = (nxt - t_begin) % STAGES;
        load_kv_rows(k_s + ns * BN * LDS, v_s + ns * BN * LDS, pages, nxt * BN, key_lo, key_hi, kvh, p, tid, true);
      }
      cp_async_commit();
    }
    if (tix == t_begin) {
      trace_mark(0);   // the queries and the first tile are in shared memory
#pragma unroll
      for (int k0 = 0; k0 < HD; k0 += 16) ldmatrix_x4(qf[k0 / 16], q_s + (lane & 15) * LDS + k0 + (lane >> 4) * 8);
    }
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int k0 = 0; k0 < HD; k0 += 16) {
      uint32_t b[4];
      ldmatrix_x4(b, kt + ((lane & 7) + (lane >> 4) * 8) * LDS + k0 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], qf[k0 / 16], b[0], b[1]);
      mma_bf16(s[1], qf[k0 / 16], b[2], b[3]);
    }
    const int j_base = tix * BN + warp * 16;
    const float c = p.scale_log2;
    if (!(j_base + 15 <= start && j_base >= lo_max)) {   // else every row sees these 16 keys
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j_base + i * 8 + t4 * 2 + e;
          if (!(live_a && j <= pos_a && j >= lo_a)) s[i][e] = -CUDART_INF_F;
          if (!(live_b && j <= pos_b && j >= lo_b)) s[i][2 + e] = -CUDART_INF_F;
        }
      }
    }
    float mx_a = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    float mx_b = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a * c), mn_b = fmaxf(m_b, mx_b * c);
    const float ms_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, ms_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
    const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);
    m_a = mn_a; m_b = mn_b;
    uint32_t pf[4];
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float p0 = ex2(fmaf(s[i][0], c, -ms_a)), p1 = ex2(fmaf(s[i][1], c, -ms_a));
      const float p2 = ex2(fmaf(s[i][2], c, -ms_b)), p3 = ex2(fmaf(s[i][3], c, -ms_b));
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      pf[i * 2] = pack_bf16(p0, p1);
      pf[i * 2 + 1] = pack_bf16(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
#pragma unroll
    for (int d0 = 0; d0 < HD; d0 += 16) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + d0 + (lane >> 4) * 8);
      mma_bf16(o[d0 / 8], pf, b[0], b[1]);
      mma_bf16(o[d0 / 8 + 1], pf, b[2], b[3]);
    }
  }
  cp_async_wait<0>();
  trace_mark(1);       // the tiles of this slice are done
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

  // ---- merge the four warps' running softmaxes through shared memory (the tile buffers are free now)
  sync();
  float* o_sh = reinterpret_cast<float*>(k_s);        // [4 warps][16 rows][HD]
  float* ml_sh = o_sh + 4 * 16 * HD;                  // [4 warps][16 rows][2]
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    *reinterpret_cast<float2*>(o_sh + (warp * 16 + g) * HD + i * 8 + t4 * 2) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(o_sh + (warp * 16 + g + 8) * HD + i * 8 + t4 * 2) = make_float2(o[i][2], o[i][3]);
  }
  if (t4 == 0) {
    ml_sh[(warp * 16 + g) * 2] = m_a; ml_sh[(warp * 16 + g) * 2 + 1] = l_a;
    ml_sh[(warp * 16 + g + 8) * 2] = m_b; ml_sh[(warp * 16 + g + 8) * 2 + 1] = l_b;
  }
  sync();
  for (int idx = tid; idx < rows_total * (HD / 2); idx += 128) {
    const int r = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, ml_sh[(w * 16 + r) * 2]);
    const float m_ref = m == -CUDART_INF_F ? 0.f : m;
    float l = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(ml_sh[(w * 16 + r) * 2] - m_ref);   // 0 for a warp that saw no key of the row
      l += f * ml_sh[(w * 16 + r) * 2 + 1];
      const float2 ov = *reinterpret_cast<const float2*>(o_sh + (w * 16 + r) * HD + d);
      acc0 += f * ov.x;
      acc1 += f * ov.y;
    }
    const size_t th = (size_t)(tok0 + r / group) * p.nq + (size_t)(kvh * group + r % group);
    if (p.splits == 1) {
      const float inv = 1.f / l;
      *reinterpret_cast<uint32_t*>(p.out + th * HD + d) = pack_bf16(acc0 * inv, acc1 * inv);
    } else {
      *reinterpret_cast<float2*>(p.part_o + (th * p.splits + split) * HD + d) = make_float2(acc0, acc1);
      if (d == 0) {
        p.part_ml[(th * p.splits + split) * 2] = m;
        p.part_ml[(th * p.splits + split) * 2 + 1] = l;
      }
    }
  }
  trace_mark(2);       // merged and written
}

// One warp's share of a tile loader: the 64 key rows and 64 value rows of the tile at j0, gathered by the 32 lanes
// of ONE warp into its own buffers (four passes of 32 rows; within a pass consecutive lanes fetch consecutive
// 16-byte pieces of a row, the row's address coming from its lane by shuffle).
__device__ __forceinline__ void load_kv_rows_warp(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst, const PageLookup& pages, int j0,
                                                  int j_begin, int j_end, int kvh, const AttnParams& p, int lane) {
  const uint64_t once = l2_evict_first();
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const bool is_v = pass >= 2;
    const int j = j0 + (pass & 1) * 32 + lane;
    bool ok = j >= j_begin && j <= j_end;
    const int page = ok ? pages(j / p.page_size) : -1;
    ok = ok && page >= 0;
    const __nv_bfloat16* src = is_v ? p.vcache : p.kcache;
    if (ok) src += (long long)page * p.page_stride + (long long)kvh * p.head_stride + (long long)(j % p.page_size) * HD;
    __nv_bfloat16* dst = (is_v ? v_dst : k_dst) + (pass & 1) * 32 * LDS;
#pragma unroll
    for (int idx = lane; idx < 32 * CHUNKS; idx += 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, r);
      const int okr = __shfl_sync(0xffffffffu, (int)ok, r);
      cp_async16_hint(dst + r * LDS + c * 8, reinterpret_cast<const __nv_bfloat16*>(a) + (okr ? c * 8 : 0), okr != 0, once);
    }
  }
}

// Decoded tokens, short slices: the same work as attention_decode_item for a slice of at most four 64-key tiles, with
// ONE WARP PER TILE instead of four warps per tile.  Every warp gathers its own tile into buffers of its own (all
// copies of the slice are in flight at once; tiles older than the step before `dep()`), the block meets once when
// everything has landed, each warp runs S = Q K^T, the softmax and P V for 16 rows x 64 keys by itself, and the four
// results are merged through shared memory as before.  The walk over the tiles of a slice, one block barrier and one
// chain of dependent MMAs per tile, was what a slice's time consisted of; here that chain is one tile long.
// Shared memory: 16 query rows, then per warp 64 key rows and 64 value rows, then TABLE_SLOTS ints.
// CLUSTER: the slices of one (request, key/value head) are the CTAs of one thread-block cluster (2 to 8 of them, the
// slice index being the rank).  Each leaves its merged result in its own shared memory, the cluster meets, and every
// CTA finishes a share of the output elements from all the peers' results over distributed shared memory: no partial
// results in global memory and no merging kernel after this one.
template <bool CLUSTER, typename Dep>
__device__ __forceinline__ void attention_decode_item_wide(const AttnParams& p, int req, int kvh, int split, int tid,
                                                           uint8_t* smem_raw, Dep dep) {
  static_assert(BN == 64, "a warp owns a tile of 64 keys");
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // 16 rows
  __nv_bfloat16* kv_s = q_s + 16 * LDS;                              // [4 warps][64 key rows, 64 value rows]
  const int group = p.nq / p.nkv;
  const int tok0 = p.cu_q[req];
  const int q_len = p.cu_q[req + 1] - tok0;
  const int rows_total = q_len * group;        // <= 16 by the launch condition
  const int start = p.q_start[req];
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int* table = p.block_table + (size_t)req * p.max_blocks;

  const int key_hi = start + q_len - 1;
  const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int first_tile = key_lo / BN, last_tile = key_hi / BN;
  const int n_tiles = last_tile - first_tile + 1;
  const int per_split = (n_tiles + p.splits - 1) / p.splits;     // <= 4 by the launch condition
  const int t_begin = first_tile + split * per_split;
  const int t_end = min(last_tile + 1, t_begin + per_split);
  int* page_slots = reinterpret_cast<int*>(kv_s + 4 * 2 * BN * LDS);
  const PageLookup pages = stage_pages(table, page_slots, t_begin * BN, t_end * BN, p.page_size, p.max_blocks, tid, 128);
  __syncthreads();

  const int tix = t_begin + warp;                         // this warp's tile
  const bool has_tile = tix < t_end;
  __nv_bfloat16* kt = kv_s + warp * 2 * BN * LDS;
  __nv_bfloat16* vt = kt + BN * LDS;
  const bool early = has_tile && (tix + 1) * BN <= start;  // the tile ends before the step's first token: older than the step
  if (early) load_kv_rows_warp(kt, vt, pages, tix * BN, key_lo, key_hi, kvh, p, lane);
  dep();
  for (int idx = tid; idx < 16 * CHUNKS; idx += 128) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < rows_total;
    const __nv_bfloat16* src = p.q;
    if (ok) src = p.q + (size_t)(tok0 + r / group) * p.q_row_stride + (size_t)(kvh * group + r % group) * HD + c * 8;
    cp_async16(q_s + r * LDS + c * 8, src, ok);
  }
  if (has_tile && !early) load_kv_rows_warp(kt, vt, pages, tix * BN, key_lo, key_hi, kvh, p, lane);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();     // the queries and every warp's tile have landed
  trace_mark(0);

  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  if (has_tile) {
    const int pos_a = start + g / group, pos_b = start + (g + 8) / group;
    const bool live_a = g < rows_total, live_b = g + 8 < rows_total;
    const int lo_a = p.window > 0 ? pos_a - p.window + 1 : 0, lo_b = p.window > 0 ? pos_b - p.window + 1 : 0;
    const int lo_max = p.window > 0 ? start + q_len - 1 - p.window + 1 : 0;
    // ---- S = Q K^T for the 16 rows x this warp's 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int k0 = 0; k0 < HD; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (lane & 15) * LDS + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n0 = 0; n0 < BN; n0 += 16) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (n0 + (lane & 7) + (lane >> 4) * 8) * LDS + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n0 / 8], a, b[0], b[1]);
        mma_bf16(s[n0 / 8 + 1], a, b[2], b[3]);
      }
    }
    const int j_base = tix * BN;
    const float c = p.scale_log2;
    if (!(j_base + BN - 1 <= start && j_base >= lo_max)) {   // else every row sees these 64 keys
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
    m_a = mx_a * c; m_b = mx_b * c;                                           // in scaled (log2) units
    const float ms_a = m_a == -CUDART_INF_F ? 0.f : m_a, ms_b = m_b == -CUDART_INF_F ? 0.f : m_b;
    uint32_t pfrag[BN / 16][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      const float p0 = ex2(fmaf(s[i][0], c, -ms_a)), p1 = ex2(fmaf(s[i][1], c, -ms_a));
      const float p2 = ex2(fmaf(s[i][2], c, -ms_b)), p3 = ex2(fmaf(s[i][3], c, -ms_b));
      l_a += p0 + p1;
      l_b += p2 + p3;
      pfrag[i / 2][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
      pfrag[i / 2][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // ---- O = P V
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
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  }
  trace_mark(1);       // the tiles of this slice are done

  // ---- merge the four warps' results through shared memory (every warp has finished reading its tile)
  __syncthreads();
  float* o_sh = reinterpret_cast<float*>(kv_s);       // [4 warps][16 rows][HD]
  float* ml_sh = o_sh + 4 * 16 * HD;                  // [4 warps][16 rows][2]
  float* c_o = ml_sh + 4 * 16 * 2;                    // [16 rows][HD]: this CTA's result, for the cluster
  float* c_ml = c_o + 16 * HD;                        // [16 rows][2]
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    *reinterpret_cast<float2*>(o_sh + (warp * 16 + g) * HD + i * 8 + t4 * 2) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(o_sh + (warp * 16 + g + 8) * HD + i * 8 + t4 * 2) = make_float2(o[i][2], o[i][3]);
  }
  if (t4 == 0) {
    ml_sh[(warp * 16 + g) * 2] = m_a; ml_sh[(warp * 16 + g) * 2 + 1] = l_a;
    ml_sh[(warp * 16 + g + 8) * 2] = m_b; ml_sh[(warp * 16 + g + 8) * 2 + 1] = l_b;
  }
  __syncthreads();
  for (int idx = tid; idx < rows_total * (HD / 2); idx += 128) {
    const int r = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, ml_sh[(w * 16 + r) * 2]);
    const float m_ref = m == -CUDART_INF_F ? 0.f : m;
    float l = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(ml_sh[(w * 16 + r) * 2] - m_ref);   // 0 for a warp that saw no key of the row
      l += f * ml_sh[(w * 16 + r) * 2 + 1];
      const float2 ov = *reinterpret_cast<const float2*>(o_sh + (w * 16 + r) * HD + d);
      acc0 += f * ov.x;
      acc1 += f * ov.y;
    }
    const size_t th = (size_t)(tok0 + r / group) * p.nq + (size_t)(kvh * group + r % group);
    if (CLUSTER) {
      *reinterpret_cast<float2*>(c_o + r * HD + d) = make_float2(acc0, acc1);
      if (d == 0) *reinterpret_cast<float2*>(c_ml + r * 2) = make_float2(m, l);
    } else if (p.splits == 1) {
      const float inv = 1.f / l;
      *reinterpret_cast<uint32_t*>(p.out + th * HD + d) = pack_bf16(acc0 * inv, acc1 * inv);
    } else {
      *reinterpret_cast<float2*>(p.part_o + (th * p.splits + split) * HD + d) = make_float2(acc0, acc1);
      if (d == 0) {
        p.part_ml[(th * p.splits + split) * 2] = m;
        p.part_ml[(th * p.splits + split) * 2 + 1] = l;
      }
    }
  }
  trace_mark(2);       // merged and written
  if (CLUSTER) cluster_merge_and_write(p, c_o, c_ml, split, tid, rows_total, tok0, group, kvh);
}

// Merges the slices of one (token, head) `th` by one warp: out = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s.
// Lane s reads the maximum and sum of slices s, s + 32, ...; the weights 2^(m_s - m) go round by
// shuffle while every lane gathers its elements of o, so no load waits for another.  A slice that
// saw no key of the row has m_s = -inf and l_s = 0 and drops out.  The partials are read past L1:
// inside a persistent kernel other SMs wrote them, and the same addresses held another layer's
// partials a moment ago.  All 32 lanes must call this together.
__device__ __forceinline__ void attention_combine_row(const float* part_o, const float* part_ml, __nv_bfloat16* out,
                                                      int splits, size_t th, int lane) {
  const size_t base = th * splits;
  float m = -CUDART_INF_F;
  for (int s0 = 0; s0 < splits; s0 += 32)
    if (s0 + lane < splits) m = fmaxf(m, __ldcg(part_ml + (base + s0 + lane) * 2));
  m = warp_max(m);
  float l = 0.f;
  float acc[(HD + 31) / 32];
#pragma unroll
  for (int i = 0; i < (HD + 31) / 32; ++i) acc[i] = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 32) {
    float f = 0.f;
    if (s0 + lane < splits) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + base + s0 + lane);
      f = ml.x == -CUDART_INF_F ? 0.f : exp2f(ml.x - m);
      l += f * ml.y;
    }
    const int n = min(32, splits - s0);
#pragma unroll 4
    for (int sl = 0; sl < n; ++sl) {
      const float fs = __shfl_sync(0xffffffffu, f, sl);
#pragma unroll
      for (int i = 0; i < (HD + 31) / 32; ++i) {
        const int d = i * 32 + lane;
        if (d < HD) acc[i] += fs * __ldcg(part_o + (base + s0 + sl) * HD + d);
      }
    }
  }
  const float inv = 1.f / warp_sum(l);
#pragma unroll
  for (int i = 0; i < (HD + 31) / 32; ++i) {
    const int d = i * 32 + lane;
    if (d < HD) out[th * HD + d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

}  // namespace tllm
