// bfloat16 attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (tcgen05), for head size 64 or 128 (-DTLLM_HEAD_DIM=64 / 128).
//
// A CTA serves 128 rows of one (request, key/value head); a row is a (new token, query head of the
// group) pair, so the heads of a group share every key/value tile.  Keys are walked in tiles of 64:
//
//   warp 0: TMA.  The query tile comes as one 3-D box (head size x heads of the group x
//     tokens) of the step's Q/K/V rows; a key tile and a value tile come page by page (one 2-D box of
//     page_size rows each, looked up in the request's block table, which sits in shared memory) into a
//     ring of four stages; every copy of a tile is issued by a lane of its own.
//   warps 1 and 6 (one thread each): tcgen05.mma.  Warp 1: S = Q K^T (M 128, N 64, K = head size; both
//     operands K-major in 128-byte-swizzled shared memory) into one of two S buffers in tensor memory, up
//     to two tiles ahead of the softmax; warp 6: O += P V (M 128, N = head
//     size, K 64) with P from tensor memory (the A operand) and V taken as it lies in the cache (rows =
//     keys: the MN-major form of the B operand).  tcgen05.commit hands each result over on an mbarrier.
//   warps 2-5: softmax.  A thread owns one row: it reads its 64 scores from tensor memory, applies
//     the causal rule (key j is visible to the token at position p iff j <= p), keeps the running
//     maximum and sum in 32-bit with the scale folded into exp2, writes P as bfloat16 pairs into one
//     of two P buffers in tensor memory, and rescales its row of O in tensor memory when the maximum
//     moved far.  Rows of a value tile beyond the request's last key are zeroed first (a
//     page may hold anything there, and 0 x NaN would spoil the product).
//
// Two such CTAs share an SM, so one CTA's softmax overlaps the other's MMAs.  Every wait is
// bounded (two seconds), after which the kernel records a code in the status word and stops.
//
// Head size 128: a row of 128 values is two 128-byte swizzle rows, so every operand lies in shared
// memory as two panels of 64 columns (Q: 128 rows each, a key or value tile: 64 rows each), fetched by
// two copies per page, and the ring has two stages so that two CTAs still fit an SM.  S = Q K^T walks
// both panels (eight steps of K = 16); O += P V is one product of N = 128 per 16 keys whose descriptor
// names the distance between the two value panels (the leading byte offset of an MN-major operand).
// Tensor memory: O takes 128 columns, so P of a tile is written over that tile's own S (which the
// softmax has read into registers by then): S/P of even tiles [0, 64), of odd tiles [64, 128), O
// [128, 256).
//
// Sizes: head size 64 or 128; heads per key/value head a power of two up to 128; page size 8, 16, 32
// or 64; no window.  Other cases run on the mma.sync kernels of attention_mma.cu.
//
// Reference counterpart: tiny_llm/ops/cuda/flash_attention.cu:338-442 (32-bit SIMT, one lane per
// key, 64-key tiles, chunk-local causal mask).
#include <math_constants.h>

#include <map>
#include <tuple>

#include "tc_common.cuh"

#ifndef TLLM_HEAD_DIM
#error "compile with -DTLLM_HEAD_DIM=64 or 128"
#endif

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int HD = TLLM_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "a row of keys is one or two 128-byte swizzle rows");
constexpr int PANELS = HD / 64;  // panels of 64 columns (one swizzle row wide) per operand
constexpr int BM = 128;          // rows per CTA = MMA M
constexpr int BNK = 64;          // keys per tile
constexpr int KV_STAGES = HD == 64 ? 4 : 2;
constexpr int THREADS = 224;     // warp 0: TMA, warp 1: S = Q K^T + tensor memory, warps 2-5: softmax, warp 6: O += P V
constexpr int UMMA_K = 16;
constexpr int Q_BYTES = BM * HD * 2, K_BYTES = BNK * HD * 2, V_BYTES = BNK * HD * 2;
constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + KV_STAGES * K_BYTES;
constexpr int OFF_BAR = OFF_V + KV_STAGES * V_BYTES;
constexpr int MAX_TABLE = 1024;                    // block-table entries kept in shared memory (longer tables are read from global)
constexpr int OFF_TABLE = OFF_BAR + 160;
constexpr int SMEM_TOTAL = OFF_TABLE + MAX_TABLE * 4 + 1024;   // + alignment slack
constexpr int Q_PANEL = BM * 128, KV_PANEL = BNK * 128;   // bytes of one panel of Q / of a key or value tile
constexpr uint32_t TMEM_COLS = 256;                // S of even tiles: columns [0, 64); of odd tiles: [64, 128); O: [128, 128 + HD);
// P (bfloat16 pairs): head size 64: even tiles [192, 224), odd tiles [224, 256); head size 128: over the tile's own S
constexpr uint32_t TMEM_O = 2 * BNK, TMEM_P = HD == 64 ? TMEM_O + HD : 0, TMEM_P_STEP = HD == 64 ? BNK / 2 : BNK;
static_assert(TMEM_O + HD <= TMEM_COLS && TMEM_P + TMEM_P_STEP + BNK / 2 <= TMEM_COLS, "S, O and P share 256 columns of tensor memory");
constexpr float RESCALE_STEP = 8.f;
constexpr int ERR_ATT_PRODUCER = 7, ERR_ATT_MMA = 8, ERR_ATT_SOFTMAX = 9;

struct TcAttnParams {
  const int* block_table;   // [R, max_blocks]
  const int* cu_q;          // [R + 1]
  const int* q_start;       // [R]: position of the request's first token in this step
  __nv_bfloat16* out;       // [T, nq * HD]
  int* status;
  int max_blocks, nq, nkv, page_size, tiles_per_req, n_requests;
  float scale_log2;         // scale * log2(e)
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Optional phase timing of the softmax (-DTLLM_ATT_TIMING=1, a build for measurements): lane 0 of the first
// softmax warp of CTA 0 adds up clock64() differences per phase of its loop over the key tiles.
#ifdef TLLM_ATT_TIMING
__device__ unsigned long long g_att_cycles[16];   // [8..15]: the MMA thread of the same CTA
#define ATT_T(k)                                                  \
  if (timed) {                                                    \
    const long long t_now_ = clock64();                           \
    att_acc[k] += (unsigned long long)(t_now_ - att_prev);        \
    att_prev = t_now_;                                            \
  }
#else
#define ATT_T(k)
#endif

__global__ void __launch_bounds__(THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* k_full = bars + 1;                   // [KV_STAGES]
  uint64_t* v_full = k_full + KV_STAGES;         // [KV_STAGES]
  uint64_t* kv_empty = v_full + KV_STAGES;       // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;       // [2]: S of an even / odd tile is in tensor memory
  uint64_t* p_full = s_full + 2;                 // [2]: P of an even / odd tile is in tensor memory (its S has been read), O rescaled (one arrival per softmax warp)
  uint64_t* o_done = p_full + 2;                 // [2]: O holds an even / odd tile too, and its P buffer is free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* table_s = reinterpret_cast<int*>(smem + OFF_TABLE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { tma_prefetch_map(&map_q); tma_prefetch_map(&map_k); tma_prefetch_map(&map_v); }
  // CTAs start in the order of blockIdx.x.  The tiles of the latest tokens see the most keys, so the
  // order is: the last tile of every request and key/value head, then the tiles before them, and so
  // on; the short ones fill the gaps at the end instead of the long ones trailing behind.
  const int kvh = blockIdx.x % p.nkv;
  const int req = (blockIdx.x / p.nkv) % p.n_requests;
  const int tile = p.tiles_per_req - 1 - blockIdx.x / (p.nkv * p.n_requests);
  const int group = p.nq / p.nkv;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_full[0], 4);
    mbar_init(&p_full[1], 4);
    mbar_init(&o_done[0], 1);
    mbar_init(&o_done[1], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  // The step's tables (request lengths, block table) were written before the step's first kernel: they are
  // read before the wait for the kernel in front.  The block table goes to shared memory, so that the
  // producer's page lookups are not a chain of global loads.
  for (int b = threadIdx.x; b < min(p.max_blocks, MAX_TABLE); b += THREADS)
    table_s[b] = p.block_table[(size_t)req * p.max_blocks + b];
  const int tok0 = p.cu_q[req];
  const int q_len = p.cu_q[req + 1] - tok0;
  const int start = p.q_start[req];
  __syncthreads();
  pdl_wait();

  const int rows_total = q_len * group;
  const int row0 = tile * BM;
  const int tok_lo = row0 / group;
  const int tok_hi = min(q_len - 1, (row0 + BM - 1) / group);
  const int kv_end = start + q_len;                         // keys that exist once this step's are written
  const int n_tiles = row0 < rows_total ? (start + tok_hi) / BNK + 1 : 0;

  if (warp == 0) {
    // ---------------- TMA producer.  A tile of 64 keys is up to eight pages, each a copy for K and one for V:
    // lane 2 g fetches the keys of the tile's page g, lane 2 g + 1 its values, so that the copies of a tile
    // are issued side by side (one thread issuing them all was the slowest part of the whole kernel).
    const int* table = p.block_table + (size_t)req * p.max_blocks;
    const int pages_per_tile = BNK / p.page_size;
    const uint32_t panel_page_bytes = (uint32_t)p.page_size * 128u;          // one page inside one panel
    const uint32_t page_bytes = panel_page_bytes * PANELS;
    // lane = (page of the tile, keys or values, panel): 2 * PANELS copies per page, at most eight pages per tile
    const int g = lane / (2 * PANELS);
    const bool is_v = (lane / PANELS) & 1;
    const int panel = lane % PANELS;
    if (lane < PANELS && n_tiles > 0) {
      if (lane == 0) mbar_expect_tx(q_full, Q_BYTES);
      __syncwarp(PANELS == 1 ? 1u : 3u);
      tma_load_3d(smem + lane * Q_PANEL, &map_q, lane * 64, kvh * group, tok0 + tok_lo, q_full);
    }
    __syncwarp();
#ifdef TLLM_ATT_TIMING
    const bool timed = blockIdx.x == 0 && lane == 0;
    unsigned long long att_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long att_prev = clock64();
#endif
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % KV_STAGES;
      ATT_T(5)   // producer: issuing
      if (i >= KV_STAGES) {
        bool ok = true;
        if (lane == 0) ok = mbar_wait(&kv_empty[s], ((i / KV_STAGES) & 1) ^ 1, abort_flag);
        if (!__shfl_sync(0xffffffffu, (int)ok, 0)) {
          if (lane == 0) { *abort_flag = 1; atomicExch(p.status, ERR_ATT_PRODUCER); }
          break;
        }
      }
      ATT_T(4)   // producer: waited for a free stage
      // this lane's page of keys [i * 64, i * 64 + 64), if it holds at least one existing key
      int page = -1;
      const int blk = i * pages_per_tile + g;
      if (g < pages_per_tile && blk < p.max_blocks && blk * p.page_size < kv_end) page = blk < MAX_TABLE ? table_s[blk] : table[blk];
      const int n_valid = __popc(__ballot_sync(0xffffffffu, page >= 0 && !is_v && panel == 0));
      if (lane == 0) {
        mbar_expect_tx(&k_full[s], (uint32_t)n_valid * page_bytes);
        mbar_expect_tx(&v_full[s], (uint32_t)n_valid * page_bytes);
      }
      __syncwarp();
      if (page >= 0) {
        const int row = (page * p.nkv + kvh) * p.page_size;
        const uint32_t off = panel * KV_PANEL + g * panel_page_bytes;
        if (is_v) tma_load_2d(smem + OFF_V + s * V_BYTES + off, &map_v, panel * 64, row, &v_full[s]);
        else tma_load_2d(smem + OFF_K + s * K_BYTES + off, &map_k, panel * 64, row, &k_full[s]);
      }
    }
#ifdef TLLM_ATT_TIMING
    if (timed)
      for (int k = 4; k < 6; ++k) atomicAdd(&g_att_cycles[8 + k], att_acc[k]);
#endif
  } else if (warp == 1) {
    // ---------------- S = Q K^T of tile t into the S buffer of its parity, as soon as its keys are there and
    // the softmax of tile t - 2 has read that buffer: up to two tiles ahead of the softmax.  The whole warp
    // walks the loop and waits; one elected lane issues (operands computed by the converged warp are warp-wide
    // values: a loop walked by a single lane took nearly twice as long per tile).
    const uint32_t idesc_qk = instr_desc_bf16(BM, BNK);
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(smem)), k_lo = smem_desc_sw128_lo(smem_u32(smem + OFF_K));
    bool ok = n_tiles == 0 || mbar_wait(q_full, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
#ifdef TLLM_ATT_TIMING
    const bool timed = blockIdx.x == 0 && lane == 0;
    unsigned long long att_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long att_prev = clock64();
#endif
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t % KV_STAGES;
      ATT_T(3)   // issuing
      if (t >= 2)   // tile t - 2: its S has been read, and its product has read the P buffer that the softmax of tile t will write
        ok = mbar_wait(&p_full[t & 1], ((t >> 1) - 1) & 1, abort_flag) && mbar_wait(&o_done[t & 1], ((t >> 1) - 1) & 1, abort_flag);
      ATT_T(1)   // waited for the S buffer
      ok = ok && mbar_wait(&k_full[s], (t / KV_STAGES) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      ATT_T(0)   // waited for K
      const uint32_t d = tmem_u + (t & 1) * BNK, kt_lo = k_lo + s * (K_BYTES >> 4);   // descriptors count in 16-byte units
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < HD / UMMA_K; ++k) {   // 16 columns = 32 bytes inside a swizzle row; every fourth step enters the next panel
          const uint32_t in_panel = (uint32_t)((k & 3) * UMMA_K * 2) >> 4;
          umma_bf16_lo(d, q_lo + (uint32_t)(k >> 2) * (Q_PANEL >> 4) + in_panel, kt_lo + (uint32_t)(k >> 2) * (KV_PANEL >> 4) + in_panel,
                       idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t & 1]);
      }
      __syncwarp();
    }
#ifdef TLLM_ATT_TIMING
    if (timed)
      for (int k = 0; k < 4; ++k) atomicAdd(&g_att_cycles[8 + k], att_acc[k]);
#endif
    if (!ok && lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, ERR_ATT_MMA); }
  } else if (warp == 6) {
    // ---------------- O += P V of tile i, when the softmax has written P (the same way: warp-wide loop, one lane issues)
    const uint32_t idesc_pv = instr_desc_bf16(BM, HD, true);   // V as it lies: rows = keys (MN-major B)
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    // head size 128: the values' second panel of 64 columns lies KV_PANEL bytes after the first
    const uint32_t v_lo = smem_desc_sw128_lo(smem_u32(smem + OFF_V), PANELS == 1 ? 16u : (uint32_t)KV_PANEL);
    const uint32_t tmem_o = tmem_u + TMEM_O;
    bool ok = true;
#ifdef TLLM_ATT_TIMING
    const bool timed = blockIdx.x == 0 && lane == 0;
    unsigned long long att_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long att_prev = clock64();
#endif
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % KV_STAGES;
      ATT_T(7)   // issuing
      ok = mbar_wait(&p_full[i & 1], (i >> 1) & 1, abort_flag);
      ATT_T(6)   // waited for P
      ok = ok && mbar_wait(&v_full[s], (i / KV_STAGES) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      ATT_T(2)   // waited for V
      const uint32_t a = tmem_u + TMEM_P + (i & 1) * TMEM_P_STEP, vt_lo = v_lo + s * (V_BYTES >> 4);
      const uint32_t acc0 = i > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BNK / UMMA_K; ++kk)   // 16 keys per step: eight columns of P pairs, two 8-row groups of V
          umma_bf16_ts_lo(tmem_o, a + kk * (UMMA_K / 2), vt_lo + (kk * UMMA_K * 128 >> 4), idesc_pv, kk > 0 ? 1u : acc0);
        umma_commit(&kv_empty[s]);
        umma_commit(&o_done[i & 1]);
      }
      __syncwarp();
    }
#ifdef TLLM_ATT_TIMING
    if (timed) {
      atomicAdd(&g_att_cycles[8 + 2], att_acc[2]);
      atomicAdd(&g_att_cycles[8 + 6], att_acc[6]);
      atomicAdd(&g_att_cycles[8 + 7], att_acc[7]);
    }
#endif
    if (!ok && lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, ERR_ATT_MMA); }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- softmax: this thread owns row `row` of the tile (tensor-memory lane)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int grow = row0 + row;
    const bool live = grow < rows_total;
    const int pos = start + grow / group;
    const uint32_t t_s0 = tmem_base + ((uint32_t)(quad * 32) << 16), t_o = t_s0 + TMEM_O, t_p0 = t_s0 + TMEM_P;
    const int soft_tid = (warp - 2) * 32 + lane;   // 0..127 among the softmax threads
    const float c = p.scale_log2;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    bool ok = true;
#ifdef TLLM_ATT_TIMING
    const bool timed = blockIdx.x == 0 && warp == 2 && lane == 0;
    unsigned long long att_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long att_prev = clock64();
#endif
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % KV_STAGES;
      ok = mbar_wait(&s_full[i & 1], (i >> 1) & 1, abort_flag);   // (a wait that gave up is seen at this tile's vote below)
      tc_fence_after();
      ATT_T(0)   // waited for S
      const uint32_t t_s = t_s0 + (i & 1) * BNK;
      float sc[BNK];
      {
        uint32_t raw[BNK];
        tmem_ld32_issue(t_s, raw);          // both halves in flight, one wait
        tmem_ld32_issue(t_s + 32, raw + 32);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < BNK; ++j) sc[j] = __uint_as_float(raw[j]);
      }
      ATT_T(1)   // S in registers
      const int j0 = i * BNK;
      if (!live || j0 + BNK - 1 > pos) {   // the tile touches this row's causal edge (or the row does not exist)
#pragma unroll
        for (int j = 0; j < BNK; ++j)
          if (!(live && j0 + j <= pos)) sc[j] = -CUDART_INF_F;
      }
      // maximum and sum as four interleaved chains: 64 dependent steps would cost more than the arithmetic
      float mx4[4] = {sc[0], sc[1], sc[2], sc[3]};
#pragma unroll
      for (int j = 4; j < BNK; j += 4) {
        mx4[0] = fmaxf(mx4[0], sc[j]); mx4[1] = fmaxf(mx4[1], sc[j + 1]);
        mx4[2] = fmaxf(mx4[2], sc[j + 2]); mx4[3] = fmaxf(mx4[3], sc[j + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The running maximum only has to bound the exponents: it follows the true one when that has moved by
      // more than RESCALE_STEP (in log2 units), so P stays below 2^RESCALE_STEP and O is rescaled rarely.
      // The result is the same quotient sum(p v) / sum(p): p carries the same factor above and below.
      const float mn = mx * c > m_run + RESCALE_STEP ? mx * c : m_run;
      const float ms = mn == -CUDART_INF_F ? 0.f : mn;
      const float corr = ex2(m_run - ms);   // 0 while nothing was seen
      m_run = mn;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < BNK; j += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sc[j + e] = ex2(fmaf(sc[j + e], c, -ms));
          sum4[e] += sc[j + e];
        }
      }
      l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      ATT_T(2)   // maximum, exponentials, sum
      // P as bfloat16 pairs in the P buffer of this tile's parity: the A operand of O += P V, taken from tensor
      // memory.  The product of tile i - 2 has read that buffer: S of this tile was issued after it had finished.
      {
        uint32_t pk[BNK / 2];
#pragma unroll
        for (int j = 0; j < BNK / 2; ++j) pk[j] = pack_bf16(sc[2 * j], sc[2 * j + 1]);
        tmem_st32_raw(t_p0 + (i & 1) * TMEM_P_STEP, pk);
      }
      ATT_T(3)   // P on its way to tensor memory
      if (!__all_sync(0xffffffffu, ok && (i == 0 || corr == 1.f))) {   // the maximum of some row of this warp moved far
        ok = __all_sync(0xffffffffu, ok);                               // (or a wait gave up)
        if (!ok) break;
#ifdef TLLM_ATT_TIMING
        if (timed) att_acc[7] += 1;
#endif
        ok = mbar_wait(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag);   // the product before this one has finished O
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < HD; h += 32) {
          float o[32];
          tmem_ld32(t_o + h, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= corr;
          tmem_st32(t_o + h, o);
        }
      }
      tmem_st_wait();
      ATT_T(5)   // O rescaled
      if (j0 + BNK > kv_end) {   // value rows past the last key hold whatever the page held: zero them
        ok = mbar_wait(&v_full[s], (i / KV_STAGES) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (soft_tid < BNK && j0 + soft_tid >= kv_end) {
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) {
            uint4* vrow = reinterpret_cast<uint4*>(smem + OFF_V + s * V_BYTES + pn * KV_PANEL + soft_tid * 128);
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) vrow[ch] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // V was written by ordinary stores
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i & 1]);
      ATT_T(6)   // fences, arrival
    }
#ifdef TLLM_ATT_TIMING
    if (timed)
      for (int k = 0; k < 8; ++k) atomicAdd(&g_att_cycles[k], att_acc[k]);
#endif
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&o_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, ERR_ATT_SOFTMAX); }
    } else if (n_tiles > 0) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      const size_t th = (size_t)(tok0 + grow / group) * p.nq + (size_t)(kvh * group + grow % group);
#pragma unroll
      for (int h = 0; h < HD; h += 32) {
        float o[32];
        tmem_ld32(t_o + h, o);   // warp-wide: rows that do not exist read too, and store nothing
        if (live) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + th * HD + h);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            v.x = pack_bf16(o[ch * 8 + 0] * inv, o[ch * 8 + 1] * inv);
            v.y = pack_bf16(o[ch * 8 + 2] * inv, o[ch * 8 + 3] * inv);
            v.z = pack_bf16(o[ch * 8 + 4] * inv, o[ch * 8 + 5] * inv);
            v.w = pack_bf16(o[ch * 8 + 6] * inv, o[ch * 8 + 7] * inv);
            dst[ch] = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------- host side
// Tensor maps are cached by what they describe; the step's buffers and the cache keep their addresses.
static bool make_map_rows(CUtensorMap* map, const void* ptr, long long rows, int box_rows) {
  using Key = std::tuple<const void*, long long, int>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  const Key key(ptr, rows, box_rows);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};   // one panel: a swizzle row of 128 bytes
  cuuint32_t elem[2] = {1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 1024) cache.clear();
  cache[key] = *map;
  return true;
}

// Queries: [tokens][heads][HD] inside rows of q_row_stride elements; a box is the heads of one group for 128 / group tokens.
static bool make_map_q(CUtensorMap* map, const void* ptr, int tokens, int nq, int q_row_stride, int group) {
  using Key = std::tuple<const void*, int, int, int, int>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  const Key key(ptr, tokens, nq, q_row_stride, group);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nq, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_row_stride * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)group, (cuuint32_t)(BM / group)};
  cuuint32_t elem[3] = {1, 1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 1024) cache.clear();
  cache[key] = *map;
  return true;
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_attention_tc_head_dim() { return HD; }

#ifdef TLLM_ATT_TIMING
// Cycles per phase of the timed softmax lane since the last call: waited for S, S to registers, maximum +
// exponentials + sum, waited for the product before, P stored, O rescaled, fences + arrival; [7] counts the rescales.
extern "C" int tllm_attention_tc_timing(unsigned long long* host) {
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(host, ::tllm::g_att_cycles, 16 * sizeof(unsigned long long)) != cudaSuccess) return 1;
  const unsigned long long zero[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  return cudaMemcpyToSymbol(::tllm::g_att_cycles, zero, sizeof(zero)) != cudaSuccess;
}
#endif

// 1 if the kernel takes these sizes (the caller then need not try and fail).
extern "C" int tllm_attention_tc_fits(int nq, int nkv, int hd, int page_size, int window) {
  if (hd != HD || nq <= 0 || nkv <= 0 || nq % nkv != 0 || window != 0) return 0;
  const int group = nq / nkv;
  if (group > BM || (group & (group - 1)) != 0) return 0;
  return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64;
}

extern "C" int tllm_attention_tc(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                 long long cache_pages, const int* block_table, int max_blocks, const int* cu_q,
                                 const int* q_start, void* out, int n_tokens, int n_requests, int max_q_len, int nq,
                                 int nkv, int hd, int page_size, float scale, int* status, void* stream) {
  TLLM_REQUIRE(tllm_attention_tc_fits(nq, nkv, hd, page_size, 0), "attention_tc: %d heads, %d key/value heads, head size %d, page size %d "
               "(takes head size %d, a power-of-two group up to 128, pages of 8 to 64)", nq, nkv, hd, page_size, HD);
  TLLM_REQUIRE(n_tokens > 0 && n_requests > 0 && max_q_len > 0 && max_blocks > 0 && cache_pages > 0 && scale > 0.f && status != nullptr,
               "attention_tc: %d tokens, %d requests, %d blocks, %lld pages", n_tokens, n_requests, max_blocks, cache_pages);
  TLLM_REQUIRE(((uintptr_t)q % 16) == 0 && (q_row_stride % 8) == 0 && ((uintptr_t)kcache % 128) == 0 && ((uintptr_t)vcache % 128) == 0 &&
               ((uintptr_t)out % 16) == 0, "attention_tc: operands are not aligned for TMA");
  const int group = nq / nkv;
  CUtensorMap mq, mk, mv;
  const long long rows = cache_pages * nkv * page_size;
  if (!make_map_q(&mq, q, n_tokens, nq, q_row_stride, group) || !make_map_rows(&mk, kcache, rows, page_size) ||
      !make_map_rows(&mv, vcache, rows, page_size))
    TLLM_FAIL(TLLM_ERR_CUDA, "attention_tc: cuTensorMapEncodeTiled failed");
  TcAttnParams p;
  p.block_table = block_table; p.cu_q = cu_q; p.q_start = q_start; p.out = (__nv_bfloat16*)out; p.status = status;
  p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
  p.tiles_per_req = (int)(((long long)max_q_len * group + BM - 1) / BM);
  p.n_requests = n_requests;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long gx = (long long)n_requests * p.tiles_per_req * nkv;
  TLLM_REQUIRE(gx <= 2147483647LL, "attention_tc: grid too large");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_tc: cannot reserve %d bytes of shared memory: %s", SMEM_TOTAL, cudaGetErrorString(e));
    configured = true;
  }
  TLLM_LAUNCH("attention_tc", attention_tc_kernel, dim3((unsigned)gx), THREADS, SMEM_TOTAL, (cudaStream_t)stream, mq, mk, mv, p);
  return TLLM_OK;
}
