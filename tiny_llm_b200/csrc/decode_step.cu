// One kernel for a whole decode step of at most eight requests, one token each: embedding, every
// layer (RMSNorm -> Q/K/V projection -> rotation and cache write -> attention over the pages ->
// output projection -> RMSNorm -> SwiGLU feed-forward), final norm and LM head, in bfloat16 with
// 32-bit statistics, residual stream and accumulators.  Compiled for one head size
// (-DTLLM_HEAD_DIM=...).
//
// Why one kernel: a decode step of a small batch is a chain of some ten short, dependent kernels per
// layer, each of which needs a few microseconds to fill the SMs and to drain them, while the work
// itself is streaming every weight once.  Here one persistent CTA per SM keeps the weight stream
// running across all of them:
//
//   * warp 8 of each CTA is the producer.  It walks the step's schedule, which is fixed before the
//     kernel starts (which 16-row tiles of which weight matrix this CTA multiplies, in order), and
//     copies the tiles into a ring of shared-memory stages with cp.async.bulk (the TMA engine; 16
//     row pieces of up to 256 elements per stage), throttled only by the ring's empty barriers.
//     It runs ahead of the math: while the CTA waits at a grid barrier or computes attention, the
//     next projection's weights are already arriving.
//   * warps 0-7 are the consumers.  A projection phase loads the (normalised) activations of all
//     tokens into shared memory, then multiplies each tile as it lands: mma.sync.m16n8k16 with the
//     16 weight rows as A and the eight tokens as B, the warps splitting each stage's K range; the
//     eight partial accumulators are summed through shared memory and warp 0 applies the phase's
//     epilogue.  A weight tile spans the whole K, so no sums cross CTAs: the residual update is a
//     plain read-modify-write by the one thread that owns the element, and results do not depend on
//     timing.
//   * Phases that read what other CTAs wrote are separated by a grid barrier (a 64-bit ticket
//     counter in global memory; the launch is cooperative so every CTA is resident).  Data written
//     inside the kernel is read with L2-only loads.
//
// Tiles pair rows so that an epilogue finds what it combines in one thread: a Q/K/V tile holds
// dimensions [8j, 8j+8) and [hd/2 + 8j, hd/2 + 8j + 8) of one head (the two halves of the rotation
// pairs); a gate/up tile holds eight gate rows and the matching eight up rows.  For RMSNorm, the
// thread that adds a projection into the residual stream (32-bit) also writes its tile's share of
// sum(x^2); the next phase copies the 32-bit rows into shared memory (one bulk copy per token), adds
// the shares in a fixed order and converts the rows in place to bf16((w * x) / sqrt(mean + eps)),
// the same rounding point as the stand-alone norm kernel.
//
// Attention of a phase is the same device function as the stand-alone decode kernel
// (attention_tiles.cuh), run by teams of four warps over (request, key/value head, slice of keys)
// items, followed by the merge of the slices.
//
// Every wait (ring barriers, grid barrier) gives up after two seconds, records a code in the status
// word and raises an abort flag that ends all CTAs; the producer then waits for its copies in
// flight before the CTA leaves.
//
// Reference counterpart: the decode branch of tiny_llm/runtime/cuda/cuda_runtime.cpp:658-802 with
// the per-layer launches of tiny_llm/runtime/cuda/cuda_kernels.cpp:336-385.
#include "attention_tiles.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;
constexpr int MAX_TOKENS = 8;                  // the N of mma.m16n8k16
static_assert(MAX_TOKENS == CONSUMER_WARPS, "one warp normalises one token");
#ifndef TLLM_STEP_KC
#define TLLM_STEP_KC 1024   // measured: copies of 2 KB stream three times faster than copies of 512 bytes
#endif
constexpr int KC = TLLM_STEP_KC;               // K elements of a ring stage (one bulk copy per row and stage)
constexpr int ROW_BYTES = KC * 2 + 16;         // +16 bytes: ldmatrix over 8 rows touches every bank once
constexpr int STAGE_BYTES = 16 * ROW_BYTES;
constexpr int MAX_STAGES = 16;
constexpr int MIN_STAGES = 2;
constexpr int RED_BYTES = 2 * CONSUMER_WARPS * 32 * 16;   // two buffers of one float4 per consumer thread
constexpr int ATT_STAGES = 3;
constexpr int TEAM_BYTES = (16 + 2 * ATT_STAGES * BN) * LDS * 2 + TABLE_SLOTS * 4;
constexpr int TEAMS = 2 * TEAM_BYTES <= 120 * 1024 ? 2 : 1;
constexpr unsigned long long WAIT_NS = 2000000000ull;
constexpr int ERR_STEP_PRODUCER = 4, ERR_STEP_CONSUMER = 5, ERR_STEP_GRID = 6;

enum Kind { K_QKV = 0, K_O = 1, K_GATE_UP = 2, K_DOWN = 3, K_LM_HEAD = 4 };

// One run-order entry.  The Python side writes the same layout (twelve pointers, four 32-bit values).
struct DecodeLayer {
  const __nv_bfloat16* w_qkv;      // [(nq + 2 nkv) hd, hidden]
  const __nv_bfloat16* w_o;        // [hidden, nq hd]
  const __nv_bfloat16* w_gate_up;  // [2 inter, hidden], gate and up rows alternating in blocks of gu_block
  const __nv_bfloat16* w_down;     // [hidden, inter]
  const float* norm1;
  const float* norm2;
  const float* cos;                // [positions, hd / 2] or null: no rotation
  const float* sin;
  __nv_bfloat16* kcache;           // [pages, nkv, page_size, hd]
  __nv_bfloat16* vcache;
  const int* block_table;          // [requests, max_blocks] of this layer's cache group
  const int* slot_mapping;         // [requests]
  float eps1, eps2, scale_log2;
  int window;
};

struct DecodeParams {
  const DecodeLayer* layers;       // device memory
  const int* tokens;
  const int* positions;            // [m]: tokens the request held before this one
  const int* cu_q;                 // [m + 1] = 0, 1, ..., m
  const __nv_bfloat16* embed;
  const float* final_norm;
  const __nv_bfloat16* lm_head;
  float* resid;                    // [m, hidden]
  __nv_bfloat16* q_buf;            // [m, nq hd]
  __nv_bfloat16* attn_out;         // [m, nq hd]
  __nv_bfloat16* ffn_act;          // [m, inter]
  float* logits;                   // [m, vocab]
  float* part_o;                   // attention partials (splits > 1)
  float* part_ml;
  float* ssq_part;                 // [ceil(hidden / 16), 8]: each residual tile's share of sum(x^2) per token
  unsigned long long* sync_words;  // [0]: grid barrier arrivals; [1]: abort flag; [2]: CTAs that have finished
  int* status;
  int n_layers, m, hidden, nq, nkv, inter, gu_block, vocab;
  int page_size, max_blocks, splits, stages, act_ld;
  float final_eps;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  False if the phase did not complete within WAIT_NS (then `code` goes to the status
// word and the CTA's abort flag is raised) or the CTA is already giving up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* s_abort, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*s_abort) return false;
    if (global_timer_ns() - t0 > WAIT_NS) {
      atomicCAS(status, 0, code);
      *s_abort = 1;
      return false;
    }
  }
}
// 16-byte-granular copy global -> shared by the TMA engine; completion is counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ unsigned long long load_acquire(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// ---------------------------------------------------------------- optional phase timing (-DTLLM_STEP_TIMING=1)
#ifdef TLLM_STEP_TIMING
__device__ unsigned long long g_step_timing[16];
#define T_BEGIN() long long t_mark = clock64()
#define T_ADD(slot)                                                      \
  do {                                                                   \
    if (blockIdx.x == TLLM_STEP_TIMING - 1 && threadIdx.x == 0) {        \
      const long long now = clock64();                                   \
      g_step_timing[slot] += (unsigned long long)(now - t_mark);         \
      t_mark = now;                                                      \
    }                                                                    \
  } while (0)
#else
#define T_BEGIN()
#define T_ADD(slot)
#endif

// ---------------------------------------------------------------- the schedule
// Tiles of a phase are dealt to the CTAs round-robin, continuing where the phase before stopped, so
// that over a step every CTA streams the same number of tiles to within one per phase.
__device__ __forceinline__ int phase_tiles(const DecodeParams& p, int kind) {
  switch (kind) {
    case K_QKV: return (p.nq + 2 * p.nkv) * (HD / 16);
    case K_GATE_UP: return (p.inter + 7) / 8;
    case K_LM_HEAD: return (p.vocab + 15) / 16;
    default: return (p.hidden + 15) / 16;
  }
}
__device__ __forceinline__ int phase_k(const DecodeParams& p, int kind) {
  return kind == K_O ? p.nq * HD : kind == K_DOWN ? p.inter : p.hidden;
}
// Row r (0..15) of tile t: where its K elements start.  Rows past the matrix repeat its last row;
// their results are dropped.
__device__ __forceinline__ const __nv_bfloat16* tile_row(const DecodeParams& p, const DecodeLayer* L, int kind, int t, int r) {
  switch (kind) {
    case K_QKV: {
      const int head = t / (HD / 16), j = t % (HD / 16);
      const int dim = (r < 8 ? 0 : HD / 2) + 8 * j + (r & 7);
      return L->w_qkv + (size_t)(head * HD + dim) * p.hidden;
    }
    case K_O: return L->w_o + (size_t)min(16 * t + r, p.hidden - 1) * (p.nq * HD);
    case K_GATE_UP: {
      const int col = min(8 * t + (r & 7), p.inter - 1);
      const int row = (col / p.gu_block) * 2 * p.gu_block + col % p.gu_block + (r < 8 ? 0 : p.gu_block);
      return L->w_gate_up + (size_t)row * p.hidden;
    }
    case K_DOWN: return L->w_down + (size_t)min(16 * t + r, p.hidden - 1) * p.inter;
    default: return p.lm_head + (size_t)min(16 * t + r, p.vocab - 1) * p.hidden;
  }
}
__device__ __forceinline__ int first_tile(int rr) {
  const int g = (int)gridDim.x;
  return ((int)blockIdx.x - rr % g + g) % g;
}

// ---------------------------------------------------------------- producer
__device__ void produce(const DecodeParams& p, uint8_t* ring, uint64_t* full_bar, uint64_t* empty_bar, volatile int* s_abort) {
  const int lane = threadIdx.x & 31, G = (int)gridDim.x;
  const uint32_t S = (uint32_t)p.stages;
  uint32_t issued = 0;
  int rr = 0;
  bool ok = true;
  const int phases = 4 * p.n_layers + 1;
#ifdef TLLM_STEP_TIMING
  const long long t_start = clock64();
  long long t_wait = 0;
#endif
  for (int ph = 0; ph < phases && ok; ++ph) {
    const int kind = ph < 4 * p.n_layers ? (ph & 3) : K_LM_HEAD;
    const DecodeLayer* L = p.layers + min(ph >> 2, p.n_layers - 1);
    const int T = phase_tiles(p, kind), K = phase_k(p, kind);
    for (int t = first_tile(rr); t < T && ok; t += G) {
      const char* src = reinterpret_cast<const char*>(tile_row(p, L, kind, t, lane & 15));
      for (int k0 = 0; k0 < K; k0 += KC) {
        const int kc = min(KC, K - k0);
        const uint32_t stage = issued % S, use = issued / S;
        int good = 1;
        if (lane == 0) {
#ifdef TLLM_STEP_TIMING
          const long long w0 = clock64();
#endif
          if (use > 0) good = mbar_wait(&empty_bar[stage], (use - 1) & 1, s_abort, p.status, ERR_STEP_PRODUCER) ? 1 : 0;
#ifdef TLLM_STEP_TIMING
          t_wait += clock64() - w0;
#endif
          if (good) mbar_expect_tx(&full_bar[stage], 16u * (uint32_t)kc * 2u);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        if (lane < 16)
          bulk_load(ring + (size_t)stage * STAGE_BYTES + lane * ROW_BYTES, src + (size_t)k0 * 2, (uint32_t)kc * 2u, &full_bar[stage]);
        ++issued;
      }
    }
    rr = (rr + T) % G;
  }
#ifdef TLLM_STEP_TIMING
  if (lane == 0 && blockIdx.x == TLLM_STEP_TIMING - 1) {
    g_step_timing[10] += (unsigned long long)t_wait;
    g_step_timing[11] += (unsigned long long)(clock64() - t_start);
  }
#endif
  // nothing of this CTA's shared memory may be written after it has left: wait for the copies in flight
  if (lane == 0) {
    const uint32_t from = issued > S ? issued - S : 0;
    for (uint32_t i = from; i < issued; ++i) {
      const unsigned long long t0 = global_timer_ns();
      while (!mbar_try_wait(&full_bar[i % S], (i / S) & 1))
        if (global_timer_ns() - t0 > WAIT_NS) break;
    }
  }
}

// ---------------------------------------------------------------- consumers
struct ConsumerState {
  uint32_t taken;      // ring stages consumed so far
  uint32_t act_loads;  // activation loads so far (parity of the activation barrier)
  uint32_t barriers;   // grid barriers passed
  int rr;              // round-robin offset of the next phase
  int red_buf;
#ifdef TLLM_STEP_TIMING
  long long t_full, t_epi;
#endif
};

__device__ __forceinline__ void consumer_sync() { named_sync(1, CONSUMERS); }

// All CTAs' consumers meet: arrivals are counted in sync_words[0], which the last CTA to finish the
// step sets back to zero.  Returns false when the step is being given up.
__device__ __forceinline__ bool grid_barrier(const DecodeParams& p, volatile int* s_abort, ConsumerState& st) {
  ++st.barriers;
  consumer_sync();
  if (threadIdx.x == 0) {
    unsigned long long* arrivals = p.sync_words;
    const volatile unsigned long long* abort_word = p.sync_words + 1;
    __threadfence();   // the CTA's writes (ordered before this thread by the barrier above) go out first
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(arrivals) : "memory");
    const unsigned long long target = (unsigned long long)st.barriers * gridDim.x;
    const unsigned long long t0 = global_timer_ns();
    bool done = false;
    while (!done) {
#pragma unroll 1
      for (int i = 0; i < 64 && !done; ++i) done = load_acquire(arrivals) >= target;
      if (done) break;
      if (*abort_word != 0 || *s_abort) { *s_abort = 1; break; }
      if (global_timer_ns() - t0 > WAIT_NS) {
        atomicCAS(p.status, 0, ERR_STEP_GRID);
        *s_abort = 1;
        break;
      }
    }
    if (*s_abort) {
      p.sync_words[1] = 1;   // the other CTAs stop waiting for this one
      __threadfence();
    }
  }
  consumer_sync();
  return *s_abort == 0;
}

// Copies m rows of `row_bytes` bytes that other CTAs wrote into the rows of the shared-memory
// activations, one bulk copy per token (and `extra`, a vector of the model, behind the rows), and
// waits for them.  Rows of tokens that do not exist keep
// what they held: column n of the product depends on row n alone and is never stored for n >= m.
__device__ __forceinline__ void fetch_rows_issue(const DecodeParams& p, __nv_bfloat16* act, const void* src, uint32_t row_bytes,
                                                 const float* extra, uint32_t extra_bytes, uint64_t* act_bar) {
  if (threadIdx.x == 0) {
    // what the generic proxy did to this shared memory (attention tiles, the first layer's rows) comes first
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_tx(act_bar, (uint32_t)p.m * row_bytes + extra_bytes);
    for (int n = 0; n < p.m; ++n)
      bulk_load(act + (size_t)n * p.act_ld, reinterpret_cast<const char*>(src) + (size_t)n * row_bytes, row_bytes, act_bar);
    if (extra_bytes) bulk_load(act + (size_t)MAX_TOKENS * p.act_ld, extra, extra_bytes, act_bar);   // behind the last row
  }
}
__device__ __forceinline__ void fetch_rows_wait(const DecodeParams& p, uint64_t* act_bar, volatile int* s_abort, ConsumerState& st) {
  mbar_wait(act_bar, st.act_loads & 1, s_abort, p.status, ERR_STEP_CONSUMER);
  ++st.act_loads;
}

// Activations of a projection that follows an RMSNorm: the 32-bit residual rows land in the
// activation rows (a row holds at least 2 * hidden bfloat16 values), warp n turns row n into
// bf16((w * x) / sqrt(mean(x^2) + eps)) in place, front to back, so that a value is overwritten only
// after it was read; mean(x^2) comes from the shares the residual stream's writers left.
__device__ __forceinline__ void load_act_norm(const DecodeParams& p, __nv_bfloat16* act, const float* norm_w, float eps,
                                              uint64_t* act_bar, volatile int* s_abort, ConsumerState& st) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.hidden;
  float denom = 1.f;
  fetch_rows_issue(p, act, p.resid, (uint32_t)K * 4u, norm_w, (uint32_t)K * 4u, act_bar);
  if (warp < p.m) {
    const int tiles = (K + 15) / 16;
    float ssq = 0.f;
    for (int t = lane; t < tiles; t += 32) ssq += __ldcg(p.ssq_part + (size_t)t * MAX_TOKENS + warp);
    denom = sqrtf(warp_sum(ssq) / (float)K + eps);
  }
  fetch_rows_wait(p, act_bar, s_abort, st);
  if (warp < p.m) {
    __nv_bfloat16* row = act + (size_t)warp * p.act_ld;
    const float4* in = reinterpret_cast<const float4*>(row);
    const float4* w_s = reinterpret_cast<const float4*>(act + (size_t)MAX_TOKENS * p.act_ld);
    constexpr int UNR = 2;
    for (int base = 0; base < K / 4; base += 32 * UNR) {
      float4 x[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = base + u * 32 + lane;
        if (k4 < K / 4) x[u] = in[k4];
      }
      __syncwarp();   // every lane has read its values before any lane writes over them
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = base + u * 32 + lane;
        if (k4 >= K / 4) continue;
        const float4 w = w_s[k4];
        uint2 packed;
        packed.x = pack_bf16((w.x * x[u].x) / denom, (w.y * x[u].y) / denom);
        packed.y = pack_bf16((w.z * x[u].z) / denom, (w.w * x[u].w) / denom);
        *reinterpret_cast<uint2*>(row + 4 * k4) = packed;
      }
      __syncwarp();
    }
  }
  consumer_sync();
}

// The first layer's norm reads the embedding rows of the step's tokens instead, one warp per token, in
// two passes (the sum, then the values); the CTA that owns a token also writes its row to the
// residual stream.
__device__ __forceinline__ void load_act_embedding(const DecodeParams& p, __nv_bfloat16* act, const float* norm_w, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.hidden, n = warp;
  if (n < p.m) {
    __nv_bfloat16* dst = act + (size_t)n * p.act_ld;
    const uint2* src = reinterpret_cast<const uint2*>(p.embed + (size_t)p.tokens[n] * K);
    const bool owner = (int)blockIdx.x == n % (int)gridDim.x;
    constexpr int UNR = 4;   // loads in flight per lane
    float ssq = 0.f;
    for (int base = 0; base < K / 4; base += 32 * UNR) {
      uint2 raw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = base + u * 32 + lane;
        raw[u] = k4 < K / 4 ? __ldg(src + k4) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = base + u * 32 + lane;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].y);
        const float4 x = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
        if (owner && k4 < K / 4) __stcg(reinterpret_cast<float4*>(p.resid + (size_t)n * K) + k4, x);
        ssq += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
      }
    }
    const float denom = sqrtf(warp_sum(ssq) / (float)K + eps);
    for (int base = 0; base < K / 4; base += 32 * UNR) {
      uint2 raw[UNR];
      float4 w[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = min(base + u * 32 + lane, K / 4 - 1);
        raw[u] = __ldg(src + k4);
        w[u] = __ldg(reinterpret_cast<const float4*>(norm_w) + k4);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k4 = base + u * 32 + lane;
        if (k4 >= K / 4) continue;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].y);
        uint2 packed;
        packed.x = pack_bf16((w[u].x * __low2float(lo)) / denom, (w[u].y * __high2float(lo)) / denom);
        packed.y = pack_bf16((w[u].z * __low2float(hi)) / denom, (w[u].w * __high2float(hi)) / denom);
        *reinterpret_cast<uint2*>(dst + 4 * k4) = packed;
      }
    }
  }
  consumer_sync();
}

// act[n, :] = src[n, :] (bfloat16 rows of K elements written earlier in this kernel)
__device__ __forceinline__ void load_act_plain(const DecodeParams& p, __nv_bfloat16* act, const __nv_bfloat16* src, int K,
                                               uint64_t* act_bar, volatile int* s_abort, ConsumerState& st) {
  fetch_rows_issue(p, act, src, (uint32_t)K * 2u, nullptr, 0u, act_bar);
  fetch_rows_wait(p, act_bar, s_abort, st);
  consumer_sync();
}

// What warp 0 does with a finished tile: c[0], c[1] are row g of the tile for tokens 2 t4, 2 t4 + 1;
// c[2], c[3] are row g + 8.
template <int KIND>
__device__ __forceinline__ void epilogue(const DecodeParams& p, const DecodeLayer* L, int t, const float* c) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  if constexpr (KIND == K_O || KIND == K_DOWN) {
    // the residual stream's owner of each element adds the product and leaves the tile's share of
    // sum(x^2) for the norm that follows
    float sq[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int n = t4 * 2 + e;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = 16 * t + g + 8 * h;
        if (n < p.m && row < p.hidden) {
          float* at = p.resid + (size_t)n * p.hidden + row;
          const float v = __ldcg(at) + c[2 * h + e];
          __stcg(at, v);
          sq[e] += v * v;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      sq[e] += __shfl_xor_sync(0xffffffffu, sq[e], 4);
      sq[e] += __shfl_xor_sync(0xffffffffu, sq[e], 8);
      sq[e] += __shfl_xor_sync(0xffffffffu, sq[e], 16);
      if (g == 0 && t4 * 2 + e < p.m) p.ssq_part[(size_t)t * MAX_TOKENS + t4 * 2 + e] = sq[e];
    }
  } else {
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int n = t4 * 2 + e;
    if (n >= p.m) continue;
    if (KIND == K_QKV) {
      const int head = t / (HD / 16), j = t % (HD / 16);
      const int d_lo = 8 * j + g, d_hi = HD / 2 + d_lo;
      // the projection's output is a bfloat16 tensor of the model: rounded before the rotation
      const float x_lo = __bfloat162float(__float2bfloat16_rn(c[e])), x_hi = __bfloat162float(__float2bfloat16_rn(c[2 + e]));
      float o_lo = x_lo, o_hi = x_hi;
      if (head < p.nq + p.nkv && L->cos != nullptr) {
        const size_t at = (size_t)p.positions[n] * (HD / 2) + d_lo;
        const float cs = L->cos[at], sn = L->sin[at];
        o_lo = cs * x_lo - sn * x_hi;
        o_hi = sn * x_lo + cs * x_hi;
      }
      __nv_bfloat16* dst;
      if (head < p.nq) {
        dst = p.q_buf + (size_t)n * p.nq * HD + (size_t)head * HD;
      } else {
        const int slot = L->slot_mapping[n];
        if (slot < 0) continue;
        const bool is_v = head >= p.nq + p.nkv;
        const int kvh = head - p.nq - (is_v ? p.nkv : 0);
        dst = (is_v ? L->vcache : L->kcache) +
              ((size_t)(slot / p.page_size) * p.nkv + kvh) * p.page_size * HD + (size_t)(slot % p.page_size) * HD;
      }
      dst[d_lo] = __float2bfloat16_rn(o_lo);
      dst[d_hi] = __float2bfloat16_rn(o_hi);
    } else if (KIND == K_GATE_UP) {
      const int col = 8 * t + g;
      if (col < p.inter) {
        const float gate = c[e], up = c[2 + e];
        p.ffn_act[(size_t)n * p.inter + col] = __float2bfloat16_rn(silu_f(gate) * up);
      }
    } else {   // K_LM_HEAD
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = 16 * t + g + 8 * h;
        if (row < p.vocab) p.logits[(size_t)n * p.vocab + row] = c[2 * h + e];
      }
    }
  }
  }
}

// One projection phase: this CTA's tiles of one weight matrix against the activations in `act`.
template <int KIND>
__device__ __forceinline__ void project(const DecodeParams& p, const DecodeLayer* L, const uint8_t* ring, float* red,
                                        const __nv_bfloat16* act, uint64_t* full_bar, uint64_t* empty_bar, volatile int* s_abort,
                                        ConsumerState& st) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int T = phase_tiles(p, KIND), K = phase_k(p, KIND), G = (int)gridDim.x;
  const uint32_t S = (uint32_t)p.stages;
  for (int t = first_tile(st.rr); t < T; t += G) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += KC) {
      const int kc = min(KC, K - k0);
      const uint32_t stage = st.taken % S, use = st.taken / S;
      // after a give-up the wait returns at once and the numbers no longer matter
#ifdef TLLM_STEP_TIMING
      const long long w0 = clock64();
#endif
      mbar_wait(&full_bar[stage], use & 1, s_abort, p.status, ERR_STEP_CONSUMER);
#ifdef TLLM_STEP_TIMING
      st.t_full += clock64() - w0;
#endif
      const uint8_t* chunk = ring + (size_t)stage * STAGE_BYTES;
      for (int ks = warp; ks < kc / 16; ks += CONSUMER_WARPS) {
        uint32_t a[4];
        ldmatrix_x4(a, chunk + (lane & 15) * ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
        const __nv_bfloat16* bp = act + (size_t)g * p.act_ld + k0 + ks * 16 + t4 * 2;
        mma_bf16(acc, a, *reinterpret_cast<const uint32_t*>(bp), *reinterpret_cast<const uint32_t*>(bp + 8));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      ++st.taken;
    }
#ifdef TLLM_STEP_TIMING
    const long long e0 = clock64();
#endif
    float4* mine = reinterpret_cast<float4*>(red) + (st.red_buf * CONSUMER_WARPS + warp) * 32 + lane;
    *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
    consumer_sync();
    if (warp == 0) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < CONSUMER_WARPS; ++w) {
        const float4 v = reinterpret_cast<const float4*>(red)[(st.red_buf * CONSUMER_WARPS + w) * 32 + lane];
        c[0] += v.x; c[1] += v.y; c[2] += v.z; c[3] += v.w;
      }
      epilogue<KIND>(p, L, t, c);
    }
#ifdef TLLM_STEP_TIMING
    st.t_epi += clock64() - e0;
#endif
    st.red_buf ^= 1;
  }
  st.rr = (st.rr + T) % G;
}

__device__ __forceinline__ void attention_phase(const DecodeParams& p, const DecodeLayer* L, uint8_t* team_smem) {
  const int team = threadIdx.x >> 7, tid = threadIdx.x & 127;
  if (team >= TEAMS) return;
  AttnParams ap;
  ap.q = p.q_buf; ap.kcache = L->kcache; ap.vcache = L->vcache; ap.block_table = L->block_table;
  ap.cu_q = p.cu_q; ap.q_start = p.positions; ap.out = p.attn_out; ap.part_o = p.part_o; ap.part_ml = p.part_ml;
  ap.head_stride = (long long)p.page_size * HD; ap.page_stride = ap.head_stride * p.nkv;
  ap.q_row_stride = p.nq * HD; ap.max_blocks = p.max_blocks; ap.nq = p.nq; ap.nkv = p.nkv; ap.page_size = p.page_size;
  ap.window = L->window; ap.tiles_per_req = 1; ap.splits = p.splits; ap.n_requests = p.m; ap.scale_log2 = L->scale_log2;
  const int items = p.m * p.nkv * p.splits;
  auto team_sync = [team] { named_sync(2 + team, 128); };
  for (int it = (int)blockIdx.x * TEAMS + team; it < items; it += (int)gridDim.x * TEAMS) {
    const int split = it % p.splits, kvh = (it / p.splits) % p.nkv, req = it / (p.splits * p.nkv);
    attention_decode_item<ATT_STAGES>(ap, req, kvh, split, tid, team_smem + (size_t)team * TEAM_BYTES, team_sync, [] {});
    team_sync();
  }
}

// Merges the slices of every (token, head), one warp per row.
__device__ __forceinline__ void combine_phase(const DecodeParams& p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = p.m * p.nq;
  for (int row = (int)blockIdx.x * CONSUMER_WARPS + warp; row < rows; row += (int)gridDim.x * CONSUMER_WARPS)
    attention_combine_row(p.part_o, p.part_ml, p.attn_out, p.splits, (size_t)row, lane);
}

__device__ void consume(const DecodeParams& p, uint8_t* ring, float* red, uint8_t* uni, uint64_t* full_bar,
                        uint64_t* empty_bar, uint64_t* act_bar, volatile int* s_abort) {
  ConsumerState st = {};
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(uni);
  T_BEGIN();
  for (int layer = 0; layer < p.n_layers; ++layer) {
    const DecodeLayer* L = p.layers + layer;
    if (layer == 0) load_act_embedding(p, act, L->norm1, L->eps1);
    else load_act_norm(p, act, L->norm1, L->eps1, act_bar, s_abort, st);
    T_ADD(0);
    project<K_QKV>(p, L, ring, red, act, full_bar, empty_bar, s_abort, st);
    T_ADD(1);
    if (!grid_barrier(p, s_abort, st)) return;
    T_ADD(2);
    attention_phase(p, L, uni);
    T_ADD(3);
    if (!grid_barrier(p, s_abort, st)) return;
    T_ADD(2);
    if (p.splits > 1) {
      combine_phase(p);
      T_ADD(4);
      if (!grid_barrier(p, s_abort, st)) return;
      T_ADD(2);
    }
    load_act_plain(p, act, p.attn_out, p.nq * HD, act_bar, s_abort, st);
    T_ADD(5);
    project<K_O>(p, L, ring, red, act, full_bar, empty_bar, s_abort, st);
    T_ADD(6);
    if (!grid_barrier(p, s_abort, st)) return;
    T_ADD(2);
    load_act_norm(p, act, L->norm2, L->eps2, act_bar, s_abort, st);
    T_ADD(0);
    project<K_GATE_UP>(p, L, ring, red, act, full_bar, empty_bar, s_abort, st);
    T_ADD(7);
    if (!grid_barrier(p, s_abort, st)) return;
    T_ADD(2);
    load_act_plain(p, act, p.ffn_act, p.inter, act_bar, s_abort, st);
    T_ADD(5);
    project<K_DOWN>(p, L, ring, red, act, full_bar, empty_bar, s_abort, st);
    T_ADD(8);
    if (!grid_barrier(p, s_abort, st)) return;
    T_ADD(2);
  }
  load_act_norm(p, act, p.final_norm, p.final_eps, act_bar, s_abort, st);
  T_ADD(0);
  project<K_LM_HEAD>(p, nullptr, ring, red, act, full_bar, empty_bar, s_abort, st);
  T_ADD(9);
  // the last CTA to get here has seen every CTA pass every barrier: it clears the counters for the next step
  if (threadIdx.x == 0) {
    const unsigned long long finished = atomicAdd(p.sync_words + 2, 1ull);
    if (finished == gridDim.x - 1) {
      p.sync_words[0] = 0ull;
      p.sync_words[2] = 0ull;
      __threadfence();
    }
  }
#ifdef TLLM_STEP_TIMING
  if (blockIdx.x == TLLM_STEP_TIMING - 1 && threadIdx.x == 0) {
    g_step_timing[12] += (unsigned long long)st.t_full;
    g_step_timing[13] += (unsigned long long)st.t_epi;
  }
#endif
}

__global__ void __launch_bounds__(THREADS, 1) decode_step_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t act_bar;
  __shared__ int s_abort;
  uint8_t* ring = smem;
  float* red = reinterpret_cast<float*>(smem + (size_t)p.stages * STAGE_BYTES);
  uint8_t* uni = reinterpret_cast<uint8_t*>(red) + RED_BYTES;   // activations, or the attention teams' tiles
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], CONSUMER_WARPS); }
    mbar_init(&act_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x >= CONSUMERS) {
    produce(p, ring, full_bar, empty_bar, &s_abort);
  } else {
    consume(p, ring, red, uni, full_bar, empty_bar, &act_bar, &s_abort);
  }
}

inline int union_bytes(int act_ld, int hidden) {
  const int act = MAX_TOKENS * act_ld * 2 + hidden * 4, att = TEAMS * TEAM_BYTES;   // rows, then a norm's weight
  return act > att ? act : att;
}

}  // namespace tllm

using namespace tllm;

#ifdef TLLM_STEP_TIMING
// Cycles CTA (TLLM_STEP_TIMING - 1)'s thread 0 spent per phase kind since the last call; clears them.
extern "C" int tllm_decode_step_timing(unsigned long long* out16) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out16, g_step_timing, sizeof(unsigned long long) * 16);
  unsigned long long zero[16] = {};
  cudaMemcpyToSymbol(g_step_timing, zero, sizeof(zero));
  return 0;
}
#endif

extern "C" int tllm_decode_step_head_dim() { return HD; }
extern "C" int tllm_decode_step_max_tokens() { return MAX_TOKENS; }
extern "C" int tllm_decode_step_teams() { return TEAMS; }
extern "C" int tllm_decode_step_layer_bytes() { return (int)sizeof(DecodeLayer); }
extern "C" int tllm_decode_step_params_bytes() { return (int)sizeof(DecodeParams); }

// Fills in what the kernel derives from the sizes (stages of the ring, row stride of the activations)
// and says whether the step can run as this kernel.  `launch` = 0 only checks.
extern "C" int tllm_decode_step(DecodeParams* hp, int launch, void* stream) {
  DecodeParams& p = *hp;
  TLLM_REQUIRE(p.m >= 1 && p.m <= MAX_TOKENS, "decode_step: %d tokens (takes 1 to %d)", p.m, MAX_TOKENS);
  TLLM_REQUIRE(p.n_layers >= 1 && p.nq >= 1 && p.nkv >= 1 && p.nq % p.nkv == 0 && p.nq / p.nkv <= 16,
               "decode_step: %d layers, %d heads, %d key/value heads (at most 16 heads per key/value head)", p.n_layers, p.nq, p.nkv);
  TLLM_REQUIRE(p.hidden >= 16 && p.hidden % 16 == 0 && p.inter >= 16 && p.inter % 16 == 0 && p.vocab >= 1,
               "decode_step: width %d and feed-forward width %d must be multiples of 16", p.hidden, p.inter);
  TLLM_REQUIRE(p.gu_block >= 1 && p.inter % p.gu_block == 0, "decode_step: gate/up block %d does not divide %d", p.gu_block, p.inter);
  TLLM_REQUIRE(p.page_size >= 1 && p.max_blocks >= 1 && p.splits >= 1 && p.splits <= 32,
               "decode_step: page size %d, %d blocks, %d slices of keys (at most 32)", p.page_size, p.max_blocks, p.splits);
  int device = 0, sms = 0, smem_max = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  int widest = p.hidden > p.inter ? p.hidden : p.inter;
  if (p.nq * HD > widest) widest = p.nq * HD;
  if (2 * p.hidden > widest) widest = 2 * p.hidden;   // a row also takes its token's 32-bit residual row on the way in
  p.act_ld = widest + 8;
  const int fixed = RED_BYTES + union_bytes(p.act_ld, p.hidden) + 1024;   // 1024: the static shared memory, rounded up
  int stages = (smem_max - fixed) / STAGE_BYTES;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  TLLM_REQUIRE(stages >= MIN_STAGES, "decode_step: activations of %d values per token leave no room for the weight ring", widest);
  p.stages = stages;
  const int smem = stages * STAGE_BYTES + RED_BYTES + union_bytes(p.act_ld, p.hidden);
  static int configured = 0;
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "decode_step: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, THREADS, smem);
  if (e != cudaSuccess || per_sm < 1) TLLM_FAIL(TLLM_ERR_CUDA, "decode_step: the kernel does not fit an SM (%d bytes of shared memory)", smem);
  if (!launch) return TLLM_OK;
  TLLM_REQUIRE(p.layers && p.tokens && p.positions && p.cu_q && p.embed && p.final_norm && p.lm_head && p.resid && p.q_buf &&
               p.attn_out && p.ffn_act && p.logits && p.ssq_part && p.sync_words && p.status && (p.splits == 1 || (p.part_o && p.part_ml)),
               "decode_step: a buffer is missing");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sms);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident: the grid barrier cannot starve
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
  if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "decode_step: %s", cudaGetErrorString(e));
  return TLLM_OK;
}
