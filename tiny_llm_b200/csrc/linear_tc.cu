// bfloat16 matrix products on the 5th-generation tensor cores: C[M,N] = A[M,K] . W[N,K]^T with
// 32-bit accumulation in tensor memory.
//
//   * operands reach shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast),
//     STAGES deep, signalled on mbarriers;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN, K = 16 per
//     instruction); tcgen05.commit releases each stage and, at the end, hands the accumulator over;
//   * four warps read the accumulator back with tcgen05.ld and run the epilogue on 32-bit values:
//     store bfloat16 / store float32 / add into a float32 output / SiLU(gate) * up / split-K
//     atomics into a float32 output.
//
// Two orientations share the main loop.  NORMAL: the 128-row operand is A (tokens), the BN-row
// operand is W: one CTA makes a 128 x BN tile of C (prefill).  SWAP: the 128-row operand is W and the
// BN-row operand is A, BN = the token count rounded up to 16: one CTA makes C^T for 128 weight rows,
// so that at decode the weights fill the 128-wide side of the MMA and stream through the pipeline;
// grid.z splits K so that every SM streams a slice, and two such CTAs fit an SM.
//
// Sizes: any M and N; K a multiple of 8 (the 16-byte rule of TMA row strides); tails of all three
// are zero-filled by TMA and masked in the epilogue.  Every wait on an mbarrier is bounded: on
// expiry the kernel records a code in `status`, stops issuing, frees its tensor memory and returns.
//
// Reference counterparts: tiny_llm/ops/cuda/gemm.cu:67-106 (SIMT tile product) and
// gemm_q1_helper.cu:15-124 (warp-per-output GEMV for one row).
#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int BM = 128;        // rows of the 128-row operand per CTA = MMA M
constexpr int BK = 64;         // K elements per stage = one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;   // warp 0: TMA, warp 1: MMA + tensor-memory allocation, warps 2-5: epilogue

enum Epilogue { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3, EPI_ATOMIC_F32 = 4,
                // cluster kernel: K slices reduced through distributed shared memory
                EPI_CL_ADD_F32 = 5, EPI_CL_ROPE_KV = 6, EPI_CL_SWIGLU = 7, EPI_CL_BF16 = 8,
                // NORMAL orientation: Q/K/V projection with rotation and cache write (head size 64 or 128)
                EPI_ROPE_KV = 9 };

constexpr int ERR_PRODUCER = 1, ERR_MMA = 2, ERR_EPILOGUE = 3;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;   // + alignment slack
};

// What the rotate-and-cache epilogues need (either orientation); cy, cz only concern the cluster kernel.
struct ClusterArgs {
  int cy, cz;                      // cluster extent over row tiles (1, or 2 for gate/up pairs) and over K slices
  const int* positions;            // [tokens]
  const float* cos;                // [positions, hd / 2] or null: no rotation
  const float* sin;
  __nv_bfloat16* kcache;           // [pages, nkv, page_size, hd]
  __nv_bfloat16* vcache;
  const int* slot_mapping;         // [tokens] or null: the rows hold queries only
  long long page_stride, head_stride;
  int nq, nkv, hd, page_size;
  // persistent kernel: the tiles of the last, incomplete round are cut into strips of `tail_width` columns so
  // that they spread over all SMs (0: no cutting); tiles [0, tail_from) are whole
  int tail_from, tail_width;
  // persistent kernel, residual-adding epilogue only: every tile is cut into `k_splits` runs of k-blocks that
  // different CTAs add into the output (0 or 1: whole K per tile); fills the SMs when there are few tiles
  int k_splits, k_per;             // runs per tile and k-blocks per run (the last run may be shorter, never empty)
  int out_by_tma;                  // residual-adding epilogue: the sums leave as TMA reductions (the output's map is valid)
};

// Epilogue of one 128 x BN tile of C in the NORMAL orientation: this thread owns row `row` of the
// tile (tensor-memory lane), walks its BN columns in chunks of 32 and stores them as EPI says.
// Q/K/V projection, NORMAL orientation: this thread owns token `m`; the tile's BN columns are whole
// heads.  Per head the two halves of the rotation pairs are read 32 columns at a time, rounded to
// bfloat16 (the projection's output is a bfloat16 tensor of the model), rotated in 32-bit and
// written: queries to the row of `out`, keys and values to the token's slot of the cache.
template <int BN>
__device__ __forceinline__ void store_tile_rope_kv(uint32_t taddr, int m, int n_first, int width, int rows_a, int rows_b,
                                                   void* __restrict__ out, int ldo, const ClusterArgs& ca) {
  const int hd = ca.hd, half = hd / 2;   // 64 or 128: half = 32 or 64
  const bool row_ok = m < rows_a;
  int pos = 0, slot = -1;
  if (row_ok) {
    pos = ca.positions ? ca.positions[m] : 0;
    slot = ca.slot_mapping ? ca.slot_mapping[m] : -1;
  }
  // 32 rotation pairs at a time: their cosines and sines are loaded once (16-byte loads from this token's
  // row of the tables) and serve every head of the tile
#pragma unroll 1
  for (int sub = 0; sub < half; sub += 32) {
    float cs[32], sn[32];
    const bool tables = row_ok && ca.cos != nullptr;
    if (tables) {
      const float4* c4 = reinterpret_cast<const float4*>(ca.cos + (size_t)pos * half + sub);
      const float4* s4 = reinterpret_cast<const float4*>(ca.sin + (size_t)pos * half + sub);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 c = c4[j], s = s4[j];
        cs[4 * j] = c.x; cs[4 * j + 1] = c.y; cs[4 * j + 2] = c.z; cs[4 * j + 3] = c.w;
        sn[4 * j] = s.x; sn[4 * j + 1] = s.y; sn[4 * j + 2] = s.z; sn[4 * j + 3] = s.w;
      }
    }
#pragma unroll 1
    for (int h0 = 0; h0 < width; h0 += hd) {
      const int n0 = n_first + h0;              // first column of this head
      const int head = n0 / hd;
      float lo[32], hi[32];
      tmem_ld32(taddr + h0 + sub, lo);          // warp-wide: every lane reads, whatever it stores
      tmem_ld32(taddr + h0 + half + sub, hi);
      if (!row_ok || n0 >= rows_b) continue;
      const bool is_q = head < ca.nq, is_v = head >= ca.nq + ca.nkv;
      __nv_bfloat16* dst;
      if (is_q) {
        dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n0;
      } else {
        if (slot < 0) continue;
        dst = (is_v ? ca.vcache : ca.kcache) + (long long)(slot / ca.page_size) * ca.page_stride +
              (long long)(head - ca.nq - (is_v ? ca.nkv : 0)) * ca.head_stride + (long long)(slot % ca.page_size) * hd;
      }
      const bool rotate = !is_v && tables;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pl, ph;
        __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&pl);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&ph);
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float o_lo[2], o_hi[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float x = __bfloat162float(__float2bfloat16_rn(lo[j + e + u])), y = __bfloat162float(__float2bfloat16_rn(hi[j + e + u]));
            o_lo[u] = rotate ? cs[j + e + u] * x - sn[j + e + u] * y : x;
            o_hi[u] = rotate ? sn[j + e + u] * x + cs[j + e + u] * y : y;
          }
          l2[e / 2] = __floats2bfloat162_rn(o_lo[0], o_lo[1]);
          h2[e / 2] = __floats2bfloat162_rn(o_hi[0], o_hi[1]);
        }
        *reinterpret_cast<uint4*>(dst + sub + j) = pl;
        *reinterpret_cast<uint4*>(dst + half + sub + j) = ph;
      }
    }
  }
}

template <int BN, int EPI>
__device__ __forceinline__ void store_tile_normal(uint32_t taddr, int row, int tile_a, int tile_b, int rows_a,
                                                  int rows_b, void* __restrict__ out, int ldo) {
  // 16-byte stores need an aligned base and row stride
  const bool vec_ok = (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                      ((EPI == EPI_BF16 || EPI == EPI_SWIGLU) ? (ldo & 7) == 0 : (ldo & 3) == 0);
  const int m = tile_a * BM + row;
  if (EPI == EPI_SWIGLU) {
    // columns [0, BN/2) are gate, [BN/2, BN) the matching up columns; output tile is BN/2 wide
    const int n0 = tile_b * (BN / 2);
    const int n_out = rows_b / 2;
#pragma unroll 1
    for (int c = 0; c < BN / 2; c += 32) {
      float g[32], u[32];
      tmem_ld32(taddr + c, g);
      tmem_ld32(taddr + BN / 2 + c, u);
      if (m < rows_a && n0 + c < n_out) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n0 + c;
        if (n0 + c + 32 <= n_out && vec_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h[e] = __floats2bfloat162_rn(silu_f(g[j + 2 * e]) * u[j + 2 * e], silu_f(g[j + 2 * e + 1]) * u[j + 2 * e + 1]);
            *reinterpret_cast<uint4*>(dst + j) = pk;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (n0 + c + j < n_out) dst[j] = __float2bfloat16_rn(silu_f(g[j]) * u[j]);
        }
      }
    }
  } else {
    const int n0 = tile_b * BN;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      float v[32];
      tmem_ld32(taddr + c, v);
      if (m < rows_a && n0 + c < rows_b) {
        const bool full = n0 + c + 32 <= rows_b;
        if (EPI == EPI_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n0 + c;
          if (full && vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
              *reinterpret_cast<uint4*>(dst + j) = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c + j < rows_b) dst[j] = __float2bfloat16_rn(v[j]);
          }
        } else {
          float* dst = reinterpret_cast<float*>(out) + (size_t)m * ldo + n0 + c;
          if (full && vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (EPI == EPI_ADD_F32) {
                // the add happens in L2 (a 16-byte reduction, nothing comes back): a load, an add and a store
                // per chunk would make the epilogue a chain of round trips
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]),
                             "f"(v[j + 3]) : "memory");
              } else {
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c + j < rows_b) {
                if (EPI == EPI_ADD_F32) atomicAdd(dst + j, v[j]);   // (runs of K of the same tile add side by side)
                else dst[j] = v[j];
              }
          }
        }
      }
    }
  }
}

// SiLU(gate) * up for a STRIP of a gate/up tile: the accumulator holds `w` gate columns and, behind them, the `w`
// matching up columns; the strip's results go to output columns [out_col, out_col + w).  This thread owns row m.
__device__ __forceinline__ void store_strip_swiglu(uint32_t taddr, int m, int out_col, int w, int rows_a, int n_out,
                                                   __nv_bfloat16* __restrict__ out, int ldo) {
  const bool vec_ok = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ldo & 7) == 0;
#pragma unroll 1
  for (int c = 0; c < w; c += 32) {
    float g[32], u[32];
    tmem_ld32(taddr + c, g);
    tmem_ld32(taddr + w + c, u);
    if (m < rows_a && out_col + c < n_out) {
      __nv_bfloat16* dst = out + (size_t)m * ldo + out_col + c;
      if (out_col + c + 32 <= n_out && vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            h[e] = __floats2bfloat162_rn(silu_f(g[j + 2 * e]) * u[j + 2 * e], silu_f(g[j + 2 * e + 1]) * u[j + 2 * e + 1]);
          *reinterpret_cast<uint4*>(dst + j) = pk;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (out_col + c + j < n_out) dst[j] = __float2bfloat16_rn(silu_f(g[j]) * u[j]);
      }
    }
  }
}

// rows_a / rows_b: extents of the 128-row operand and of the BN-row operand.  NORMAL: rows_a = M,
// rows_b = N, out[M, N].  SWAP: rows_a = N (weights), rows_b = M (tokens), out[M, N] all the same.
template <int BN, int STAGES, bool SWAP, int EPI>
__global__ void __launch_bounds__(THREADS, SWAP ? 2 : 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 void* __restrict__ out, int rows_a, int rows_b, int k_blocks, int k_blocks_per_split, int ldo,
                 int* __restrict__ status) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }   // the descriptors are on their way while the barriers are set up
  const int tile_a = blockIdx.y, tile_b = blockIdx.x;
  const int kb_begin = blockIdx.z * k_blocks_per_split;
  const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
  const int n_kb = kb_end - kb_begin;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The weight operand (A when SWAP, else B) depends on no earlier kernel: its first STAGES tiles are
  // requested before this grid waits for its predecessors, so they stream in under their tail.
  pdl_trigger();
  const int n_pre = min(n_kb, STAGES);
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < n_pre; ++i) {
      mbar_expect_tx(&full_bar[i], L::STAGE_BYTES);
      uint8_t* a_dst = smem + i * L::STAGE_BYTES;
      if (SWAP) tma_load_2d_hint(a_dst, &map_a, (kb_begin + i) * BK, tile_a * BM, &full_bar[i], l2_evict_first_policy());
      else tma_load_2d(a_dst + L::A_BYTES, &map_b, (kb_begin + i) * BK, tile_b * BN, &full_bar[i]);
    }
  }
  pdl_wait();
  trace_tag(((unsigned long long)rows_a << 40) | ((unsigned long long)rows_b << 20) | (unsigned long long)k_blocks);   // which product (timeline builds only)

  if (n_kb > 0) {
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % STAGES;
        uint8_t* a_dst = smem + s * L::STAGE_BYTES;
        const bool pre = i < n_pre;   // the weight tile of this stage is already on its way
        if (!pre) {
          const uint32_t parity = ((i / STAGES) & 1) ^ 1;
          if (!mbar_wait(&empty_bar[s], parity, abort_flag)) { *abort_flag = 1; atomicExch(status, ERR_PRODUCER); break; }
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
        }
        if (!pre || !SWAP) {
          if (SWAP) tma_load_2d_hint(a_dst, &map_a, (kb_begin + i) * BK, tile_a * BM, &full_bar[s], l2_evict_first_policy());   // weights: read once per step
          else tma_load_2d(a_dst, &map_a, (kb_begin + i) * BK, tile_a * BM, &full_bar[s]);
        }
        if (!pre || SWAP) tma_load_2d(a_dst + L::A_BYTES, &map_b, (kb_begin + i) * BK, tile_b * BN, &full_bar[s]);
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer: the whole warp walks the loop and waits, one elected lane issues (a loop
      // walked by one lane alone spends about twice as long between two stages)
      const uint32_t idesc = instr_desc_bf16(BM, BN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t lo0 = smem_desc_sw128_lo(smem_u32(smem));
      bool ok = true;
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t parity = (i / STAGES) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = lo0 + s * (L::STAGE_BYTES >> 4), b_lo = a_lo + (L::A_BYTES >> 4);   // descriptors count in 16-byte units
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_lo(tmem_u, a_lo + (k * UMMA_K * 2 >> 4), b_lo + (k * UMMA_K * 2 >> 4), idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
        }
        __syncwarp();
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, ERR_MMA); }
      if (elect_one()) umma_commit(acc_bar);   // arrives when every MMA issued so far has completed
      __syncwarp();
    } else if (warp >= 2) {
      // ---------------- epilogue: warp w reads tensor-memory lanes [32 (w % 4), +32)
      const int quad = warp & 3;
      const int row = quad * 32 + lane;             // row of the 128-row operand within the tile
      bool ok = mbar_wait(acc_bar, 0, abort_flag);
      if (!ok) { *abort_flag = 1; atomicExch(status, ERR_EPILOGUE); }
      ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-wide: all lanes or none
      tc_fence_after();
      if (ok) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
        if (!SWAP) {
          store_tile_normal<BN, EPI>(taddr, row, tile_a, tile_b, rows_a, rows_b, out, ldo);
        } else {
          // SWAP: this thread's row is weight row n; tensor-memory column j is token tile_b*BN + j.
          // For a fixed token the 32 lanes of a warp write 32 consecutive n: coalesced.
          const int n = tile_a * BM + row;
          const int m0 = tile_b * BN;
#pragma unroll 1
          for (int c = 0; c < BN; c += 16) {
            float v[16];
            tmem_ld16(taddr + c, v);
            if (n < rows_a) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c + j;
                if (m < rows_b) {
                  const size_t o = (size_t)m * ldo + n;
                  if (EPI == EPI_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v[j]);
                  else if (EPI == EPI_F32) reinterpret_cast<float*>(out)[o] = v[j];
                  else if (EPI == EPI_ADD_F32) reinterpret_cast<float*>(out)[o] += v[j];
                  else if (EPI == EPI_ATOMIC_F32) atomicAdd(reinterpret_cast<float*>(out) + o, v[j]);
                }
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------- cluster kernel, SWAP orientation
// Few rows of A (decode): a weight tile of 128 rows has too little work for an SM unless K is split,
// and there are too few tiles for all SMs unless K is split too.  Here the CZ slices of K of one tile
// (and, for SiLU*up, the gate tile and the up tile beside it: CY = 2) run as one thread-block
// cluster.  Every CTA accumulates its slice in tensor memory as in linear_tc_kernel, leaves the
// 128 x BN accumulators in its own shared memory, and after a cluster barrier each CTA reduces its
// share of the tile's rows over the peers' shared memory (ld.shared::cluster) and applies the
// epilogue once: no atomics, no float32 scratch for a later kernel to convert, and the order of the
// sum is fixed.  Epilogues: add into the float32 residual stream; round to bfloat16, rotate Q and K
// by position and write K, V into their pages (a tile holds whole heads, so both halves of a rotation
// pair are at hand); SiLU(gate) * up; plain bfloat16 store.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// four floats at byte address `addr` of this CTA's shared memory, read from the CTA of rank `rank` in the cluster
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// One work item of the rotate-and-cache epilogue: four neighbouring rotation pairs of one token.  What it
// needs from global memory (position, slot, cosines, sines) depends on the step's tables only, so the
// first item of every thread is fetched when the kernel starts and waits in registers.
struct RopeItem {
  bool valid;
  bool rotate;
  int j, r_lo, d, head, m;
  int slot;
  float4 cs, sn;
};
template <int BN>
__device__ __forceinline__ RopeItem rope_item(const ClusterArgs& ca, int idx, int tile_a, int m0, int rows_a, int rows_b) {
  RopeItem it;
  const int half = ca.hd / 2, CZ = ca.cz;
  const int pairs_per = ((BM / 2 + CZ - 1) / CZ + 3) & ~3, p0 = (int)blockIdx.z * pairs_per, quads = pairs_per / 4;
  it.j = idx / quads;
  const int q = p0 + (idx % quads) * 4;
  it.r_lo = (q / half) * ca.hd + q % half;
  it.m = m0 + it.j;
  const int n_lo = tile_a * BM + it.r_lo;
  it.valid = idx < quads * BN && it.m < rows_b && q < BM / 2 && n_lo + half < rows_a;   // heads are whole: the four pairs exist together
  it.head = n_lo / ca.hd;
  it.d = n_lo % ca.hd;
  it.rotate = false;
  it.slot = -1;
  it.cs = it.sn = make_float4(0.f, 0.f, 0.f, 0.f);
  if (it.valid) {
    it.rotate = it.head < ca.nq + ca.nkv && ca.cos != nullptr;
    if (it.head >= ca.nq && ca.slot_mapping != nullptr) it.slot = ca.slot_mapping[it.m];
    if (it.rotate) {
      const size_t t = (size_t)ca.positions[it.m] * half + it.d;   // d is a multiple of four: 16-byte loads
      it.cs = *reinterpret_cast<const float4*>(ca.cos + t);
      it.sn = *reinterpret_cast<const float4*>(ca.sin + t);
    }
  }
  return it;
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 2)
linear_tc_cluster_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         void* __restrict__ out, int rows_a, int rows_b, int k_blocks, int k_blocks_per_split, int ldo,
                         const ClusterArgs ca, int* __restrict__ status) {
  using L = SmemLayout<BN, STAGES>;
  static_assert(BN * BM * 4 <= STAGES * L::STAGE_BYTES, "the accumulators are parked in the pipeline's stages");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* parked = reinterpret_cast<float*>(smem);   // [BN tokens][128 rows] once the MMAs are done

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }   // the descriptors are on their way while the barriers are set up
  const int tile_a = blockIdx.y, tile_b = blockIdx.x;
  const int kb_begin = blockIdx.z * k_blocks_per_split;
  const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
  const int n_kb = max(0, kb_end - kb_begin);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  RopeItem first_item = {};
  if (EPI == EPI_CL_ROPE_KV) first_item = rope_item<BN>(ca, threadIdx.x, tile_a, tile_b * BN, rows_a, rows_b);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // the first weight tiles are requested before this grid waits for its predecessors
  pdl_trigger();
  const int n_pre = min(n_kb, STAGES);
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < n_pre; ++i) {
      mbar_expect_tx(&full_bar[i], L::STAGE_BYTES);
      tma_load_2d_hint(smem + i * L::STAGE_BYTES, &map_a, (kb_begin + i) * BK, tile_a * BM, &full_bar[i], l2_evict_first_policy());
    }
  }
  pdl_wait();
  trace_tag(((unsigned long long)rows_a << 40) | ((unsigned long long)rows_b << 20) | (unsigned long long)k_blocks);   // which product (timeline builds only)

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    const uint64_t once = l2_evict_first_policy();   // the weights are read once per step
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % STAGES;
      uint8_t* a_dst = smem + s * L::STAGE_BYTES;
      const bool pre = i < n_pre;
      if (!pre) {
        const uint32_t parity = ((i / STAGES) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[s], parity, abort_flag)) { *abort_flag = 1; atomicExch(status, ERR_PRODUCER); break; }
        mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
        tma_load_2d_hint(a_dst, &map_a, (kb_begin + i) * BK, tile_a * BM, &full_bar[s], once);
      }
      tma_load_2d(a_dst + L::A_BYTES, &map_b, (kb_begin + i) * BK, tile_b * BN, &full_bar[s]);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (warp-wide loop, one elected lane issues)
    const uint32_t idesc = instr_desc_bf16(BM, BN);
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t lo0 = smem_desc_sw128_lo(smem_u32(smem));
    bool ok = true;
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % STAGES;
      const uint32_t parity = (i / STAGES) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_lo = lo0 + s * (L::STAGE_BYTES >> 4), b_lo = a_lo + (L::A_BYTES >> 4);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16_lo(tmem_u, a_lo + (k * UMMA_K * 2 >> 4), b_lo + (k * UMMA_K * 2 >> 4), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, ERR_MMA); }
    if (elect_one()) umma_commit(acc_bar);
    __syncwarp();
  } else if (warp >= 2) {
    // ---------------- park the accumulators: warp w reads tensor-memory lanes [32 (w % 4), +32)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    bool ok = true;
    if (n_kb > 0) {
      ok = mbar_wait(acc_bar, 0, abort_flag);
      if (!ok) { *abort_flag = 1; atomicExch(status, ERR_EPILOGUE); }
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
    }
    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      float v[16];
      if (n_kb > 0 && ok) {
        tmem_ld16(taddr + c, v);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;   // a slice without K blocks adds nothing
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) parked[(c + j) * BM + row] = v[j];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);

  // ---------------- every CTA of the cluster has parked its slice: reduce and store
  // Work items are four consecutive rows of one token: one 16-byte load per peer, all peers' loads in flight.
  cluster_sync_all();
  const int CY = ca.cy, CZ = ca.cz;
  const int my_y = blockIdx.y % CY, my_z = blockIdx.z;
  const uint32_t base = smem_u32(parked);
  const int m0 = tile_b * BN;
  if (EPI == EPI_CL_SWIGLU) {
    // ranks (0, z) hold the gate tile's slices, ranks (1, z) the up tile's; the 128 rows are dealt to all CY * CZ CTAs
    // (shares are whole groups of four rows; with 6 CTAs the last share is short)
    const int rows_per = ((BM + CY * CZ - 1) / (CY * CZ) + 3) & ~3, r0 = (my_y + my_z * CY) * rows_per, quads = rows_per / 4;
    const int col0 = (tile_a / 2) * BM;            // first output column of this gate/up pair
    for (int idx = threadIdx.x; idx < quads * BN; idx += THREADS) {
      const int j = idx / quads, r = r0 + (idx % quads) * 4;
      const int m = m0 + j, col = col0 + r;
      if (m >= rows_b || r >= BM) continue;
      const uint32_t at = base + (uint32_t)(j * BM + r) * 4u;
      float4 part[8];
#pragma unroll
      for (int z = 0; z < 4; ++z) {
        if (z < CZ) { part[2 * z] = ld_cluster_f32x4(at, z * CY); part[2 * z + 1] = ld_cluster_f32x4(at, z * CY + 1); }
      }
      float gate[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int z = 0; z < 4; ++z) {
        if (z < CZ) {
          gate[0] += part[2 * z].x; gate[1] += part[2 * z].y; gate[2] += part[2 * z].z; gate[3] += part[2 * z].w;
          up[0] += part[2 * z + 1].x; up[1] += part[2 * z + 1].y; up[2] += part[2 * z + 1].z; up[3] += part[2 * z + 1].w;
        }
      }
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + col;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (2 * col0 + BM + r + e < rows_a)   // the matching up row exists
          dst[e] = __float2bfloat16_rn((gate[e] / (1.f + expf(-gate[e]))) * up[e]);
    }
  } else if (EPI == EPI_CL_ROPE_KV) {
    // pairs (d, d + hd/2) of whole heads: 64 pairs per tile, dealt to the CZ CTAs, four neighbouring pairs per item
    const int half = ca.hd / 2;
    const int pairs_per = ((BM / 2 + CZ - 1) / CZ + 3) & ~3, quads = pairs_per / 4;
    for (int idx = threadIdx.x; idx < quads * BN; idx += THREADS) {
      const RopeItem it = idx == (int)threadIdx.x ? first_item : rope_item<BN>(ca, idx, tile_a, m0, rows_a, rows_b);
      if (!it.valid) continue;
      const uint32_t at_lo = base + (uint32_t)(it.j * BM + it.r_lo) * 4u, at_hi = at_lo + (uint32_t)half * 4u;
      float4 pl[8], ph[8];
#pragma unroll
      for (int z = 0; z < 8; ++z) {
        if (z < CZ) { pl[z] = ld_cluster_f32x4(at_lo, z); ph[z] = ld_cluster_f32x4(at_hi, z); }
      }
      float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int z = 0; z < 8; ++z) {
        if (z < CZ) {
          lo[0] += pl[z].x; lo[1] += pl[z].y; lo[2] += pl[z].z; lo[3] += pl[z].w;
          hi[0] += ph[z].x; hi[1] += ph[z].y; hi[2] += ph[z].z; hi[3] += ph[z].w;
        }
      }
      __nv_bfloat16* dst;
      if (it.head < ca.nq) {
        dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)it.m * ldo + (size_t)it.head * ca.hd;
      } else {
        if (it.slot < 0) continue;
        const bool is_v = it.head >= ca.nq + ca.nkv;
        dst = (is_v ? ca.vcache : ca.kcache) + (long long)(it.slot / ca.page_size) * ca.page_stride +
              (long long)(it.head - ca.nq - (is_v ? ca.nkv : 0)) * ca.head_stride + (long long)(it.slot % ca.page_size) * ca.hd;
      }
      const float cs[4] = {it.cs.x, it.cs.y, it.cs.z, it.cs.w}, sn[4] = {it.sn.x, it.sn.y, it.sn.z, it.sn.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // the projection's output is a bfloat16 tensor of the model: rounded before the rotation
        const float x = __bfloat162float(__float2bfloat16_rn(lo[e])), y = __bfloat162float(__float2bfloat16_rn(hi[e]));
        const float o_lo = it.rotate ? cs[e] * x - sn[e] * y : x;
        const float o_hi = it.rotate ? sn[e] * x + cs[e] * y : y;
        dst[it.d + e] = __float2bfloat16_rn(o_lo);
        dst[it.d + half + e] = __float2bfloat16_rn(o_hi);
      }
    }
  } else {
    const int rows_per = ((BM + CZ - 1) / CZ + 3) & ~3, r0 = my_z * rows_per, quads = rows_per / 4;
    for (int idx = threadIdx.x; idx < quads * BN; idx += THREADS) {
      const int j = idx / quads, r = r0 + (idx % quads) * 4;
      const int m = m0 + j, n = tile_a * BM + r;
      if (m >= rows_b || r >= BM || n >= rows_a) continue;
      const uint32_t at = base + (uint32_t)(j * BM + r) * 4u;
      float4 part[8];
#pragma unroll
      for (int z = 0; z < 8; ++z)
        if (z < CZ) part[z] = ld_cluster_f32x4(at, z);
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int z = 0; z < 8; ++z)
        if (z < CZ) { sum[0] += part[z].x; sum[1] += part[z].y; sum[2] += part[z].z; sum[3] += part[z].w; }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (n + e >= rows_a) break;
        const size_t o = (size_t)m * ldo + n + e;
        if (EPI == EPI_CL_ADD_F32) reinterpret_cast<float*>(out)[o] += sum[e];
        else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(sum[e]);
      }
    }
  }
  cluster_sync_all();   // no CTA leaves while a peer still reads its shared memory
}

// ---------------------------------------------------------------- persistent kernel, NORMAL orientation
// One CTA per SM walks the 128 x BN tiles of C (tile t, t + grid, ...; the M tiles of one N tile
// are neighbours, so CTAs running side by side share the weight tile in L2).  Two accumulators of BN
// columns alternate in tensor memory: while the four epilogue warps drain tile i, the MMA thread
// already accumulates tile i + 1, and the TMA thread runs ahead of both through the ring of stages.

template <int BN, int STAGES>
struct PersistentSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // behind the stages: two staging chunks of 128 rows x 32 floats from which the residual-adding epilogue hands its
  // sums to the TMA unit (cp.reduce.async.bulk.tensor ... add), 128-byte swizzled like every other tile
  static constexpr int OUT_CHUNK_BYTES = BM * 32 * 4;
  static constexpr int OUT_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = OUT_OFFSET + 2 * OUT_CHUNK_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

// The epilogue's side of the TMA unit: a reduction of a shared-memory box into global memory, in bulk groups.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the four epilogue warps
// ... and their agreement: true only if `ok` holds in all of them (a warp that gave up a wait must not leave the
// others standing at the barriers of the staging chunks)
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)ok) : "memory");
  return r != 0;
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
linear_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const __grid_constant__ CUtensorMap map_b_strip, const __grid_constant__ CUtensorMap map_out,
                            void* __restrict__ out, int rows_a, int rows_b,
                            int k_blocks, int ldo, const ClusterArgs ca, int* __restrict__ status) {
  static_assert(2 * BN <= 512, "two accumulators must fit tensor memory");
  using L = PersistentSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;      // [2]: accumulator b holds a finished tile
  uint64_t* acc_empty = acc_full + 2;           // [2]: the epilogue has drained accumulator b
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }   // the descriptors are on their way while the barriers are set up
  const int tiles_m = (rows_a + BM - 1) / BM, tiles_n = (rows_b + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  // Work items: the whole tiles [0, tail_from), then the tiles of the last, incomplete round cut into strips
  // of tail_width columns (160 tiles on 148 SMs: 148 whole tiles, then 12 x 4 strips for 48 of the SMs,
  // instead of 12 whole tiles for 12 of them).  Item i -> (row tile, first column, width).
  // With K splits (residual-adding products of few tiles; no strips then) item i is run i / n_tiles of tile i % n_tiles.
  const int k_splits = (EPI == EPI_ADD_F32 && ca.k_splits > 1) ? ca.k_splits : 1;
  const int k_per = k_splits > 1 ? ca.k_per : k_blocks;
  const int whole = k_splits > 1 ? n_tiles * k_splits : (ca.tail_width > 0 ? ca.tail_from : n_tiles);
  const int strips = (k_splits == 1 && ca.tail_width > 0) ? BN / ca.tail_width : 1;
  const int n_items = k_splits > 1 ? whole : whole + (n_tiles - whole) * strips;
  auto item_tile = [&](int i) { return k_splits > 1 ? i % n_tiles : (i < whole ? i : whole + (i - whole) / strips); };
  auto item_kb0 = [&](int i) { return k_splits > 1 ? (i / n_tiles) * k_per : 0; };
  auto item_kbn = [&](int i) { return k_splits > 1 ? max(0, min(k_blocks, (i / n_tiles + 1) * k_per) - (i / n_tiles) * k_per) : k_blocks; };
  // (a strip of a gate/up tile: tail_width / 2 gate rows from item_col on, and the matching up rows BN / 2 further on)
  auto item_col = [&](int i) {
    return (item_tile(i) / tiles_m) * BN + (i < whole ? 0 : ((i - whole) % strips) * (EPI == EPI_SWIGLU ? ca.tail_width / 2 : ca.tail_width));
  };
  auto item_width = [&](int i) { return i < whole ? BN : ca.tail_width; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The weight operand depends on no earlier kernel: the first stages of the first tile are requested
  // before this grid waits for its predecessors.
  pdl_trigger();
  const int first_tile = blockIdx.x;
  const int n_pre = first_tile < whole ? min(item_kbn(first_tile), STAGES) : 0;   // (a CTA's first item is a whole tile, or it has none worth the trouble)
  if (warp == 0 && lane == 0) {
    const int tn = item_tile(first_tile) / tiles_m, kb0 = item_kb0(first_tile);
    for (int i = 0; i < n_pre; ++i) {
      mbar_expect_tx(&full_bar[i], L::STAGE_BYTES);
      tma_load_2d(smem + i * L::STAGE_BYTES + L::A_BYTES, &map_b, (kb0 + i) * BK, tn * BN, &full_bar[i]);
    }
  }
  pdl_wait();
  trace_tag(((unsigned long long)rows_a << 40) | ((unsigned long long)rows_b << 20) | (unsigned long long)k_blocks);   // which product (timeline builds only)

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    int it = 0;   // k-blocks issued so far, over all tiles: stage = it % STAGES
    bool ok = true;
    for (int t = first_tile; t < n_items && ok; t += gridDim.x) {
      const int tm = item_tile(t) % tiles_m, col = item_col(t), width = item_width(t);
      const int kb0 = item_kb0(t), kb1 = kb0 + item_kbn(t);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        uint8_t* a_dst = smem + s * L::STAGE_BYTES;
        const bool pre = it < n_pre;
        if (!pre) {
          if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicExch(status, ERR_PRODUCER); ok = false; break; }
          mbar_expect_tx(&full_bar[s], (uint32_t)(L::A_BYTES + width * BK * 2));
          if (EPI == EPI_SWIGLU && width != BN) {   // the strip's gate rows, then its up rows behind them
            tma_load_2d(a_dst + L::A_BYTES, &map_b_strip, kb * BK, col, &full_bar[s]);
            tma_load_2d(a_dst + L::A_BYTES + (width / 2) * BK * 2, &map_b_strip, kb * BK, col + BN / 2, &full_bar[s]);
          } else {
            tma_load_2d(a_dst + L::A_BYTES, width == BN ? &map_b : &map_b_strip, kb * BK, col, &full_bar[s]);
          }
        }
        tma_load_2d(a_dst, &map_a, kb * BK, tm * BM, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (warp-wide loop, one elected lane issues)
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t lo0 = smem_desc_sw128_lo(smem_u32(smem));
    int it = 0, local = 0;
    bool ok = true;
    for (int t = first_tile; t < n_items && ok; t += gridDim.x, ++local) {
      const uint32_t idesc = instr_desc_bf16(BM, item_width(t));
      const int buf = local & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_u + buf * BN;
      const int kb0 = item_kb0(t), kb1 = kb0 + item_kbn(t);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = lo0 + s * (L::STAGE_BYTES >> 4), b_lo = a_lo + (L::A_BYTES >> 4);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_lo(d_tmem, a_lo + (k * UMMA_K * 2 >> 4), b_lo + (k * UMMA_K * 2 >> 4), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (elect_one()) umma_commit(&acc_full[buf]);   // arrives when this tile's MMAs have completed
      __syncwarp();
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, ERR_MMA); }
  } else if (warp >= 2) {
    // ---------------- epilogue: warp w reads tensor-memory lanes [32 (w % 4), +32)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    int local = 0;
    int out_chunks = 0;   // staging chunks handed to the TMA unit so far (their buffers alternate)
    for (int t = first_tile; t < n_items; t += gridDim.x, ++local) {
      const int buf = local & 1;
      bool ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, abort_flag);
      if (!ok) { *abort_flag = 1; atomicExch(status, ERR_EPILOGUE); }
      ok = __all_sync(0xffffffffu, ok);
      if (EPI == EPI_ADD_F32 && ca.out_by_tma) ok = epilogue_all(ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
      if (EPI == EPI_ROPE_KV)
        store_tile_rope_kv<BN>(taddr, (item_tile(t) % tiles_m) * BM + row, item_col(t), item_width(t), rows_a, rows_b, out, ldo, ca);
      else if (EPI == EPI_ADD_F32 && ca.out_by_tma) {
        // The sums go to the TMA unit: 32 columns at a time every thread lays its row into a swizzled staging chunk,
        // the four warps meet, and one thread hands the chunk over as one reduction (add) into the output.  Stores of
        // 16 bytes per thread, a row apart from lane to lane, kept this epilogue at 4.8 us per tile.
        uint8_t* stage_out = smem + L::OUT_OFFSET;
        const int row0 = (item_tile(t) % tiles_m) * BM, col0 = (item_tile(t) / tiles_m) * BN;
        const bool issuer = warp == 2 && lane == 0;
#pragma unroll 1
        for (int c = 0; c < BN && col0 + c < rows_b; c += 32, ++out_chunks) {   // (columns past the output's end: no chunk)
          float v[32];
          tmem_ld32(taddr + c, v);
          uint8_t* buf = stage_out + (out_chunks & 1) * L::OUT_CHUNK_BYTES;
          if (issuer) bulk_wait_read<1>();     // the reduction that read this buffer two chunks ago has its data
          epilogue_barrier();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(buf + row * 128 + ((j ^ (row & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          epilogue_barrier();
          if (issuer) {
            tma_reduce_add_2d(&map_out, buf, col0 + c, row0);   // rows and columns past the output's end are clipped
            bulk_commit();
          }
        }
      }
      else if (EPI == EPI_SWIGLU && item_width(t) != BN)
        store_strip_swiglu(taddr, (item_tile(t) % tiles_m) * BM + row,
                           (item_tile(t) / tiles_m) * (BN / 2) + (item_col(t) - (item_tile(t) / tiles_m) * BN), item_width(t) / 2,
                           rows_a, rows_b / 2, reinterpret_cast<__nv_bfloat16*>(out), ldo);
      else store_tile_normal<BN, EPI>(taddr, row, item_tile(t) % tiles_m, item_tile(t) / tiles_m, rows_a, rows_b, out, ldo);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);   // four arrivals free the accumulator
    }
    if (EPI == EPI_ADD_F32 && warp == 2 && lane == 0) bulk_wait_all();   // every reduction of this CTA has been performed
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------- host side
// A 2-D bfloat16 tensor [rows, k] with row stride ld (elements), tiled in boxes of box_rows x 64.
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int k, long long ld, int box_rows) {
  using Key = std::tuple<const void*, int, int, long long, int>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  const Key key(ptr, rows, k, ld, box_rows);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = *map;
  return true;
}

// A 2-D float32 tensor [rows, cols] with row stride ld (elements), in boxes of 128 rows x 32 columns: the output of the
// residual-adding products as the TMA unit's reductions see it.
static bool make_out_map(CUtensorMap* map, const void* ptr, int rows, int cols, long long ld) {
  using Key = std::tuple<const void*, int, int, long long>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  const Key key(ptr, rows, cols, ld);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32u, (cuuint32_t)BM};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = *map;
  return true;
}

template <int BN, int STAGES, bool SWAP, int EPI>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int k, int splits,
                  int ldo, int* status, cudaStream_t s) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = linear_tc_kernel<BN, STAGES, SWAP, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
    configured = true;
  }
  const int k_blocks = (k + BK - 1) / BK;
  const int per_split = (k_blocks + splits - 1) / splits;
  const int used_splits = (k_blocks + per_split - 1) / per_split;
  dim3 grid((rows_b + BN - 1) / BN, (rows_a + BM - 1) / BM, used_splits);
  TLLM_LAUNCH("linear_tc", kern, grid, THREADS, L::TOTAL, s, ma, mb, out, rows_a, rows_b, k_blocks, per_split, ldo, status);
  return TLLM_OK;
}

template <int EPI>
static int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int m, int n, int k, int ldo,
                             int* status, cudaStream_t s, const ClusterArgs& ca = ClusterArgs(), const void* w_ptr = nullptr) {
  constexpr int BN = 256, STAGES = 4;
  using L = PersistentSmem<BN, STAGES>;
  auto kern = linear_tc_persistent_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  ClusterArgs args = ca;
  args.tail_from = tiles;
  args.tail_width = 0;
  // a residual-adding product of few tiles (fewer than 2,048 tokens): its K in runs of at least four k-blocks,
  // as many as fill the SMs; the runs add into the output with the same reductions as whole tiles do
  const int kb = (k + BK - 1) / BK;
  args.k_splits = 1;
  args.k_per = kb;
  if (EPI == EPI_ADD_F32 && 2 * tiles <= sm_count && kb >= 8) {
    const int want = std::min(sm_count / tiles, kb / 4);
    args.k_per = (kb + want - 1) / want;
    args.k_splits = (kb + args.k_per - 1) / args.k_per;
  }
  const int items = tiles * args.k_splits;
  const int grid = items < sm_count ? items : sm_count;
  const CUtensorMap* strip_map = &mb;
  CUtensorMap ms;
  // the residual-adding epilogue through the TMA unit where its rules hold: base and row stride on 16 bytes
  const CUtensorMap* out_map = &ma;   // (a valid map that is never used)
  CUtensorMap mo;
  args.out_by_tma = 0;
  if (EPI == EPI_ADD_F32 && ((uintptr_t)out % 16) == 0 && ldo % 4 == 0 && make_out_map(&mo, out, m, n, ldo)) {
    args.out_by_tma = 1;
    out_map = &mo;
  }
  if (EPI == EPI_ROPE_KV && tiles > sm_count && tiles % sm_count != 0) {
    // the last round is incomplete: cut its tiles into strips of whole heads if those then fit one round
    const int width = ca.hd <= 64 ? 64 : ca.hd, left = tiles % sm_count;
    if (BN % width == 0 && left * (BN / width) <= sm_count && make_map(&ms, w_ptr, n, k, k, width)) {
      args.tail_from = tiles - left;
      args.tail_width = width;
      strip_map = &ms;
    }
  }
  if (EPI == EPI_SWIGLU && tiles > sm_count && tiles % sm_count != 0 && w_ptr != nullptr && n % BN == 0) {
    // gate/up: the tiles of the incomplete last round as 4 or 2 strips (32 or 64 gate columns with their up columns),
    // as many as still fit one round
    const int left = tiles % sm_count;
    const int parts = left * 4 <= sm_count ? 4 : (left * 2 <= sm_count ? 2 : 1);
    if (parts > 1 && make_map(&ms, w_ptr, n, k, k, BN / 2 / parts)) {
      args.tail_from = tiles - left;
      args.tail_width = BN / parts;
      strip_map = &ms;
    }
  }
  TLLM_LAUNCH("linear_tc_persistent", kern, grid, THREADS, L::TOTAL, s, ma, mb, *strip_map, *out_map, out, m, n, (k + BK - 1) / BK, ldo, args, status);
  return TLLM_OK;
}

template <int BN, int STAGES, int EPI>
static int launch_cluster(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int rows_a, int rows_b, int k, int ldo,
                          const ClusterArgs& ca, int* status, cudaStream_t s) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = linear_tc_cluster_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
    configured = true;
  }
  const int k_blocks = (k + BK - 1) / BK;
  const int per_split = (k_blocks + ca.cz - 1) / ca.cz;
  const int row_tiles = (rows_a + BM - 1) / BM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((rows_b + BN - 1) / BN, (row_tiles + ca.cy - 1) / ca.cy * ca.cy, ca.cz);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ca.cy;
  attr[0].val.clusterDim.z = ca.cz;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mb, out, rows_a, rows_b, k_blocks, per_split, ldo, ca, status);
  if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc_cluster: %s", cudaGetErrorString(e));
  return TLLM_OK;
}

}  // namespace tllm

using namespace tllm;

// out[M, N] (row stride ldo) = / += a[M, K] (row stride lda) . w[N, K]^T, bfloat16 operands.
//   epi: 0 store bfloat16, 1 store float32, 2 add into float32, 3 SiLU(gate)*up with gate/up rows of w
//        interleaved in blocks of 128 (out is [M, N/2] bfloat16), 4 atomic add into float32.
//   swap: 0 = 128 x 256 tiles of C per CTA (large M); 1 = weights on the 128-row side, M <= 128,
//        `splits` slices of K per weight tile (epi 4 when splits > 1).
// `status` is a device int that receives a non-zero code if a bounded wait expired.
extern "C" int tllm_linear_tc(const void* a, const void* w, void* out, int m, int n, int k, int lda, int ldo, int epi,
                              int swap, int splits, int* status, void* stream) {
  TLLM_REQUIRE(m > 0 && n > 0 && k > 0, "linear_tc: empty product %d x %d x %d", m, n, k);
  TLLM_REQUIRE(k % 8 == 0 && lda % 8 == 0, "linear_tc: K (%d) and the row stride of A (%d) must be multiples of 8 (16-byte rule of TMA)", k, lda);
  TLLM_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0, "linear_tc: operands must be 16-byte aligned");
  TLLM_REQUIRE(status != nullptr, "linear_tc: needs a status word");
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap ma, mb;
  if (!swap) {
    TLLM_REQUIRE(splits == 1, "linear_tc: K is split only in the swapped orientation");
    TLLM_REQUIRE(epi != EPI_ATOMIC_F32, "linear_tc: atomic output belongs to the swapped orientation");
    if (epi == EPI_SWIGLU) TLLM_REQUIRE(n % 256 == 0, "linear_tc: the fused SiLU*up epilogue needs gate/up blocks of 128 rows (N = %d)", n);
    if (!make_map(&ma, a, m, k, lda, BM) || !make_map(&mb, w, n, k, k, 256))
      TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc: cuTensorMapEncodeTiled failed");
    switch (epi) {
      case EPI_BF16: return launch_persistent<EPI_BF16>(ma, mb, out, m, n, k, ldo, status, s);
      case EPI_F32: return launch_persistent<EPI_F32>(ma, mb, out, m, n, k, ldo, status, s);
      case EPI_ADD_F32: return launch_persistent<EPI_ADD_F32>(ma, mb, out, m, n, k, ldo, status, s);
      case EPI_SWIGLU: return launch_persistent<EPI_SWIGLU>(ma, mb, out, m, n, k, ldo, status, s, ClusterArgs(), w);
    }
    TLLM_FAIL(TLLM_ERR_ARG, "linear_tc: unknown epilogue %d", epi);
  }
  TLLM_REQUIRE(m <= 128, "linear_tc: the swapped orientation takes at most 128 rows of A (got %d)", m);
  TLLM_REQUIRE(epi != EPI_SWIGLU, "linear_tc: SiLU*up is fused only in the unswapped orientation");
  TLLM_REQUIRE(splits >= 1 && (splits == 1 || epi == EPI_ATOMIC_F32), "linear_tc: split K needs the atomic epilogue");
  const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
  if (!make_map(&ma, w, n, k, k, BM) || !make_map(&mb, a, m, k, lda, bn))
    TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc: cuTensorMapEncodeTiled failed");
#define TLLM_SWAP_CASE(BN_, ST_)                                                                                       \
  switch (epi) {                                                                                                      \
    case EPI_BF16: return launch<BN_, ST_, true, EPI_BF16>(ma, mb, out, n, m, k, splits, ldo, status, s);              \
    case EPI_F32: return launch<BN_, ST_, true, EPI_F32>(ma, mb, out, n, m, k, splits, ldo, status, s);                \
    case EPI_ADD_F32: return launch<BN_, ST_, true, EPI_ADD_F32>(ma, mb, out, n, m, k, splits, ldo, status, s);        \
    case EPI_ATOMIC_F32: return launch<BN_, ST_, true, EPI_ATOMIC_F32>(ma, mb, out, n, m, k, splits, ldo, status, s);  \
  }                                                                                                                   \
  break;
  // stage counts keep a CTA under half of an SM's shared memory: two CTAs stream side by side, so
  // that a grid of up to 296 CTAs is resident at once and no second wave trails behind
  switch (bn) {
    case 16: TLLM_SWAP_CASE(16, 6)
    case 32: TLLM_SWAP_CASE(32, 5)
    case 64: TLLM_SWAP_CASE(64, 4)
    case 128: TLLM_SWAP_CASE(128, 3)
  }
#undef TLLM_SWAP_CASE
  TLLM_FAIL(TLLM_ERR_ARG, "linear_tc: unknown epilogue %d", epi);
}

// The same product for at most 128 rows of A with the K slices of a weight tile reduced inside a
// thread-block cluster (`slices` = 1 to 8) and one of these epilogues:
//   5: out (float32 [M, N]) += product;
//   6: Q/K/V projection: out (bfloat16, row stride ldo) gets the rotated queries; rotated keys and the values
//      go to their pages at slot_mapping (null: the rows are queries only).  N = (nq + 2 nkv) hd (or nq hd),
//      hd 16, 32, 64 or 128; cos/sin null: no rotation.  This one also takes more than 128 rows (head size
//      64 or 128): then it runs as 128 x 256 tiles of C with the same epilogue per tile;
//   7: SiLU(gate) * up with gate/up rows of w interleaved in blocks of 128, out bfloat16 [M, N/2]
//      (slices <= 4: the cluster also spans the gate tile and the up tile);
//   8: out (bfloat16 [M, N]) = product.
extern "C" int tllm_linear_tc_cluster(const void* a, const void* w, void* out, int m, int n, int k, int lda, int ldo,
                                      int epi, int slices, const int* positions, const float* cos, const float* sin,
                                      int nq, int nkv, int hd, void* kcache, void* vcache, const int* slot_mapping,
                                      int page_size, long long page_stride, long long head_stride, int* status,
                                      void* stream) {
  TLLM_REQUIRE(m > 0 && n > 0 && k > 0 && (m <= 128 || epi == EPI_CL_ROPE_KV),
               "linear_tc_cluster: product %d x %d x %d (at most 128 rows, except for the Q/K/V projection)", m, n, k);
  TLLM_REQUIRE(k % 8 == 0 && lda % 8 == 0, "linear_tc_cluster: K (%d) and the row stride of A (%d) must be multiples of 8", k, lda);
  TLLM_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0, "linear_tc_cluster: operands must be 16-byte aligned");
  TLLM_REQUIRE(status != nullptr, "linear_tc_cluster: needs a status word");
  TLLM_REQUIRE(slices >= 1 && slices <= 8, "linear_tc_cluster: %d slices of K (1 to 8: a cluster has at most 8 CTAs)", slices);
  TLLM_REQUIRE(slices <= (k + BK - 1) / BK, "linear_tc_cluster: %d slices of a K of %d", slices, k);
  ClusterArgs ca = {};
  ca.cy = 1; ca.cz = slices;
  if (epi == EPI_CL_SWIGLU) {
    TLLM_REQUIRE(n % 256 == 0 && slices <= 4, "linear_tc_cluster: SiLU*up needs gate/up blocks of 128 rows (N = %d) and at most 4 slices", n);
    ca.cy = 2;
  } else if (epi == EPI_CL_ROPE_KV) {
    TLLM_REQUIRE(hd >= 16 && 128 % hd == 0 && nq >= 1 && nkv >= 0, "linear_tc_cluster: head size %d must be 16, 32, 64 or 128", hd);
    TLLM_REQUIRE(n == (slot_mapping ? (nq + 2 * nkv) * hd : nq * hd), "linear_tc_cluster: %d rows of weights for %d + 2 x %d heads of %d", n, nq, nkv, hd);
    TLLM_REQUIRE(positions != nullptr || cos == nullptr, "linear_tc_cluster: rotation needs positions");
    TLLM_REQUIRE(slot_mapping == nullptr || (kcache && vcache && page_size > 0), "linear_tc_cluster: cache arguments missing");
    ca.positions = positions; ca.cos = cos; ca.sin = sin; ca.kcache = (__nv_bfloat16*)kcache; ca.vcache = (__nv_bfloat16*)vcache;
    ca.slot_mapping = slot_mapping; ca.page_stride = page_stride; ca.head_stride = head_stride;
    ca.nq = nq; ca.nkv = nkv; ca.hd = hd; ca.page_size = page_size;
  } else {
    TLLM_REQUIRE(epi == EPI_CL_ADD_F32 || epi == EPI_CL_BF16, "linear_tc_cluster: unknown epilogue %d", epi);
  }
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap ma, mb;
  if (m > 128) {
    // many tokens: 128 x 256 tiles of C as in tllm_linear_tc, with the rotation and the cache write in the epilogue
    TLLM_REQUIRE(hd == 64 || hd == 128, "linear_tc_cluster: the Q/K/V epilogue for more than 128 tokens takes head size 64 or 128 (got %d)", hd);
    if (!make_map(&ma, a, m, k, lda, BM) || !make_map(&mb, w, n, k, k, 256))
      TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc_cluster: cuTensorMapEncodeTiled failed");
    return launch_persistent<EPI_ROPE_KV>(ma, mb, out, m, n, k, ldo, status, s, ca, w);
  }
  const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
  if (!make_map(&ma, w, n, k, k, BM) || !make_map(&mb, a, m, k, lda, bn))
    TLLM_FAIL(TLLM_ERR_CUDA, "linear_tc_cluster: cuTensorMapEncodeTiled failed");
#define TLLM_CL_CASE(BN_, ST_)                                                                                        \
  switch (epi) {                                                                                                     \
    case EPI_CL_ADD_F32: return launch_cluster<BN_, ST_, EPI_CL_ADD_F32>(ma, mb, out, n, m, k, ldo, ca, status, s);   \
    case EPI_CL_ROPE_KV: return launch_cluster<BN_, ST_, EPI_CL_ROPE_KV>(ma, mb, out, n, m, k, ldo, ca, status, s);   \
    case EPI_CL_SWIGLU: return launch_cluster<BN_, ST_, EPI_CL_SWIGLU>(ma, mb, out, n, m, k, ldo, ca, status, s);     \
    case EPI_CL_BF16: return launch_cluster<BN_, ST_, EPI_CL_BF16>(ma, mb, out, n, m, k, ldo, ca, status, s);         \
  }                                                                                                                  \
  break;
  switch (bn) {
    case 16: TLLM_CL_CASE(16, 6)
    case 32: TLLM_CL_CASE(32, 5)
    case 64: TLLM_CL_CASE(64, 4)
    case 128: TLLM_CL_CASE(128, 3)
  }
#undef TLLM_CL_CASE
  TLLM_FAIL(TLLM_ERR_ARG, "linear_tc_cluster: unknown epilogue %d", epi);
}
