// Device-side support for tile programs that the lowerer emits op by op.
//
// The two programs of the hot path (GEMM, attention forward) are recognised by the
// lowerer and run on the warp-specialised kernels in gemm_sm100.cuh / attn_fwd_sm100.cuh.
// Every other program built from the tile IR's ops (reference op table:
// warpir/lowering/lowering.py:427-570) is emitted as straight-line code over the helpers
// in this file, one call per op, under this execution model:
//
//   * one CTA of 128 threads per (blockIdx.x, blockIdx.y, blockIdx.z);
//   * a register tile of R x N (R = 4 x the per-warp rows of its type, R <= 128) is held
//     one row per thread -- thread t owns row t, which is also tensor-memory lane t, so
//     row reductions need no shuffles and MMA results are read back with 32x32b loads;
//     threads t >= R carry don't-care values and never store;
//   * shared tiles are filled by TMA with the 128-byte swizzle, 64 columns (128 bytes) per
//     chunk, every chunk padded to 128 rows so that a tile can serve as the A operand of
//     a 128-row tcgen05.mma whatever its own height;
//   * `mma` runs on the tensor core: the accumulator goes to tensor memory, one elected
//     thread of warp 0 issues the k-steps, everybody waits for the commit and reads the
//     result back; a register-tile A operand is packed to bf16 and fed from tensor
//     memory (the TS form);
//   * every wait is bounded (ptx.cuh); after a failed wait the CTA finishes quickly with
//     the error recorded in the status words, drains its copies and frees tensor memory.
//
// This path favours generality over speed: MMAs are synchronous and nothing overlaps.
#pragma once

#include "ptx.cuh"

namespace wir {
namespace tp {

constexpr int kThreads = 128;
constexpr int kMaxBarriers = 32;
constexpr int kRoleTile = 6;   // role id in the status words
constexpr int kChunkBytes = 128 * 128;   // one 64-column chunk of a shared tile, padded to 128 rows

template <int N>
struct Tile {
  float v[N];   // this thread's row
};

// Shared control block (declared __shared__ by the emitted kernel).
template <int NBARS>
struct Control {
  unsigned long long bars[NBARS];   // mbarriers: 0 = MMA completion, then one per tile / ring slot
  uint32_t tmem_slot;
  int abort_flag;
};

struct Ctx {
  uint32_t smem;          // shared address of the 1024-byte-aligned data area
  uint32_t bars;          // shared address of the barrier array
  uint32_t tmem;          // base of this CTA's tensor-memory columns
  uint32_t tmem_cols;
  uint32_t phases;        // bit b: parity the next wait on barrier b expects
  uint32_t outstanding;   // bit b: a load was issued on barrier b and not waited for yet
  int consumed;           // ring slots consumed by MMAs inside loops (drain slots count from here)
  bool ok;
  AbortCtx abort;
};

__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int b) { return c.bars + 8u * static_cast<uint32_t>(b); }

template <int NBARS>
__device__ __forceinline__ void begin(Ctx& c, Control<NBARS>& ctl, uint8_t* dyn, int* status, uint32_t tmem_cols) {
  static_assert(NBARS <= kMaxBarriers, "barrier bit masks are 32 bits wide");
  c.smem = (smem_u32(dyn) + 1023u) & ~1023u;
  c.bars = smem_u32(&ctl.bars[0]);
  c.tmem_cols = tmem_cols;
  c.phases = 0;
  c.outstanding = 0;
  c.consumed = 0;
  c.ok = true;
  c.abort = AbortCtx{&ctl.abort_flag, status};
  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int b = 0; b < NBARS; ++b) mbar_init(bar_addr(c, b), 1);
    fence_mbar_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(smem_u32(&ctl.tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = ctl.tmem_slot;
}

__device__ __forceinline__ void end(Ctx& c) {
  if (!c.ok || *c.abort.flag) {
    // copies still in flight must land before the shared memory is handed to the next CTA
    for (int b = 1; b < kMaxBarriers; ++b)
      if (c.outstanding & (1u << b)) mbar_wait_quiet(bar_addr(c, b), (c.phases >> b) & 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(c.tmem, c.tmem_cols);
  }
}

// Bounded wait on barrier b by every thread; flips the expected parity.
__device__ __forceinline__ void wait_bar(Ctx& c, int b, int tag) {
  const uint32_t bit = 1u << b;
  if (c.ok) {
    const bool got = mbar_wait(bar_addr(c, b), (c.phases >> b) & 1u, c.abort, kRoleTile, tag, b);
    // the outcome must be CTA-uniform: the control flow after it contains block barriers
    c.ok = __syncthreads_and(got ? 1 : 0) != 0;
    if (c.ok) {
      c.phases ^= bit;
      c.outstanding &= ~bit;
    }
  }
}

__device__ __forceinline__ void ensure_loaded(Ctx& c, int b) {
  if (c.outstanding & (1u << b)) wait_bar(c, b, 2);
}

__device__ __forceinline__ int slot_of(int value, int modulus) {
  const int r = value % modulus;
  return r < 0 ? r + modulus : r;
}

// ---- TMA load of one ROWS x COLS bf16 tile (wait op: wait_bar on the same barrier) -------------
// `map` covers the tensor as (cols, rows, batch * depth) with a 64 x ROWS x 1 box.
template <int ROWS, int COLS>
__device__ __forceinline__ void load_tile(Ctx& c, const CUtensorMap* map, uint32_t dst, int b, int col0, int row0,
                                          int plane) {
  static_assert(COLS % 64 == 0, "shared tiles are whole 128-byte swizzle rows");
  ensure_loaded(c, b);   // a second load into the same tile must not race the first
  if (c.ok && threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_addr(c, b), ROWS * COLS * 2);
#pragma unroll
    for (int ch = 0; ch < COLS / 64; ++ch)
      tma_load_3d(dst + ch * kChunkBytes, map, bar_addr(c, b), col0 + 64 * ch, row0, plane);
  }
  if (c.ok) c.outstanding |= 1u << b;
}

// ---- tensor memory <-> this thread's row ----------------------------------------------------
template <int N>
__device__ __forceinline__ void tmem_store_row(uint32_t taddr, const float* v) {
  static_assert(N % 16 == 0, "whole groups of 16 columns");
  uint32_t r[N];
#pragma unroll
  for (int i = 0; i < N; ++i) r[i] = __float_as_uint(v[i]);
#pragma unroll
  for (int i = 0; i + 32 <= N; i += 32) tmem_st32(taddr + i, r + i);
  if (N % 32) tmem_st16(taddr + (N - 16), r + (N - 16));
}
template <int N>
__device__ __forceinline__ void tmem_load_row(uint32_t taddr, float* v) {
  uint32_t r[N];
#pragma unroll
  for (int i = 0; i + 32 <= N; i += 32) tmem_ld32(taddr + i, r + i);
  if (N % 32) tmem_ld16(taddr + (N - 16), r + (N - 16));
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint32_t lane_base(const Ctx& c) {
  return c.tmem + (static_cast<uint32_t>(threadIdx.x & ~31u) << 16);
}

// Common tail of both MMA forms: wait for the commit, read the accumulator back.
template <int N>
__device__ __forceinline__ void mma_finish(Ctx& c, Tile<N>& acc) {
  wait_bar(c, 0, 1);
  tc_fence_after();
  if (c.ok) tmem_load_row<N>(lane_base(c), acc.v);
}

// acc = (accumulate ? acc : 0) + A x B with A a shared tile [128(padded) x K] (K contiguous).
// B_MN = true : B is a shared tile [K x N] (N contiguous, the row-major B of `mma`);
// B_MN = false: B is a shared tile [N x K] (K contiguous, `mma` with transpose_b).
template <int N, int K, bool B_MN>
__device__ __forceinline__ void mma_smem(Ctx& c, uint32_t a_addr, uint32_t b_addr, Tile<N>& acc, bool accumulate) {
  static_assert(N % 16 == 0 && N >= 16 && N <= 256 && K % 16 == 0, "tcgen05.mma shape");
  if (accumulate && c.ok) {
    tmem_store_row<N>(lane_base(c), acc.v);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32 && c.ok) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16_f32(128, N, 0, B_MN ? 1 : 0);
    constexpr uint32_t hi = smem_desc_hi_sw128(1024);
    const uint32_t a_lo = smem_desc_lo(a_addr, 16);
    const uint32_t b_lo = smem_desc_lo(b_addr, B_MN ? kChunkBytes : 16);
#pragma unroll
    for (int k = 0; k < K / 16; ++k) {
      const uint32_t a_off = ((k / 4) * kChunkBytes + (k % 4) * 32) >> 4;
      const uint32_t b_off = (B_MN ? k * 2048 : (k / 4) * kChunkBytes + (k % 4) * 32) >> 4;
      mma_ss_elect(c.tmem, a_lo + a_off, hi, b_lo + b_off, hi, idesc, (k > 0 || accumulate) ? 1u : 0u);
    }
    mma_commit_elect(bar_addr(c, 0));
  }
  mma_finish<N>(c, acc);
}

// Same with A a bf16 register tile [128 x K]: packed into tensor memory at column A_COL.
template <int N, int K, bool B_MN, int A_COL>
__device__ __forceinline__ void mma_regs(Ctx& c, const Tile<K>& a, uint32_t b_addr, Tile<N>& acc, bool accumulate) {
  static_assert(N % 16 == 0 && N >= 16 && N <= 256 && K % 32 == 0, "tcgen05.mma shape");
  if (c.ok) {
    uint32_t pk[K / 2];
#pragma unroll
    for (int i = 0; i < K / 2; ++i) pk[i] = pack_bf16(a.v[2 * i], a.v[2 * i + 1]);
#pragma unroll
    for (int i = 0; i + 32 <= K / 2; i += 32) tmem_st32(lane_base(c) + A_COL + i, pk + i);
    if ((K / 2) % 32) tmem_st16(lane_base(c) + A_COL + (K / 2 - 16), pk + (K / 2 - 16));
    if (accumulate) tmem_store_row<N>(lane_base(c), acc.v);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32 && c.ok) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16_f32(128, N, 0, B_MN ? 1 : 0);
    constexpr uint32_t hi = smem_desc_hi_sw128(1024);
    const uint32_t b_lo = smem_desc_lo(b_addr, B_MN ? kChunkBytes : 16);
#pragma unroll
    for (int k = 0; k < K / 16; ++k) {
      const uint32_t b_off = (B_MN ? k * 2048 : (k / 4) * kChunkBytes + (k % 4) * 32) >> 4;
      mma_ts_elect(c.tmem, c.tmem + A_COL + k * 8, b_lo + b_off, hi, idesc, (k > 0 || accumulate) ? 1u : 0u);
    }
    mma_commit_elect(bar_addr(c, 0));
  }
  mma_finish<N>(c, acc);
}

// ---- elementwise and row-wise ops (reference semantics: warpir/ir/ops.py:103-190) ------------
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int N> __device__ __forceinline__ Tile<N> fill(float x) {
  Tile<N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = x;
  return r;
}
#define WIR_TP_MAP1(NAME, EXPR)                                                     \
  template <int N> __device__ __forceinline__ Tile<N> NAME(const Tile<N>& a) {       \
    Tile<N> r;                                                                      \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const float x = a.v[i]; r.v[i] = (EXPR); } \
    return r;                                                                       \
  }                                                                                 \
  __device__ __forceinline__ float NAME(float x) { return (EXPR); }
#define WIR_TP_MAP2(NAME, EXPR)                                                     \
  template <int N> __device__ __forceinline__ Tile<N> NAME(const Tile<N>& a, const Tile<N>& b) { \
    Tile<N> r;                                                                      \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const float x = a.v[i], y = b.v[i]; r.v[i] = (EXPR); } \
    return r;                                                                       \
  }                                                                                 \
  __device__ __forceinline__ float NAME(float x, float y) { return (EXPR); }
// tile (op) per-row scalar, and tile (op) compile-time scalar
#define WIR_TP_ROW(NAME, EXPR)                                                      \
  template <int N> __device__ __forceinline__ Tile<N> NAME(const Tile<N>& a, float y) { \
    Tile<N> r;                                                                      \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const float x = a.v[i]; r.v[i] = (EXPR); } \
    return r;                                                                       \
  }

WIR_TP_MAP1(copy, x)
WIR_TP_MAP1(to_bf16, round_bf16(x))
WIR_TP_MAP1(exp2, exp2f(x))
WIR_TP_MAP2(sub, x - y)
WIR_TP_MAP2(mul, x * y)
WIR_TP_ROW(mul_scalar, x * y)
WIR_TP_ROW(sub_row, x - y)
WIR_TP_ROW(mul_row, x * y)
WIR_TP_ROW(div_row, x / y)
__device__ __forceinline__ float mul_scalar(float x, float y) { return x * y; }

template <int N> __device__ __forceinline__ float row_max(const Tile<N>& a, float prev) {
  float m = prev;
#pragma unroll
  for (int i = 0; i < N; ++i) m = fmaxf(m, a.v[i]);
  return m;
}
template <int N> __device__ __forceinline__ float row_sum(const Tile<N>& a, float prev) {
  // four partial sums keep the dependent-add chain short; the order is fixed, so results repeat
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int i = 0; i + 4 <= N; i += 4) {
    s0 += a.v[i];
    s1 += a.v[i + 1];
    s2 += a.v[i + 2];
    s3 += a.v[i + 3];
  }
  return prev + ((s0 + s1) + (s2 + s3));
}

// ---- store of a register tile as bf16 ------------------------------------------------------
// `base` addresses a [planes, rows, cols] bf16 tensor; the tile's first element is
// (plane, row0, col0); rows and columns past the extents are dropped (ragged edges).
template <int N>
__device__ __forceinline__ void store_tile(const Ctx& c, const Tile<N>& t, __nv_bfloat16* base, long long rows,
                                           long long cols, long long plane, long long row0, long long col0,
                                           int tile_rows) {
  if (!c.ok) return;
  const long long r = row0 + threadIdx.x;
  if (static_cast<int>(threadIdx.x) >= tile_rows || r >= rows) return;
  __nv_bfloat16* dst = base + (plane * rows + r) * cols + col0;
  const bool vec_ok = (cols % 8 == 0) && (col0 % 8 == 0);
#pragma unroll
  for (int g = 0; g < N / 8; ++g) {
    if (col0 + 8 * g >= cols) break;
    if (vec_ok && col0 + 8 * g + 8 <= cols) {
      uint4 q;
      q.x = pack_bf16(t.v[8 * g + 0], t.v[8 * g + 1]);
      q.y = pack_bf16(t.v[8 * g + 2], t.v[8 * g + 3]);
      q.z = pack_bf16(t.v[8 * g + 4], t.v[8 * g + 5]);
      q.w = pack_bf16(t.v[8 * g + 6], t.v[8 * g + 7]);
      *reinterpret_cast<uint4*>(dst + 8 * g) = q;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col0 + 8 * g + e < cols) dst[8 * g + e] = __float2bfloat16_rn(t.v[8 * g + e]);
    }
  }
}

}  // namespace tp
}  // namespace wir
