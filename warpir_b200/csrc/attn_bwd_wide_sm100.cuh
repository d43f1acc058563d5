// Attention backward for sm_100a in steps of 128 streamed rows (the library's choice; the 64-row kernel of
// attn_bwd_sm100.cuh remains as the other variant).  Same mathematics and the same two launches of one template:
//
//   DKV = false (grid over 128-row Q tiles):  X0 = Q, X1 = dO resident; streams K, V tiles; accumulates dQ.
//   (delta = rowsum(dO * O), which both need, comes from a third, small kernel that runs first: attn_bwd_delta.)
//   DKV = true  (grid over 128-key K/V tiles): X0 = K, X1 = V resident; streams the Q, dO tiles of every query
//     head of the group; accumulates dV and dK.
//
// With c = scale * log2(e), per step j (Y0, Y1 the streamed 128 x D tiles):
//
//   A1:  T0 = X0 Y0^T            A2:  T1 = X1 Y1^T                       (128 x 128 each, operands in shared memory)
//   P  = 2^(c T0 - LSE log2e)    dS = P (T1 - delta) scale               (compute warps; packed to bf16 into T1)
//   DKV:  B1: acc0 += P Y1 (dV)  B2: acc1 += dS Y0 (dK)       else  B: acc0 += dS Y0 (dQ)     (A from tensor memory)
//
// In the dQ launch LSE and delta belong to the thread's row and sit in two registers.  In the dK / dV launch they
// belong to the COLUMN (the streamed query), 128 of each per step; there the tensor core subtracts them: one more
// k-step per score tile multiplies rows of ones with rows that hold -LSE / scale (for A1) and -delta (for A2) in
// three bf16 pieces, so that T0 = S - LSE / scale and T1 = dP - delta arrive ready (AttnBwdWideSmem::kExtraOffset).
//
// Why 128 rows per step: the warp that issues the MMAs is the kernel's clock.  It gets through its own dependent
// instructions at 6-12 clocks each and pays 75-150 for every look at a barrier, and the tensor core's queue is
// only about four MMAs deep; with 64-row steps (16 MMAs of 128 x 64 x 16, which from shared memory take 48 clocks
// for 32 of arithmetic, and 4-8 of 128 x 128 x 16) it spent twice the tensor core's time per step.  Here a step
// is 24 or 32 MMAs of 128 x 128 x 16 at the full rate, with the same number of hand-offs as a 64-row step had.
//
// Tensor memory has no room to double-buffer 128-column score tiles next to the accumulators (T0 128 + T1 128 +
// acc0 D + acc1 D = 512 at D = 128), so the overlap comes from the order of issue and from where the packed values
// go.
//
// dQ launch:   A1(j+1)  B(j)  A2(j+1).  P stays in registers, so T0 is released as soon as it has been read and the
//   next scores are computed under the whole of step j; dS (packed bf16) goes over T1 columns 32-95, which B(j)
//   reads before A2(j+1) overwrites them (MMAs execute in issue order).
// dK / dV launch:   A1(j+1) | B1(j) | B2(j)  A2(j+1).  Both packed tiles go into T1, which is dead once both groups
//   have read it: P over columns 32-95, dS over the outer columns (0-31 and 96-127).  T0 is released as soon as it
//   has been read, as in the dQ launch, so the exponentials of step j+1 never wait for an MMA of step j; what is
//   left in line is dS(j) -> B2(j), A2(j+1) -> dS(j+1), with the exponentials of step j+1 running under those MMAs.
//   (Before, P went back into T0: the next scores then had to follow B1(j), and the compute warps waited 1000 of
//   3500 clocks per step for them.)
//
// Shared memory: X0, X1, then a ring of STREAMED TILES (not steps): Y0(0), Y1(0), Y0(1), ...; a tile goes back to
// the producer behind the last MMA group that reads it (Y1(j) after B1(j), or after A2(j) in the dQ launch; Y0(j)
// after B2(j) / B(j)).  Warp 0 is the TMA producer, warp 1 issues every MMA (whole warp, one elected lane, four
// MMAs per instruction block), warps 2-9 are two compute warpgroups: thread = one tensor-memory lane (row), group
// g takes columns 64 g ... of T0 / T1 and overwrites only columns of T1 that it has read itself (group 0 reads
// 0-63 and writes 0-63, group 1 reads 64-127 and writes 64-127).  Every wait is bounded.
#pragma once

#include <type_traits>

#include "attn_bwd_sm100.cuh"

namespace wir {

constexpr int kBw2Rows = 128;   // rows of the resident AND of the streamed tiles

template <int D, bool DKV>
struct AttnBwdWideSmem {
  // ring of streamed tiles; the dK / dV launch gives one 32 KB slot up for the chunk of extra operands below
  static constexpr int kSlots = (D == 128) ? (DKV ? 4 : 5) : 10;
  static constexpr int kChunkBytes = kBw2Rows * 128;                 // 128 rows x 64 bf16
  static constexpr int kTileBytes = (D / 64) * kChunkBytes;
  static constexpr int kRingOffset = 2 * kTileBytes;
  // dK / dV launch: one K-major chunk (128 rows x 64 columns, 128-byte swizzle) whose k-steps 0, 1, 2 are three
  // operands of their own: rows of (1, 1, 1, 0 ...); rows of -LSE / scale of the step's queries in three bf16
  // pieces; rows of -delta likewise.  One more MMA per score tile adds ones x (-LSE / scale)^T to Q K^T and
  // ones x (-delta)^T to dO V^T, so the compute warps get c S - LSE log2e and dP - delta without reading a
  // statistic per column from shared memory (which cost the launch a sixth of its step).
  static constexpr int kExtraOffset = kRingOffset + kSlots * kTileBytes;
  static constexpr int kExtraBytes = DKV ? kChunkBytes : 0;
  static constexpr int kBarOffset = kExtraOffset + kExtraBytes;
  // x_full, y_full[S], y_empty[S], t0_full, t1_full, p_ready, ds_ready, acc_done, drain, e_ready, t0_free
  static constexpr int kNumBars = 2 * kSlots + 9;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

template <int D, bool CAUSAL, bool DKV>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_wide_sm100(const __grid_constant__ CUtensorMap tmap_x0, const __grid_constant__ CUtensorMap tmap_x1,
                    const __grid_constant__ CUtensorMap tmap_y0, const __grid_constant__ CUtensorMap tmap_y1,
                    const AttnBwdParams p) {
  using L = AttnBwdWideSmem<D, DKV>;
  constexpr int SLOTS = L::kSlots;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kT1Col = 128, kAccCol = 256;
  constexpr uint32_t kPackCol = 32;    // packed dS (dQ launch) / packed P (dK / dV launch) start here inside T1
  // One pair of exponentials in so many takes the FMA pipe (a cubic) instead of the exponential unit; 0: none.
  // Measured: the dQ launch takes 2730 clocks per step with one pair in four and 3410 with none (a third is level,
  // a half slower).  The dK / dV launch, whose exponentials run under the chain of MMAs anyway, is 0.6-1.4 %
  // faster with none at D = 128 (under the power cap fewer instructions buy clock) and 1 % faster with one in
  // four at D = 64.
#if defined(WIR_BWD_POLY_DQ) && defined(WIR_BWD_POLY_DKV)
  constexpr int kPolyEvery = DKV ? WIR_BWD_POLY_DKV : WIR_BWD_POLY_DQ;
#else
  constexpr int kPolyEvery = (DKV && D == 128) ? 0 : 4;
#endif

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  const uint32_t x_full = bar_base;
  auto y_full = [&](uint32_t s) { return bar_base + 8u * (1 + s); };
  auto y_empty = [&](uint32_t s) { return bar_base + 8u * (1 + SLOTS + s); };
  const uint32_t t0_full = bar_base + 8u * (1 + 2 * SLOTS);
  const uint32_t t1_full = bar_base + 8u * (2 + 2 * SLOTS);
  const uint32_t p_ready = bar_base + 8u * (3 + 2 * SLOTS);
  const uint32_t ds_ready = bar_base + 8u * (4 + 2 * SLOTS);
  const uint32_t acc_done = bar_base + 8u * (5 + 2 * SLOTS);
  const uint32_t drain_bar = bar_base + 8u * (6 + 2 * SLOTS);
  const uint32_t e_ready = bar_base + 8u * (7 + 2 * SLOTS);     // dK / dV launch: the first step's extra operands are written
  const uint32_t t0_free = bar_base + 8u * (8 + 2 * SLOTS);     // dK / dV launch: every compute thread has read T0
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which tile, which steps ---------------------------------------------------------
  const int group = p.H / p.Hkv;
  const int batch = blockIdx.z;
  const int ny = (p.S + kBw2Rows - 1) / kBw2Rows;      // 128-row tiles along the sequence
  // DKV = false: blockIdx.x (heaviest causal tiles first) is the Q tile, blockIdx.y the query head.
  // DKV = true : blockIdx.x is the K/V tile, blockIdx.y the K/V head.
  const int xt = (!DKV && CAUSAL) ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int x_row0 = xt * kBw2Rows;
  const int head = blockIdx.y;
  const int x_plane = DKV ? (batch * p.Hkv + head) : (batch * p.H + head);
  // steps: DKV = false walks K/V tiles 0 .. y_end-1 of the head's K/V head;
  //        DKV = true  walks, for each query head of the group, Q tiles y_begin .. ny-1
  const int y_begin = (DKV && CAUSAL) ? xt : 0;
  const int y_end = (!DKV && CAUSAL) ? min(ny, xt + 1) : ny;
  const int per_head = max(0, y_end - y_begin);
  const int n_it = DKV ? per_head * group : per_head;
  auto y_tile_of = [&](int it) { return y_begin + (DKV ? it % per_head : it); };
  auto y_plane_of = [&](int it) {
    return DKV ? (batch * p.H + head * group + it / per_head) : (batch * p.Hkv + head / group);
  };

  // Ring position of a streamed tile: slot and phase parity, carried along by additions.
  struct RingPos { uint32_t slot, phase; };
  auto ring_next = [](RingPos r, uint32_t by) {
    r.slot += by;
    if (r.slot >= static_cast<uint32_t>(SLOTS)) { r.slot -= SLOTS; r.phase ^= 1u; }
    return r;
  };
  auto tile_addr = [&](RingPos r) { return smem_base + L::kRingOffset + r.slot * L::kTileBytes; };
  // Where tile `which` (0: Y0, 1: Y1) of step `it` sits.  Normally the ring is a FIFO of tiles in the order they are
  // loaded (tile k = 2 it + which in slot k % SLOTS).  A ring of four slots (dK / dV launch at D = 128) is only two
  // steps deep, and a FIFO would give Y0(it), the tile that is needed FIRST (its scores start as soon as the previous
  // ones have been read), the slot that is released LAST (Y0(it-2), after B2).  There the two tiles of a step trade
  // places every other step: Y0(it) takes the slot of Y1(it-2), which B1 releases a third of a step earlier.
  constexpr bool kCross = DKV && SLOTS == 4;
  auto pos_of = [](int it, int which) {
    if constexpr (kCross) {
      const uint32_t turn = (static_cast<uint32_t>(it) >> 1) & 1u;
      return RingPos{2u * (static_cast<uint32_t>(it) & 1u) + (static_cast<uint32_t>(which) ^ turn), turn};
    } else {
      const uint32_t k = 2u * static_cast<uint32_t>(it) + static_cast<uint32_t>(which);
      return RingPos{k % SLOTS, (k / SLOTS) & 1u};
    }
  };

  // Producer (thread 0, which also initialises the barriers): streamed tile `which` (0: Y0, 1: Y1) of step `it`
  // into the ring at `pos`.  The resident tiles and the first step go out before the CTA-wide barrier below.
  auto load_tile = [&](int it, int which, RingPos pos) -> bool {
    if (!mbar_wait(y_empty(pos.slot), pos.phase ^ 1, ctx, kRoleProducer, pos.slot, it)) return false;
    mbar_arrive_expect_tx(y_full(pos.slot), L::kTileBytes);
    const uint32_t dst = tile_addr(pos);
    const int row = y_tile_of(it) * kBw2Rows, plane = y_plane_of(it);
#pragma unroll
    for (int c = 0; c < D / 64; ++c)
      tma_load_3d(dst + c * L::kChunkBytes, which == 0 ? &tmap_y0 : &tmap_y1, y_full(pos.slot), c * 64, row, plane);
    return true;
  };
  bool p_ok = true;
  RingPos p_pos{0u, 0u};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(x_full, 1);
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(y_full(s), 1);
      mbar_init(y_empty(s), 1);
    }
    mbar_init(t0_full, 1);
    mbar_init(t1_full, 1);
    mbar_init(p_ready, kBwdComputeThreads);
    mbar_init(ds_ready, kBwdComputeThreads);
    mbar_init(acc_done, 1);
    mbar_init(drain_bar, 1);
    mbar_init(e_ready, kBwdComputeThreads);
    mbar_init(t0_free, kBwdComputeThreads);
    fence_mbar_init();
    fence_proxy_async_smem();
    if (n_it > 0) {
      mbar_arrive_expect_tx(x_full, 2 * L::kTileBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_3d(smem_base + c * L::kChunkBytes, &tmap_x0, x_full, c * 64, x_row0, x_plane);
        tma_load_3d(smem_base + L::kTileBytes + c * L::kChunkBytes, &tmap_x1, x_full, c * 64, x_row0, x_plane);
      }
      p_ok = load_tile(0, 0, p_pos);        // (step 0 sits in slots 0 and 1 either way)
      p_pos = ring_next(p_pos, 1);
      if (p_ok) {
        p_ok = load_tile(0, 1, p_pos);
        p_pos = ring_next(p_pos, 1);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && n_it > 0) {
      bool ok = p_ok;
      int issued = ok ? 2 : 0;    // tiles handed to the copy engine so far (step 0 went out before the barrier)
      for (int it = 1; ok && it < n_it; ++it) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          if (!ok) break;
          ok = load_tile(it, which, kCross ? pos_of(it, which) : p_pos);
          if (ok) {
            p_pos = ring_next(p_pos, 1);
            ++issued;
          }
        }
      }
      if (!ok || *abort_flag) {
        // every copy in flight must have landed before the CTA may exit
        mbar_wait_quiet(x_full, 0);
        const int n = issued < SLOTS ? issued : SLOTS;
        for (int back = 1; back <= n; ++back) {
          const int k = issued - back;
          const RingPos r = pos_of(k >> 1, k & 1);
          mbar_wait_quiet(y_full(r.slot), r.phase);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_t = idesc_bf16_f32(kBw2Rows, kBw2Rows, 0, 0);   // X Y^T: both K-major, N = 128
    constexpr uint32_t idesc_acc = idesc_bf16_f32(kBw2Rows, D, 0, 1);        // (P | dS) Y: B is MN-major, N = D
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    const uint64_t x0d = desc64(smem_desc_lo(smem_base, 16), desc_hi);
    const uint64_t x1d = desc64(smem_desc_lo(smem_base + L::kTileBytes, 16), desc_hi);
    auto wait_tile = [&](RingPos r, int it) { return mbar_wait_warp(y_full(r.slot), r.phase, ctx, kRoleMma, 10, it); };
    // T = X Y^T: D/16 k-steps, four (one 64-element chunk of the head dimension, 32 bytes per step) per block
    auto issue_a = [&](uint32_t t_col, uint64_t xd, RingPos r) {
      const uint64_t yd = desc64(smem_desc_lo(tile_addr(r), 16), desc_hi);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const uint64_t o = static_cast<uint64_t>((c * L::kChunkBytes) >> 4);
        mma_ss_elect_x4(tmem_base + t_col, xd + o, xd + o + 2, xd + o + 4, xd + o + 6, yd + o, yd + o + 2, yd + o + 4,
                        yd + o + 6, idesc_t, c > 0 ? 1u : 0u);
      }
    };
    // acc += (P | dS) Y: the 128 streamed rows are the K dimension, eight k-steps of 16 rows (2048 bytes of an
    // MN-major tile whose 64-column chunks are kChunkBytes apart), A = 8 packed columns of tensor memory per step
    // (a_col0 / a_col1: where the packed values of streamed rows 0-63 / 64-127 sit)
    auto issue_b = [&](uint32_t acc_col, uint32_t a_col0, uint32_t a_col1, RingPos r, uint32_t accumulate) {
      const uint64_t yd = desc64(smem_desc_lo(tile_addr(r), L::kChunkBytes), desc_hi);
#pragma unroll
      for (int m = 0; m < kBw2Rows / 64; ++m) {
        const uint64_t y = yd + static_cast<uint64_t>(512 * m);
        mma_ts_elect_x4(tmem_base + acc_col, tmem_base + (m == 0 ? a_col0 : a_col1), y, y + 128, y + 256, y + 384,
                        idesc_acc, (accumulate != 0u || m > 0) ? 1u : 0u);
      }
    };
    // dK / dV launch: one more k-step per score tile, ones x (statistic)^T (see AttnBwdWideSmem::kExtraOffset);
    // which = 1: -LSE / scale into T0, 2: -delta into T1
    const uint32_t extra_lo = smem_desc_lo(smem_base + L::kExtraOffset, 16);
    auto issue_extra = [&](uint32_t t_col, uint32_t which) {
      if constexpr (DKV) mma_ss_elect(tmem_base + t_col, extra_lo, desc_hi, extra_lo + 2u * which, desc_hi, idesc_t, 1u);
    };
    bool ok = true;
    WIR_TRACE_DECL;
    RingPos pos0{0u, 0u}, pos1{1u, 0u};     // Y0(j), Y1(j) of the current step; the next step's are two tiles on

    if (n_it > 0) ok = mbar_wait_warp(x_full, 0, ctx, kRoleMma, 1, 0);
    if (DKV && ok && n_it > 0) ok = mbar_wait_warp(e_ready, 0, ctx, kRoleMma, 2, 0);
    if (ok && n_it > 0) ok = wait_tile(pos0, 0);
    if (ok && n_it > 0) {
      tc_fence_after();
      issue_a(0, x0d, pos0);
      issue_extra(0, 1);
      mma_commit_elect(t0_full);
      ok = wait_tile(pos1, 0);
      if (ok) {
        tc_fence_after();
        issue_a(kT1Col, x1d, pos1);
        issue_extra(kT1Col, 2);
        mma_commit_elect(t1_full);
        if (!DKV) mma_commit_elect(y_empty(pos1.slot));      // dQ launch: A2 is the last reader of V(j)
      }
    }
    for (int it = 0; ok && it < n_it; ++it) {
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const bool more = it + 1 < n_it;
      const RingPos nxt0 = kCross ? pos_of(it + 1, 0) : ring_next(pos0, 2);
      const RingPos nxt1 = kCross ? pos_of(it + 1, 1) : ring_next(pos1, 2);
      const uint32_t acc = it > 0 ? 1u : 0u;
      // the next step's tiles were asked for long ago: look at their barriers before the waits that are true
      // dependencies, so that nothing but a fence stands between those and the MMAs
      // (both tiles' barriers tested together: one vote, one branch; the full waits only if one is still open)
      bool landed1 = !more;
      if (!DKV && more) {
        const bool both = mbar_test_wait(y_full(nxt0.slot), nxt0.phase) & mbar_test_wait(y_full(nxt1.slot), nxt1.phase);
        landed1 = __all_sync(0xffffffffu, both);
      }
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 0, it);
      if constexpr (DKV) {
        // the next scores as soon as every thread has read the current ones (P goes into T1, not back into T0) and
        // their Q tile has landed; if it has not, B1 goes first
        auto next_scores = [&]() {
          tc_fence_after();
          issue_a(0, x0d, nxt0);
          issue_extra(0, 1);
          mma_commit_elect(t0_full);
        };
        bool scores_out = !more;
        if (more) {
          if (!mbar_wait_warp(t0_free, ph, ctx, kRoleMma, 15, it)) { ok = false; break; }
          if (__all_sync(0xffffffffu, mbar_test_wait(y_full(nxt0.slot), nxt0.phase))) {
            next_scores();
            scores_out = true;
          }
        }
        if (!mbar_wait_warp(p_ready, ph, ctx, kRoleMma, 20, it)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 1, it);
        issue_b(kAccCol, kT1Col + kPackCol, kT1Col + kPackCol + 32, pos1, acc);      // dV += P^T dO
        mma_commit_elect(y_empty(pos1.slot));
        if (!scores_out) {
          if (!wait_tile(nxt0, it + 1)) { ok = false; break; }
          next_scores();
        }
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 2, it);
        if (!mbar_wait_warp(ds_ready, ph, ctx, kRoleMma, 30, it)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 3, it);
        issue_b(kAccCol + D, kT1Col, kT1Col + 96, pos0, acc);                         // dK += dS^T Q
        mma_commit_elect(y_empty(pos0.slot));
        if (!more) mma_commit_elect(acc_done);
        if (more) {
          if (!wait_tile(nxt1, it + 1)) { ok = false; break; }    // (B2 is executing meanwhile)
          tc_fence_after();
          issue_a(kT1Col, x1d, nxt1);                             // next dP, behind the MMAs that read P and dS
          issue_extra(kT1Col, 2);
          mma_commit_elect(t1_full);
        }
      } else {
        if (!landed1 && !wait_tile(nxt0, it + 1)) { ok = false; break; }
        if (!mbar_wait_warp(p_ready, ph, ctx, kRoleMma, 20, it)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 1, it);
        if (more) {
          issue_a(0, x0d, nxt0);                                  // next scores (T0 has been read)
          mma_commit_elect(t0_full);
        }
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 2, it);
        if (!landed1 && !wait_tile(nxt1, it + 1)) { ok = false; break; }
        if (!mbar_wait_warp(ds_ready, ph, ctx, kRoleMma, 30, it)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 3, it);
        issue_b(kAccCol, kT1Col + kPackCol, kT1Col + kPackCol + 32, pos0, acc);       // dQ += dS K
        mma_commit_elect(y_empty(pos0.slot));
        if (!more) mma_commit_elect(acc_done);
        if (more) {
          issue_a(kT1Col, x1d, nxt1);                             // next dP, behind the MMAs that read dS
          mma_commit_elect(t1_full);
          mma_commit_elect(y_empty(nxt1.slot));                   // A2 is the last reader of V(j+1)
        }
      }
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 4, it);
      pos0 = nxt0;
      pos1 = nxt1;
    }
    if (!ok || *abort_flag) {
      mma_commit_elect(drain_bar);
      mbar_wait_quiet(drain_bar, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    const int quarter = warp & 3;                       // tensor-memory lanes 32*quarter .. +31
    const int half = (warp - 2) >> 2;                   // warpgroup: columns 64 half ... of T0 / T1
    const int tid = quarter * 32 + lane;                // row of the resident tiles owned by this thread
    const int x_row = x_row0 + tid;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float c = p.scale_log2;
    constexpr float kLog2e = 1.4426950408889634f;
    bool ok = true;
    WIR_TRACE_DECL;
    const bool traced = (quarter == 0 && lane == 0);
    if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 90, 0);     // set-up done, prologue starts

    // per-row statistics (DKV = false): L2 = LSE log2 e, ds = delta * scale.  delta = rowsum(dO * O) comes from a
    // small kernel of its own that runs before this launch (attn_bwd_delta below): computed here, per thread from
    // its own row, it was a chain of round trips to memory of 13000 clocks per CTA, an eighth of the launch.
    float row_l2 = 0.f, row_ds = 0.f;
    if constexpr (!DKV) {
      if (x_row < p.S) {
        const size_t r = static_cast<size_t>(x_plane) * p.S + x_row;
        row_ds = p.delta[r] * p.scale;
        row_l2 = p.LSE[r] * kLog2e;
      }
    }

    // DKV: the statistics of a step's 128 queries (LSE, delta) reach the scores through one more MMA per score
    // tile (see AttnBwdWideSmem::kExtraOffset): thread t of group 0 writes -LSE / scale of query t, thread t of
    // group 1 -delta of query t, as three bf16 pieces into row t of its k-step of the extra chunk, for the NEXT
    // step, once the MMA that read the current step's values has completed.  The values are fetched from global
    // memory a step before that.
    auto fetch_stat = [&](int it) -> float {
      const int q = y_tile_of(it) * kBw2Rows + tid;
      const size_t r = static_cast<size_t>(y_plane_of(it)) * p.S + min(q, p.S - 1);
      return (half == 0) ? p.LSE[r] : p.delta[r];
    };
    const float stat_factor = (half == 0) ? -1.0f / p.scale : -1.0f;
    // k-step `slot` of row `row` of the extra chunk: 16 bf16 = two 16-byte units, swizzled like every K-major tile
    // here (unit u of row r at r / 8 * 1024 + r % 8 * 128 + (u ^ r % 8) * 16)
    auto write_extra = [&](int slot, int row, uint32_t w0, uint32_t w1) {
      uint8_t* base = smem + L::kExtraOffset + (row >> 3) * 1024 + (row & 7) * 128;
      *reinterpret_cast<uint4*>(base + (((2 * slot) ^ (row & 7)) << 4)) = make_uint4(w0, w1, 0u, 0u);
      *reinterpret_cast<uint4*>(base + (((2 * slot + 1) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
    };
    auto write_stat = [&](float raw) {         // three bf16 pieces whose sum is raw * stat_factor to 24 bits
      const float v = raw * stat_factor;
      const __nv_bfloat16 h = __float2bfloat16_rn(v);
      const float r1 = v - __bfloat162float(h);
      const __nv_bfloat16 m = __float2bfloat16_rn(r1);
      const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
      const uint32_t w0 = static_cast<uint32_t>(__bfloat16_as_ushort(h)) | (static_cast<uint32_t>(__bfloat16_as_ushort(m)) << 16);
      write_extra(1 + half, tid, w0, static_cast<uint32_t>(__bfloat16_as_ushort(l)));
    };
    float stat_next = 0.f, stat_fetched = 0.f;
    if constexpr (DKV) {
      if (n_it > 0) {
        if (half == 0) write_extra(0, tid, 0x3f803f80u, 0x00003f80u);      // (1, 1, 1, 0 ...)
        write_stat(fetch_stat(0));
        fence_proxy_async_smem();
        mbar_arrive(e_ready);
        if (n_it > 1) stat_next = fetch_stat(1);
      }
    }
    if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 91, 0);     // prologue done

    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const int y_row0 = y_tile_of(it) * kBw2Rows;
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 10, it);
      // ---- P from T0
      bool got = mbar_wait(t0_full, ph, ctx, kRoleSoftmax, 0, it);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      if constexpr (DKV) {
        // the MMA that read this step's -LSE / scale is done: the next step's may take its place
        if (half == 0 && it + 1 < n_it) {
          write_stat(stat_next);
          fence_proxy_async_smem();
        }
      }
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 11, it);

      // masks are only needed on tiles that touch the diagonal or the end of the sequence
      const bool ragged = (y_row0 + kBw2Rows > p.S) || (x_row0 + kBw2Rows > p.S);
      const bool diagonal = CAUSAL && (y_row0 == x_row0);
      const bool masked = ragged || diagonal;

      float pv[64];      // this thread's 64 values of P, kept for the dS phase
      uint32_t pk[DKV ? 32 : 1];   // dK / dV launch: and packed to bf16, stored once T1 has been read
      {
        uint32_t t0[64];
        tmem_ld32(lane_base + half * 64, t0);
        tmem_ld32(lane_base + half * 64 + 32, t0 + 32);
        tmem_wait_ld();
        // T0 is free as soon as it has been read, and the next scores start now: P stays in registers (dQ launch)
        // or goes into T1 (dK / dV launch)
        tc_fence_before();
        mbar_arrive(DKV ? t0_free : p_ready);
        if constexpr (DKV) {
          // The statistic for the step after the next is fetched HERE, with the exponentials between the load and
          // the next fence or arrival: both wait for every earlier access of the thread, a load from global memory
          // included, and right behind the load they kept the thread waiting for it.
          if (it + 2 < n_it) stat_fetched = fetch_stat(it + 2);
        }
        if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 15, it);
        // in pairs (packed f32x2 arithmetic); one pair in kPolyEvery takes its exponentials on the FMA pipe
        // (a cubic, relative error below 6e-4, far inside bf16's 4e-3)
        const float2 c2 = make_float2(c, c);
        const float2 l2 = make_float2(-row_l2, -row_l2);       // (dK / dV launch: zero, the tensor core subtracted it)
        // The loop exists twice, with and without the mask: a test of `masked` inside it, once per pair, is a
        // branch per pair, across which the compiler does not move instructions.
        auto p_phase = [&](auto masked_c) {
          constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int col = half * 64 + 2 * k;
            const float2 t = make_float2(__uint_as_float(t0[2 * k]), __uint_as_float(t0[2 * k + 1]));
            const float2 x = DKV ? __fmul2_rn(t, c2) : __ffma2_rn(t, c2, l2);
            float2 e;
            if (kPolyEvery > 0 && (k % (kPolyEvery > 0 ? kPolyEvery : 1)) == 0) {
              e = ex2_fma2(x);
            } else {
              e.x = ex2_approx(x.x);
              e.y = ex2_approx(x.y);
            }
            if constexpr (kMasked) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int y = y_row0 + col + h;             // index along the streamed tile
                const int qi = DKV ? y : x_row;             // query index
                const int ki = DKV ? x_row : y;             // key index
                if (qi >= p.S || ki >= p.S || (CAUSAL && ki > qi)) (h == 0 ? e.x : e.y) = 0.f;
              }
            }
            pv[2 * k] = e.x;
            pv[2 * k + 1] = e.y;
            if constexpr (DKV) pk[k] = pack_bf16(e.x, e.y);
          }
        };
        if (masked) p_phase(std::true_type{});
        else p_phase(std::false_type{});
        if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 16, it);
      }

      // ---- dS from T1 and P
      got = mbar_wait(t1_full, ph, ctx, kRoleSoftmax, 1, it);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      if constexpr (DKV) {
        if (half == 1 && it + 1 < n_it) {      // as above, for -delta
          write_stat(stat_next);
          fence_proxy_async_smem();
        }
      }
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 13, it);
      {
        uint32_t t1[64];
        tmem_ld32(lane_base + kT1Col + half * 64, t1);
        tmem_ld32(lane_base + kT1Col + half * 64 + 32, t1 + 32);
        tmem_wait_ld();
        if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 17, it);
        if constexpr (DKV) {
          // P, packed, over T1 columns 32-95 (each group over columns it has just read): B1 reads it from there
          tmem_st16(lane_base + kT1Col + kPackCol + half * 32, pk);
          tmem_st16(lane_base + kT1Col + kPackCol + half * 32 + 16, pk + 16);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_ready);
          if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 12, it);
        }
        const float2 s2 = make_float2(p.scale, p.scale);
        const float2 d2 = make_float2(-row_ds, -row_ds);
        uint32_t dk[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const float2 t = make_float2(__uint_as_float(t1[2 * k]), __uint_as_float(t1[2 * k + 1]));
          const float2 u = DKV ? __fmul2_rn(t, s2) : __ffma2_rn(t, s2, d2);
          const float2 d = __fmul2_rn(make_float2(pv[2 * k], pv[2 * k + 1]), u);
          dk[k] = pack_bf16(d.x, d.y);
        }
        // dS, packed: dQ launch over T1 columns 32-95; dK / dV launch, where P sits there, over the outer columns
        // (group 0: 0-31, group 1: 96-127)
        const uint32_t ds_col = kT1Col + (DKV ? half * 96 : kPackCol + half * 32);
        tmem_st16(lane_base + ds_col, dk);
        tmem_st16(lane_base + ds_col + 16, dk + 16);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(ds_ready);
      stat_next = stat_fetched;
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 14, it);
    }

    if (ok && n_it > 0) {
      const bool got = mbar_wait(acc_done, 0, ctx, kRoleEpilogue, 0, n_it);
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 92, 0);   // accumulators complete
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        // each warp turns its 32 x 32 blocks around in shared memory (XOR-swizzled; the ring is idle by now) and
        // stores whole 128-byte rows, four rows per instruction
        uint8_t* stage = smem + L::kRingOffset + (warp - 2) * 4096;
        const int row0 = x_row0 + quarter * 32;
        const int rows_valid = min(32, p.S - row0);
        const size_t r0 = static_cast<size_t>(x_plane) * p.S + row0;
#pragma unroll 1
        for (int a = 0; a < (DKV ? 2 : 1); ++a) {
          float* dst = (a == 0 ? p.out0 : p.out1) + r0 * D;
#pragma unroll 1
          for (int cidx = half * (D / 64); cidx < (half + 1) * (D / 64); ++cidx) {   // each group stores half the columns
            uint32_t o[32];
            tmem_ld32(lane_base + kAccCol + a * D + cidx * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(stage + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                  make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            __syncwarp();
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
              const int rl = rr * 4 + (lane >> 3);
              const uint4 q = *reinterpret_cast<const uint4*>(stage + rl * 128 + (((lane & 7) ^ (rl & 7)) << 4));
              if (rl < rows_valid)
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rl) * D + cidx * 32 + (lane & 7) * 4) = q;
            }
            __syncwarp();
          }
        }
      }
    } else if (ok && n_it == 0) {
      // nothing attends here (only possible past the end of the sequence): gradients are zero
      if (x_row < p.S && half == 0) {
        const size_t r = static_cast<size_t>(x_plane) * p.S + x_row;
        for (int a = 0; a < (DKV ? 2 : 1); ++a) {
          float* dst = (a == 0 ? p.out0 : p.out1) + r * D;
          for (int v = 0; v < D / 4; ++v) reinterpret_cast<uint4*>(dst)[v] = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
#ifdef WIR_TRACE
  if (threadIdx.x == 64) {
    WIR_TRACE_DECL;
    WIR_TRACE_EVENT(p.trace, 3, 93, 0);   // epilogue done
  }
#endif
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[r] = sum over the head dimension of dO[r][:] * O[r][:] for every row r of [B, H, S, D] (bf16, D = 64 or 128).
// Sixteen bytes per lane: D / 8 lanes share a row, a warp takes 256 / D ... rows per step; memory-bound, one pass
// over O and dO.
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_delta(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                                      float* __restrict__ delta, long long rows) {
  constexpr int kLanesPerRow = D / 8;                 // 16 (D = 128) or 8 (D = 64)
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;
  const int lane = threadIdx.x & 31;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int sub = lane / kLanesPerRow, piece = lane % kLanesPerRow;
  for (long long r0 = warp_global * kRowsPerWarp; r0 < rows; r0 += n_warps * kRowsPerWarp) {
    const long long r = r0 + sub;
    float acc = 0.f;
    if (r < rows) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(O + r * D) + piece);
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(dO + r * D) + piece);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 af = __bfloat1622float2(a2[e]), gf = __bfloat1622float2(g2[e]);
        acc = fmaf(af.x, gf.x, acc);
        acc = fmaf(af.y, gf.y, acc);
      }
    }
#pragma unroll
    for (int off = kLanesPerRow / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (r < rows && piece == 0) delta[r] = acc;
  }
}

}  // namespace wir
