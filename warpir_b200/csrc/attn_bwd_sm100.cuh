// Attention backward for sm_100a: given Q, K, V, O, dO and the forward's LSE, computes
// dQ, dK, dV (fp32), the counterpart of the reference's hand-written Hopper backward
// (kernel_examples/attention/mha_h100.cu:239-642: a preparation kernel for
// delta = rowsum(dO * O), then the gradient kernel; host wrapper attention_backward,
// mha_h100.cu:799-1010, which also returns fp32 gradients).
//
// With c = scale * log2(e):  P = 2^(c Q K^T - LSE log2 e),  dP = dO V^T,
// dS = P * (dP - delta) * scale,  dV = P^T dO,  dK = dS^T Q,  dQ = dS K.
//
// The reference accumulates dQ with atomics from the CTAs that own the K/V tiles.  Here
// the work is two launches of ONE kernel template, each deterministic and atomic-free:
//
//   DKV = false (grid over 128-row Q tiles):  streams 64-key K/V tiles, recomputes S and
//     dP, accumulates dQ in tensor memory.  Its prologue also computes delta and stores
//     it for the second launch.
//   DKV = true  (grid over 128-key K/V tiles): streams 64-row Q/dO tiles of every query
//     head of the group, recomputes S^T and dP^T, accumulates dV and dK.
//
// Both are the same pipeline on different operands.  With X0, X1 the two resident
// 128 x D tiles and Y0, Y1 the streamed 64 x D tiles of step `it`:
//
//   stage 1 (tcgen05.mma, SS):  T0 = X0 Y0^T,  T1 = X1 Y1^T          (128 x 64 each)
//   compute warps:              P = 2^(c T0 - L2),  dS = P (T1 - delta) scale, both
//                               packed to bf16 over columns 16..47 of T0 / T1
//   stage 2 (tcgen05.mma, TS):  DKV:  acc0 += P  Y1   (dV),  acc1 += dS Y0   (dK)
//                               else: acc0 += dS Y0   (dQ)
//
//   (DKV = false: X = Q, dO and Y = K, V, statistics per row.
//    DKV = true:  X = K, V  and Y = Q, dO, statistics per column.)
//
// Tensor memory: T0[2] at columns 0 / 64, T1[2] at 128 / 192 (double-buffered so stage 1
// of step it+1 runs while the compute warps work on step it), acc0 at 256, acc1 at
// 256 + D.  Warp 0 is the TMA producer, warp 1 issues every MMA (whole warp, one elected
// lane), warps 2-9 are two compute warpgroups: thread = one tensor-memory lane (row).  The
// groups take the steps in turn (group g the steps of parity g, which are the steps of score
// buffer g), each doing all 64 columns of its step in two passes of 32.  That keeps the groups
// out of phase: while one waits for its scores, loads them or hands P / dS over, the other is
// in its arithmetic, so the exponential and conversion units (the compute warps' bottleneck)
// stay busy.  With both groups on the same step (splitting its columns) every one of those
// waits was paid once per step by all eight warps at once.
// MMAs execute in issue order, which makes the aliasing safe: stage 1 of step it+2
// overwrites T0/T1[b] only after stage 2 of step it, which reads P/dS from them.
#pragma once

#include "ptx.cuh"

namespace wir {

constexpr int kBwdBX = 128;        // rows of the resident tiles = MMA M
constexpr int kBwdBY = 64;         // rows of the streamed tiles = MMA N of stage 1, K of stage 2
constexpr int kBwdThreads = 320;        // producer warp, MMA warp, two compute warpgroups
constexpr int kBwdComputeThreads = 256;

struct AttnBwdParams {
  int B, H, Hkv, S;
  float scale;             // softmax scale
  float scale_log2;        // scale * log2(e)
  const __nv_bfloat16* Q;  // [B, H, S, D]   (DKV = false: copied into tensor memory)
  const __nv_bfloat16* O;  // [B, H, S, D]   (DKV = false: for delta)
  const __nv_bfloat16* dO; // [B, H, S, D]
  const float* LSE;        // [B, H, S] natural-log logsumexp of the scaled scores
  float* delta;            // [B, H, S] written by the DKV = false launch, read by the other
  float* out0;             // DKV = false: dQ [B, H, S, D];  DKV = true: dV [B, Hkv, S, D]
  float* out1;             // DKV = true: dK [B, Hkv, S, D]
  int* status;
  unsigned long long* trace;   // event trace buffer of debug builds (-DWIR_TRACE), else unused
};

template <int D, bool DKV>
struct AttnBwdSmem {
  // DKV = false keeps its resident operands (Q, dO) in tensor memory, not in shared memory
  static constexpr int kStages = DKV ? ((D == 128) ? 4 : 8) : ((D == 128) ? 6 : 12);
  static constexpr int kXChunkBytes = kBwdBX * 128;
  static constexpr int kXTileBytes = (D / 64) * kXChunkBytes;
  static constexpr int kYChunkBytes = kBwdBY * 128;
  static constexpr int kYTileBytes = (D / 64) * kYChunkBytes;
  static constexpr int kYOffset = DKV ? 2 * kXTileBytes : 0;
  static constexpr int kStatsOffset = kYOffset + kStages * 2 * kYTileBytes;   // [2 groups][2 buffers][2 vectors][64] floats
  static constexpr int kBarOffset = kStatsOffset + 2 * 2 * 2 * kBwdBY * 4;
  // x_full, y_full[S], y_empty[S], t_full[2], pds_full[2], acc_done, drain
  static constexpr int kNumBars = 1 + 2 * kStages + 6;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

template <int D, bool CAUSAL, bool DKV>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_sm100(const __grid_constant__ CUtensorMap tmap_x0, const __grid_constant__ CUtensorMap tmap_x1,
               const __grid_constant__ CUtensorMap tmap_y0, const __grid_constant__ CUtensorMap tmap_y1,
               const AttnBwdParams p) {
  using L = AttnBwdSmem<D, DKV>;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kAccCol = 256;
  constexpr uint32_t kXCol = 256 + D;   // DKV = false: Q and dO rows as packed bf16, D/2 columns each

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  const uint32_t x_full = bar_base;
  auto y_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto y_empty = [&](int s) { return bar_base + 8u * (1 + STAGES + s); };
  auto t_full = [&](int b) { return bar_base + 8u * (1 + 2 * STAGES + b); };
  auto pds_full = [&](int b) { return bar_base + 8u * (3 + 2 * STAGES + b); };
  const uint32_t acc_done = bar_base + 8u * (5 + 2 * STAGES);
  const uint32_t drain_bar = bar_base + 8u * (6 + 2 * STAGES);
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  float* stats = reinterpret_cast<float*>(smem + L::kStatsOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which tile, which steps ---------------------------------------------------------
  const int group = p.H / p.Hkv;
  const int batch = blockIdx.z;
  const int ny = (p.S + kBwdBY - 1) / kBwdBY;          // 64-row tiles along the sequence
  // DKV = false: blockIdx.x (heaviest causal tiles first) is the Q tile, blockIdx.y the query head.
  // DKV = true : blockIdx.x is the K/V tile, blockIdx.y the K/V head.
  const int xt = (!DKV && CAUSAL) ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int x_row0 = xt * kBwdBX;
  const int head = blockIdx.y;
  const int x_plane = DKV ? (batch * p.Hkv + head) : (batch * p.H + head);
  // steps: DKV = false walks K/V tiles 0 .. y_end-1 of the head's K/V head;
  //        DKV = true  walks, for each query head of the group, Q tiles y_begin .. ny-1
  const int y_begin = (DKV && CAUSAL) ? (x_row0 / kBwdBY) : 0;
  const int y_end = (!DKV && CAUSAL) ? min(ny, (x_row0 + kBwdBX) / kBwdBY) : ny;
  const int per_head = max(0, y_end - y_begin);
  const int n_it = DKV ? per_head * group : per_head;
  auto y_tile_of = [&](int it) { return y_begin + (DKV ? it % per_head : it); };
  auto y_plane_of = [&](int it) {
    return DKV ? (batch * p.H + head * group + it / per_head) : (batch * p.Hkv + head / group);
  };

  // Producer (thread 0, which also initialises the barriers): loads of the streamed tiles of step
  // `it` into ring slot it % STAGES.  The resident tiles and the first step go out before the
  // CTA-wide barrier below, so their latency overlaps the rest of the set-up.
  auto load_y = [&](int it) -> bool {
    const int s = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1;
    if (!mbar_wait(y_empty(s), ph ^ 1, ctx, kRoleProducer, s, it)) return false;
    mbar_arrive_expect_tx(y_full(s), 2 * L::kYTileBytes);
    const uint32_t dst = smem_base + L::kYOffset + s * 2 * L::kYTileBytes;
    const int row = y_tile_of(it) * kBwdBY, plane = y_plane_of(it);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      tma_load_3d(dst + c * L::kYChunkBytes, &tmap_y0, y_full(s), c * 64, row, plane);
      tma_load_3d(dst + L::kYTileBytes + c * L::kYChunkBytes, &tmap_y1, y_full(s), c * 64, row, plane);
    }
    return true;
  };
  bool p_ok = true;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(x_full, DKV ? 1 : kBwdComputeThreads);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(y_full(s), 1);
      mbar_init(y_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(t_full(b), 1);
      mbar_init(pds_full(b), kBwdComputeThreads / 2);   // the one warpgroup that owns buffer b
    }
    mbar_init(acc_done, 1);
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    if (n_it > 0) {
      if constexpr (DKV) {
        mbar_arrive_expect_tx(x_full, 2 * L::kXTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_3d(smem_base + c * L::kXChunkBytes, &tmap_x0, x_full, c * 64, x_row0, x_plane);
          tma_load_3d(smem_base + L::kXTileBytes + c * L::kXChunkBytes, &tmap_x1, x_full, c * 64, x_row0, x_plane);
        }
      }
      p_ok = load_y(0);
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
      int it = 1;   // step 0 went out before the barrier
      for (; ok && it < n_it; ++it) ok = load_y(it);
      if (!ok) --it;   // the step whose wait ran out issued nothing
      if (!ok || *abort_flag) {
        if (DKV) mbar_wait_quiet(x_full, 0);
        const int n = it < STAGES ? it : STAGES;
        for (int back = 1; back <= n; ++back) {
          const int i = it - back;
          mbar_wait_quiet(y_full(i % STAGES), (i / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_t = idesc_bf16_f32(kBwdBX, kBwdBY, 0, 0);   // X Y^T: both K-major
    constexpr uint32_t idesc_acc = idesc_bf16_f32(kBwdBX, D, 0, 1);      // (P | dS) Y: B is MN-major
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    const uint32_t x0_lo = smem_desc_lo(smem_base, 16);
    const uint32_t x1_lo = smem_desc_lo(smem_base + L::kXTileBytes, 16);
    // Ring position (slot, phase parity) of a step's streamed tiles, carried along by additions: the issuing
    // warp takes 6-12 clocks over every dependent instruction, and `it % STAGES`, `it / STAGES` with six or
    // twelve stages are a dozen of them each.
    struct RingPos { uint32_t slot, phase; };
    auto ring_next = [](RingPos r) {
      if (++r.slot == static_cast<uint32_t>(STAGES)) { r.slot = 0; r.phase ^= 1u; }
      return r;
    };
    auto y_addr = [&](RingPos r) { return smem_base + L::kYOffset + r.slot * (2 * L::kYTileBytes); };
    auto wait_y = [&](RingPos r, int it) { return mbar_wait_warp(y_full(r.slot), r.phase, ctx, kRoleMma, 10, it); };
    bool ok = true;
    WIR_TRACE_DECL;
    // stage 1 of step `it`, whose streamed tiles (ring position r) have landed
    auto stage1 = [&](int it, RingPos r) {
      const int b = it & 1;
      const uint32_t y0_lo = smem_desc_lo(y_addr(r), 16);
      const uint32_t y1_lo = smem_desc_lo(y_addr(r) + L::kYTileBytes, 16);
      // groups of four k-steps (one 64-column chunk of the head dimension: 32 bytes per step)
#pragma unroll
      for (int c4 = 0; c4 < D / 64; ++c4) {
        const uint32_t xo = (c4 * L::kXChunkBytes) >> 4, yo = (c4 * L::kYChunkBytes) >> 4;
        const uint32_t acc = c4 > 0 ? 1u : 0u;
        const uint64_t y0d = desc64(y0_lo + yo, desc_hi), y1d = desc64(y1_lo + yo, desc_hi);
        if constexpr (DKV) {
          const uint64_t x0d = desc64(x0_lo + xo, desc_hi), x1d = desc64(x1_lo + xo, desc_hi);
          mma_ss_elect_x4(tmem_base + b * 64, x0d, x0d + 2, x0d + 4, x0d + 6, y0d, y0d + 2, y0d + 4, y0d + 6, idesc_t, acc);
          mma_ss_elect_x4(tmem_base + 128 + b * 64, x1d, x1d + 2, x1d + 4, x1d + 6, y1d, y1d + 2, y1d + 4, y1d + 6,
                          idesc_t, acc);
        } else {   // A operands (Q, dO) from tensor memory
          mma_ts_elect_x4(tmem_base + b * 64, tmem_base + kXCol + c4 * 32, y0d, y0d + 2, y0d + 4, y0d + 6, idesc_t, acc);
          mma_ts_elect_x4(tmem_base + 128 + b * 64, tmem_base + kXCol + D / 2 + c4 * 32, y1d, y1d + 2, y1d + 4, y1d + 6,
                          idesc_t, acc);
        }
      }
      mma_commit_elect(t_full(b));
    };

    if (n_it > 0) ok = mbar_wait_warp(x_full, 0, ctx, kRoleMma, 1, 0);
    tc_fence_after();
    RingPos cur{0u, 0u}, ahead{0u, 0u};      // positions of step it and of step it + 2
    for (int it = 0; ok && it < 2 && it < n_it; ++it) {
      ok = wait_y(ahead, it);
      if (ok) {
        tc_fence_after();
        stage1(it, ahead);
      }
      ahead = ring_next(ahead);
    }
    if (n_it == 1) ahead = ring_next(ahead);
    for (int it = 0; ok && it < n_it; ++it) {
      const int b = it & 1;
      const bool more = it + 2 < n_it;
      // The tiles of step it + 2 were asked for some steps ago.  Their barrier is tested here, before the one
      // wait that is a true dependency (a look at a barrier costs the issuing warp 75-150 clocks even when it is
      // long complete, and the tensor core's queue is about four MMAs deep); only if they have not landed yet
      // is there a wait between the two stages.
      const bool landed = !more || __all_sync(0xffffffffu, mbar_test_wait(y_full(ahead.slot), ahead.phase));
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 0, it);
      if (!mbar_wait_warp(pds_full(b), (it >> 1) & 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 1, it);
      // as B operands the streamed tiles are read with the 64 tile rows as K: chunks of 64
      // columns kYChunkBytes apart, 16 rows (2048 bytes) per k-step
      const uint32_t y0_mn = smem_desc_lo(y_addr(cur), L::kYChunkBytes);
      const uint32_t y1_mn = smem_desc_lo(y_addr(cur) + L::kYTileBytes, L::kYChunkBytes);
      const uint32_t p_tmem = tmem_base + b * 64 + 16;          // bf16 P inside T0[b]
      const uint32_t ds_tmem = tmem_base + 128 + b * 64 + 16;   // bf16 dS inside T1[b]
      {
        // four k-steps of 16 streamed rows (2048 bytes of an MN-major tile) each
        const uint32_t acc = it > 0 ? 1u : 0u;
        const uint64_t y0d = desc64(y0_mn, desc_hi), y1d = desc64(y1_mn, desc_hi);
        if constexpr (DKV) {
          mma_ts_elect_x4(tmem_base + kAccCol, p_tmem, y1d, y1d + 128, y1d + 256, y1d + 384, idesc_acc, acc);
          mma_ts_elect_x4(tmem_base + kAccCol + D, ds_tmem, y0d, y0d + 128, y0d + 256, y0d + 384, idesc_acc, acc);
        } else {
          mma_ts_elect_x4(tmem_base + kAccCol, ds_tmem, y0d, y0d + 128, y0d + 256, y0d + 384, idesc_acc, acc);
        }
      }
      // No commit for the ring slot here: a step has exactly one commit (stage 1's, below, which also covers
      // this stage 2), and the compute warps, who wait for it anyway, release the slot.
      if (it + 1 == n_it) mma_commit_elect(acc_done);
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 2, it);
      if (more) {
        if (!landed && !wait_y(ahead, it + 2)) { ok = false; break; }
        stage1(it + 2, ahead);
      }
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 3, it);
      cur = ring_next(cur);
      ahead = ring_next(ahead);
    }
    if (!ok || *abort_flag) {
      mma_commit_elect(drain_bar);
      mbar_wait_quiet(drain_bar, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute warps
    const int quarter = warp & 3;                       // tensor-memory lanes 32*quarter .. +31
    const int half = (warp - 2) >> 2;                   // warpgroup: takes the steps of this parity (score buffer `half`)
    const int tid = quarter * 32 + lane;                // row of the resident tiles owned by this thread
    const int x_row = x_row0 + tid;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float c = p.scale_log2;
    constexpr float kLog2e = 1.4426950408889634f;
    bool ok = true;
    WIR_TRACE_DECL;
    const bool traced = (quarter == 0 && lane == 0);
    if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 90, 0);     // set-up done, prologue starts

    // per-row statistics (DKV = false): L2 = LSE log2 e, ds = delta * scale; delta is computed here
    float row_l2 = 0.f, row_ds = 0.f;
    if constexpr (!DKV) {
      // Each thread copies its row of one of the two resident operands into tensor memory as the A operand of
      // stage 1 (group 0 the Q row, group 1 the dO row; a row of D bf16 is D/2 32-bit words, exactly the packed
      // layout the MMA reads) and computes half of delta = rowsum(dO * O), group g over columns g D/2 ...; the
      // halves meet in shared memory.  All loads of a batch are issued before the first use: the prologue is a
      // chain of round trips to L2 or HBM, and a CTA has nothing else to do meanwhile.
      uint32_t xw[D / 2];
#pragma unroll
      for (int i = 0; i < D / 2; ++i) xw[i] = 0u;
      float part = 0.f, lse = 0.f;
      const bool live = x_row < p.S;
      const size_t r = static_cast<size_t>(x_plane) * p.S + (live ? x_row : 0);
      if (live) {
        const uint4* x4 = reinterpret_cast<const uint4*>((half == 0 ? p.Q : p.dO) + r * D);
        const uint4* o4 = reinterpret_cast<const uint4*>(p.O + r * D) + half * (D / 16);
        const uint4* g4 = reinterpret_cast<const uint4*>(p.dO + r * D) + half * (D / 16);
#pragma unroll
        for (int v = 0; v < D / 8; ++v) {
          const uint4 x = __ldg(x4 + v);
          xw[4 * v + 0] = x.x;
          xw[4 * v + 1] = x.y;
          xw[4 * v + 2] = x.z;
          xw[4 * v + 3] = x.w;
        }
        uint4 a[D / 16], g[D / 16];
#pragma unroll
        for (int v = 0; v < D / 16; ++v) {
          a[v] = __ldg(o4 + v);
          g[v] = __ldg(g4 + v);
        }
        lse = p.LSE[r];
#pragma unroll
        for (int v = 0; v < D / 16; ++v) {
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[v]);
          const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g[v]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 af = __bfloat1622float2(a2[e]), gf = __bfloat1622float2(g2[e]);
            part = fmaf(af.x, gf.x, part);
            part = fmaf(af.y, gf.y, part);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < D / 2; i += 32) tmem_st32(lane_base + kXCol + half * (D / 2) + i, xw + i);
      stats[half * kBwdBX + tid] = part;
      asm volatile("bar.sync 2, 256;" ::: "memory");
      const float delta = stats[tid] + stats[kBwdBX + tid];
      if (live && half == 0) p.delta[r] = delta;
      row_ds = delta * p.scale;
      row_l2 = lse * kLog2e;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(x_full);
    }

    // DKV: the 64 per-column statistics (LSE, delta) of a step's Q tile are staged in shared memory by the
    // warpgroup that owns the step (threads 0-63 LSE, 64-127 delta), fetched from global memory one of its
    // steps ahead so that the round trip is off the critical path
    auto fetch_stat = [&](int it) -> float {
      const int q = y_tile_of(it) * kBwdBY + (tid & 63);
      const size_t r = static_cast<size_t>(y_plane_of(it)) * p.S + min(q, p.S - 1);
      return (tid < 64) ? p.LSE[r] * kLog2e : p.delta[r] * p.scale;
    };
    float stat_next = 0.f;
    if (DKV && half < n_it) stat_next = fetch_stat(half);

    if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 91, 0);     // prologue done
    const int b = half;                                   // this group's score buffer
    for (int it = half; it < n_it; it += 2) {
      const int y_row0 = y_tile_of(it) * kBwdBY;
      // the group's own double buffer: every warp of the group has passed the previous step's barrier, hence
      // finished reading this buffer two steps ago
      float* st = stats + (half * 2 + ((it >> 1) & 1)) * 2 * kBwdBY;
      if constexpr (DKV) {
        st[tid] = stat_next;
        if (it + 2 < n_it) stat_next = fetch_stat(it + 2);
      }
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 10, it);
      const bool got = mbar_wait(t_full(b), (it >> 1) & 1, ctx, kRoleSoftmax, b, it);
      if (DKV) {
        // the group's warps meet at a named barrier every step (it also publishes st), so they must agree on going on
        uint32_t all;
        asm volatile(
            "{\n\t.reg .pred a, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred a, %2, 128, q;\n\t"
            "selp.u32 %0, 1, 0, a;\n\t}"
            : "=r"(all)
            : "r"(got ? 1u : 0u), "r"(2 + half)
            : "memory");
        if (all == 0) { ok = false; break; }
      } else if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // stage 1 of this step was committed after stage 2 of step it - 2: that step's ring slot is free
      if (it >= 2 && tid == 0) mbar_arrive(y_empty((it - 2) % STAGES));
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 11, it);
#if defined(WIR_BWD_ABLATE) && WIR_BWD_ABLATE == 3   // measurement build 3: the compute warps only pass the hand-offs on
      mbar_arrive(pds_full(b));
      continue;
#endif

      // masks are only needed on tiles that touch the diagonal or the end of the sequence
      const bool ragged = (y_row0 + kBwdBY > p.S) || (x_row0 + kBwdBX > p.S);
      const bool diagonal = CAUSAL && (DKV ? (y_row0 < x_row0 + kBwdBX) : (y_row0 + kBwdBY > x_row0));
      const bool masked = ragged || diagonal;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {              // 32 of the 64 columns of T0 / T1 at a time
        uint32_t t0[32], t1[32];
        tmem_ld32(lane_base + b * 64 + pass * 32, t0);
        tmem_ld32(lane_base + 128 + b * 64 + pass * 32, t1);
        tmem_wait_ld();
        if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 12, it);
        uint32_t pk[16], dk[16];
#if defined(WIR_BWD_ABLATE) && WIR_BWD_ABLATE == 1    // measurement build 1: tensor-memory traffic as is, no arithmetic
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk[i] = t0[2 * i] & 0x3f003f00u;
          dk[i] = t1[2 * i] & 0x3f003f00u;
        }
#else
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float pv[2], dv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col = pass * 32 + 2 * i + h;        // column of T0 / T1
            const float l2 = DKV ? st[col] : row_l2;
            const float dsc = DKV ? st[kBwdBY + col] : row_ds;
#if defined(WIR_BWD_ABLATE) && WIR_BWD_ABLATE == 4    // measurement build 4: no exponentials
            float pe = fmaf(__uint_as_float(t0[2 * i + h]), c, -l2);
#else
            float pe = ex2_approx(fmaf(__uint_as_float(t0[2 * i + h]), c, -l2));
#endif
            if (masked) {
              const int y = y_row0 + col;                 // index along the streamed tile
              const int qi = DKV ? y : x_row;             // query index
              const int ki = DKV ? x_row : y;             // key index
              if (qi >= p.S || ki >= p.S || (CAUSAL && ki > qi)) pe = 0.f;
            }
            pv[h] = pe;
            dv[h] = pe * fmaf(__uint_as_float(t1[2 * i + h]), p.scale, -dsc);
          }
#if defined(WIR_BWD_ABLATE) && WIR_BWD_ABLATE == 5    // measurement build 5: bf16 by truncation (a byte permute), no conversions
          pk[i] = __byte_perm(__float_as_uint(pv[0]), __float_as_uint(pv[1]), 0x7632);
          dk[i] = __byte_perm(__float_as_uint(dv[0]), __float_as_uint(dv[1]), 0x7632);
#else
          pk[i] = pack_bf16(pv[0], pv[1]);
          dk[i] = pack_bf16(dv[0], dv[1]);
#endif
        }
#endif
        // Packed bf16: a pass's 32 values fill 16 columns.  The 32 packed columns sit at columns 16..47 of
        // the buffer, so each pass overwrites only columns that have been read already (pass 0 read 0..31
        // and writes 16..31, pass 1 read 32..63 and writes 32..47).
        if constexpr (DKV) tmem_st16(lane_base + b * 64 + 16 + pass * 16, pk);
        tmem_st16(lane_base + 128 + b * 64 + 16 + pass * 16, dk);
      }
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 13, it);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(pds_full(b));
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 14, it);
    }

    if (ok && n_it > 0) {
      const bool got = mbar_wait(acc_done, 0, ctx, kRoleEpilogue, 0, n_it);
      if (traced) WIR_TRACE_EVENT(p.trace, 1 + half, 92, 0);   // accumulators complete
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        // A store instruction of a warp with one row per lane writes 32 separate 16-byte pieces, and the
        // memory pipeline takes them one cache line at a time (the epilogue of the dK / dV launch took 10000
        // clocks for 128 KB that way).  So each warp turns its 32 x 32 block around in shared memory
        // (XOR-swizzled, conflict-free both ways; the ring is idle by now) and stores whole 128-byte rows, four
        // rows per instruction.
        uint8_t* stage = smem + L::kYOffset + (warp - 2) * 4096;
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
    WIR_TRACE_EVENT(p.trace, 3, 93, 0);   // epilogue done (its own region: this thread's counter starts anew)
  }
#endif
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace wir
