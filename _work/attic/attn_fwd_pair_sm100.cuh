// Attention forward for head dimension 128 on CTA pairs (thread-block clusters of two).
//
// Same algorithm, roles and tensor-memory layout as attn_fwd_sm100.cuh (two 128-row Q tiles
// per CTA, one softmax warpgroup per tile, 64-key K/V blocks, double-buffered scores, P fed
// to the second MMA from tensor memory, lazy rescale).  What changes is who issues the MMAs
// and what one instruction covers: the two CTAs of a cluster form a pair (tcgen05
// cta_group::2), tile t of the leader and tile t of its peer are the two halves of ONE
// 256-row MMA stream issued by the leader's MMA warp t for both, and each CTA loads only
// half of every K/V block (the B operand of a pair-MMA is split between the two shared
// memories: 32 of the 64 keys of a K block, 64 of the 128 columns of a V block).
// Measured, this is slower than the single-CTA kernel (830 vs 1137 TFLOP/s on the non-causal
// benchmark shape): shared-memory traffic was not the limit, each SM's tensor core still
// works through as many instructions per block, and every completion is committed twice.
// The kernel is kept, selectable and tested, as the worked example of the pair protocol.
//
// Q tiles of a cluster c: CTA r holds tiles 4c + r and 4c + 2 + r; stream t = tiles
// (4c + 2t, 4c + 2t + 1).  With a causal mask a stream runs as many K/V blocks as its later
// tile needs; the earlier tile sees its last two blocks fully masked.
//
// Barriers: full (TMA) and P-ready barriers live in the leader, because its MMA warps wait
// on them; the peer's copies and softmax threads arrive there through shared::cluster
// addresses.  Everything an MMA completion releases (score buffers, K/V slots, O) exists in
// both CTAs, and the leader commits to both.  The cluster synchronises once after set-up
// (barriers initialised and tensor memory allocated in both CTAs before anything remote
// happens) and once before exit (no CTA leaves while its pair may still touch its memory).
#pragma once

#include "attn_fwd_sm100.cuh"

namespace wir {

struct AttnPairSmem {
  static constexpr int kD = 128;
  static constexpr int kStages = 16;
  static constexpr int kQChunkBytes = kAttnBQ * 128;
  static constexpr int kQTileBytes = 2 * kQChunkBytes;             // 128 rows x 128 bf16
  static constexpr int kSlotBytes = 8192;                           // half a K block (32 keys x 128) or half a V block (64 keys x 64)
  static constexpr int kKChunkBytes = 32 * 128;                     // 32 keys x 64 bf16
  static constexpr int kKVOffset = 2 * kQTileBytes;
  static constexpr int kBarOffset = kKVOffset + kStages * kSlotBytes;
  // q_full, kv_full[S], kv_empty[S], s_full[2][2], p_full[2][2], pv_done[2][2], drain[2]
  static constexpr int kNumBars = 1 + 2 * kStages + 14;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

template <bool CAUSAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kAttnThreads, 1)
attn_fwd_pair_sm100(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = AttnPairSmem;
  constexpr int D = 128;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256;        // O_t at columns 256 + t*D

  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory window starts at the same offset in both CTAs, so aligning the
  // shared address gives both the same layout
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - raw_addr);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + STAGES + s); };
  auto s_full = [&](int t, int b) { return bar_base + 8u * (1 + 2 * STAGES + 2 * t + b); };
  auto p_full = [&](int t, int b) { return bar_base + 8u * (5 + 2 * STAGES + 2 * t + b); };
  auto pv_done = [&](int t, int b) { return bar_base + 8u * (9 + 2 * STAGES + 2 * t + b); };
  const uint32_t drain_bar = bar_base + 8u * (13 + 2 * STAGES);
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
  auto in_leader = [&](uint32_t addr) { return mapa_shared(addr, 0); };
  auto in_other = [&](uint32_t addr) { return mapa_shared(addr, rank ^ 1u); };

  // ---- which rows / how many KV tiles -----------------------------------------
  const int clusters = gridDim.x >> 1;
  const int cl = CAUSAL ? (clusters - 1 - static_cast<int>(blockIdx.x >> 1)) : static_cast<int>(blockIdx.x >> 1);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int bh = batch * p.H + head;
  const int bh_kv = batch * p.Hkv + head / (p.H / p.Hkv);
  const int nkv = (p.S + kAttnBKV - 1) / kAttnBKV;
  // stream t = Q tiles 4 cl + 2t (leader) and 4 cl + 2t + 1 (peer); it runs as many blocks as the later tile needs
  auto stream_blocks = [&](int t) {
    const int first = 4 * cl + 2 * t;
    if (first * kAttnBQ >= p.S) return 0;
    return CAUSAL ? min(nkv, 2 * (first + 1) + 2) : nkv;
  };
  const int n0 = stream_blocks(0), n1 = stream_blocks(1);
  const int n_max = max(n0, n1);
  auto k_index = [&](int j) -> uint32_t { return j == 0 ? 0u : static_cast<uint32_t>(2 * j - 1); };
  auto v_index = [&](int j) -> uint32_t { return static_cast<uint32_t>(j + 1 < n_max ? 2 * j + 2 : 2 * j + 1); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 2);   // one arrival per MMA issuer (both live in the leader)
    }
    for (int t = 0; t < 2; ++t)
      for (int b = 0; b < 2; ++b) {
        mbar_init(s_full(t, b), 1);
        mbar_init(p_full(t, b), 256);   // the softmax warpgroup of tile t in both CTAs
        mbar_init(pv_done(t, b), 1);
      }
    mbar_init(drain_bar, 1);
    mbar_init(drain_bar + 8u, 1);
    fence_mbar_init();
  }
  if (warp == kAttnMmaWarp) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == kAttnMmaWarp + 2) {
    // ------------------------------------------------------------------ producer (one per CTA)
    if (lane == 0 && n_max > 0) {
      // both CTAs' Q tiles are counted on the leader's barrier
      if (rank == 0) mbar_arrive_expect_tx(q_full, 2 * 2 * L::kQTileBytes);
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d_pair(smem_base + t * L::kQTileBytes + c * L::kQChunkBytes, &tmap_q, in_leader(q_full), c * 64,
                           (4 * cl + 2 * t + static_cast<int>(rank)) * kAttnBQ, bh);
      uint32_t idx = 0;
      bool ok = true;
      // this CTA's half of K(j): keys j*64 + rank*32 .. +31, both 64-column chunks
      auto load_k = [&](int j) -> bool {
        const int s = idx % STAGES;
        if (!mbar_wait(kv_empty(s), ((idx / STAGES) & 1) ^ 1, ctx, kRoleProducer, s, j)) return false;
        if (rank == 0) mbar_arrive_expect_tx(kv_full(s), 2 * L::kSlotBytes);
        const uint32_t dst = smem_base + L::kKVOffset + s * L::kSlotBytes;
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d_pair(dst + c * L::kKChunkBytes, &tmap_k, in_leader(kv_full(s)), c * 64,
                           j * kAttnBKV + static_cast<int>(rank) * 32, bh_kv);
        ++idx;
        return true;
      };
      // this CTA's half of V(j): all 64 keys, columns rank*64 .. +63
      auto load_v = [&](int j) -> bool {
        const int s = idx % STAGES;
        if (!mbar_wait(kv_empty(s), ((idx / STAGES) & 1) ^ 1, ctx, kRoleProducer, s, j)) return false;
        if (rank == 0) mbar_arrive_expect_tx(kv_full(s), 2 * L::kSlotBytes);
        tma_load_3d_pair(smem_base + L::kKVOffset + s * L::kSlotBytes, &tmap_v, in_leader(kv_full(s)),
                         static_cast<int>(rank) * 64, j * kAttnBKV, bh_kv);
        ++idx;
        return true;
      };
      ok = load_k(0);
      for (int j = 0; ok && j < n_max; ++j) {
        if (j + 1 < n_max) ok = load_k(j + 1);
        if (ok) ok = load_v(j);
      }
      if (!ok || *abort_flag) {
        // The copies in flight are counted on the leader's barriers, which the peer cannot wait on.
        // After a failure give them time to land (they take microseconds) before the CTA may exit
        // and its shared memory go to another CTA.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if ((warp == kAttnMmaWarp || warp == kAttnMmaWarp + 1) && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer of stream t (leader only)
    const int t = warp - kAttnMmaWarp;
    const int n = (t == 0) ? n0 : n1;
    constexpr uint32_t idesc_qk = idesc_bf16_f32(2 * kAttnBQ, kAttnBKV, 0, 0);
    constexpr uint32_t idesc_pv = idesc_bf16_f32(2 * kAttnBQ, D, 0, 1);
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    const uint32_t q_lo = smem_desc_lo(smem_base + t * L::kQTileBytes, 16);
    const uint32_t o_tmem = tmem_base + kOCol + t * D;
    bool ok = true;
    auto kv_addr = [&](uint32_t idx) { return smem_base + L::kKVOffset + (idx % STAGES) * L::kSlotBytes; };
    auto wait_kv = [&](uint32_t idx, int tag) {
      return mbar_wait_warp(kv_full(idx % STAGES), (idx / STAGES) & 1, ctx, kRoleMma, tag, idx);
    };
    // completions are announced in both CTAs
    auto commit_both = [&](uint32_t bar) {
      mma_commit_pair_elect(mapa_shared(bar, 0));
      mma_commit_pair_elect(mapa_shared(bar, 1));
    };
    auto skip_tile = [&](uint32_t idx) -> bool {
      if (!wait_kv(idx, 40 + t)) return false;
      mbar_arrive_elect(kv_empty(idx % STAGES));
      if (elect_one()) mbar_arrive_cluster(mapa_shared(kv_empty(idx % STAGES), 1));
      __syncwarp();
      return true;
    };
    auto issue_qk = [&](int j) -> bool {
      const uint32_t idx = k_index(j);
      if (!wait_kv(idx, 10 + t)) return false;
      tc_fence_after();
      const uint32_t k_lo = smem_desc_lo(kv_addr(idx), 16);
      const uint32_t d_tmem = tmem_base + t * 128 + (j & 1) * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {   // the two 64-element chunks of the head dimension, four k-steps each
        const uint64_t qd = desc64(q_lo + ((c * L::kQChunkBytes) >> 4), desc_hi);
        const uint64_t kd = desc64(k_lo + ((c * L::kKChunkBytes) >> 4), desc_hi);
        mma_ss_pair_x4(d_tmem, qd, qd + 2, qd + 4, qd + 6, kd, kd + 2, kd + 4, kd + 6, idesc_qk, c > 0 ? 1u : 0u);
      }
      commit_both(s_full(t, j & 1));
      commit_both(kv_empty(idx % STAGES));
      return true;
    };

    if (n_max > 0) ok = mbar_wait_warp(q_full, 0, ctx, kRoleMma, 1, 0);
    for (int j = 0; ok && j < 2 && j < n_max; ++j) ok = (j < n) ? issue_qk(j) : skip_tile(k_index(j));

    for (int j = 0; ok && j < n_max; ++j) {
      const uint32_t idx = v_index(j);
      if (j < n) {
        if (!mbar_wait_warp(p_full(t, j & 1), (j >> 1) & 1, ctx, kRoleMma, 20 + t, j)) { ok = false; break; }
        if (!wait_kv(idx, 30 + t)) { ok = false; break; }
        tc_fence_after();
        // this CTA's half of V is one 64-column chunk: 16 keys (2048 bytes) per k-step
        const uint64_t vd = desc64(smem_desc_lo(kv_addr(idx), L::kSlotBytes), desc_hi);
        const uint32_t p_tmem = tmem_base + t * 128 + (j & 1) * 64;
        mma_ts_pair_x4(o_tmem, p_tmem, vd, vd + 128, vd + 256, vd + 384, idesc_pv, j > 0 ? 1u : 0u);
        commit_both(pv_done(t, j & 1));
        commit_both(kv_empty(idx % STAGES));
      } else {
        ok = skip_tile(idx);
      }
      if (ok && j + 2 < n_max) ok = (j + 2 < n) ? issue_qk(j + 2) : skip_tile(k_index(j + 2));
    }
    if (!ok || *abort_flag) {
      mma_commit_pair_elect(mapa_shared(drain_bar + 8u * t, 0));
      mbar_wait_quiet(drain_bar + 8u * t, 0);
    }
    __syncwarp();
  } else if (warp < kAttnMmaWarp) {
    // ------------------------------------------------------------------ softmax + epilogue (both CTAs)
    const int t = warp >> 2;            // which Q tile of this CTA = which stream
    const int quarter = warp & 3;
    const int qt = 4 * cl + 2 * t + static_cast<int>(rank);
    const int q_row = qt * kAttnBQ + quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_addr = lane_base + kOCol + t * D;
    const float c = p.scale_log2;
    const int n = (t == 0) ? n0 : n1;
    const int first_masked = CAUSAL ? 2 * qt : (p.S % kAttnBKV != 0 ? nkv - 1 : nkv);

    float m = -INFINITY;
    float l = 0.f;
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      const int b = j & 1;
      const uint32_t s_addr = lane_base + t * 128 + b * 64;
      const bool got = mbar_wait(s_full(t, b), (j >> 1) & 1, ctx, kRoleSoftmax, t, j);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      if (j == 0 && t == 1 && p.stagger_clocks > 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < p.stagger_clocks) {
        }
      }

      uint32_t sb[64];
      tmem_ld32(s_addr, sb);
      tmem_ld32(s_addr + 32, sb + 32);
      tmem_wait_ld();
#define WIR_S(i) __uint_as_float(sb[i])

      if (j >= first_masked || (j == nkv - 1 && p.S % kAttnBKV != 0)) {
        const int k0 = j * kAttnBKV;
        const int limit = CAUSAL ? min(q_row, p.S - 1) : (p.S - 1);
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (k0 + i > limit) sb[i] = 0xff800000u;
      }

      float mx0 = WIR_S(0), mx1 = WIR_S(1), mx2 = WIR_S(2), mx3 = WIR_S(3);
#pragma unroll
      for (int i = 4; i < 64; i += 4) {
        mx0 = fmaxf(mx0, WIR_S(i));
        mx1 = fmaxf(mx1, WIR_S(i + 1));
        mx2 = fmaxf(mx2, WIR_S(i + 2));
        mx3 = fmaxf(mx3, WIR_S(i + 3));
      }
      const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
      const bool grow = (m_new - m) * c > kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        if (j > 0) {
          const bool done = mbar_wait(pv_done(t, (j - 1) & 1), ((j - 1) >> 1) & 1, ctx, kRoleSoftmax, 8 + t, j);
          if (!__all_sync(0xffffffffu, done)) { ok = false; break; }
          tc_fence_after();
          const float alpha = ex2_approx((m - m_new) * c);
          l *= alpha;
#pragma unroll 1
          for (int cidx = 0; cidx < D / 32; ++cidx) {
            uint32_t o[32];
            tmem_ld32(o_addr + cidx * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + cidx * 32, o);
          }
        }
        m = m_new;
      }

      // rows whose every key so far is masked (past the end of a ragged tile) keep m = -inf; use 0 there
      const float neg_mc = (m == -INFINITY) ? 0.f : -m * c;
      const float2 c2 = make_float2(c, c), neg_mc2 = make_float2(neg_mc, neg_mc);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float2 x = __ffma2_rn(make_float2(WIR_S(2 * i), WIR_S(2 * i + 1)), c2, neg_mc2);
        float2 e;
        if ((i & 3) == 3) {
          e = ex2_fma2(x);
        } else {
          e.x = ex2_approx(x.x);
          e.y = ex2_approx(x.y);
        }
        if (i & 1) lb = __fadd2_rn(lb, e);
        else la = __fadd2_rn(la, e);
        pk[i] = pack_bf16(e.x, e.y);
      }
      const float l0 = la.x + lb.x, l1 = la.y + lb.y;
#undef WIR_S
      tmem_st32(s_addr, pk);
      l += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_cluster(in_leader(p_full(t, b)));   // the leader's MMA warp waits for both CTAs' P
    }

    if (ok && n > 0) {
      const bool got = mbar_wait(pv_done(t, (n - 1) & 1), ((n - 1) >> 1) & 1, ctx, kRoleEpilogue, t, n);
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        const float inv_l = 1.0f / l;
        const bool live = q_row < p.S;
        __nv_bfloat16* dst = p.O + (static_cast<size_t>(bh) * p.S + (live ? q_row : 0)) * D;
#pragma unroll 1
        for (int cidx = 0; cidx < D / 32; ++cidx) {
          uint32_t o[32];
          tmem_ld32(o_addr + cidx * 32, o);
          tmem_wait_ld();
          if (live) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(o[8 * v + 0]) * inv_l, __uint_as_float(o[8 * v + 1]) * inv_l);
              q.y = pack_bf16(__uint_as_float(o[8 * v + 2]) * inv_l, __uint_as_float(o[8 * v + 3]) * inv_l);
              q.z = pack_bf16(__uint_as_float(o[8 * v + 4]) * inv_l, __uint_as_float(o[8 * v + 5]) * inv_l);
              q.w = pack_bf16(__uint_as_float(o[8 * v + 6]) * inv_l, __uint_as_float(o[8 * v + 7]) * inv_l);
              reinterpret_cast<uint4*>(dst + cidx * 32)[v] = q;
            }
          }
        }
        if (live && p.LSE != nullptr)
          p.LSE[static_cast<size_t>(bh) * p.S + q_row] = m * c * 0.6931471805599453f + logf(l);
      }
    }
  }

  // No CTA may leave (or free its tensor memory) while its pair can still read its shared
  // memory, write its tensor memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == kAttnMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace wir
