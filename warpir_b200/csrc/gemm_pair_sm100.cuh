// bf16 GEMM on CTA pairs (thread-block clusters of two, tcgen05 cta_group::2): the kernel the large
// problems run on.
//
// A pair computes a 256 x 256 output tile with one stream of 256 x 256 x 16 MMAs issued by the pair's
// leader (cluster rank 0).  CTA r holds rows 128 r .. 128 r + 127 of the A tile and rows
// 128 r .. 128 r + 127 of the B tile (B stored [N,K]: its half of the tile's N extent) in its own
// shared memory, and ends up with rows 128 r .. of the output tile, all 256 columns, in its own
// tensor memory.  Compared with the 256 x 256 tile of one CTA (gemm_bf16_sm100 with MT = 2):
//
//   * each SM's tensor core reads A (4 KB) + half of B (4 KB) per 128-clock MMA instead of
//     A (4 KB) + B (8 KB): a third less shared-memory traffic for the same FLOPs, which under the
//     power cap is clock frequency;
//   * an accumulator is 256 tensor-memory columns per CTA instead of 512, so there are two, and the
//     epilogue of one tile runs under the main loop of the next;
//   * a stage is 32 KB per CTA instead of 64 KB: six stages instead of three.
//
// Every TMA copy lands in the shared memory of the CTA that issues it (no cluster-wide copy form is
// used anywhere); only the barrier a copy signals may be the leader's.  Barriers:
//
//   full[s]      in the leader; the leader's producer arms it with the bytes of BOTH CTAs' copies, the
//                peer's copies complete on it through its shared::cluster address
//   empty[s]     in each CTA, for its own producer; the leader's MMA warp commits to both at once
//   acc_full[a]  in each CTA, for its own epilogue warps; committed to both at once
//   acc_empty[a] in the leader; eight arrivals, one per epilogue warp of either CTA
//
// One cluster barrier after set-up (no remote arrival or copy before the partner's barriers exist and its
// tensor memory is allocated) and one before exit (no CTA leaves while its partner may still read
// its shared memory, write its tensor memory or signal its barriers).  All waits are bounded.
#pragma once

#include "gemm_sm100.cuh"

namespace wir {

constexpr int kPairThreads = 192;   // producer warp, MMA warp, four epilogue warps (per CTA)
constexpr int kPairBN = 256;        // output tile width = MMA N
constexpr int kPairRows = 128;      // rows of A, of B and of the output tile per CTA

// Role table of the pair kernel (checked against the lowering's, see GemmRoles): per CTA a producer
// warp, the MMA warp (it issues in the pair's leader only) and one epilogue warpgroup.
struct GemmPairRoles {
  static constexpr int kProducerWarp = 0;
  static constexpr int kMmaWarp = 1;
  static constexpr int kFirstEpilogueWarp = 2;
  static constexpr int kEpilogueWarps = 4;
  static constexpr int kThreads = kPairThreads;
  static constexpr int kCtasPerTile = 2;
};
static_assert(GemmPairRoles::kThreads == 32 * (2 + GemmPairRoles::kEpilogueWarps), "thread count");

template <int STAGES>
struct GemmPairSmem {
  static constexpr int kABytes = kPairRows * kGemmBK * 2;   // 16 KB
  static constexpr int kBBytes = kPairRows * kGemmBK * 2;   // 16 KB: this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBOffset = STAGES * kABytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * STAGES + 5;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

// Work of cluster `cl` of `ncl`: output tiles cl, cl + ncl, ... in the rasterised order of decode_tile
// (p.tiles_m counts 256-row tiles, p.tiles_n 256-column tiles).
template <int STAGES, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_sm100(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmParams p) {
  using L = GemmPairSmem<STAGES>;
  constexpr uint32_t kTmemCols = 512;   // two accumulators of 256 columns

  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory window starts at the same offset in both CTAs, so aligning the shared
  // address gives both the same layout
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - raw_addr);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cl = blockIdx.x >> 1;
  const int ncl = gridDim.x >> 1;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);   // four epilogue warps in each CTA
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (one per CTA)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      TileCoord t;
      const uint64_t pol_a = l2_policy_evict_last(), pol_b = l2_policy_evict_first();
      for (int tile = cl; ok && tile < total_tiles; tile += ncl) {
        decode_tile(tile, p, t);
        const int row_a = t.m_blk * 2 * kPairRows + static_cast<int>(rank) * kPairRows;
        const int row_b = t.n_blk * kPairBN + static_cast<int>(rank) * kPairRows;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, ctx, kRoleProducer, s, kb)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * L::kStageBytes);   // both CTAs' bytes
          const uint32_t full_leader = mapa_shared(full_bar(s), 0);
          const uint32_t a_dst = smem_base + s * L::kABytes;
          const uint32_t b_dst = smem_base + L::kBOffset + s * L::kBBytes;
          if (p.l2_hints & 1) tma_load_2d_pair_hint(a_dst, &tmap_a, full_leader, kb * kGemmBK, row_a, pol_a);
          else tma_load_2d_pair(a_dst, &tmap_a, full_leader, kb * kGemmBK, row_a);
          if constexpr (!B_MN) {
            if (p.l2_hints & 2) tma_load_2d_pair_hint(b_dst, &tmap_b, full_leader, kb * kGemmBK, row_b, pol_b);
            else tma_load_2d_pair(b_dst, &tmap_b, full_leader, kb * kGemmBK, row_b);
          } else {
#pragma unroll
            for (int c = 0; c < kPairRows / 64; ++c)
              tma_load_2d_pair(b_dst + c * 8192, &tmap_b, full_leader, row_b + c * 64, kb * kGemmBK);
          }
        }
      }
      if (!ok || *abort_flag) {
        // The copies in flight are counted on the leader's barriers, which the peer cannot wait on.
        // After a failure give them time to land (they take microseconds) before the CTA may exit.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0) {
      constexpr uint32_t idesc = idesc_bf16_f32(2 * kPairRows, kPairBN, 0, B_MN ? 1 : 0);
      constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
      constexpr uint32_t kBStep = B_MN ? (2048 >> 4) : (32 >> 4);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = cl; ok && tile < total_tiles; tile += ncl, ++acc_it) {
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait_warp(acc_empty_bar(acc), acc_ph ^ 1, ctx, kRoleMma, 100 + acc, tile)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_warp(full_bar(s), ph, ctx, kRoleMma, s, kb)) { ok = false; break; }
          tc_fence_after();
          const uint64_t ad = desc64(smem_desc_lo(smem_base + s * L::kABytes, 16), desc_hi);
          const uint64_t bd = desc64(smem_desc_lo(smem_base + L::kBOffset + s * L::kBBytes, B_MN ? 8192 : 16), desc_hi);
          // the stage's four k-steps: 32 bytes further along a K-major row, 16 rows (2048 B) of an N-major tile
          mma_ss_pair_x4(d_tmem, ad, ad + 2, ad + 4, ad + 6, bd, bd + kBStep, bd + 2 * kBStep, bd + 3 * kBStep, idesc,
                         kb > 0 ? 1u : 0u);
          mma_commit_pair_both_elect(empty_bar(s));   // both producers may refill the stage once these MMAs have read it
        }
        if (ok) mma_commit_pair_both_elect(acc_full_bar(acc));
      }
      if (!ok || *abort_flag) {
        mma_commit_pair_elect(mapa_shared(drain_bar, 0));
        mbar_wait_quiet(drain_bar, 0);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs: own 128 rows, 256 columns)
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, 32*quarter+32) belong to this warp
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const uint32_t acc_empty_leader0 = mapa_shared(acc_empty_bar(0), 0);
    const uint32_t acc_empty_leader1 = mapa_shared(acc_empty_bar(1), 0);
    uint32_t acc_it = 0;
    bool ok = true;
    TileCoord t;
    for (int tile = cl; ok && tile < total_tiles; tile += ncl, ++acc_it) {
      decode_tile(tile, p, t);
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      bool got = mbar_wait(acc_full_bar(acc), acc_ph, ctx, kRoleEpilogue, acc, tile);
      got = __all_sync(0xffffffffu, got);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const int row = t.m_blk * 2 * kPairRows + static_cast<int>(rank) * kPairRows + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kPairBN;
#pragma unroll 1
      for (int c = 0; c < kPairBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = t.n_blk * kPairBN + c * 32;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* dst = p.C + static_cast<size_t>(row) * p.ldc + col0;
          if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              q.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              q.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              q.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              if (p.l2_hints & 4) __stcs(reinterpret_cast<uint4*>(dst) + v, q);
              else reinterpret_cast<uint4*>(dst)[v] = q;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
        }
      }
      // this warp has read its lanes of the accumulator: one arrival on the leader's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? acc_empty_leader0 : acc_empty_leader1);
    }
  }

  // No CTA may leave (or free its tensor memory) while its partner can still read its shared memory,
  // write its tensor memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace wir
