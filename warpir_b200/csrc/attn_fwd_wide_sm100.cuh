// Attention forward with 128-key blocks: variant 4 of warpir_attn_fwd_bf16_ex, and what the
// library picks when there is no causal mask.
//
// The 64-key kernel (attn_fwd_sm100.cuh) double-buffers its scores and is bound by the rate at
// which the tensor core retires 128 x 64 x 16 MMAs (~71 clocks each, against ~100 for a
// 128 x 128 x 16 one, so twice the work for 1.4x the time).  With 128-key blocks tensor memory
// holds exactly one score tile and one accumulator per Q tile (2 x 128 + 2 x D columns), so the
// Q K^T of a tile's next block cannot run ahead of its softmax; the overlap comes from the two
// Q tiles of the CTA taking turns: while one is in its softmax, the tensor core works through
// the other's batch (P V of this block, then Q K^T of the next).
//
//   warps 0-3 / 4-7    softmax of tile 0 / 1: thread = row = tensor-memory lane, the whole row
//                      of 128 scores in registers (one pass: max, exponentials, P written over
//                      score columns 0-63 as packed bf16)
//   warp 8             MMA issuer of both tiles, strictly alternating between them
//   warp 10            producer (Q once, then K(j), V(j) tiles of 128 keys into a ring)
//   warps 9, 11        idle: they only complete the warpgroup whose registers move to the
//                      softmax warps (setmaxnreg 168 -> 104 / 200)
//
// D = 64: the two accumulators need only 128 columns, which leaves room for a THIRD score tile.  The three rotate
// between the two Q tiles (the k-th Q K^T of the CTA, in the order the issuer sends them, goes into score tile
// k % 3; the issuer sends P V number m and then Q K^T number m + 3 into the tile that P V has just read), so a
// Q tile finds its next scores waiting when its softmax ends and the two softmaxes run all the time: the
// exponential unit, which bounds this head dimension (16384 exponentials per 128 x 128 block against 512 clocks
// of MMAs), went from 63 % busy to what 750 TFLOP/s need (660 before; causal B4 H32 S8192).  A Q tile announces P
// of block j only once P V of block j - 1 has completed: otherwise it could get two blocks ahead of a held-up
// issuer and the parity of the "P ready" barrier would alias (seen once in a few hundred runs, as a timed-out wait).
//
// Why one issuer: with an issuer per tile the two batches interleaved in the tensor core's
// queue, which pulled the tiles into lockstep (both softmaxes at once at half speed, then both
// batches queued; 1049 TFLOP/s).  Alternating batches make the tiles settle half a period apart.
// MMAs execute in issue order, so the next Q K^T, issued right after P V, overwrites S only once
// P has been read.
//
// Measured on a B200 (bf16, TFLOP/s, this kernel against the 64-key one): B16 H16 S4096 D128
// 1177 vs 1134, D64 635 vs 581-616; causal B4 H32 S8192 D128 1052-1104 vs 1123, D64 550 vs 607.
// A step of both tiles takes ~3690 clocks for 3218 clocks of MMAs (87 %): a tile's chain is its
// softmax (~2050 clocks: tensor-memory load 220, row max ~300, 128 exponentials at the
// exponential unit's 8 clocks per warp instruction ~1150 with the arithmetic around them,
// store and signalling ~250) followed by its batch (1609), and only the other tile's batch
// hides under the softmax.  Tried and not kept: two softmax warpgroups per tile (64 columns
// each; the halves run in lockstep, so max and exponentials still add up: 1140), P V starting
// on the first half or quarters of P (the issuer trails the tensor core's queue, so the early
// start is not used: 1170 and 1039), a polynomial share of the exponentials on the FMA pipe
// (one warp per scheduler is short of issue slots, not of exponential throughput: 1144-1190),
// three-input max and rounding P by byte permute (no change), exponentials against the stale max
// with the row max taken alongside (softmax 1900 clocks, but the batches stretch to 1715-1833 and
// the step stays at 3700: the tensor core is then ~96 % busy, so this is the instruction-rate
// bound of 128-wide MMAs).
#pragma once

#include "attn_fwd_sm100.cuh"

namespace wir {

constexpr int kWideThreads = 384;   // 8 softmax warps, 2 MMA warps, 1 producer warp, 1 idle warp (whole warpgroups)
constexpr int kWideMmaWarp = 8;
constexpr int kWideBKV = 128;       // keys per block

// Role table of the 128-key kernel: softmax warps 0-7, ONE MMA-issuing warp for both Q tiles, the
// producer warp; warps 9 and 11 only complete the warpgroup whose registers move to the softmax warps.
struct AttnWideRoles {
  static constexpr int kSoftmaxWarps = 8;
  static constexpr int kFirstMmaWarp = kWideMmaWarp;
  static constexpr int kMmaWarps = 1;
  static constexpr int kProducerWarp = kWideMmaWarp + 2;
  static constexpr int kIdleWarps = 2;
  static constexpr int kThreads = kWideThreads;
};
static_assert(AttnWideRoles::kThreads == 32 * (AttnWideRoles::kSoftmaxWarps + AttnWideRoles::kMmaWarps + 1 + AttnWideRoles::kIdleWarps), "thread count");

template <int D>
struct AttnWideSmem {
  static constexpr int kChunkBytes = 128 * 128;                  // 128 rows x 64 bf16 (Q, K and V tiles alike)
  static constexpr int kTileBytes = (D / 64) * kChunkBytes;
  static constexpr int kStages = (D == 128) ? 4 : 8;             // K and V tiles alternate in the ring
  static constexpr int kQOffset = 0;
  static constexpr int kKVOffset = 2 * kTileBytes;
  static constexpr int kBarOffset = kKVOffset + kStages * kTileBytes;
  // q_full, kv_full[S], kv_empty[S], s_full[3], p_full[2], pv_done[2], drain
  static constexpr int kNumBars = 1 + 2 * kStages + 8;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kWideThreads, 1)
attn_fwd_wide_sm100(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = AttnWideSmem<D>;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  // Tensor memory.  D = 128: score tile S_t at columns 128 t, O_t at 256 + 128 t: all 512, one score tile per
  // Q tile.  D = 64: the accumulators need only 128 columns, which leaves room for a THIRD score tile: the three
  // rotate between the two Q tiles (the k-th Q K^T of the CTA, in the order the issuer sends them, goes into tile
  // k % 3), so that a Q tile's next scores are already waiting when its softmax ends; O_t at 384 + 64 t.
  constexpr bool kThird = (D == 64);
  constexpr uint32_t kOCol = kThird ? 384 : 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + STAGES + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (1 + 2 * STAGES + b); };      // per score tile
  auto p_full = [&](int t) { return bar_base + 8u * (4 + 2 * STAGES + t); };      // per Q tile
  auto pv_done = [&](int t) { return bar_base + 8u * (6 + 2 * STAGES + t); };
  const uint32_t drain_bar = bar_base + 8u * (8 + 2 * STAGES);
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which rows / how many K/V blocks ------------------------------------------------
  const int pair = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heaviest causal tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int bh = batch * p.H + head;
  const int bh_kv = batch * p.Hkv + head / (p.H / p.Hkv);
  const int nkv = (p.S + kWideBKV - 1) / kWideBKV;
  const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
  const int n0 = (qt0 * kAttnBQ >= p.S) ? 0 : (CAUSAL ? min(nkv, qt0 + 1) : nkv);
  const int n1 = (qt1 * kAttnBQ >= p.S) ? 0 : (CAUSAL ? min(nkv, qt1 + 1) : nkv);
  const int n_max = max(n0, n1);
  // Order of the CTA's Q K^T (and P V): the two Q tiles alternate while both have blocks left, then the one with
  // more goes on alone.  Block j of tile t is number seq_of(t, j) in that order.
  const int n_min = min(n0, n1);
  auto seq_of = [&](int t, int j) { return j < n_min ? 2 * j + t : n_min + j; };
  // ring positions: K(j) at 2j, V(j) at 2j + 1

  // Producer state (one lane of the producer warp, which also initialises the barriers and issues
  // Q and K(0) before the CTA-wide barrier).
  uint32_t p_idx = 0;
  auto load_tile = [&](const CUtensorMap* map, int j) -> bool {
    const int s = p_idx % STAGES;
    const uint32_t ph = (p_idx / STAGES) & 1;
    if (!mbar_wait(kv_empty(s), ph ^ 1, ctx, kRoleProducer, s, j)) return false;
    mbar_arrive_expect_tx(kv_full(s), L::kTileBytes);
    const uint32_t dst = smem_base + L::kKVOffset + s * L::kTileBytes;
#pragma unroll
    for (int c = 0; c < D / 64; ++c)
      tma_load_3d(dst + c * L::kChunkBytes, map, kv_full(s), c * 64, j * kWideBKV, bh_kv);
    ++p_idx;
    return true;
  };
  bool p_ok = true;

  if (threadIdx.x == (kWideMmaWarp + 2) * 32) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 3; ++b) mbar_init(s_full(b), 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(p_full(t), 128);   // one arrival per row
      mbar_init(pv_done(t), 1);
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    const int n_q = (n0 > 0) + (n1 > 0);
    mbar_arrive_expect_tx(q_full, n_q * L::kTileBytes);
    for (int t = 0; t < 2; ++t)
      if ((t == 0 ? n0 : n1) > 0)
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(smem_base + L::kQOffset + t * L::kTileBytes + c * L::kChunkBytes, &tmap_q, q_full, c * 64,
                      (2 * pair + t) * kAttnBQ, bh);
    if (n_max > 0) p_ok = load_tile(&tmap_k, 0);
  }
  if (warp == kWideMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  // Registers move from the warpgroup of the issuers and the producer to the softmax warpgroups,
  // whose threads hold a whole row of 128 scores (168 each at launch: 3 x 128 x 168 = 2 x 128 x 200 + 128 x 104).
  if (warp >= kWideMmaWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
  if (warp == kWideMmaWarp + 2) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = p_ok;
      // K(0) went out before the barrier; then V(j), K(j+1): the order in which the MMA warps consume them
      for (int j = 0; ok && j < n_max; ++j) {
        ok = load_tile(&tmap_v, j);
        if (ok && j + 1 < n_max) ok = load_tile(&tmap_k, j + 1);
      }
      if (!ok || *abort_flag) {
        mbar_wait_quiet(q_full, 0);
        const uint32_t n = p_idx < STAGES ? p_idx : STAGES;
        for (uint32_t back = 1; back <= n; ++back) {
          const uint32_t i = p_idx - back;
          mbar_wait_quiet(kv_full(i % STAGES), (i / STAGES) & 1);
        }
      }
    }
  } else if (warp == kWideMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer of both Q tiles
    // The whole warp runs the loop (warp-uniform operands), one elected lane issues.  The tiles
    // are served in strict alternation, each with its P V of this block and its Q K^T of the next
    // as one batch: the tensor core then works through one tile's batch while the other tile is
    // in its softmax, and the two settle half a period apart.  (Two independent issuers let the
    // batches interleave in the tensor core's queue, which pulled the tiles into lockstep: both
    // softmaxes ran at once at half speed, then both batches queued.)
    constexpr uint32_t idesc_qk = idesc_bf16_f32(kAttnBQ, kWideBKV, 0, 0);
    constexpr uint32_t idesc_pv = idesc_bf16_f32(kAttnBQ, D, 0, 1);
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    bool ok = true;
    WIR_TRACE_DECL;
    auto kv_addr = [&](uint32_t idx) { return smem_base + L::kKVOffset + (idx % STAGES) * L::kTileBytes; };
    auto wait_kv = [&](uint32_t idx, int tag) {
      return mbar_wait_warp(kv_full(idx % STAGES), (idx / STAGES) & 1, ctx, kRoleMma, tag, idx);
    };
    // a ring slot goes back to the producer behind the MMAs of the last tile that reads it
    auto last_user = [&](int j) { return j < n1 ? 1 : 0; };
    // S_t = Q_t K(j)^T: D/16 MMAs of 128 x 128 x 16, four (one 64-element chunk of the head dimension) per
    // instruction block.  K(j) must have landed (the caller made sure).
    auto issue_qk = [&](int t, int j, int buf) {
      const uint32_t idx = 2u * j;
      const uint64_t qd = desc64(smem_desc_lo(smem_base + L::kQOffset + t * L::kTileBytes, 16), desc_hi);
      const uint64_t kd = desc64(smem_desc_lo(kv_addr(idx), 16), desc_hi);
      const uint32_t s_tmem = tmem_base + buf * 128;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const uint64_t o = static_cast<uint64_t>((c * L::kChunkBytes) >> 4);   // 32 bytes per k-step inside a chunk
        mma_ss_elect_x4(s_tmem, qd + o, qd + o + 2, qd + o + 4, qd + o + 6, kd + o, kd + o + 2, kd + o + 4, kd + o + 6,
                        idesc_qk, c > 0 ? 1u : 0u);
      }
      mma_commit_elect(s_full(buf));
      if (t == last_user(j)) mma_commit_elect(kv_empty(idx % STAGES));
    };
    // O_t += P_t(j) V(j): 8 MMAs of 128 x D x 16, P from tensor memory (columns 0-63 of the score tile),
    // four per instruction block.  V(j) must have landed and P_t(j) be complete.
    auto issue_pv = [&](int t, int j, int buf) {
      const uint32_t idx = 2u * j + 1;
      const uint64_t vd = desc64(smem_desc_lo(kv_addr(idx), L::kChunkBytes), desc_hi);
      const uint32_t s_tmem = tmem_base + buf * 128;
      const uint32_t o_tmem = tmem_base + kOCol + t * D;
#pragma unroll
      for (int m = 0; m < kWideBKV / 64; ++m) {
        // 16 keys further: 8 packed columns of P, 16 rows (2048 bytes = 128 descriptor units) of V
        const uint64_t v = vd + static_cast<uint64_t>(512 * m);
        mma_ts_elect_x4(o_tmem, s_tmem + 32 * m, v, v + 128, v + 256, v + 384, idesc_pv, (j > 0 || m > 0) ? 1u : 0u);
      }
      mma_commit_elect(pv_done(t));
      if (t == last_user(j)) mma_commit_elect(kv_empty(idx % STAGES));
    };
    // One tile's batch: P V of block j and Q K^T of block j + 1.  A wait costs the issuing warp 75-150 clocks
    // even when the barrier is long complete, and the tensor core's queue is only about four MMAs deep, so
    // every wait that can be had early is taken BEFORE the one wait that is a true dependency (P from the
    // softmax warps): the K and V tiles are loaded well ahead.  Between P becoming ready and the sixteen MMAs
    // there is then nothing but the fence.
    // (t2, j2): whose scores go into the score tile that this P V frees (D = 128: the same Q tile's next block;
    // D = 64: the third Q K^T from here in the CTA's order)
    auto issue_batch = [&](int t, int j, int buf, bool next_scores, int t2, int j2) -> bool {
      const uint32_t vidx = 2u * j + 1, kidx = next_scores ? 2u * j2 : vidx;
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 1 + 10 * t, j);
      // the three barriers tested together (one vote, one branch); full waits only if one is still open
      const bool ready = mbar_test_wait(kv_full(vidx % STAGES), (vidx / STAGES) & 1) &
                         mbar_test_wait(kv_full(kidx % STAGES), (kidx / STAGES) & 1) &
                         mbar_test_wait(p_full(t), j & 1);
      if (!__all_sync(0xffffffffu, ready)) {
        if (!wait_kv(vidx, 30 + t)) return false;
        if (next_scores && !wait_kv(kidx, 10 + t)) return false;
        if (!mbar_wait_warp(p_full(t), j & 1, ctx, kRoleMma, 20 + t, j)) return false;
      }
      tc_fence_after();
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 2 + 10 * t, j);
      issue_pv(t, j, buf);
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 3 + 10 * t, j);
      // the next scores overwrite the score tile (and P inside it): in issue order behind P V, which reads P
      if (next_scores) issue_qk(t2, j2, buf);
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 4 + 10 * t, j);
      return true;
    };

    if (n_max > 0) ok = mbar_wait_warp(q_full, 0, ctx, kRoleMma, 1, 0);
    if (ok && n_max > 0) ok = wait_kv(0, 10);
    if constexpr (kThird) {
      const int total = n0 + n1, longer = (n1 > n0) ? 1 : 0;
      auto tile_of = [&](int m) { return m < 2 * n_min ? (m & 1) : longer; };
      auto block_of = [&](int m) { return m < 2 * n_min ? (m >> 1) : m - n_min; };
      // three Q K^T ahead (K(0) has landed; the third needs K(1))
      for (int m = 0; ok && m < min(3, total); ++m) {
        if (block_of(m) > 0) ok = wait_kv(2u * block_of(m), 10);
        if (ok) {
          tc_fence_after();
          issue_qk(tile_of(m), block_of(m), m);
        }
      }
      int buf = 0;
      for (int m = 0; ok && m < total; ++m) {
        const bool more = m + 3 < total;
        ok = issue_batch(tile_of(m), block_of(m), buf, more, more ? tile_of(m + 3) : 0, more ? block_of(m + 3) : 0);
        buf = (buf == 2) ? 0 : buf + 1;
      }
    } else {
      if (ok) {
        tc_fence_after();
        if (n0 > 0) issue_qk(0, 0, 0);
        if (n1 > 0) issue_qk(1, 0, 1);
      }
      for (int j = 0; ok && j < n_max; ++j) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int n = (t == 0) ? n0 : n1;
          if (ok && j < n) ok = issue_batch(t, j, t, j + 1 < n, t, j + 1);
        }
      }
    }
    if (!ok || *abort_flag) {
      mma_commit_elect(drain_bar);
      mbar_wait_quiet(drain_bar, 0);
    }
    __syncwarp();
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;            // which Q tile
    const int quarter = warp & 3;       // tensor-memory lanes 32*quarter .. +31
    const int qt = 2 * pair + t;
    const int q_row = qt * kAttnBQ + quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_addr = lane_base + kOCol + t * D;
    const float c = p.scale_log2;
    const int n = (t == 0) ? n0 : n1;
    const int first_masked = CAUSAL ? qt : (p.S % kWideBKV != 0 ? nkv - 1 : nkv);

    WIR_TRACE_DECL;
    float m = -INFINITY;  // running (possibly stale) max of the raw scores
    float l = 0.f;        // running sum of 2^(s c - m c)
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      if (quarter == 0 && lane == 0) WIR_TRACE_EVENT(p.trace, 1 + t, 100, j);
      // which score tile, and which of its completions (D = 128: the Q tile's own, one completion per block)
      const int k_seq = kThird ? seq_of(t, j) : 0;
      const int buf = kThird ? k_seq % 3 : t;
      const uint32_t s_phase = kThird ? static_cast<uint32_t>(k_seq / 3) & 1u : static_cast<uint32_t>(j) & 1u;
      const uint32_t s_addr = lane_base + buf * 128;
      if (!mbar_wait_warp(s_full(buf), s_phase, ctx, kRoleSoftmax, t, j)) { ok = false; break; }
      tc_fence_after();
      if (quarter == 0 && lane == 0) WIR_TRACE_EVENT(p.trace, 1 + t, 101, j);

#if defined(WIR_ABLATE) && WIR_ABLATE == 3
      // measurement build: no softmax at all, only the barrier handshake (results are meaningless)
      tc_fence_before();
      mbar_arrive(p_full(t));
      continue;
#endif
      uint32_t sb[128];  // this thread's row of raw scores, as fp32 bit patterns
      tmem_ld32(s_addr, sb);
      tmem_ld32(s_addr + 32, sb + 32);
      tmem_ld32(s_addr + 64, sb + 64);
      tmem_ld32(s_addr + 96, sb + 96);
      tmem_wait_ld();
      if (quarter == 0 && lane == 0) WIR_TRACE_EVENT(p.trace, 1 + t, 102, j);
#define WIR_S(i) __uint_as_float(sb[i])

      if (j >= first_masked || (j == nkv - 1 && p.S % kWideBKV != 0)) {
        const int k0 = j * kWideBKV;
        const int limit = CAUSAL ? min(q_row, p.S - 1) : (p.S - 1);  // last visible key
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > limit) sb[i] = 0xff800000u;  // -inf
      }

      float mx0 = WIR_S(0), mx1 = WIR_S(1), mx2 = WIR_S(2), mx3 = WIR_S(3);
      float mx4 = WIR_S(4), mx5 = WIR_S(5), mx6 = WIR_S(6), mx7 = WIR_S(7);
      // measurement builds (-DWIR_ABLATE=1|2|3, results meaningless): 2 also drops the row max
#if defined(WIR_ABLATE) && WIR_ABLATE == 2
#pragma unroll
      for (int i = 8; i < 16; i += 8) {
#else
#pragma unroll
      for (int i = 8; i < 128; i += 8) {
#endif
        mx0 = fmaxf(mx0, WIR_S(i));
        mx1 = fmaxf(mx1, WIR_S(i + 1));
        mx2 = fmaxf(mx2, WIR_S(i + 2));
        mx3 = fmaxf(mx3, WIR_S(i + 3));
        mx4 = fmaxf(mx4, WIR_S(i + 4));
        mx5 = fmaxf(mx5, WIR_S(i + 5));
        mx6 = fmaxf(mx6, WIR_S(i + 6));
        mx7 = fmaxf(mx7, WIR_S(i + 7));
      }
      const float m_new = fmaxf(fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3))), fmaxf(fmaxf(mx4, mx5), fmaxf(mx6, mx7)));
      const bool grow = (m_new - m) * c > kRescaleThreshold;  // true on the first block (m = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        if (j > 0) {
          // O_t was accumulated into by P V(j-1), which ran ahead of the Q K^T these scores came from
          if (!mbar_wait_warp(pv_done(t), (j - 1) & 1, ctx, kRoleSoftmax, 8 + t, j)) { ok = false; break; }
          tc_fence_after();
          const float alpha = ex2_approx((m - m_new) * c);
          l *= alpha;
#pragma unroll 1
          for (int cidx = 0; cidx < D / 16; ++cidx) {   // 16 columns at a time: the scores stay in registers
            uint32_t o[16];
            tmem_ld16(o_addr + cidx * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(o_addr + cidx * 16, o);
          }
        }
        m = m_new;
      }

      const float neg_mc = -m * c;
      // packed f32x2 arithmetic; all exponentials on the exponential unit (a polynomial share on the
      // FMA pipe, which pays in the 64-key kernel, measured slower here: one warp per scheduler is
      // short of issue slots, not of exponential throughput).
      // P goes over score columns 0-63, 16 packed columns per store; all scores are in registers by now.
      const float2 c2 = make_float2(c, c), neg_mc2 = make_float2(neg_mc, neg_mc);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(make_float2(WIR_S(ch * 32 + 2 * i), WIR_S(ch * 32 + 2 * i + 1)), c2, neg_mc2);
          float2 e;
#if defined(WIR_ABLATE) && (WIR_ABLATE == 1 || WIR_ABLATE == 2)
          e = x;   // measurement build: no exponentials
#else
          e.x = ex2_approx(x.x);
          e.y = ex2_approx(x.y);
#endif
          if (i & 1) lb = __fadd2_rn(lb, e);
          else la = __fadd2_rn(la, e);
          pk[i] = pack_bf16(e.x, e.y);
        }
        tmem_st16(s_addr + ch * 16, pk);
      }
#undef WIR_S
      l += (la.x + lb.x) + (la.y + lb.y);
      if constexpr (kThird) {
        // With its next scores computed ahead, a Q tile could finish block j + 1 before the issuing warp (held up by
        // a K or V tile, say) has looked at "P ready" of block j, and the barrier's parity would then read as "not
        // yet" for good.  So block j is only announced once P V of block j - 1 has completed, which the issuing warp
        // sends after it has seen block j - 1: the barrier is never more than one completion ahead of its reader.
        if (j > 0 && !mbar_wait_warp(pv_done(t), (j - 1) & 1, ctx, kRoleSoftmax, 8 + t, j)) { ok = false; break; }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(t));
      if (quarter == 0 && lane == 0) WIR_TRACE_EVENT(p.trace, 1 + t, 103, j);
    }

    if (ok && n > 0) {
      if (mbar_wait_warp(pv_done(t), (n - 1) & 1, ctx, kRoleEpilogue, t, n)) {
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

  tc_fence_before();
  __syncthreads();
  if (warp == kWideMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace wir
