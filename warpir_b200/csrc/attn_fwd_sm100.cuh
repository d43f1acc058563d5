// Attention forward for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V and
// LSE = logsumexp(scale * Q K^T), bf16 in, fp32 accumulate, bf16 O, fp32 LSE.
//
// This is the device kernel that the reference's attention tile program lowers to
// (tests/attention_baseline.py:147-177): per KV tile S = Q K^T; m' = max(m, rowmax S);
// P = 2^(S c - m' c); alpha = 2^(m c - m' c); l = l alpha + rowsum P; O = O alpha + bf16(P) V;
// finally O / l, with c = scale * log2(e) folded into the exponent
// (attention_baseline.py:42-43).  The reference lowers it to one 64-row tile per CTA
// with every step serialised by block barriers; its hand-written Hopper target adds a
// K/V ring, a producer warpgroup and causal / 4-D / log-sum-exp handling
// (kernel_examples/attention/mha_h100.cu:52-232).  Here:
//
//   warps 0-3, 4-7  one softmax warpgroup per 128-row Q tile (two tiles per CTA, so the
//                   tensor core works on one tile while the other is in softmax); one
//                   row per thread, so row max / row sum need no shuffles;
//   warp 8          MMA issuer: S_t = Q_t K^T and O_t += P_t V as tcgen05.mma into
//                   tensor memory, P_t read straight from tensor memory;
//   warp 9          producer: TMA loads of Q (once) and of the K/V tiles into a ring.
//
// Tensor memory (512 columns): S_0, S_1 (128 each; P_t overwrites the low 64 columns
// of S_t as packed bf16) and O_0, O_1 (D columns each).
//
// The O rescale is lazy: the running max m is only advanced when some row of the warp
// saw its max grow by more than 2^8 in the exponent domain; then that warp multiplies
// its O rows and l by alpha.  Until then P, l and O are all relative to the same stale
// m, so the final O / l and LSE = m c ln2 + ln l are exact.
#pragma once

#include "ptx.cuh"

namespace wir {

constexpr int kAttnBQ = 128;       // rows of one Q tile = MMA M
constexpr int kAttnBKV = 128;      // keys per KV tile
constexpr int kAttnThreads = 320;  // 2 softmax warpgroups + MMA warp + producer warp
constexpr float kRescaleThreshold = 8.0f;

struct AttnParams {
  int B, H, Hkv, S;        // S = query length = key length
  int D;
  float scale_log2;        // softmax_scale * log2(e)
  __nv_bfloat16* O;        // [B, H, S, D]
  float* LSE;              // [B, H, S] or nullptr
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int kStages = (D == 128) ? 5 : 8;
  static constexpr int kChunkBytes = 128 * 128;           // 128 rows x 64 bf16
  static constexpr int kTileBytes = (D / 64) * kChunkBytes;
  static constexpr int kQOffset = 0;
  static constexpr int kKVOffset = 2 * kTileBytes;
  static constexpr int kBarOffset = kKVOffset + kStages * kTileBytes;
  // q_full, kv_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2], drain
  static constexpr int kNumBars = 1 + 2 * kStages + 7;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kBytes = kAbortOffset + 4;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_sm100(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSCol = 0;          // S_t at columns t*128
  constexpr uint32_t kOCol = 256;        // O_t at columns 256 + t*D

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + STAGES + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 2 * STAGES + t); };
  auto p_full = [&](int t) { return bar_base + 8u * (3 + 2 * STAGES + t); };
  auto o_full = [&](int t) { return bar_base + 8u * (5 + 2 * STAGES + t); };
  const uint32_t drain_bar = bar_base + 8u * (7 + 2 * STAGES);
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
  const AbortCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which rows / how many KV tiles -----------------------------------------
  const int pair = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heaviest causal tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int bh = batch * p.H + head;
  const int bh_kv = batch * p.Hkv + head / (p.H / p.Hkv);
  const int nkv = (p.S + kAttnBKV - 1) / kAttnBKV;
  int n_trip[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = 2 * pair + t;
    n_trip[t] = (qt * kAttnBQ >= p.S) ? 0 : (CAUSAL ? min(nkv, qt + 1) : nkv);
  }
  const int n_max = max(n_trip[0], n_trip[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 128);
      mbar_init(o_full(t), 1);
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;

  if (warp == 9) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int n_q = (n_trip[0] > 0) + (n_trip[1] > 0);
      mbar_arrive_expect_tx(q_full, n_q * L::kTileBytes);
      for (int t = 0; t < 2; ++t)
        if (n_trip[t] > 0)
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_3d(smem_base + L::kQOffset + t * L::kTileBytes + c * L::kChunkBytes, &tmap_q, q_full,
                        c * 64, (2 * pair + t) * kAttnBQ, bh);
      uint32_t idx = 0;
      bool ok = true;
      for (int j = 0; ok && j < n_max; ++j) {
#pragma unroll
        for (int which = 0; which < 2; ++which, ++idx) {  // K(j) then V(j)
          const int s = idx % STAGES;
          const uint32_t ph = (idx / STAGES) & 1;
          if (!mbar_wait(kv_empty(s), ph ^ 1, ctx, kRoleProducer, s, j)) { ok = false; break; }
          mbar_arrive_expect_tx(kv_full(s), L::kTileBytes);
          const uint32_t dst = smem_base + L::kKVOffset + s * L::kTileBytes;
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_3d(dst + c * L::kChunkBytes, which == 0 ? &tmap_k : &tmap_v, kv_full(s), c * 64,
                        j * kAttnBKV, bh_kv);
        }
      }
      if (!ok || *abort_flag) {
        mbar_wait_quiet(q_full, 0);
        const uint32_t n = idx < STAGES ? idx : STAGES;
        for (uint32_t back = 1; back <= n; ++back) {
          const uint32_t i = idx - back;
          mbar_wait_quiet(kv_full(i % STAGES), (i / STAGES) & 1);
        }
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_bf16_f32(kAttnBQ, kAttnBKV, 0, 0);
      constexpr uint32_t idesc_pv = idesc_bf16_f32(kAttnBQ, D, 0, 1);
      bool ok = true;

      auto kv_stage_addr = [&](uint32_t idx) { return smem_base + L::kKVOffset + (idx % STAGES) * L::kTileBytes; };
      auto wait_kv = [&](uint32_t idx, int tag) {
        return mbar_wait(kv_full(idx % STAGES), (idx / STAGES) & 1, ctx, kRoleMma, tag, idx);
      };
      // S_t = Q_t K(j)^T
      auto issue_qk = [&](int t, int j) -> bool {
        const uint32_t idx = 2 * j;
        if (!wait_kv(idx, 10 + t)) return false;
        tc_fence_after();
        const uint32_t q_src = smem_base + L::kQOffset + t * L::kTileBytes;
        const uint32_t k_src = kv_stage_addr(idx);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * L::kChunkBytes + (k % 4) * 32;
          mma_ss(tmem_base + kSCol + t * 128, smem_desc_sw128(q_src + off, 16, 1024),
                 smem_desc_sw128(k_src + off, 16, 1024), idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(s_full(t));
        // K(j) is free once the last tile that needs it has been issued
        const bool last_user = (t == 1) || !(j < n_trip[1]);
        if (last_user) mma_commit(kv_empty(idx % STAGES));
        return true;
      };

      ok = mbar_wait(q_full, 0, ctx, kRoleMma, 1, 0);
      for (int t = 0; ok && t < 2; ++t)
        if (n_trip[t] > 0) ok = issue_qk(t, 0);

      for (int j = 0; ok && j < n_max; ++j) {
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= n_trip[t]) continue;
          // O_t += P_t(j) V(j)
          if (!mbar_wait(p_full(t), j & 1, ctx, kRoleMma, 20 + t, j)) { ok = false; break; }
          const uint32_t idx = 2 * j + 1;
          if (!wait_kv(idx, 30 + t)) { ok = false; break; }
          tc_fence_after();
          const uint32_t v_src = kv_stage_addr(idx);
#pragma unroll
          for (int k = 0; k < kAttnBKV / 16; ++k) {
            // 16 keys further: 8 packed-bf16 columns of P, 16 rows (2048 B) of V
            mma_ts(tmem_base + kOCol + t * D, tmem_base + kSCol + t * 128 + k * 8,
                   smem_desc_sw128(v_src + k * 2048, L::kChunkBytes, 1024), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
          const bool last_user = (t == 1) || !(j < n_trip[1]);
          if (last_user) mma_commit(kv_empty(idx % STAGES));
          if (j + 1 == n_trip[t]) mma_commit(o_full(t));
          else ok = issue_qk(t, j + 1);
        }
      }
      if (!ok || *abort_flag) {
        mma_commit(drain_bar);
        mbar_wait_quiet(drain_bar, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;            // which Q tile
    const int quarter = warp & 3;       // tensor-memory lanes 32*quarter .. +31
    const int row_in_tile = quarter * 32 + lane;
    const int q_row = (2 * pair + t) * kAttnBQ + row_in_tile;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_base + kSCol + t * 128;
    const uint32_t o_addr = lane_base + kOCol + t * D;
    const float c = p.scale_log2;
    const int n = n_trip[t];

    float m = -INFINITY;  // running (possibly stale) max of the raw scores
    float l = 0.f;        // running sum of 2^(s c - m c)
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      const bool got = mbar_wait(s_full(t), j & 1, ctx, kRoleSoftmax, t, j);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();

      uint32_t sb[128];  // this thread's row of raw scores, as fp32 bit patterns
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx) tmem_ld32(s_addr + cidx * 32, sb + cidx * 32);
      tmem_wait_ld();
#define WIR_S(i) __uint_as_float(sb[i])

      const bool diag = CAUSAL && (j == (2 * pair + t));
      const bool tail = (j == nkv - 1) && (p.S % kAttnBKV != 0);
      if (diag || tail) {
        const int k0 = j * kAttnBKV;
        const int limit = CAUSAL ? min(q_row, p.S - 1) : (p.S - 1);  // last visible key
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > limit) sb[i] = 0xff800000u;  // -inf
      }

      float mx0 = WIR_S(0), mx1 = WIR_S(1), mx2 = WIR_S(2), mx3 = WIR_S(3);
#pragma unroll
      for (int i = 4; i < 128; i += 4) {
        mx0 = fmaxf(mx0, WIR_S(i));
        mx1 = fmaxf(mx1, WIR_S(i + 1));
        mx2 = fmaxf(mx2, WIR_S(i + 2));
        mx3 = fmaxf(mx3, WIR_S(i + 3));
      }
      const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
      const bool grow = (m_new - m) * c > kRescaleThreshold;  // true on the first tile (m = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        if (j > 0) {
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

      const float neg_mc = -m * c;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2_approx(fmaf(WIR_S(cidx * 32 + 2 * i), c, neg_mc));
          const float p1 = ex2_approx(fmaf(WIR_S(cidx * 32 + 2 * i + 1), c, neg_mc));
          l0 += p0;
          l1 += p1;
          pk[i] = pack_bf16(p0, p1);
        }
        tmem_st16(s_addr + cidx * 16, pk);
      }
#undef WIR_S
      l += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(t));
    }

    if (ok && n > 0) {
      const bool got = mbar_wait(o_full(t), 0, ctx, kRoleEpilogue, t, 0);
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

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace wir
