// bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B, fp32 accumulation in tensor memory.
//
// This is the device kernel that the reference's GEMM tile program
// (tests/gemm_baseline_v2.py:62-88: zero; k-loop of two TMA loads, wait, MMA;
// store) lowers to.  The reference emits a 64x64 tile per CTA with every k-step
// serialised by block barriers (warpir/lowering/lowering.py:436-470); its
// hand-written targets add a two-slot ring (kernel_examples/gemm_pipelined.cu:21-78)
// and a producer/consumer split with full/empty semaphores
// (kernel_examples/gemm_warp_specialized.cu:22-77).  On Blackwell the same program
// becomes a persistent, warp-specialised kernel:
//
//   warp 0   producer: one lane issues TMA loads of A (128 x 64) and B (BN x 64)
//            tiles into a STAGES-deep shared-memory ring guarded by full/empty
//            mbarriers;
//   warp 1   MMA issuer: one lane issues tcgen05.mma (128 x BN x 16, four per
//            stage) into one of two accumulators in tensor memory, frees each
//            stage with tcgen05.commit and publishes the finished accumulator;
//   warps 2-5 epilogue: tcgen05.ld the accumulator (one row per thread), convert
//            to bf16 and store C, overlapping the next tile's main loop.
//
// MT = 2 makes the CTA tile 256 rows tall: two 128-row MMAs per k-step share one B tile, which
// halves the B bytes each SM pulls from L2 per FLOP (the 128 x 256 tile moves 96 B/clk/SM, about
// what L2 can feed to 148 SMs at once; 256 x 256 moves 64).  The two accumulators then fill all
// 512 tensor-memory columns, so the epilogue (two warpgroups) is not overlapped with the next
// tile's MMAs; at large K that costs a few percent, at small K the 128-row tile is preferred.
//
// Work items (output tile x K-split) are handed out statically, `gridDim.x`
// apart, walking the tile grid in bands of kGroupM row-blocks so that the CTAs
// running at any moment share A and B panels in L2.  (DRAM traffic stays near "every wave of
// tiles reads its own rows of A and columns of B once": ~1.1-1.2 GB per 8192^3 launch for 0.4 GB
// of operands, whatever the band height, the K direction of alternate tiles or the L2
// eviction hints; the reuse that is left on the table is ACROSS waves, and L2 does not
// keep a 33-67 MB row band alive under the 60 MB that stream through per wave.)
#pragma once

#include "ptx.cuh"

namespace wir {

constexpr int kGemmBM = 128;      // rows of an output tile = MMA M
constexpr int kGemmBK = 64;       // K extent of one pipeline stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192; // producer warp + MMA warp + 4 epilogue warps (per 128 rows of the tile)
__host__ __device__ constexpr int gemm_threads(int mt) { return 64 + 128 * mt; }
constexpr int kGroupM = 8;        // rasterisation band height in row-blocks (measured on 8192^3: least DRAM traffic of 4/8/12/16/32)

// Which warp does what.  The lowering writes its role table into every translation unit it emits as
// static_asserts against these constants, so a table that drifts from the kernel fails to compile.
template <int MT>
struct GemmRoles {
  static constexpr int kProducerWarp = 0;        // one elected lane issues the TMA loads
  static constexpr int kMmaWarp = 1;             // one elected lane issues tcgen05.mma / commit
  static constexpr int kFirstEpilogueWarp = 2;   // one warpgroup per 128 rows of the CTA tile
  static constexpr int kEpilogueWarps = 4 * MT;
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps);
};
static_assert(GemmRoles<1>::kThreads == gemm_threads(1) && GemmRoles<2>::kThreads == gemm_threads(2), "thread counts");

struct GemmParams {
  int M, N, K;
  int ldc;            // leading dimension of C in elements
  int tiles_m, tiles_n;   // tiles_m counts CTA tiles of MT * 128 rows
  int num_kb;         // ceil(K / 64)
  int splits;         // K-splits per output tile (1 = none)
  int kb_per_split;
  __nv_bfloat16* C;
  float* partial;     // [splits][M][N] fp32 partial sums when splits > 1 (stream-K: one slot per tile segment)
  int* status;        // 4 device status words
  // Stream-K (sk_units > 0): the tiles_m * tiles_n * num_kb k-blocks of the problem are dealt out as
  // `gridDim.x` contiguous runs of sk_units, so every CTA streams the same amount of B whatever the
  // number of tiles.  A run covers the tail of one tile, whole tiles, and the head of another; each
  // piece (segment) of a tile shared between CTAs goes to its own fp32 slot, and the CTA whose
  // segment lands last sums the slots in segment order and stores the tile.
  int sk_units = 0;       // k-blocks per CTA, 0 = off
  int sk_max_seg = 0;     // slots reserved per tile
  int sk_rows = 0;        // rows of a slot (min(M, 128))
  int* sk_counters = nullptr;   // one arrival counter per tile; zero between launches
  // Fused all-gather of the output (n_dst > 1): every finished tile is stored to each of the n_dst
  // destinations, which are the places of this GPU's block of C in the full C of every GPU of the
  // job (its own and its peers', mapped into this GPU's address space).  The stores to peers travel
  // over NVLink while the tensor core works on the next tile.  C is dst[0] when n_dst == 0.
  static constexpr int kMaxDst = 8;
  int n_dst = 0;
  __nv_bfloat16* dst[kMaxDst] = {};
  unsigned long long* trace;   // event trace buffer of debug builds (-DWIR_TRACE), else unused
  // Rasterisation: tiles are walked in bands of group_m row-blocks (column by column inside a band).
  int group_m = kGroupM;
  // 1: every other tile of a CTA walks K backwards, so that a wave starts on the K end the
  // previous wave finished on, which is what an LRU cache still holds of the shared panel
  int k_serpentine = 0;
  // L2 hints of the pair kernel (bit 0: A tiles evict_last, bit 1: B tiles evict_first, bit 2: streaming
  // stores of C).  Measured on 8192^3 (DRAM read + write per launch, band of 8): none 1186 MB, A evict_last
  // 1157 MB and ~1 % faster, B evict_first 2137 MB (a B tile is still wanted by the other clusters of the
  // wave when it goes), streaming stores no change.  No setting brings a row band of A (33 MB) through
  // to the next wave of tiles.
  int l2_hints = 1;
};

// Shared memory: the A tiles of all stages first, then the B tiles, then barriers.  A_ROWS < 128
// (problems with few rows) loads only the rows of A that exist; the MMA still reads 128 rows
// starting at the tile, i.e. runs on into the tiles behind it, which only produces values for
// rows of C that are never stored.  The B area behind the A area keeps those reads inside the
// allocation.
template <int BN, int STAGES, int MT = 1, int A_ROWS = kGemmBM>
struct GemmSmem {
  static_assert(A_ROWS % 8 == 0 && A_ROWS <= kGemmBM && (A_ROWS == kGemmBM || MT == 1), "A rows");
  static constexpr int kABytes = (A_ROWS == kGemmBM ? MT * kGemmBM : A_ROWS) * kGemmBK * 2;
  static constexpr int kBBytes = BN * kGemmBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBOffset = STAGES * kABytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static_assert(STAGES * kBBytes >= kGemmBM * kGemmBK * 2, "B area must cover the MMA's over-read of A");
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * STAGES + 5;
  static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
  static constexpr int kAbortOffset = kTmemPtrOffset + 4;
  static constexpr int kTicketOffset = kAbortOffset + 4;
  // 4 KB per epilogue warp: 32 rows x 128 bytes of output, turned from one row per lane into
  // whole 128-byte row segments per store when the tile also goes to peer GPUs
  static constexpr int kStageOutOffset = (kTicketOffset + 4 + 127) & ~127;
  static constexpr int kBytes = kStageOutOffset + 4 * MT * 4096;
  static constexpr int kDynamicBytes = kBytes + 1024;  // room to align the base to 1024 B
};

struct TileCoord {
  int m_blk, n_blk, kb_begin, kb_end, split;
  int tile;   // linear tile index (rasterised order)
  int nseg;   // pieces this tile's K range is computed in (1: this piece is the whole tile)
};

// Tile index -> block coordinates, walking the tile grid in bands of kGroupM row-blocks.
// (The work decomposition below is plain integer arithmetic, callable from the host so that
// it can be checked exhaustively without a GPU.)
__host__ __device__ __forceinline__ void decode_tile(int tile, const GemmParams& p, TileCoord& t) {
  const int band = p.group_m * p.tiles_n;
  const int g = tile / band;
  const int first_m = g * p.group_m;
  const int rest = p.tiles_m - first_m;
  const int rows = rest < p.group_m ? rest : p.group_m;
  const int in_band = tile - g * band;
  t.m_blk = first_m + in_band % rows;
  t.n_blk = in_band / rows;
  t.tile = tile;
}

// The sequence of work items of CTA `cta` of `grid`; producer, MMA issuer and epilogue each walk their own copy.
struct WorkIter {
  int w;          // next item (tile x K-split), static round-robin
  int g, g_end;   // stream-K: next k-block of this CTA's run, and its end
  int cta, grid;
};

__host__ __device__ __forceinline__ WorkIter work_begin(const GemmParams& p, int cta, int grid) {
  WorkIter it;
  it.cta = cta;
  it.grid = grid;
  it.w = cta;
  it.g = cta * p.sk_units;
  const int total = p.tiles_m * p.tiles_n * p.num_kb;
  it.g_end = (it.g + p.sk_units < total) ? it.g + p.sk_units : total;
  return it;
}

__host__ __device__ __forceinline__ bool work_next(WorkIter& it, const GemmParams& p, TileCoord& t) {
  if (p.sk_units == 0) {
    if (it.w >= p.tiles_m * p.tiles_n * p.splits) return false;
    const int tile = it.w / p.splits;
    decode_tile(tile, p, t);
    t.split = it.w - tile * p.splits;
    t.nseg = p.splits;
    t.kb_begin = t.split * p.kb_per_split;
    t.kb_end = (t.kb_begin + p.kb_per_split < p.num_kb) ? t.kb_begin + p.kb_per_split : p.num_kb;
    it.w += it.grid;
    return true;
  }
  if (it.g >= it.g_end) return false;
  const int tile = it.g / p.num_kb;
  decode_tile(tile, p, t);
  t.kb_begin = it.g - tile * p.num_kb;
  const int left = it.g_end - it.g;
  t.kb_end = (t.kb_begin + left < p.num_kb) ? t.kb_begin + left : p.num_kb;
  const int first_cta = (tile * p.num_kb) / p.sk_units;
  const int last_cta = ((tile + 1) * p.num_kb - 1) / p.sk_units;
  t.split = it.cta - first_cta;
  t.nseg = last_cta - first_cta + 1;
  it.g += t.kb_end - t.kb_begin;
  return true;
}

// B_MN = false: B stored [N,K] (K contiguous), one TMA box of BN rows per stage.
// B_MN = true : B stored [K,N] (N contiguous), BN/64 boxes of 64(k) x 64(n) per stage.
template <int BN, int STAGES, bool B_MN, int MT = 1, int A_ROWS = kGemmBM>
__global__ void __launch_bounds__(gemm_threads(MT), 1)
gemm_bf16_sm100(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmParams p) {
  using L = GemmSmem<BN, STAGES, MT, A_ROWS>;
  constexpr int kAccBufs = (2 * MT * BN <= 512) ? 2 : 1;   // double-buffer the accumulator when it fits
  constexpr uint32_t kTmemCols = (kAccBufs * MT * BN < 32) ? 32 : kAccBufs * MT * BN;
  constexpr int kTileM = MT * kGemmBM;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "MMA N");
  static_assert(!B_MN || BN % 64 == 0, "N-contiguous B is loaded in 64-column boxes");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
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
#ifdef WIR_TRACE
  { WIR_TRACE_DECL; if (threadIdx.x == 64) WIR_TRACE_EVENT(p.trace, 2, 20, 0); }
#endif

  // Producer state (thread 0 only).  The first loads are issued right here, before the rest of the
  // CTA has allocated tensor memory and met at the barrier, so the start-up latency of the first
  // copies overlaps the rest of the prologue.
  WorkIter p_work = work_begin(p, blockIdx.x, gridDim.x);
  TileCoord p_tile;
  int p_kb = 0, p_kb_end = 0;
  uint32_t p_it = 0;
  bool p_rev = true;   // flipped before the first tile
  // 1: one stage issued, 0: no work left, -1: a wait ran out
  auto producer_step = [&](bool slot_known_free) -> int {
    if (p_kb >= p_kb_end) {
      if (!work_next(p_work, p, p_tile)) return 0;
      p_kb = p_tile.kb_begin;
      p_kb_end = p_tile.kb_end;
      p_rev = !p_rev;
    }
    // K coordinate of this step (the MMA warp only counts stages, so the order is the producer's choice)
    const int kc = (p.k_serpentine && p_rev) ? (p_tile.kb_begin + p_tile.kb_end - 1 - p_kb) : p_kb;
    const int s = p_it % STAGES;
    const uint32_t ph = (p_it / STAGES) & 1;
    if (!slot_known_free && !mbar_wait(empty_bar(s), ph ^ 1, ctx, kRoleProducer, s, p_kb)) return -1;
    mbar_arrive_expect_tx(full_bar(s), L::kStageBytes);
    const uint32_t a_dst = smem_base + s * L::kABytes;
    const uint32_t b_dst = smem_base + L::kBOffset + s * L::kBBytes;
    tma_load_2d(a_dst, &tmap_a, full_bar(s), kc * kGemmBK, p_tile.m_blk * kTileM);
    if constexpr (!B_MN) {
      tma_load_2d(b_dst, &tmap_b, full_bar(s), kc * kGemmBK, p_tile.n_blk * BN);
    } else {
#pragma unroll
      for (int c = 0; c < BN / 64; ++c)
        tma_load_2d(b_dst + c * 8192, &tmap_b, full_bar(s), p_tile.n_blk * BN + c * 64, kc * kGemmBK);
    }
    ++p_kb;
    ++p_it;
    return 1;
  };

  if (threadIdx.x == 0) {
    WIR_TRACE_DECL;
    WIR_TRACE_EVENT(p.trace, 4, 30, 0);
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 128 * MT);
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    WIR_TRACE_EVENT(p.trace, 4, 31, 0);
    // two stages only: issuing a stage costs this thread ~280 clocks, and the rest of the CTA is
    // waiting for it at the barrier below; the remaining slots are filled right after it
    for (int n = 0; n < 2 && n < STAGES; ++n)
      if (producer_step(true) <= 0) break;
    WIR_TRACE_EVENT(p.trace, 4, 32, 0);
  }
  static_assert(GemmRoles<MT>::kProducerWarp == 0 && GemmRoles<MT>::kMmaWarp == 1 && GemmRoles<MT>::kFirstEpilogueWarp == 2, "roles");
  if (warp == 1) {
    WIR_TRACE_DECL;
    if (lane == 0) WIR_TRACE_EVENT(p.trace, 5, 40, 0);
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
    if (lane == 0) WIR_TRACE_EVENT(p.trace, 5, 41, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
#ifdef WIR_TRACE
  { WIR_TRACE_DECL; if (threadIdx.x == 64) WIR_TRACE_EVENT(p.trace, 6, 21, 0); }
#endif

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int r;
      while ((r = producer_step(false)) > 0) {
      }
      if (r < 0 || *abort_flag) {
        // wait (bounded, silently) for the copies still in flight before the CTA may exit
        const uint32_t n = p_it < STAGES ? p_it : STAGES;
        for (uint32_t back = 1; back <= n; ++back) {
          const uint32_t idx = p_it - back;
          mbar_wait_quiet(full_bar(idx % STAGES), (idx / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs this loop (warp-uniform operands); one elected lane issues.
    constexpr uint32_t idesc = idesc_bf16_f32(kGemmBM, BN, 0, B_MN ? 1 : 0);
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    WIR_TRACE_DECL;
    WorkIter work = work_begin(p, blockIdx.x, gridDim.x);
    TileCoord t;
    for (; ok && work_next(work, p, t); ++acc_it) {
      const int w = t.tile;
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 1, w);
      long long waited = 0;
      const uint32_t acc = kAccBufs == 2 ? (acc_it & 1) : 0;
      const uint32_t acc_ph = kAccBufs == 2 ? ((acc_it >> 1) & 1) : (acc_it & 1);
      if (!mbar_wait_warp(acc_empty_bar(acc), acc_ph ^ 1, ctx, kRoleMma, 100 + acc, w)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * (MT * BN);
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 2, w);
      for (int kb = t.kb_begin; kb < t.kb_end; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
#ifdef WIR_TRACE
        const long long w0 = clock64();
#endif
        if (!mbar_wait_warp(full_bar(s), ph, ctx, kRoleMma, s, kb)) { ok = false; break; }
#ifdef WIR_TRACE
        waited += clock64() - w0;
#endif
        tc_fence_after();
        const uint32_t a_lo = smem_desc_lo(smem_base + s * L::kABytes, 16);
        const uint32_t b_lo = smem_desc_lo(smem_base + L::kBOffset + s * L::kBBytes, B_MN ? 8192 : 16);
        // The stage's four k-steps go out as one instruction block per 128-row half (issued one by
        // one, an MMA costs the issuing warp ~80 clocks, more than the tensor core needs for the
        // 64- and 128-wide tiles).  16 K-elements further: 32 bytes along a K-major row, 16 rows
        // (2048 B) of an N-major tile.
        static_assert(kGemmBK == 64, "four k-steps per stage");
        constexpr uint32_t kBStep = B_MN ? (2048 >> 4) : (32 >> 4);
        const uint64_t bd = desc64(b_lo, desc_hi);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {   // the row halves of the CTA tile: 16 KB apart in the A stage
          const uint64_t ad = desc64(a_lo + ((mt * kGemmBM * 128) >> 4), desc_hi);
          mma_ss_elect_x4(d_tmem + mt * BN, ad, ad + 2, ad + 4, ad + 6, bd, bd + kBStep, bd + 2 * kBStep, bd + 3 * kBStep,
                          idesc, kb > t.kb_begin ? 1u : 0u);
        }
        mma_commit_elect(empty_bar(s));  // stage reusable once these MMAs have read it
      }
      if (ok) mma_commit_elect(acc_full_bar(acc));
      if (lane == 0) WIR_TRACE_EVENT(p.trace, 0, 3, static_cast<int>(waited));
    }
    if (!ok || *abort_flag) {
      mma_commit_elect(drain_bar);
      mbar_wait_quiet(drain_bar, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, 32*quarter+32) belong to this warp
    const int mt = (warp - 2) >> 2;  // which 128-row half of the CTA tile this warpgroup drains
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    uint32_t acc_it = 0;
    bool ok = true;
    WIR_TRACE_DECL;
    WorkIter work = work_begin(p, blockIdx.x, gridDim.x);
    TileCoord t;
    for (; ok && work_next(work, p, t); ++acc_it) {
      const int w = t.tile;
      const uint32_t acc = kAccBufs == 2 ? (acc_it & 1) : 0;
      const uint32_t acc_ph = kAccBufs == 2 ? ((acc_it >> 1) & 1) : (acc_it & 1);
      if (warp == 2 && lane == 0) WIR_TRACE_EVENT(p.trace, 1, 10, w);
      bool got = mbar_wait(acc_full_bar(acc), acc_ph, ctx, kRoleEpilogue, acc, w);
      got = __all_sync(0xffffffffu, got);
      if (p.sk_units != 0) {
        // the four epilogue warps meet at named barriers below, so they must agree on whether to go on
        uint32_t all;
        asm volatile(
            "{\n\t.reg .pred a, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred a, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, a;\n\t}"
            : "=r"(all)
            : "r"(got ? 1u : 0u)
            : "memory");
        got = all != 0;
      }
      if (!got) { ok = false; break; }
      tc_fence_after();
      if (warp == 2 && lane == 0) WIR_TRACE_EVENT(p.trace, 1, 11, w);
      const int row = t.m_blk * kTileM + mt * kGemmBM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * (MT * BN) + mt * BN;
      constexpr int kChunk = (BN % 32 == 0) ? 32 : 16;
      if constexpr (BN % 64 == 0 && MT == 1) {   // the host only gathers with 128-row tiles
        if (p.n_dst > 0) {
          // Gathered output.  A store instruction of a warp with one row per lane writes 32 separate
          // 16-byte pieces, which is harmless in local memory (L2 merges them) but wastes most of an
          // NVLink packet.  So the warp turns its 32 x 64 block around in shared memory (XOR-swizzled,
          // conflict-free both ways) and stores 128 contiguous bytes per row, four rows per instruction.
          uint8_t* stage = smem + L::kStageOutOffset + (warp - 2) * 4096;
          const int row_base = t.m_blk * kTileM + mt * kGemmBM + quarter * 32;
#pragma unroll 1
          for (int c2 = 0; c2 < BN / 64; ++c2) {
            uint32_t r[64];
            tmem_ld32(t_row + c2 * 64, r);
            tmem_ld32(t_row + c2 * 64 + 32, r + 32);
            tmem_wait_ld();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              q.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              q.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              q.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              *reinterpret_cast<uint4*>(stage + lane * 128 + ((v ^ (lane & 7)) << 4)) = q;
            }
            __syncwarp();
            const int gcol = t.n_blk * BN + c2 * 64 + (lane & 7) * 8;
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
              const int rl = rr * 4 + (lane >> 3);
              const uint4 q = *reinterpret_cast<const uint4*>(stage + rl * 128 + (((lane & 7) ^ (rl & 7)) << 4));
              const int grow = row_base + rl;
              if (grow < p.M && gcol + 8 <= p.N)
                for (int d = 0; d < p.n_dst; ++d)
                  *reinterpret_cast<uint4*>(p.dst[d] + static_cast<size_t>(grow) * p.ldc + gcol) = q;
            }
            __syncwarp();
          }
          tc_fence_before();
          mbar_arrive(acc_empty_bar(acc));
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / kChunk; ++c) {
        uint32_t r[kChunk];
        if constexpr (kChunk == 32) tmem_ld32(t_row + c * kChunk, r);
        else tmem_ld16(t_row + c * kChunk, r);
        tmem_wait_ld();
        const int col0 = t.n_blk * BN + c * kChunk;
        if (row < p.M && col0 < p.N) {
          if (t.nseg == 1) {
            __nv_bfloat16* dst = p.C + static_cast<size_t>(row) * p.ldc + col0;
            if (vec_ok && col0 + kChunk <= p.N) {
#pragma unroll
              for (int v = 0; v < kChunk / 8; ++v) {
                uint4 q;
                q.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                q.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                q.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                q.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                reinterpret_cast<uint4*>(dst)[v] = q;
              }
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (col0 + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else if (p.sk_units != 0) {
            // stream-K: slot [tile][segment] of sk_rows x BN floats, whole chunks (columns past N are never read)
            float* dst = p.partial + ((static_cast<size_t>(t.tile) * p.sk_max_seg + t.split) * p.sk_rows +
                                      (mt * kGemmBM + quarter * 32 + lane)) * BN + c * kChunk;
#pragma unroll
            for (int v = 0; v < kChunk / 4; ++v)
              reinterpret_cast<uint4*>(dst)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          } else {
            float* dst = p.partial + (static_cast<size_t>(t.split) * p.M + row) * p.N + col0;
            if ((p.N % 4 == 0) && col0 + kChunk <= p.N) {
#pragma unroll
              for (int v = 0; v < kChunk / 4; ++v)
                reinterpret_cast<uint4*>(dst)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (col0 + j < p.N) dst[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty_bar(acc));
      if (warp == 2 && lane == 0) WIR_TRACE_EVENT(p.trace, 1, 12, w);
      if (MT == 1 && p.sk_units != 0 && t.nseg > 1) {   // (the host deals k-blocks out only with 128-row tiles)
        // Whoever brings the last segment of a tile finishes it.  Nobody waits: each CTA publishes
        // its slot, takes a ticket, and only the holder of the last ticket reads the slots back
        // (in segment order, so the sum does not depend on who arrived when).
        volatile int* ticket_slot = reinterpret_cast<volatile int*>(smem + L::kTicketOffset);
        const int epi_tid = threadIdx.x - 64;
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi_tid == 0) *ticket_slot = atomicAdd(p.sk_counters + t.tile, 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = (*ticket_slot == t.nseg - 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the slot is free for the next item
        if (last) {
          __threadfence();
          const int row0 = t.m_blk * kTileM, col0 = t.n_blk * BN;
          const int rows = min(p.sk_rows, p.M - row0);
          const float* slot0 = p.partial + static_cast<size_t>(t.tile) * p.sk_max_seg * p.sk_rows * BN;
          // all loads of a batch (kFixU float4 per thread x up to kFixSeg segments) are issued before
          // the first add, so a batch costs about one L2 round trip
          constexpr int kFixU = 8, kFixSeg = 4;
          const int n4 = (rows * BN) >> 2;
          const size_t seg_stride4 = (static_cast<size_t>(p.sk_rows) * BN) >> 2;
          const float4* base4 = reinterpret_cast<const float4*>(slot0);
          for (int first = epi_tid; first < n4; first += 128 * kFixU) {
            float4 v[kFixSeg][kFixU];
#pragma unroll
            for (int sgm = 0; sgm < kFixSeg; ++sgm)
#pragma unroll
              for (int u = 0; u < kFixU; ++u) {
                const int idx = first + u * 128;
                v[sgm][u] = (sgm < t.nseg && idx < n4) ? __ldcg(base4 + sgm * seg_stride4 + idx)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
            for (int u = 0; u < kFixU; ++u) {
              const int idx = first + u * 128;
              if (idx >= n4) break;
              float4 sum = v[0][u];
#pragma unroll
              for (int sgm = 1; sgm < kFixSeg; ++sgm)
                if (sgm < t.nseg) { sum.x += v[sgm][u].x; sum.y += v[sgm][u].y; sum.z += v[sgm][u].z; sum.w += v[sgm][u].w; }
              for (int sgm = kFixSeg; sgm < t.nseg; ++sgm) {   // tiles cut into more pieces than a batch holds
                const float4 w4 = __ldcg(base4 + sgm * seg_stride4 + idx);
                sum.x += w4.x; sum.y += w4.y; sum.z += w4.z; sum.w += w4.w;
              }
              const int e = idx << 2;
              const int r_in = e / BN, c_in = e - r_in * BN;
              const int col = col0 + c_in;
              __nv_bfloat16* dst = p.C + static_cast<size_t>(row0 + r_in) * p.ldc + col;
              if (vec_ok && col + 4 <= p.N) {
                uint2 q;
                q.x = pack_bf16(sum.x, sum.y);
                q.y = pack_bf16(sum.z, sum.w);
                *reinterpret_cast<uint2*>(dst) = q;
              } else {
                const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
                for (int k4 = 0; k4 < 4; ++k4)
                  if (col + k4 < p.N) dst[k4] = __float2bfloat16_rn(vals[k4]);
              }
            }
          }
          if (epi_tid == 0) p.sk_counters[t.tile] = 0;   // ready for the next launch
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
#ifdef WIR_TRACE
  { WIR_TRACE_DECL; if (threadIdx.x == 32) WIR_TRACE_EVENT(p.trace, 7, 22, 0); }
#endif
}

// Deterministic second pass of a split-K GEMM: sums the fp32 partials in split
// order and rounds to bf16.  One thread per four consecutive columns.
__global__ void splitk_reduce_bf16(const float* __restrict__ partial, __nv_bfloat16* __restrict__ C,
                                   int M, int N, int ldc, int splits) {
  const size_t total4 = (static_cast<size_t>(M) * N) >> 2;
  const size_t plane = static_cast<size_t>(M) * N;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(partial)[i];
    for (int s = 1; s < splits; ++s) {
      const float4 v = reinterpret_cast<const float4*>(partial + s * plane)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const size_t e = i << 2;
    const int row = static_cast<int>(e / N);
    const int col = static_cast<int>(e - static_cast<size_t>(row) * N);
    __nv_bfloat16* dst = C + static_cast<size_t>(row) * ldc + col;
    uint2 q;
    q.x = pack_bf16(acc.x, acc.y);
    q.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(dst) = q;
  }
}

}  // namespace wir
