// Micro-benchmark of the tensor core's instruction rate on sm_100a: how many SM clocks one
// tcgen05.mma of a given shape takes when the issuing thread keeps the queue full.
//
// One CTA per SM (or one CTA pair per two SMs) issues `batches` x 4 back-to-back MMAs into one
// accumulator, operands laid out exactly as the GEMM and attention kernels lay them out (K-major
// tiles of 64 bf16 per row, 128-byte swizzle; the A operand either in shared memory, "SS", or in
// tensor memory, "TS"), commits once at the end and waits.  clock64 brackets the whole run, so
// clocks / MMA = the rate the tensor core retires that shape at, provided the issue loop itself
// is faster (the time at which the last MMA was issued is reported too).  Optional background
// load separates the two suspects for a rate below the arithmetic one:
//   bg_tmem: four warps stream tcgen05.ld / tcgen05.st over other tensor-memory columns, as the
//            softmax warpgroups of the attention kernels do while the other tile's MMAs run;
//   bg_tma : one thread keeps four TMA tile loads (16 KB each) in flight into spare shared
//            memory, as a producer warp does.
// The arithmetic needs M x N x 16 / 4096 clocks per SM for an instruction (64 for 128 x 128 x 16).
// An SS instruction reads (128 + N_local) x 32 bytes of shared memory per SM, N_local = N for
// cta_group::1 and N / 2 for a pair.
//
// Exported as warpir_probe_mma_rate (see the prototype below); built as its own small library
// next to the product library, used by tests/test_mma_issue_rate_gpu.py.
#include "host_common.cuh"
#include "ptx.cuh"

namespace wir {

struct ProbeParams {
  int n;          // MMA N (whole instruction; a pair splits it between the two CTAs)
  int ts;         // 1: A operand from tensor memory
  int batches;    // groups of four MMAs (the four 16-element k-steps of one 64-element chunk)
  int bg_tmem;
  int bg_tma;
  int b_mn;       // 1: B operand N-major (64-element chunks of N, 8 KB apart, 128 bytes per K row), as V is in P V
  int single;     // 1: one MMA per instruction block (elect, descriptor moves and predicate set per MMA)
  int random_data;   // 1: operands hold pseudo-random values in +-[0.5, 1) instead of zeros
  int bg_alu;        // 1: eight more warps run the softmax's arithmetic (packed FMA, exponentials, bf16 packing) on registers
  int commit_every;  // > 0: a tcgen05.commit (to a barrier nobody waits on) after every so many instruction blocks
  int issuers;       // 2: warp 1 issues the same stream into a second accumulator (columns 128..), with its own commits
  // Pattern mode (n_blocks > 0): instead of one uniform stream, every step issues this list of instruction
  // blocks (four MMAs each, TS or SS as `ts` says): {N (64 or 128), accumulator column, 1 = the block's first
  // MMA overwrites the accumulator, 1 = commit after the block}.  B is read N-major for N = 128 blocks when
  // b_mn is set.  This is how a kernel's real issue order (several accumulators, mixed widths) is replayed.
  int n_blocks;
  int blocks[16][4];
  // Loop-shape mode (shape > 0): the issue loop of the attention backward's dQ kernel (per step one block of four
  // 128-wide MMAs, a commit, four blocks of four 64-wide MMAs, a commit; operand addresses that change with the
  // step as ring slots and buffers do), written in several ways -- see issue_dq_like below.
  int shape;
  float* sink;       // the arithmetic warps' results (never read)
  unsigned long long* out;   // per CTA: clocks until the last MMA was issued, clocks until all completed
  int* status;
};

constexpr int kProbeThreads = 448;          // warp 0 issuer, warp 1 TMA background, warps 2-5 tensor-memory background, warps 6-13 arithmetic background
constexpr int kProbeABytes = 128 * 128;     // 128 rows x 64 bf16
constexpr int kProbeBBytes = 256 * 128;     // up to 256 rows x 64 bf16
constexpr int kProbeBgBytes = 4 * 16384;    // four background TMA slots
constexpr int kProbeBarOffset = kProbeABytes + kProbeBBytes + kProbeBgBytes;
constexpr int kProbeSmem = kProbeBarOffset + 128 + 1024;

// The dQ kernel's issue loop in different shapes.  What changes with the step as in the kernel: the ring slot
// of the streamed tiles (step % 6) and the score buffer (step & 1).  `ready` is a barrier whose waited-for phase
// is always complete, so the waits return at once, as they do in the kernel's steady state.
//   1  as the kernel writes it: the loop ends early when a bounded wait fails (`ok && it < n`, `break`)
//   2  fixed trip count; a failed wait only switches the rest of the work off
//   3  no waits and no fences at all
//   4  waits that cannot fail (plain polling), fixed trip count
//   5  as 1, with the ring slot kept in a counter instead of `it % 6`
//   6  as 3, with every operand address computed before the block list is issued (two steps' worth of
//      descriptors held in registers)
//   7  as 1 without the tcgen05 fences after the waits
//   8  as 3 plus the two fences per step (no waits)
//   9  as 1, every lane waiting for itself and no vote on the outcome (a __syncwarp instead)
//  10  as 1, the ring-slot barrier tested before stage 2 is issued and the outcome used after it (the full
//      wait only if that early test failed)
//  11  as 1, stage 1 in two blocks of eight MMAs (all of T0, then all of T1) instead of four of four
//  12  10 and 11 together
//  13  as 1, one elected lane issuing a whole step's MMAs and its commits from inside one branch
// Eight MMAs with A in tensor memory in one instruction block: k-steps 0-3 read A at a0 + 8 j, 4-7 at a1 + 8 j.
__device__ __forceinline__ void mma_ts_elect_x8(uint32_t d_tmem, uint32_t a0, uint32_t a1, uint64_t b0, uint64_t b1,
                                                uint64_t b2, uint64_t b3, uint64_t b4, uint64_t b5, uint64_t b6,
                                                uint64_t b7, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t.reg .b32 x1, x2, x3, y1, y2, y3;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %12, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 x1, %1, 8;\n\t"
      "add.u32 x2, %1, 16;\n\t"
      "add.u32 x3, %1, 24;\n\t"
      "add.u32 y1, %2, 8;\n\t"
      "add.u32 y2, %2, 16;\n\t"
      "add.u32 y3, %2, 24;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %11, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [x1], %4, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [x2], %5, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [x3], %6, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %7, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [y1], %8, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [y2], %9, %11, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [y3], %10, %11, t;\n\t}"
      ::"r"(d_tmem), "r"(a0), "r"(a1), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "l"(b4), "l"(b5), "l"(b6), "l"(b7),
        "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int SHAPE>
__device__ __forceinline__ void issue_dq_like(uint32_t tmem_base, uint32_t smem_base, int n, uint32_t ready,
                                              uint32_t extra_bar, const AbortCtx& ctx) {
  constexpr int STAGES = 6;
  constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
  constexpr uint32_t idesc_t = idesc_bf16_f32(128, 64, 0, 0);
  constexpr uint32_t idesc_acc = idesc_bf16_f32(128, 128, 0, 1);
  const uint32_t b_base = smem_base + kProbeABytes;
  const uint32_t a_tmem = tmem_base + 256;     // 64 columns of packed A
  const uint32_t acc = tmem_base + 320;        // 128-column accumulator
  auto stage2 = [&](int it, uint32_t y) {
    const int b = it & 1;
    const uint64_t y0d = desc64(smem_desc_lo(y, 8192), desc_hi);
    mma_ts_elect_x4(acc, tmem_base + 128 + b * 64 + 16, y0d, y0d + 128, y0d + 256, y0d + 384, idesc_acc, it > 0 ? 1u : 0u);
    mma_commit_elect(extra_bar);
  };
  auto stage1 = [&](int it, uint32_t y) {
    const int b = it & 1;
    const uint32_t y0_lo = smem_desc_lo(y, 16), y1_lo = smem_desc_lo(y + 16384, 16);
#pragma unroll
    for (int c4 = 0; c4 < 2; ++c4) {
      const uint32_t yo = (c4 * 4096) >> 4;
      const uint64_t y0d = desc64(y0_lo + yo, desc_hi), y1d = desc64(y1_lo + yo, desc_hi);
      mma_ts_elect_x4(tmem_base + b * 64, a_tmem + c4 * 32, y0d, y0d + 2, y0d + 4, y0d + 6, idesc_t, c4 > 0 ? 1u : 0u);
      mma_ts_elect_x4(tmem_base + 128 + b * 64, a_tmem + c4 * 32, y1d, y1d + 2, y1d + 4, y1d + 6, idesc_t, c4 > 0 ? 1u : 0u);
    }
    mma_commit_elect(extra_bar);
  };
  auto stage1_x8 = [&](int it, uint32_t y) {
    const int b = it & 1;
    const uint64_t y0d = desc64(smem_desc_lo(y, 16), desc_hi), y1d = desc64(smem_desc_lo(y + 16384, 16), desc_hi);
    mma_ts_elect_x8(tmem_base + b * 64, a_tmem, a_tmem + 32, y0d, y0d + 2, y0d + 4, y0d + 6, y0d + 256, y0d + 258,
                    y0d + 260, y0d + 262, idesc_t, 0u);
    mma_ts_elect_x8(tmem_base + 128 + b * 64, a_tmem, a_tmem + 32, y1d, y1d + 2, y1d + 4, y1d + 6, y1d + 256, y1d + 258,
                    y1d + 260, y1d + 262, idesc_t, 0u);
    mma_commit_elect(extra_bar);
  };
  auto y_of = [&](int it) { return b_base + static_cast<uint32_t>(it % STAGES) * 2048u; };
  if constexpr (SHAPE == 10 || SHAPE == 11 || SHAPE == 12) {
    bool ok = true;
    for (int it = 0; ok && it < n; ++it) {
      if (!mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      tc_fence_after();
      bool y_ready = false;
      if constexpr (SHAPE != 11) y_ready = mbar_test_wait(ready, 1);
      stage2(it, y_of(it));
      if (it + 2 < n) {
        if (!__all_sync(0xffffffffu, y_ready)) ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
        if (ok) {
          if constexpr (SHAPE == 10) stage1(it + 2, y_of(it + 2));
          else stage1_x8(it + 2, y_of(it + 2));
        }
      }
    }
  } else if constexpr (SHAPE == 13) {
    bool ok = true;
    for (int it = 0; ok && it < n; ++it) {
      if (!mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      tc_fence_after();
      ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
      if (!ok) break;
      if (elect_one()) {
        const int b = it & 1;
        const uint32_t ya = y_of(it), yb = y_of(it + 2);
        const uint64_t w = desc64(smem_desc_lo(ya, 8192), desc_hi);
        const uint64_t n0 = desc64(smem_desc_lo(yb, 16), desc_hi), n1 = desc64(smem_desc_lo(yb + 16384, 16), desc_hi);
        const uint32_t t0 = tmem_base + b * 64, t1 = tmem_base + 128 + b * 64;
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ts(acc, t1 + 16 + 8 * k, w + 128 * k, idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        mma_commit(extra_bar);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ts(t0, a_tmem + 8 * k, n0 + (k < 4 ? 2 * k : 256 + 2 * (k - 4)), idesc_t, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ts(t1, a_tmem + 8 * k, n1 + (k < 4 ? 2 * k : 256 + 2 * (k - 4)), idesc_t, k > 0 ? 1u : 0u);
        mma_commit(extra_bar);
      }
      __syncwarp();
    }
  } else if constexpr (SHAPE == 1) {
    bool ok = true;
    for (int it = 0; ok && it < n; ++it) {
      if (!mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      tc_fence_after();
      stage2(it, y_of(it));
      if (it + 2 < n) {
        ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
        if (ok) {
          tc_fence_after();
          stage1(it + 2, y_of(it + 2));
        }
      }
    }
  } else if constexpr (SHAPE == 2) {
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      if (ok) ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it);
      if (ok) {
        tc_fence_after();
        stage2(it, y_of(it));
        ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
        if (ok) {
          tc_fence_after();
          stage1(it + 2, y_of(it + 2));
        }
      }
    }
  } else if constexpr (SHAPE == 3) {
    for (int it = 0; it < n; ++it) {
      stage2(it, y_of(it));
      stage1(it + 2, y_of(it + 2));
    }
  } else if constexpr (SHAPE == 4) {
    for (int it = 0; it < n; ++it) {
      mbar_wait_quiet(ready, 1);
      tc_fence_after();
      stage2(it, y_of(it));
      mbar_wait_quiet(ready, 1);
      tc_fence_after();
      stage1(it + 2, y_of(it + 2));
    }
  } else if constexpr (SHAPE == 7) {
    bool ok = true;
    for (int it = 0; ok && it < n; ++it) {
      if (!mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      stage2(it, y_of(it));
      if (it + 2 < n) {
        ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
        if (ok) stage1(it + 2, y_of(it + 2));
      }
    }
  } else if constexpr (SHAPE == 8) {
    for (int it = 0; it < n; ++it) {
      tc_fence_after();
      stage2(it, y_of(it));
      tc_fence_after();
      stage1(it + 2, y_of(it + 2));
    }
  } else if constexpr (SHAPE == 9) {
    bool ok = true;
    for (int it = 0; ok && it < n; ++it) {
      ok = mbar_wait(ready, 1, ctx, kRoleMma, 20, it);
      __syncwarp();
      if (!ok) break;
      tc_fence_after();
      stage2(it, y_of(it));
      if (it + 2 < n) {
        ok = mbar_wait(ready, 1, ctx, kRoleMma, 10, it);
        __syncwarp();
        if (ok) {
          tc_fence_after();
          stage1(it + 2, y_of(it + 2));
        }
      }
    }
  } else if constexpr (SHAPE == 5) {
    bool ok = true;
    uint32_t y = b_base, y2 = b_base + 2 * 2048u;
    for (int it = 0; ok && it < n; ++it) {
      if (!mbar_wait_warp(ready, 1, ctx, kRoleMma, 20, it)) { ok = false; break; }
      tc_fence_after();
      stage2(it, y);
      if (it + 2 < n) {
        ok = mbar_wait_warp(ready, 1, ctx, kRoleMma, 10, it);
        if (ok) {
          tc_fence_after();
          stage1(it + 2, y2);
        }
      }
      y = (y == b_base + (STAGES - 1) * 2048u) ? b_base : y + 2048u;
      y2 = (y2 == b_base + (STAGES - 1) * 2048u) ? b_base : y2 + 2048u;
    }
  } else {
    // every descriptor of a step computed first, then the blocks issued back to back
    for (int it = 0; it < n; ++it) {
      const int b = it & 1;
      const uint32_t ya = y_of(it), yb = y_of(it + 2);
      const uint64_t w = desc64(smem_desc_lo(ya, 8192), desc_hi);
      const uint64_t n00 = desc64(smem_desc_lo(yb, 16), desc_hi), n10 = desc64(smem_desc_lo(yb + 16384, 16), desc_hi);
      const uint64_t n01 = n00 + 256, n11 = n10 + 256;
      const uint32_t t0 = tmem_base + b * 64, t1 = tmem_base + 128 + b * 64;
      mma_ts_elect_x4(acc, t1 + 16, w, w + 128, w + 256, w + 384, idesc_acc, it > 0 ? 1u : 0u);
      mma_commit_elect(extra_bar);
      mma_ts_elect_x4(t0, a_tmem, n00, n00 + 2, n00 + 4, n00 + 6, idesc_t, 0u);
      mma_ts_elect_x4(t1, a_tmem, n10, n10 + 2, n10 + 4, n10 + 6, idesc_t, 0u);
      mma_ts_elect_x4(t0, a_tmem + 32, n01, n01 + 2, n01 + 4, n01 + 6, idesc_t, 1u);
      mma_ts_elect_x4(t1, a_tmem + 32, n11, n11 + 2, n11 + 4, n11 + 6, idesc_t, 1u);
      mma_commit_elect(extra_bar);
    }
  }
}

template <bool PAIR>
__global__ void __launch_bounds__(kProbeThreads, 1)
probe_mma_rate_kernel(const __grid_constant__ CUtensorMap tmap_bg, const ProbeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - raw_addr);
  const uint32_t bar_base = smem_base + kProbeBarOffset;
  const uint32_t done_bar = bar_base;                       // all MMAs completed
  auto bg_bar = [&](int s) { return bar_base + 8u * (1 + s); };
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem + kProbeBarOffset + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kProbeBarOffset + 68);
  volatile int* stop_flag = reinterpret_cast<volatile int*>(smem + kProbeBarOffset + 72);
  const AbortCtx ctx{abort_flag, p.status, 200000000ull};   // 0.2 s per wait

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;

  // operands: zeros, or pseudo-random bf16 pairs in +-[0.5, 1) (does the rate depend on the values?)
  auto rnd = [&](uint32_t i) {
    uint32_t h = (i + 1u + blockIdx.x * 65536u) * 2654435761u;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    return p.random_data ? ((h & 0x807f807fu) | 0x3f003f00u) : 0u;
  };
  for (int i = threadIdx.x; i < (kProbeABytes + kProbeBBytes) / 16; i += kProbeThreads)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(rnd(4 * i), rnd(4 * i + 1), rnd(4 * i + 2), rnd(4 * i + 3));
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *stop_flag = 0;
    mbar_init(done_bar, 1);
    for (int s = 0; s < 4; ++s) mbar_init(bg_bar(s), 1);
    mbar_init(bar_base + 8u * 5, 1);   // target of the extra commits
    mbar_init(bar_base + 8u * 6, 1);   // second issuer: all MMAs completed
    mbar_init(bar_base + 8u * 7, 1);   // second issuer: target of its extra commits
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  if (warp >= 2 && warp < 6) {
    // A operand of the TS form (32 packed columns at column 256) and a zeroed accumulator
    uint32_t r[32];
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = rnd(threadIdx.x * 32 + i);
    tmem_st32(lane_addr + 256, r);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = 0u;
    for (int c = 0; c < 8; ++c) tmem_st32(lane_addr + c * 32, r);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // One issuing warp's run: `batches` blocks of four MMAs into the accumulator at `d_tmem`, an extra commit to
  // `extra_bar` after every commit_every blocks, one commit to `done` at the end.  t[0]: clocks until the last
  // MMA was issued, t[1]: the starting clock.  (No clock reads inside the loop: reading the clock after every
  // block was tried and by itself nearly doubled the time per block.)
  auto issue_stream = [&](uint32_t d_tmem, uint32_t done, uint32_t extra_bar, long long* t) {
    const int m = PAIR ? 256 : 128;
    const uint32_t idesc = idesc_bf16_f32(m, p.n, 0, p.b_mn);
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    const uint64_t ad = desc64(smem_desc_lo(smem_base, 16), desc_hi);
    const uint64_t bd = desc64(smem_desc_lo(smem_base + kProbeABytes, p.b_mn ? 8192 : 16), desc_hi);
    // 16 K-elements further: 32 bytes along a K-major row, 16 rows (2048 bytes) of an N-major chunk
    const uint64_t bs = p.b_mn ? 128 : 2;
    const uint32_t a_tmem = tmem_base + 256;    // TS form: A as 32 packed columns
    __syncwarp();
    const long long t0 = clock64();
    // a countdown, not `(b + 1) % commit_every`: a division by a run-time value is some thirty dependent
    // instructions, which the issuing warp takes 6-12 clocks each over -- more than the MMAs it would
    // separate last (an earlier version of this probe measured that division and called it the commit's cost)
    int left = p.commit_every > 0 ? p.commit_every : 0x7fffffff;
    const uint32_t extra_cluster = PAIR ? mapa_shared(extra_bar, 0) : extra_bar;
    auto maybe_commit = [&](int) {
      if (--left == 0) {
        left = p.commit_every;
        if (PAIR) mma_commit_pair_elect(extra_cluster);
        else mma_commit_elect(extra_bar);
      }
    };
    // one loop per form, so that each is as tight as a kernel's own (the choice is not re-made per block)
    if (p.single) {
      const uint32_t a_lo = static_cast<uint32_t>(ad), b_lo = static_cast<uint32_t>(bd);
      for (int b = 0; b < p.batches; ++b) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (p.ts) mma_ts_elect(d_tmem, a_tmem + k * 8, b_lo + k * static_cast<uint32_t>(bs), desc_hi, idesc, 1u);
          else mma_ss_elect(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * static_cast<uint32_t>(bs), desc_hi, idesc, 1u);
        }
        maybe_commit(b);
      }
    } else if (p.ts) {
      for (int b = 0; b < p.batches; ++b) {
        if (PAIR) mma_ts_pair_x4(d_tmem, a_tmem, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, 1u);
        else mma_ts_elect_x4(d_tmem, a_tmem, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, 1u);
        maybe_commit(b);
      }
    } else {
      for (int b = 0; b < p.batches; ++b) {
        if (PAIR) mma_ss_pair_x4(d_tmem, ad, ad + 2, ad + 4, ad + 6, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, 1u);
        else mma_ss_elect_x4(d_tmem, ad, ad + 2, ad + 4, ad + 6, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, 1u);
        maybe_commit(b);
      }
    }
    t[0] = clock64() - t0;
    if (PAIR) mma_commit_pair_both_elect(done);
    else mma_commit_elect(done);
    t[1] = t0;
  };

  // Pattern mode: `batches` steps of the block list.  No clock reads inside the loop.
  auto issue_pattern = [&](uint32_t done, uint32_t extra_bar, long long* t) {
    constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
    const uint64_t ad = desc64(smem_desc_lo(smem_base, 16), desc_hi);
    const uint64_t bd_k = desc64(smem_desc_lo(smem_base + kProbeABytes, 16), desc_hi);
    const uint64_t bd_n = desc64(smem_desc_lo(smem_base + kProbeABytes, 8192), desc_hi);
    const uint32_t a_tmem = tmem_base + 256;
    const uint32_t idesc64 = idesc_bf16_f32(128, 64, 0, 0);
    const uint32_t idesc128 = idesc_bf16_f32(128, 128, 0, p.b_mn);
    __syncwarp();
    const long long t0 = clock64();
    for (int step = 0; step < p.batches; ++step) {
      for (int i = 0; i < p.n_blocks; ++i) {
        const int n = p.blocks[i][0];
        const uint32_t d = tmem_base + static_cast<uint32_t>(p.blocks[i][1]);
        const uint32_t acc = p.blocks[i][2] ? 0u : 1u;
        const bool wide = n == 128;
        const uint32_t idesc = wide ? idesc128 : idesc64;
        const uint64_t bd = (wide && p.b_mn) ? bd_n : bd_k;
        const uint64_t bs = (wide && p.b_mn) ? 128 : 2;
        if (p.ts) mma_ts_elect_x4(d, a_tmem, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, acc);
        else mma_ss_elect_x4(d, ad, ad + 2, ad + 4, ad + 6, bd, bd + bs, bd + 2 * bs, bd + 3 * bs, idesc, acc);
        if (p.blocks[i][3]) mma_commit_elect(extra_bar);
      }
    }
    t[0] = clock64() - t0;
    mma_commit_elect(done);
    t[1] = t0;
  };

  if (warp == 0) {
    if (rank == 0) {
      // ---------------------------------------------------------------- issuer (whole warp, one elected lane)
      long long t[2];
      if (!PAIR && p.shape > 0) {
        __syncwarp();
        const long long t0 = clock64();
        const uint32_t ready = bg_bar(0), extra = bar_base + 8u * 5;   // nothing ever arrives on bg_bar(0) in this mode
        switch (p.shape) {
          case 1: issue_dq_like<1>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 2: issue_dq_like<2>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 3: issue_dq_like<3>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 4: issue_dq_like<4>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 5: issue_dq_like<5>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 7: issue_dq_like<7>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 8: issue_dq_like<8>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 9: issue_dq_like<9>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 10: issue_dq_like<10>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 11: issue_dq_like<11>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 12: issue_dq_like<12>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          case 13: issue_dq_like<13>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
          default: issue_dq_like<6>(tmem_base, smem_base, p.batches, ready, extra, ctx); break;
        }
        t[0] = clock64() - t0;
        mma_commit_elect(done_bar);
        t[1] = t0;
      } else if (!PAIR && p.n_blocks > 0) issue_pattern(done_bar, bar_base + 8u * 5, t);
      else issue_stream(tmem_base, done_bar, bar_base + 8u * 5, t);
      bool ok = mbar_wait_warp(done_bar, 0, ctx, kRoleMma, 1, 0);
      if (p.issuers == 2) ok = mbar_wait_warp(bar_base + 8u * 6, 0, ctx, kRoleMma, 3, 0) && ok;
      const long long t2 = clock64();
      *stop_flag = 1;
      if (lane == 0 && ok) {
        p.out[2 * blockIdx.x] = static_cast<unsigned long long>(t[0]);
        p.out[2 * blockIdx.x + 1] = static_cast<unsigned long long>(t2 - t[1]);
      }
    } else {
      // the peer only lends its shared and tensor memory; it waits for the same completion
      mbar_wait_warp(done_bar, 0, ctx, kRoleMma, 2, 0);
      *stop_flag = 1;
    }
  } else if (warp == 1 && p.issuers == 2) {
    // ------------------------------------------------------------------ second issuing warp (cta_group::1 only)
    if (!PAIR) {
      long long t[2];
      issue_stream(tmem_base + 128, bar_base + 8u * 6, bar_base + 8u * 7, t);
      mbar_wait_warp(bar_base + 8u * 6, 0, ctx, kRoleMma, 4, 0);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ background TMA loads
    if (p.bg_tma && lane == 0) {
      uint32_t issued = 0;
      for (; issued < 4; ++issued) {
        mbar_arrive_expect_tx(bg_bar(issued), 16384);
        tma_load_2d(smem_base + kProbeABytes + kProbeBBytes + issued * 16384, &tmap_bg, bg_bar(issued), 0,
                    static_cast<int>((blockIdx.x * 4 + issued) % 64) * 128);
      }
      uint32_t it = 0;
      bool ok = true;
      for (; ok && !*stop_flag && it < (1u << 20); ++it) {
        const int s = it & 3;
        ok = mbar_wait(bg_bar(s), (it >> 2) & 1, ctx, kRoleProducer, s, it);
        if (ok && !*stop_flag) {
          mbar_arrive_expect_tx(bg_bar(s), 16384);
          tma_load_2d(smem_base + kProbeABytes + kProbeBBytes + s * 16384, &tmap_bg, bg_bar(s), 0,
                      static_cast<int>((blockIdx.x * 4 + it) % 64) * 128);
          ++issued;
        }
      }
      // every copy issued must have landed before the CTA may exit: copy k completes phase k / 4 of barrier k % 4
      for (uint32_t back = 1; back <= 4; ++back) {
        const uint32_t k = issued - back;
        mbar_wait_quiet(bg_bar(k & 3), (k >> 2) & 1);
      }
    }
  } else if (warp >= 6) {
    // -------------------------------------------------------------------- background arithmetic
    if (p.bg_alu == 3) {
      // eight warps waiting on a barrier that never completes, the way compute warps wait for their input
      for (uint32_t it = 0; !*stop_flag && it < (1u << 22); ++it) mbar_try_wait(bg_bar(1), 0);
    } else if (p.bg_alu == 1 || (p.bg_alu == 2 && (warp & 3) != 0)) {   // 2: not on the issuing warp's scheduler
      float2 x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = make_float2(-0.001f * (threadIdx.x + i), -0.002f * (threadIdx.x + i));
      float2 acc = make_float2(0.f, 0.f);
      uint32_t packed = 0;
      for (uint32_t it = 0; !*stop_flag && it < (1u << 22); ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 y = __ffma2_rn(x[i], make_float2(1.0001f, 1.0001f), make_float2(-0.01f, -0.01f));
          float2 e;
          e.x = ex2_approx(y.x);
          e.y = ex2_approx(y.y);
          acc = __fadd2_rn(acc, e);
          packed ^= pack_bf16(e.x, e.y);
          x[i] = make_float2(y.x * 0.5f, y.y * 0.5f);
        }
      }
      if (acc.x + acc.y == 12345.f) p.sink[threadIdx.x] = acc.x + __uint_as_float(packed);
    }
  } else {
    // -------------------------------------------------------------------- background tensor-memory traffic
    if (p.bg_tmem == 1 || (p.bg_tmem == 2 && (warp & 3) != 0)) {
      const int quarter = warp & 3;
      // columns 384-511 (pattern and loop-shape modes, whose accumulators reach further: 448-511, two loads per round)
      const bool narrow = p.n_blocks > 0 || p.shape > 0;
      const uint32_t addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (narrow ? 448 : 384);
      const int n_ld = narrow ? 2 : 4;
      uint32_t r[32];
      for (uint32_t it = 0; !*stop_flag && it < (1u << 22); ++it) {
        // a softmax step's traffic: load 128 columns, store 64
#pragma unroll 1
        for (int c = 0; c < n_ld; ++c) {
          tmem_ld32(addr + c * 32, r);
          tmem_wait_ld();
        }
#pragma unroll 1
        for (int c = 0; c < 2; ++c) tmem_st32(addr + c * 32, r);
        tmem_wait_st();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  if (warp == 0) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace wir

using namespace wir::host;

// Runs the probe once on `device` and returns, through `clocks_out[0..1]`, the median over CTAs of
// (clocks until the last MMA was issued, clocks until all MMAs completed).  `n` in {64, 128, 256};
// pair = 1 uses cta_group::2 (256-row instructions over two SMs); b_mn = 1 reads B N-major; single = 1
// issues the MMAs one per instruction block; random_data = 1 fills the operands with random values;
// bg_alu = 1 adds eight warps of softmax-like arithmetic; commit_every = k > 0 commits after every k blocks.  `bg_buffer` is 64 x 128 x 64
// bf16 (1 MiB) of device memory for the background TMA loads (may be NULL when bg_tma = 0).
static int probe_impl(int n, int ts, int pair, int batches, int bg_tmem, int bg_tma, int b_mn, int single,
                      int random_data, int bg_alu, int commit_every, int issuers, const void* bg_buffer, int device,
                      double* clocks_out, int n_out, const int* blocks = nullptr, int n_blocks = 0, int shape = 0) {
  g_last_error[0] = 0;
  if (issuers != 1 && issuers != 2) return fail(WARPIR_EINVAL, "issuers must be 1 or 2");
  if (issuers == 2 && (pair || bg_tma || n > 128))
    return fail(WARPIR_EINVAL, "two issuing warps: cta_group::1, n <= 128 and no background TMA loads (its warp issues)");
  if (n != 64 && n != 128 && n != 256) return fail(WARPIR_EINVAL, "n must be 64, 128 or 256");
  if (batches < 1 || batches > 65536) return fail(WARPIR_EINVAL, "batches must be in [1, 65536]");
  if (bg_tma && bg_buffer == nullptr) return fail(WARPIR_EINVAL, "bg_tma needs a buffer");
  if (single && pair) return fail(WARPIR_EINVAL, "the one-by-one issue form exists for cta_group::1 only");
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  int grid = dev->sm_count;
  if (pair) grid &= ~1;

  CUtensorMap tm;
  memset(&tm, 0, sizeof tm);
  if (bg_tma) {
    const uint64_t dims[2] = {64, 64 * 128};
    const uint64_t strides[1] = {128};
    const uint32_t box[2] = {64, 128};
    if (int rc = make_tmap(&tm, bg_buffer, 2, dims, strides, box)) return rc;
  }
  unsigned long long* out = nullptr;
  WIR_CUDA(cudaMalloc(&out, sizeof(unsigned long long) * 2 * grid));
  WIR_CUDA(cudaMemset(out, 0, sizeof(unsigned long long) * 2 * grid));
  wir::ProbeParams p{n, ts, batches, bg_tmem, bg_tma, b_mn ? 1 : 0, single ? 1 : 0, random_data ? 1 : 0, bg_alu, commit_every, issuers, 0, {}, shape, nullptr, out, dev->status};
  p.sink = reinterpret_cast<float*>(out);   // never written (the guard in the kernel is never true)
  p.n_blocks = n_blocks;
  for (int i = 0; i < n_blocks; ++i)
    for (int j = 0; j < 4; ++j) p.blocks[i][j] = blocks[4 * i + j];
  cudaError_t e;
  if (pair) {
    auto kernel = wir::probe_mma_rate_kernel<true>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wir::kProbeSmem);
    if (e == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(grid);
      cfg.blockDim = dim3(wir::kProbeThreads);
      cfg.dynamicSmemBytes = wir::kProbeSmem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, kernel, tm, p);
    }
  } else {
    auto kernel = wir::probe_mma_rate_kernel<false>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wir::kProbeSmem);
    if (e == cudaSuccess) {
      kernel<<<grid, wir::kProbeThreads, wir::kProbeSmem>>>(tm, p);
      e = cudaGetLastError();
    }
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  unsigned long long* host = static_cast<unsigned long long*>(malloc(sizeof(unsigned long long) * 2 * grid));
  if (e == cudaSuccess) e = cudaMemcpy(host, out, sizeof(unsigned long long) * 2 * grid, cudaMemcpyDeviceToHost);
  cudaFree(out);
  if (e != cudaSuccess) {
    free(host);
    return fail(WARPIR_ECUDA, "probe: %s", cudaGetErrorString(e));
  }
  // median over the CTAs that measured (the leaders, for pairs)
  const int step = pair ? 2 : 1;
  const int cnt = grid / step;
  for (int which = 0; which < n_out; ++which) {
    double* v = static_cast<double*>(malloc(sizeof(double) * cnt));
    for (int i = 0; i < cnt; ++i) v[i] = static_cast<double>(host[2 * (i * step) + which]);
    for (int i = 1; i < cnt; ++i) {   // insertion sort: cnt <= 148
      const double x = v[i];
      int j = i - 1;
      for (; j >= 0 && v[j] > x; --j) v[j + 1] = v[j];
      v[j + 1] = x;
    }
    clocks_out[which] = v[cnt / 2];
    free(v);
  }
  free(host);
  int code = 0, detail = 0;
  return read_status_impl(device, nullptr, &code, &detail);
}

extern "C" int warpir_probe_mma_rate(int n, int ts, int pair, int batches, int bg_tmem, int bg_tma, int b_mn,
                                     int single, int random_data, int bg_alu, int commit_every,
                                     const void* bg_buffer, int device, double* clocks_out) {
  return probe_impl(n, ts, pair, batches, bg_tmem, bg_tma, b_mn, single, random_data, bg_alu, commit_every, 1,
                    bg_buffer, device, clocks_out, 2);
}

// The same run with `issuers` (1 or 2) warps issuing, each its own stream, accumulator and commits;
// clocks_out[1] then runs until BOTH streams completed.
extern "C" int warpir_probe_mma_rate_ex(int n, int ts, int pair, int batches, int bg_tmem, int bg_tma, int b_mn,
                                        int single, int random_data, int bg_alu, int commit_every, int issuers,
                                        const void* bg_buffer, int device, double* clocks_out) {
  return probe_impl(n, ts, pair, batches, bg_tmem, bg_tma, b_mn, single, random_data, bg_alu, commit_every, issuers,
                    bg_buffer, device, clocks_out, 2);
}

// Pattern mode: `steps` repetitions of a list of `n_blocks` (<= 16) instruction blocks, four ints each:
// {N (64 or 128), accumulator column (a multiple of 32; column + N <= 256, or 320 for a 128-wide one), first MMA
// overwrites (0/1), commit after the block (0/1)}; cta_group::1.  clocks_out[0..1]: clocks until the last MMA
// was issued / until all completed (median over SMs), for the whole run.
extern "C" int warpir_probe_mma_pattern(const int* blocks, int n_blocks, int steps, int ts, int b_mn, int bg_tmem,
                                        int bg_alu, int device, double* clocks_out) {
  g_last_error[0] = 0;
  if (blocks == nullptr || n_blocks < 1 || n_blocks > 16) return fail(WARPIR_EINVAL, "1 to 16 blocks");
  for (int i = 0; i < n_blocks; ++i) {
    const int n = blocks[4 * i], col = blocks[4 * i + 1];
    if (n != 64 && n != 128) return fail(WARPIR_EINVAL, "block %d: N must be 64 or 128", i);
    if (col < 0 || col % 32 != 0 || !(col + n <= 256 || (col == 320 && n == 128)))
      return fail(WARPIR_EINVAL, "block %d: accumulator column %d out of range", i, col);
  }
  return probe_impl(64, ts, 0, steps, bg_tmem, 0, b_mn, 0, 1, bg_alu, 0, 1, nullptr, device, clocks_out, 2, blocks, n_blocks);
}

// Loop-shape mode: `steps` steps of the attention backward's dQ issue loop written in shape 1..13 (see
// issue_dq_like); 768 clocks of tensor-core arithmetic per step.  clocks_out as above, for the whole run.
extern "C" int warpir_probe_issue_loop(int shape, int steps, int bg_tmem, int bg_alu, int device, double* clocks_out) {
  g_last_error[0] = 0;
  if (shape < 1 || shape > 13) return fail(WARPIR_EINVAL, "shape must be 1..13");
  return probe_impl(64, 1, 0, steps, bg_tmem, 0, 1, 0, 1, bg_alu, 0, 1, nullptr, device, clocks_out, 2, nullptr, 0, shape);
}

extern "C" const char* warpir_probe_last_error(void) { return g_last_error; }
