// Inline-PTX building blocks for the sm_100a kernels: mbarriers with bounded
// waits, TMA bulk-tensor copies, tensor-memory management, tcgen05 MMA issue,
// tensor-memory loads/stores and the fences that order them.
//
// No-hang rule: every wait in this file is a bounded poll.  A wait that runs
// out records an error code in the kernel's status words, raises the CTA-wide
// abort flag and returns false; callers leave their loops, the CTA drains its
// copies and MMAs (again with bounded waits), frees its tensor memory and
// returns.  Nothing traps and nothing spins forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wir {

// ---- status words written by the device ------------------------------------
// status[0] = error code (0 = ok), status[1] = linear CTA index,
// status[2] = (role << 16) | tag, status[3] = detail (stage / phase / iteration)
enum DeviceError : int {
  kDevOk = 0,
  kDevWaitTimeout = 1,   // an mbarrier wait ran out of polls
  kDevAborted = 2,       // left a loop because another role raised the abort flag
};

enum Role : int { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRoleSoftmax = 4, kRoleDrain = 5 };

// Time limit of one wait, in nanoseconds of %globaltimer.  Far longer than any
// legitimate wait in these kernels (whole launches take milliseconds) and short
// enough that a protocol bug surfaces as an error status, not as a hung GPU.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;
// Hard cap on polls in case the timer does not advance.
constexpr uint32_t kWaitPolls = 1u << 28;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Non-blocking probe (try_wait may suspend the thread for a while when the phase is still open).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

struct AbortCtx {
  volatile int* flag;   // CTA-wide abort flag in shared memory
  int* status;          // 4 status words in global memory
  uint64_t limit_ns = kWaitBudgetNs;   // how long one wait may take
};

__device__ __forceinline__ void report_error(const AbortCtx& ctx, int code, int role, int tag,
                                             int detail) {
  *ctx.flag = 1;
  if (atomicCAS(ctx.status, 0, code) == 0) {
    ctx.status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    ctx.status[2] = (role << 16) | (tag & 0xffff);
    ctx.status[3] = detail;
    __threadfence();
  }
}

// Bounded wait for the phase with parity `parity` of barrier `bar` to complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtx& ctx,
                                          int role, int tag, int detail) {
  if (mbar_test_wait(bar, parity)) return true;
  if (*ctx.flag) return false;      // the CTA is already giving up: do not start another wait
  uint64_t t0 = 0;
  for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((poll & 0x3f) == 0x3f) {
      if (*ctx.flag) return false;  // another role gave up: leave quietly
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > ctx.limit_ns) break;
    }
  }
  report_error(ctx, kDevWaitTimeout, role, tag, detail);
  return false;
}

// Bounded wait used only while draining after an abort: never reports.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity) {
  uint64_t t0 = 0;
  for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
    if (mbar_try_wait(bar, parity)) return;
    if ((poll & 0x3f) == 0x3f) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > (kWaitBudgetNs >> 3)) return;
    }
  }
}

// ---- TMA (cp.async.bulk.tensor; every copy targets the issuing CTA only) --------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor memory ------------------------------------------------------------
// Whole-warp operations.  `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- tcgen05.mma ----------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, tile base 1024-byte aligned.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) swizzle mode (2 = 128 B)
// K-major operand (K contiguous, one 128-byte row per M/N index): rows are grouped
// by eight, groups `sbo` bytes apart (1024 when rows are packed); LBO is unused.
// MN-major operand (M/N contiguous, 64 elements = 128 bytes per K index): eight K
// rows form a 1024-byte group, groups `sbo` bytes apart, and successive chunks of
// 64 M/N elements are `lbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The same descriptor as two 32-bit halves.  Only the low half depends on the address, and
// stepping through a tile only adds a constant to it, so a loop that issues many MMAs from
// one thread keeps `hi` in a register and spends one integer add per operand per MMA (a lone
// issuing thread executes dependent ALU instructions several clocks apart, so descriptor
// arithmetic is what bounds its MMA issue rate).
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3ffff) >> 4) | (((lbo_bytes >> 4) & 0x3fff) << 16);
}
__host__ __device__ constexpr uint32_t smem_desc_hi_sw128(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fff) | (1u << 14) | (2u << 29);
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   [4,6) D format (1 = f32)  [7,10) A format (1 = bf16)  [10,13) B format (1 = bf16)
//   [15] A major (0 = K)      [16] B major (0 = K, 1 = MN)
//   [17,23) N >> 3            [24,29) M >> 4
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same two instructions with the descriptors given as (low, high) halves.
__device__ __forceinline__ void mma_ss_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lh(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Warp-collective issue.  The whole (converged) warp runs the issuing loop, so barrier
// addresses, descriptors and tensor-memory addresses are warp-uniform values that the
// compiler can keep in uniform registers, which is what the MMA and commit instructions take;
// only the instruction itself is predicated on one elected lane.  Issuing from inside an
// `if (lane == 0)` region instead makes every operand a per-thread value that has to be
// moved to a uniform register before each MMA, and the issue rate of the lone thread (about
// 100 clocks per MMA) becomes the kernel's bottleneck.  elect.sync picks the same lane every
// time for a given mask, so MMAs and the commits that track them come from one thread.
__device__ __forceinline__ void mma_ss_elect(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                             uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b64 da, db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t.reg .b64 db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four MMAs into one accumulator from a single instruction block: one elect, then the four
// tcgen05.mma back to back with ready-made 64-bit descriptors.  Per MMA the issuing warp
// spends one instruction instead of an elect, two register-pair moves and a predicate set,
// which matters for narrow MMAs (N = 64 runs 32 clocks on the tensor core, less than the
// per-call overhead of the single-MMA helpers).  `accumulate` applies to the first MMA; the
// other three always accumulate.
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ void mma_ss_elect_x4(uint32_t d_tmem, uint64_t a0, uint64_t a1, uint64_t a2, uint64_t a3,
                                                uint64_t b0, uint64_t b1, uint64_t b2, uint64_t b3, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %10, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, t;\n\t}"
      ::"r"(d_tmem), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc),
        "r"(accumulate)
      : "memory");
}
// Same with the A operand in tensor memory at a_tmem, a_tmem + 8, + 16, + 24 (16 K-elements =
// 8 packed bf16 columns per MMA).
__device__ __forceinline__ void mma_ts_elect_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, uint64_t b1, uint64_t b2,
                                                uint64_t b3, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1, a2, a3;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %7, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "add.u32 a2, %1, 16;\n\t"
      "add.u32 a3, %1, 24;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %6, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %3, %6, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %4, %6, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %5, %6, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_elect(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_elect(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
      ::"r"(bar)
      : "memory");
}
// Warp-uniform bounded wait: every lane polls, the warp agrees on the outcome.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const AbortCtx& ctx, int role,
                                               int tag, int detail) {
  const bool ok = mbar_wait(bar, parity, ctx, role, tag, detail);
  return __all_sync(0xffffffffu, ok);
}

// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---- CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) ------------------------
// One MMA instruction of the pair's leader (cluster rank 0) computes a 256-row tile: rows
// 0-127 into the leader's tensor memory, rows 128-255 into the peer's, A from each CTA's own
// shared or tensor memory (same offsets in both), B split along N between the two CTAs'
// shared memories.  Nothing here names a cluster-wide TMA copy: every load lands in the
// shared memory of the CTA that issues it; only the barrier it signals may live in the leader.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of this CTA's shared address `addr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted on a barrier given by its
// shared::cluster address (the leader's, for operands a pair's MMA reads from both CTAs)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Four pair-MMAs (see mma_ss_elect_x4); issued by the leader only.
__device__ __forceinline__ void mma_ss_pair_x4(uint32_t d_tmem, uint64_t a0, uint64_t a1, uint64_t a2, uint64_t a3,
                                               uint64_t b0, uint64_t b1, uint64_t b2, uint64_t b3, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %10, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %5, %9, p;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %2, %6, %9, t;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %3, %7, %9, t;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %4, %8, %9, t;\n\t}"
      ::"r"(d_tmem), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc),
        "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_pair_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, uint64_t b1, uint64_t b2,
                                               uint64_t b3, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1, a2, a3;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %7, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "add.u32 a2, %1, 16;\n\t"
      "add.u32 a3, %1, 24;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %6, p;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [a1], %3, %6, t;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [a2], %4, %6, t;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [a3], %5, %6, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at shared::cluster address `bar_cluster` (in either CTA of the pair)
// once every pair-MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit_pair_elect(uint32_t bar_cluster) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar_cluster)
      : "memory");
}

// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once every
// pair-MMA issued so far by this thread has completed (a commit costs the issuing thread a few hundred
// clocks, so one multicast commit instead of one per CTA).
__device__ __forceinline__ void mma_commit_pair_both_elect(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t.reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar)
      : "memory");
}
// L2 eviction policies for TMA loads: an operand that the next waves of CTAs read again is worth keeping
// (evict_last), one that streams through once is not (evict_first).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted on the barrier at `bar_cluster`
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}

// ---- tensor memory <-> registers (shape 32x32b: lane = row, one column per register) ----
#define WIR_R4(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3])
#define WIR_R16(r, o) WIR_R4(r, o), WIR_R4(r, o + 4), WIR_R4(r, o + 8), WIR_R4(r, o + 12)
#define WIR_W4(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3])
#define WIR_W16(r, o) WIR_W4(r, o), WIR_W4(r, o + 4), WIR_W4(r, o + 8), WIR_W4(r, o + 12)

// 32 consecutive columns of this thread's lane into r[0..31]
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : WIR_R16(r, 0), WIR_R16(r, 16)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : WIR_R16(r, 0)
      : "r"(taddr)
      : "memory");
}
// r[0..31] into 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::WIR_W16(r, 0), WIR_W16(r, 16), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::WIR_W16(r, 0), "r"(taddr)
      : "memory");
}

// ---- optional event trace (debug builds only: -DWIR_TRACE) --------------------------------
// A traced thread of CTA (0,0,0) appends (event << 32 | index, clock64) pairs to its own
// region of a global buffer (plain stores, no round trip, so the perturbation is a few
// clocks per event).  Compiled out of the product library.
#ifdef WIR_TRACE
constexpr int kTraceRegion = 4096;   // entries per region
#define WIR_TRACE_DECL int wir_trace_n = 0
__device__ __forceinline__ void trace_event(unsigned long long* buf, int region, int& n, int ev, int idx) {
  if (buf == nullptr || blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0 || n >= kTraceRegion) return;
  unsigned long long* dst = buf + 2ull * (static_cast<unsigned long long>(region) * kTraceRegion + n);
  dst[0] = (static_cast<unsigned long long>(ev) << 32) | static_cast<unsigned int>(idx);
  dst[1] = clock64();
  ++n;
}
#define WIR_TRACE_EVENT(buf, region, ev, idx) trace_event(buf, region, wir_trace_n, ev, idx)
#else
#define WIR_TRACE_DECL ((void)0)
#define WIR_TRACE_EVENT(buf, region, ev, idx) ((void)0)
#endif

// ---- small numeric helpers -----------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two 2^x (x <= 0) on the FMA pipe instead of the exponential unit, with packed f32x2
// arithmetic: x = n + f with n the nearest integer (magic-constant rounding), 2^f by a cubic on
// [-0.5, 0.5] (relative error below 6e-4, far inside bf16's 4e-3), and n added into the
// exponent field.  The exponential unit retires 16 results per clock per SM, a quarter of what
// the tensor cores need at head dimension 128; moving a share of the exponentials here is
// what lets the two overlap.
__device__ __forceinline__ float2 ex2_fma2(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 r = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));     // 1.5 * 2^23: n in the low mantissa bits
  const float2 n = __fadd2_rn(r, make_float2(-12582912.f, -12582912.f));
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 q = __ffma2_rn(f, make_float2(0.0555041087f, 0.0555041087f), make_float2(0.2402265070f, 0.2402265070f));
  q = __ffma2_rn(q, f, make_float2(0.6931471806f, 0.6931471806f));
  q = __ffma2_rn(q, f, make_float2(1.f, 1.f));
  q.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(r.x) << 23));
  q.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(r.y) << 23));
  return q;
}

}  // namespace wir
