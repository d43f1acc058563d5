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

  if (warp == 0) {
    if (rank == 0) {
      // ---------------------------------------------------------------- issuer (whole warp, one elected lane)
      const int m = PAIR ? 256 : 128;
      const uint32_t idesc = idesc_bf16_f32(m, p.n, 0, p.b_mn);
      constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
      const uint64_t ad = desc64(smem_desc_lo(smem_base, 16), desc_hi);
      const uint64_t bd = desc64(smem_desc_lo(smem_base + kProbeABytes, p.b_mn ? 8192 : 16), desc_hi);
      // 16 K-elements further: 32 bytes along a K-major row, 16 rows (2048 bytes) of an N-major chunk
      const uint64_t bs = p.b_mn ? 128 : 2;
      const uint32_t d_tmem = tmem_base;          // accumulator: columns [0, n)
      const uint32_t a_tmem = tmem_base + 256;    // TS form: A as 32 packed columns
      __syncwarp();
      const long long t0 = clock64();
      const uint32_t extra_bar = bar_base + 8u * 5;
      auto maybe_commit = [&](int b) {
        if (p.commit_every > 0 && (b + 1) % p.commit_every == 0) {
          if (PAIR) mma_commit_pair_elect(mapa_shared(extra_bar, 0));
          else mma_commit_elect(extra_bar);
        }
      };
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
      const long long t1 = clock64();
      if (PAIR) mma_commit_pair_both_elect(done_bar);
      else mma_commit_elect(done_bar);
      const bool ok = mbar_wait_warp(done_bar, 0, ctx, kRoleMma, 1, 0);
      const long long t2 = clock64();
      *stop_flag = 1;
      if (lane == 0 && ok) {
        p.out[2 * blockIdx.x] = static_cast<unsigned long long>(t1 - t0);
        p.out[2 * blockIdx.x + 1] = static_cast<unsigned long long>(t2 - t0);
      }
    } else {
      // the peer only lends its shared and tensor memory; it waits for the same completion
      mbar_wait_warp(done_bar, 0, ctx, kRoleMma, 2, 0);
      *stop_flag = 1;
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
    if (p.bg_alu) {
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
    if (p.bg_tmem) {
      const int quarter = warp & 3;
      const uint32_t addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + 384;   // columns 384-511
      uint32_t r[32];
      for (uint32_t it = 0; !*stop_flag && it < (1u << 22); ++it) {
        // a softmax step's traffic: load 128 columns, store 64
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
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
extern "C" int warpir_probe_mma_rate(int n, int ts, int pair, int batches, int bg_tmem, int bg_tma, int b_mn,
                                     int single, int random_data, int bg_alu, int commit_every,
                                     const void* bg_buffer, int device, double* clocks_out) {
  g_last_error[0] = 0;
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
  wir::ProbeParams p{n, ts, batches, bg_tmem, bg_tma, b_mn ? 1 : 0, single ? 1 : 0, random_data ? 1 : 0, bg_alu ? 1 : 0, commit_every, nullptr, out, dev->status};
  p.sink = reinterpret_cast<float*>(out);   // never written (the guard in the kernel is never true)
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
  for (int which = 0; which < 2; ++which) {
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

extern "C" const char* warpir_probe_last_error(void) { return g_last_error; }
