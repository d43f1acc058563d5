// Host side of the GEMM and attention kernels: tile-shape choice, tensor maps and the
// launches themselves.  Included by the C-ABI library (capi.cu) and by the translation
// units that the lowering emits for a recognised GEMM / attention program, so both go
// through the same code.
#pragma once

#include "host_common.cuh"
#include "attn_bwd_sm100.cuh"
#include "attn_bwd_wide_sm100.cuh"
#include "attn_fwd_sm100.cuh"
#include "attn_fwd_wide_sm100.cuh"
#include "gemm_sm100.cuh"
#include "gemm_pair_sm100.cuh"

namespace wir {
namespace host {

// ------------------------------------------------------------------------ GEMM
using GemmLaunchFn = int (*)(const CUtensorMap&, const CUtensorMap&, const wir::GemmParams&, int, cudaStream_t);

template <int BN, int STAGES, bool B_MN, int MT = 1, int A_ROWS = wir::kGemmBM>
int launch_gemm_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const wir::GemmParams& p, int grid,
                    cudaStream_t stream) {
  auto kernel = wir::gemm_bf16_sm100<BN, STAGES, B_MN, MT, A_ROWS>;
  constexpr int smem = wir::GemmSmem<BN, STAGES, MT, A_ROWS>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  kernel<<<grid, wir::gemm_threads(MT), smem, stream>>>(ta, tb, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

// 256 x 256 tiles on CTA pairs (gemm_pair_sm100.cuh); `grid` counts CTAs (two per cluster).
template <int STAGES, bool B_MN>
int launch_gemm_pair_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const wir::GemmParams& p, int grid,
                         cudaStream_t stream) {
  auto kernel = wir::gemm_pair_sm100<STAGES, B_MN>;
  constexpr int smem = wir::GemmPairSmem<STAGES>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  kernel<<<grid, wir::kPairThreads, smem, stream>>>(ta, tb, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

struct GemmChoice {
  int block_n;
  int splits;
  bool stream_k = false;   // deal k-blocks, not tiles, out to the CTAs (few rows: HBM-bound on B)
  int mt = 1;   // CTA tile height in units of 128 rows
  int a_rows = 128;   // rows of A loaded per stage (fewer for problems with few rows)
  bool pair = false;  // the 256 x 256 tile on a CTA pair (cta_group::2) instead of one CTA
};

// One-off start-up offset between the two Q tiles' softmax warpgroups of the attention kernel,
// in SM clocks (WARPIR_ATTN_STAGGER overrides the default).
inline int env_attn_stagger() {
  static const int v = [] {
    const char* e = getenv("WARPIR_ATTN_STAGGER");
    const int c = e ? atoi(e) : 1000;
    return c < 0 ? 0 : (c > 100000 ? 100000 : c);   // the kernel spins for this long once: keep it bounded
  }();
  return v;
}

// Tuning override for experiments: WARPIR_SKINNY_BN=64|128|256 picks the tile width for problems
// with few rows (64: static tiles, no stream-K).
inline int env_skinny_bn() {
  static const int v = [] {
    const char* e = getenv("WARPIR_SKINNY_BN");
    return e ? atoi(e) : 0;
  }();
  return v;
}

// Tuning override for experiments: WARPIR_GEMM_PAIR=0|1 turns the CTA-pair kernel off / on wherever
// the 256 x 256 tile is chosen.
inline int env_gemm_pair() {
  static const int v = [] {
    const char* e = getenv("WARPIR_GEMM_PAIR");
    return e ? (atoi(e) != 0 ? 1 : 0) : -1;
  }();
  return v;
}

// Tuning override for experiments: WARPIR_GEMM_MT=1|2 forces the CTA tile height.
inline int env_gemm_mt() {
  static const int v = [] {
    const char* e = getenv("WARPIR_GEMM_MT");
    return e ? atoi(e) : 0;
  }();
  return v;
}

// Tuning overrides for experiments: WARPIR_GEMM_GROUP_M=<row-blocks per rasterisation band>,
// WARPIR_GEMM_KSERP=0|1 (every other tile of a CTA walks K backwards).
inline int env_gemm_group_m() {
  static const int v = [] {
    const char* e = getenv("WARPIR_GEMM_GROUP_M");
    const int g = e ? atoi(e) : 0;
    return g > 0 && g <= 4096 ? g : 0;
  }();
  return v;
}
inline int env_gemm_l2_hints() {
  static const int v = [] {
    const char* e = getenv("WARPIR_GEMM_L2_HINTS");
    return e ? (atoi(e) & 7) : -1;
  }();
  return v;
}
inline int env_gemm_kserp() {
  static const int v = [] {
    const char* e = getenv("WARPIR_GEMM_KSERP");
    return e ? (atoi(e) != 0 ? 1 : 0) : -1;
  }();
  return v;
}

// Tile width: the widest tile keeps the tensor core busiest per byte of shared-memory
// traffic, but the tile count must fill the SMs.  Score = fraction of SM-waves that do
// useful work x relative MMA efficiency of the tile width.
inline GemmChoice choose_gemm(int64_t M, int64_t N, int64_t K, int sms) {
  const int cands[3] = {256, 128, 64};
  const double eff[3] = {1.0, 0.65, 0.40};
  const int64_t tm = (M + wir::kGemmBM - 1) / wir::kGemmBM;
  double best = -1.0;
  GemmChoice c{256, 1};
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = tm * ((N + cands[i] - 1) / cands[i]);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double score = eff[i] * static_cast<double>(tiles) / static_cast<double>(waves * sms);
    if (score > best + 1e-9) {
      best = score;
      c.block_n = cands[i];
    }
  }
  // 256-row CTA tiles (two MMAs sharing B) when the k-loop is long enough to amortise the
  // un-overlapped epilogue and the tile count still fills the SMs as well as before.
  if (c.block_n == 256 && M >= 512 && K >= 2048) {
    const int64_t tn = (N + 255) / 256;
    const int64_t t1 = tm * tn, t2 = ((M + 255) / 256) * tn;
    const double e1 = static_cast<double>(t1) / static_cast<double>(((t1 + sms - 1) / sms) * sms);
    const double e2 = static_cast<double>(t2) / static_cast<double>(((t2 + sms - 1) / sms) * sms);
    if (e2 >= 0.97 * e1) c.mt = 2;
  }
  return c;
}

// Everything the launcher decides about a GEMM from its extents: tile width and height, the CTA pair,
// stream-K for problems with few rows.  `block_n` / `splits` != 0 are the caller's explicit choices,
// `n_dst` > 0 the fused all-gather, `fixed` a pinned instantiation (then only the K decomposition is
// left to decide).  passes/tile_planner.py states the same rules for tile programs; warpir_plan_gemm
// exposes this function so that the two can be checked against each other.
inline GemmChoice plan_gemm_choice(int64_t M, int64_t N, int64_t K, int sms, int block_n, int splits, int n_dst,
                                   bool fixed) {
  GemmChoice ch = choose_gemm(M, N, K, sms);
  if (block_n != 0) { ch.block_n = block_n; ch.mt = 1; }
  if (splits != 0) ch.splits = splits;
  // few rows: 64-wide tiles (many CTAs streaming B), only the existing rows of A are loaded and
  // the saved shared memory deepens the ring so more of B is in flight per SM
  // With splits left to the library the k-blocks are dealt out evenly over all SMs (stream-K)
  // and the tiles are wider, which makes the TMA boxes of B larger.
  if (!fixed && block_n == 0 && M <= 64 && N >= 64 * 64) {
    ch.block_n = 64;
    ch.mt = 1;
    ch.a_rows = (M <= 16) ? 16 : 64;
    const int want = n_dst > 0 ? 64 : (env_skinny_bn() ? env_skinny_bn() : 128);   // no shared tiles when gathering
    // Shared tiles cost a round trip of fp32 partial sums through L2, which grows with the row
    // count: above 32 rows the static 64-wide tiling wins unless it leaves many SMs idle.
    const int64_t tiles64 = (N + 63) / 64;
    const double static_fill = static_cast<double>(tiles64) /
                               static_cast<double>(((tiles64 + sms - 1) / sms) * sms);
    if (splits == 0 && (want == 128 || want == 256) && N % 4 == 0 && (M <= 32 || static_fill < 0.7)) {
      const int64_t tiles = (N + want - 1) / want;
      const int64_t units = tiles * ((K + wir::kGemmBK - 1) / wir::kGemmBK);
      if (tiles <= kSkMaxTiles && units >= 4 * sms) {
        ch.block_n = want;
        ch.stream_k = true;
        ch.splits = 1;
      }
    }
  }
  if (env_gemm_mt() == 1 && !fixed) ch.mt = 1;
  if (env_gemm_mt() == 2 && ch.block_n == 256 && !fixed) ch.mt = 2;
  if (ch.splits > 1 && !fixed) ch.mt = 1;
  // Gathering: the 128-row tile keeps two accumulators, so its epilogue (which now also feeds the
  // slower stores to the peers) runs under the next tile's MMAs; the 256-row tile's does not.
  if (n_dst > 0 && !fixed) ch.mt = 1;
  // the 256 x 256 tile runs on a CTA pair (needs an even number of SMs to pair up, which every sm_100 part has)
  ch.pair = (ch.mt == 2 && ch.block_n == 256 && !fixed && ch.splits <= 1 && !ch.stream_k && sms >= 2);
  if (env_gemm_pair() >= 0) ch.pair = ch.pair && env_gemm_pair() != 0;
  return ch;
}

// `fixed`: when not null, the instantiation to launch (with `block_n` its tile width,
// `fixed_mt` its tile height in units of 128 rows and `fixed_pair` whether it is the CTA-pair kernel); used by
// the translation units the lowering emits, which pin tile width and ring depth.
// `dsts` / `n_dst` (fused all-gather): instead of C, n_dst destinations for the finished tiles, each
// the start of this problem's rows in one GPU's copy of the full output (memory of this GPU or peer
// memory mapped into its address space).  K-splitting is off in that mode: a tile leaves the SM once.
inline int gemm_impl(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int b_layout, int block_n,
                     int splits, int device, void* cuda_stream, GemmLaunchFn fixed = nullptr, int fixed_mt = 1,
                     void* const* dsts = nullptr, int n_dst = 0, bool fixed_pair = false) {
  g_last_error[0] = 0;
  if (n_dst < 0 || n_dst > wir::GemmParams::kMaxDst || (n_dst > 0 && dsts == nullptr))
    return fail(WARPIR_EINVAL, "n_dst must be in [1, %d] with a destination array", wir::GemmParams::kMaxDst);
  if (n_dst > 0) {
    for (int d = 0; d < n_dst; ++d) {
      if (dsts[d] == nullptr) return fail(WARPIR_EINVAL, "destination %d is NULL", d);
      if (reinterpret_cast<uintptr_t>(dsts[d]) & 15) return fail(WARPIR_EALIGN, "destination %d is not 16-byte aligned", d);
      cudaPointerAttributes attr;
      if (cudaPointerGetAttributes(&attr, dsts[d]) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        return fail(WARPIR_EDEVICE, "destination %d is not device memory visible to this process", d);
      }
    }
    if (N % 8 != 0) return fail(WARPIR_ESHAPE, "N = %lld: the gathered output needs a row pitch that is a multiple of 16 bytes", (long long)N);
    C = dsts[0];
    splits = 1;
  }
  if (M < 0 || N < 0 || K < 0) return fail(WARPIR_EINVAL, "negative size");
  if (b_layout != 0 && b_layout != 1) return fail(WARPIR_EINVAL, "b_layout must be 0 or 1");
  if (block_n != 0 && block_n != 64 && block_n != 128 && block_n != 256)
    return fail(WARPIR_EINVAL, "block_n must be 0, 64, 128 or 256");
  if (splits < 0 || splits > 64) return fail(WARPIR_EINVAL, "splits must be in [0, 64]");
  if (M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2) return fail(WARPIR_ESHAPE, "size above 2^30");
  if (M == 0 || N == 0) return WARPIR_OK;
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  if (n_dst == 0)
    if (int rc = check_device_ptr(C, "C", device)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  if (K == 0) {
    for (int d = 0; d < (n_dst > 0 ? n_dst : 1); ++d)
      WIR_CUDA(cudaMemsetAsync(n_dst > 0 ? dsts[d] : C, 0, static_cast<size_t>(M) * N * 2, stream));
    return WARPIR_OK;
  }
  if (int rc = check_device_ptr(A, "A", device)) return rc;
  if (int rc = check_device_ptr(B, "B", device)) return rc;
  if (K % 8 != 0) return fail(WARPIR_ESHAPE, "K = %lld: the row pitch of A must be a multiple of 16 bytes (K %% 8 == 0)", (long long)K);
  if (b_layout == 0 && N % 8 != 0) return fail(WARPIR_ESHAPE, "N = %lld: with B stored [K,N] its row pitch must be a multiple of 16 bytes (N %% 8 == 0)", (long long)N);

  GemmChoice ch = plan_gemm_choice(M, N, K, dev->sm_count, block_n, splits, n_dst, fixed != nullptr);
  if (fixed != nullptr) {
    ch.mt = fixed_mt;
    ch.pair = fixed_pair;   // a pinned instantiation says which kernel it is
  }
  const int num_kb = static_cast<int>((K + wir::kGemmBK - 1) / wir::kGemmBK);
  if (ch.splits > num_kb) ch.splits = num_kb;
  if (ch.splits > 1 && N % 4 != 0) ch.splits = 1;  // the reduce pass works on groups of four columns

  wir::GemmParams p;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.ldc = p.N;
  const int tile_m = wir::kGemmBM * ch.mt;
  p.tiles_m = static_cast<int>((M + tile_m - 1) / tile_m);
  p.tiles_n = static_cast<int>((N + ch.block_n - 1) / ch.block_n);
  p.num_kb = num_kb;
  p.kb_per_split = (num_kb + ch.splits - 1) / ch.splits;
  p.splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  p.C = static_cast<__nv_bfloat16*>(C);
  p.partial = nullptr;
  p.status = dev->status;
  p.trace = g_trace;
  if (env_gemm_group_m()) p.group_m = env_gemm_group_m();
  if (env_gemm_kserp() >= 0 && !ch.stream_k) p.k_serpentine = env_gemm_kserp();
  if (env_gemm_l2_hints() >= 0) p.l2_hints = env_gemm_l2_hints();
  p.n_dst = n_dst;
  for (int d = 0; d < n_dst; ++d) p.dst[d] = static_cast<__nv_bfloat16*>(dsts[d]);

  int64_t work = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.splits;
  int grid = static_cast<int>(work < dev->sm_count ? work : dev->sm_count);
  if (ch.pair) grid = 2 * static_cast<int>(work < dev->sm_count / 2 ? work : dev->sm_count / 2);
  size_t sk_bytes = 0;
  if (ch.stream_k) {
    const int64_t units = static_cast<int64_t>(p.tiles_m) * p.tiles_n * num_kb;
    p.sk_units = static_cast<int>((units + dev->sm_count - 1) / dev->sm_count);
    grid = static_cast<int>((units + p.sk_units - 1) / p.sk_units);
    p.sk_max_seg = (num_kb + p.sk_units - 2) / p.sk_units + 1;
    p.sk_rows = static_cast<int>(M < wir::kGemmBM ? M : wir::kGemmBM);
    sk_bytes = static_cast<size_t>(p.tiles_m) * p.tiles_n * p.sk_max_seg * p.sk_rows * ch.block_n * sizeof(float);
  }

  if (p.splits > 1 || ch.stream_k) {
    const size_t need = ch.stream_k ? sk_bytes : static_cast<size_t>(p.splits) * M * N * sizeof(float);
    DeviceState::Scratch* sc = nullptr;
    if (int rc = stream_scratch(dev, stream, need, &sc)) return rc;
    p.partial = sc->partial;
    p.sk_counters = sc->counters;
  }

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {wir::kGemmBK, static_cast<uint32_t>(ch.pair ? wir::kPairRows : (ch.a_rows < 128 ? ch.a_rows : tile_m))};
    if (int rc = make_tmap(&ta, A, 2, dims, strides, box)) return rc;
  }
  if (b_layout == 1) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {wir::kGemmBK, static_cast<uint32_t>(ch.pair ? wir::kPairRows : ch.block_n)};
    if (int rc = make_tmap(&tb, B, 2, dims, strides, box)) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, wir::kGemmBK};
    if (int rc = make_tmap(&tb, B, 2, dims, strides, box)) return rc;
  }

  int rc;
  const bool mn = (b_layout == 0);
  if (fixed != nullptr) rc = fixed(ta, tb, p, grid, stream);
  else if (ch.pair) rc = mn ? launch_gemm_pair_cfg<6, true>(ta, tb, p, grid, stream) : launch_gemm_pair_cfg<6, false>(ta, tb, p, grid, stream);
  else if (ch.stream_k && ch.block_n == 128 && ch.a_rows == 16) rc = mn ? launch_gemm_cfg<128, 10, true, 1, 16>(ta, tb, p, grid, stream) : launch_gemm_cfg<128, 10, false, 1, 16>(ta, tb, p, grid, stream);
  else if (ch.stream_k && ch.block_n == 128) rc = mn ? launch_gemm_cfg<128, 8, true, 1, 64>(ta, tb, p, grid, stream) : launch_gemm_cfg<128, 8, false, 1, 64>(ta, tb, p, grid, stream);
  else if (ch.stream_k && ch.a_rows == 16) rc = mn ? launch_gemm_cfg<256, 6, true, 1, 16>(ta, tb, p, grid, stream) : launch_gemm_cfg<256, 6, false, 1, 16>(ta, tb, p, grid, stream);
  else if (ch.stream_k) rc = mn ? launch_gemm_cfg<256, 5, true, 1, 64>(ta, tb, p, grid, stream) : launch_gemm_cfg<256, 5, false, 1, 64>(ta, tb, p, grid, stream);
  else if (ch.a_rows == 16) rc = mn ? launch_gemm_cfg<64, 19, true, 1, 16>(ta, tb, p, grid, stream) : launch_gemm_cfg<64, 19, false, 1, 16>(ta, tb, p, grid, stream);
  else if (ch.a_rows == 64) rc = mn ? launch_gemm_cfg<64, 12, true, 1, 64>(ta, tb, p, grid, stream) : launch_gemm_cfg<64, 12, false, 1, 64>(ta, tb, p, grid, stream);
  else if (ch.mt == 2) rc = mn ? launch_gemm_cfg<256, 3, true, 2>(ta, tb, p, grid, stream) : launch_gemm_cfg<256, 3, false, 2>(ta, tb, p, grid, stream);
  else switch (ch.block_n) {
    case 256: rc = mn ? launch_gemm_cfg<256, 4, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<256, 4, false>(ta, tb, p, grid, stream); break;
    case 128: rc = mn ? launch_gemm_cfg<128, 6, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<128, 6, false>(ta, tb, p, grid, stream); break;
    default:  rc = mn ? launch_gemm_cfg<64, 8, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<64, 8, false>(ta, tb, p, grid, stream); break;
  }
  if (rc) return rc;
  if (p.splits > 1) {
    const size_t total4 = (static_cast<size_t>(M) * N) >> 2;
    int blocks = static_cast<int>((total4 + 255) / 256);
    if (blocks > dev->sm_count * 8) blocks = dev->sm_count * 8;
    wir::splitk_reduce_bf16<<<blocks, 256, 0, stream>>>(p.partial, p.C, p.M, p.N, p.ldc, p.splits);
    WIR_CUDA(cudaGetLastError());
  }
  return WARPIR_OK;
}

// ------------------------------------------------------------------------ attention
template <int D, bool CAUSAL>
int launch_attn_cfg(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const wir::AttnParams& p,
                    cudaStream_t stream) {
  auto kernel = wir::attn_fwd_sm100<D, CAUSAL>;
  constexpr int smem = wir::AttnSmem<D>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  const int pairs = (p.S + 2 * wir::kAttnBQ - 1) / (2 * wir::kAttnBQ);
  dim3 grid(pairs, p.H, p.B);
  kernel<<<grid, wir::kAttnThreads, smem, stream>>>(tq, tk, tv, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

// 128-key blocks, two Q tiles taking turns on the tensor core (attn_fwd_wide_sm100.cuh).
template <int D, bool CAUSAL>
int launch_attn_wide_cfg(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const wir::AttnParams& p,
                         cudaStream_t stream) {
  auto kernel = wir::attn_fwd_wide_sm100<D, CAUSAL>;
  constexpr int smem = wir::AttnWideSmem<D>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  const int pairs = (p.S + 2 * wir::kAttnBQ - 1) / (2 * wir::kAttnBQ);
  dim3 grid(pairs, p.H, p.B);
  kernel<<<grid, wir::kWideThreads, smem, stream>>>(tq, tk, tv, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

// WARPIR_ATTN_WIDE=0|1 overrides the choice between the 64-key and the 128-key forward (read once per process).
inline int env_attn_wide() {
  static const int v = [] {
    const char* e = getenv("WARPIR_ATTN_WIDE");
    return e ? (atoi(e) != 0 ? 1 : 0) : -1;
  }();
  return v;
}

inline int attn_impl(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B, int64_t Hq,
                     int64_t Hkv, int64_t S, int64_t D, float softmax_scale, int causal, int device,
                     void* cuda_stream, int variant = 0) {
  g_last_error[0] = 0;
  if (B < 0 || Hq < 0 || Hkv < 0 || S < 0) return fail(WARPIR_EINVAL, "negative size");
  if (D != 64 && D != 128) return fail(WARPIR_ESHAPE, "D = %lld: head dimension must be 64 or 128", (long long)D);
  if (variant != 0 && variant != 1 && variant != 4)
    return fail(WARPIR_EINVAL, "variant must be 0 (choose), 1 (64-key blocks) or 4 (128-key blocks)");
  if (B == 0 || Hq == 0 || S == 0) return WARPIR_OK;
  if (Hkv <= 0 || Hq % Hkv != 0) return fail(WARPIR_ESHAPE, "Hq = %lld must be a positive multiple of Hkv = %lld", (long long)Hq, (long long)Hkv);
  if (!(softmax_scale > 0.f) || !std::isfinite(softmax_scale)) return fail(WARPIR_EINVAL, "softmax_scale must be positive and finite");
  if (B > 65535 || Hq > 65535) return fail(WARPIR_ESHAPE, "B and Hq must be at most 65535");
  if (S > (1 << 24) || B * Hq * S > INT32_MAX) return fail(WARPIR_ESHAPE, "sequence too long");
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  if (int rc = check_device_ptr(Q, "Q", device)) return rc;
  if (int rc = check_device_ptr(K, "K", device)) return rc;
  if (int rc = check_device_ptr(V, "V", device)) return rc;
  if (int rc = check_device_ptr(O, "O", device)) return rc;
  if (LSE != nullptr)
    if (int rc = check_device_ptr(LSE, "LSE", device)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));

  CUtensorMap tq, tk, tv;
  const uint32_t box[3] = {64, wir::kAttnBQ, 1};       // one 128-row Q tile chunk
  const uint32_t box_kv[3] = {64, wir::kAttnBKV, 1};   // one K/V tile chunk
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(B * Hq)};
    const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(S) * D * 2};
    if (int rc = make_tmap(&tq, Q, 3, dims, strides, box)) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(B * Hkv)};
    const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(S) * D * 2};
    if (int rc = make_tmap(&tk, K, 3, dims, strides, box_kv)) return rc;
    if (int rc = make_tmap(&tv, V, 3, dims, strides, box_kv)) return rc;
  }
  wir::AttnParams p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(Hq);
  p.Hkv = static_cast<int>(Hkv);
  p.S = static_cast<int>(S);
  p.D = static_cast<int>(D);
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.O = static_cast<__nv_bfloat16*>(O);
  p.LSE = LSE;
  p.status = dev->status;
  p.trace = g_trace;
  p.stagger_clocks = env_attn_stagger();
  // Measured (sustained TFLOP/s, 128-key kernel vs 64-key kernel): without a causal mask 1077 vs 1077 at head
  // dimension 128 and 706 vs 659 at 64; with one 1005 vs 1044 at 128 (the tiles of a CTA end a block apart and
  // a 128-key diagonal block is masked whole) and 660 vs 644 at 64.
  bool wide = !causal || D == 64;
  if (env_attn_wide() >= 0) wide = env_attn_wide() != 0;
  if (variant != 0) wide = (variant == 4);
  if (wide) {
    CUtensorMap tk128, tv128;   // K and V in tiles of 128 keys
    const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(B * Hkv)};
    const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(S) * D * 2};
    if (int rc = make_tmap(&tk128, K, 3, dims, strides, box)) return rc;
    if (int rc = make_tmap(&tv128, V, 3, dims, strides, box)) return rc;
    if (D == 128) return causal ? launch_attn_wide_cfg<128, true>(tq, tk128, tv128, p, stream) : launch_attn_wide_cfg<128, false>(tq, tk128, tv128, p, stream);
    return causal ? launch_attn_wide_cfg<64, true>(tq, tk128, tv128, p, stream) : launch_attn_wide_cfg<64, false>(tq, tk128, tv128, p, stream);
  }
  if (D == 128) return causal ? launch_attn_cfg<128, true>(tq, tk, tv, p, stream) : launch_attn_cfg<128, false>(tq, tk, tv, p, stream);
  return causal ? launch_attn_cfg<64, true>(tq, tk, tv, p, stream) : launch_attn_cfg<64, false>(tq, tk, tv, p, stream);
}

// ------------------------------------------------------------------------ attention backward
template <int D, bool CAUSAL, bool DKV>
int launch_attn_bwd_cfg(const CUtensorMap& x0, const CUtensorMap& x1, const CUtensorMap& y0, const CUtensorMap& y1,
                        const wir::AttnBwdParams& p, cudaStream_t stream) {
  auto kernel = wir::attn_bwd_sm100<D, CAUSAL, DKV>;
  constexpr int smem = wir::AttnBwdSmem<D, DKV>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  dim3 grid((p.S + wir::kBwdBX - 1) / wir::kBwdBX, DKV ? p.Hkv : p.H, p.B);
  kernel<<<grid, wir::kBwdThreads, smem, stream>>>(x0, x1, y0, y1, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

template <int D, bool CAUSAL, bool DKV>
int launch_attn_bwd_wide_cfg(const CUtensorMap& x0, const CUtensorMap& x1, const CUtensorMap& y0, const CUtensorMap& y1,
                             const wir::AttnBwdParams& p, cudaStream_t stream) {
  auto kernel = wir::attn_bwd_wide_sm100<D, CAUSAL, DKV>;
  constexpr int smem = wir::AttnBwdWideSmem<D, DKV>::kDynamicBytes;
  static_assert(smem <= 232448, "shared memory limit per CTA");
  static_assert(smem > 116 * 1024, "one CTA per SM is what keeps the tensor-memory allocation from blocking");
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  dim3 grid((p.S + wir::kBw2Rows - 1) / wir::kBw2Rows, DKV ? p.Hkv : p.H, p.B);
  kernel<<<grid, wir::kBwdThreads, smem, stream>>>(x0, x1, y0, y1, p);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

// Tuning override for experiments: WARPIR_ATTN_BWD_ROWS=64|128 picks the backward kernel by the rows it streams per step.
inline int env_attn_bwd_rows() {
  static const int v = [] {
    const char* e = getenv("WARPIR_ATTN_BWD_ROWS");
    return e ? atoi(e) : 0;
  }();
  return v;
}

inline int attn_bwd_impl(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* LSE,
                         float* dQ, float* dK, float* dV, float* delta, int64_t B, int64_t Hq, int64_t Hkv, int64_t S,
                         int64_t D, float softmax_scale, int causal, int device, void* cuda_stream) {
  g_last_error[0] = 0;
  if (B < 0 || Hq < 0 || Hkv < 0 || S < 0) return fail(WARPIR_EINVAL, "negative size");
  if (D != 64 && D != 128) return fail(WARPIR_ESHAPE, "D = %lld: head dimension must be 64 or 128", (long long)D);
  if (B == 0 || Hq == 0 || S == 0) return WARPIR_OK;
  if (Hkv <= 0 || Hq % Hkv != 0) return fail(WARPIR_ESHAPE, "Hq = %lld must be a positive multiple of Hkv = %lld", (long long)Hq, (long long)Hkv);
  if (!(softmax_scale > 0.f) || !std::isfinite(softmax_scale)) return fail(WARPIR_EINVAL, "softmax_scale must be positive and finite");
  if (B > 65535 || Hq > 65535) return fail(WARPIR_ESHAPE, "B and Hq must be at most 65535");
  if (S > (1 << 24) || B * Hq * S > INT32_MAX) return fail(WARPIR_ESHAPE, "sequence too long");
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  const void* ptrs[10] = {Q, K, V, O, dO, LSE, dQ, dK, dV, delta};
  const char* names[10] = {"Q", "K", "V", "O", "dO", "LSE", "dQ", "dK", "dV", "delta"};
  for (int i = 0; i < 10; ++i)
    if (int rc = check_device_ptr(ptrs[i], names[i], device)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));

  // every bf16 operand is read both as resident 128-row tiles and as streamed 64-row tiles
  auto maps = [&](const void* base, int64_t planes, CUtensorMap* big, CUtensorMap* small) -> int {
    const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(planes)};
    const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(S) * D * 2};
    const uint32_t box_x[3] = {64, wir::kBwdBX, 1}, box_y[3] = {64, wir::kBwdBY, 1};
    if (int rc = make_tmap(big, base, 3, dims, strides, box_x)) return rc;
    return make_tmap(small, base, 3, dims, strides, box_y);
  };
  CUtensorMap q_x, q_y, k_x, k_y, v_x, v_y, g_x, g_y;
  if (int rc = maps(Q, B * Hq, &q_x, &q_y)) return rc;
  if (int rc = maps(dO, B * Hq, &g_x, &g_y)) return rc;
  if (int rc = maps(K, B * Hkv, &k_x, &k_y)) return rc;
  if (int rc = maps(V, B * Hkv, &v_x, &v_y)) return rc;

  wir::AttnBwdParams p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(Hq);
  p.Hkv = static_cast<int>(Hkv);
  p.S = static_cast<int>(S);
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.Q = static_cast<const __nv_bfloat16*>(Q);
  p.O = static_cast<const __nv_bfloat16*>(O);
  p.dO = static_cast<const __nv_bfloat16*>(dO);
  p.LSE = LSE;
  p.delta = delta;
  p.status = dev->status;
  p.trace = g_trace;
  const bool c = causal != 0;
  int rc;
  const bool wide = env_attn_bwd_rows() ? env_attn_bwd_rows() == 128 : true;
  if (wide) {
    // steps of 128 streamed rows: every operand is read as 128-row tiles, resident or streamed
    {
      // delta = rowsum(dO * O) first, in a small kernel of its own (one pass over O and dO)
      const long long rows = static_cast<long long>(B) * Hq * S;
      const int rows_per_block = 8 * (32 / static_cast<int>(D / 8));
      long long blocks = (rows + rows_per_block - 1) / rows_per_block;
      if (blocks > static_cast<long long>(dev->sm_count) * 16) blocks = static_cast<long long>(dev->sm_count) * 16;
      if (D == 128) wir::attn_bwd_delta<128><<<static_cast<int>(blocks), 256, 0, stream>>>(p.O, p.dO, delta, rows);
      else wir::attn_bwd_delta<64><<<static_cast<int>(blocks), 256, 0, stream>>>(p.O, p.dO, delta, rows);
      WIR_CUDA(cudaGetLastError());
    }
    p.out0 = dQ;
    p.out1 = nullptr;
    if (D == 128) rc = c ? launch_attn_bwd_wide_cfg<128, true, false>(q_x, g_x, k_x, v_x, p, stream) : launch_attn_bwd_wide_cfg<128, false, false>(q_x, g_x, k_x, v_x, p, stream);
    else rc = c ? launch_attn_bwd_wide_cfg<64, true, false>(q_x, g_x, k_x, v_x, p, stream) : launch_attn_bwd_wide_cfg<64, false, false>(q_x, g_x, k_x, v_x, p, stream);
    if (rc) return rc;
#if defined(WIR_TRACE) || defined(WIR_BWD_ABLATE)
    if (getenv("WARPIR_BWD_DQ_ONLY")) return rc;   // debug and measurement builds: the first launch alone
#endif
    p.out0 = dV;
    p.out1 = dK;
    if (D == 128) rc = c ? launch_attn_bwd_wide_cfg<128, true, true>(k_x, v_x, q_x, g_x, p, stream) : launch_attn_bwd_wide_cfg<128, false, true>(k_x, v_x, q_x, g_x, p, stream);
    else rc = c ? launch_attn_bwd_wide_cfg<64, true, true>(k_x, v_x, q_x, g_x, p, stream) : launch_attn_bwd_wide_cfg<64, false, true>(k_x, v_x, q_x, g_x, p, stream);
    return rc;
  }
  // 1: dQ (and delta) per Q tile, streaming K and V
  p.out0 = dQ;
  p.out1 = nullptr;
  if (D == 128) rc = c ? launch_attn_bwd_cfg<128, true, false>(q_x, g_x, k_y, v_y, p, stream) : launch_attn_bwd_cfg<128, false, false>(q_x, g_x, k_y, v_y, p, stream);
  else rc = c ? launch_attn_bwd_cfg<64, true, false>(q_x, g_x, k_y, v_y, p, stream) : launch_attn_bwd_cfg<64, false, false>(q_x, g_x, k_y, v_y, p, stream);
  if (rc) return rc;
#if defined(WIR_TRACE) || defined(WIR_BWD_ABLATE)
  if (getenv("WARPIR_BWD_DQ_ONLY")) return rc;   // debug and measurement builds: the first launch alone
#endif
  // 2: dV and dK per K/V tile, streaming Q and dO of the head group
  p.out0 = dV;
  p.out1 = dK;
  if (D == 128) rc = c ? launch_attn_bwd_cfg<128, true, true>(k_x, v_x, q_y, g_y, p, stream) : launch_attn_bwd_cfg<128, false, true>(k_x, v_x, q_y, g_y, p, stream);
  else rc = c ? launch_attn_bwd_cfg<64, true, true>(k_x, v_x, q_y, g_y, p, stream) : launch_attn_bwd_cfg<64, false, true>(k_x, v_x, q_y, g_y, p, stream);
  return rc;
}

// Self-test of the bounded-wait machinery: one CTA waits, with a limit of `limit_ns`, on an
// mbarrier that nothing ever arrives on.  The wait runs out, the kernel records the error in the
// device's status words exactly as the GEMM / attention kernels would, and returns normally.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = wir::smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    wir::mbar_init(bar_addr, 1);
    wir::fence_mbar_init();
  }
  __syncthreads();
  wir::AbortCtx ctx{&abort_flag, status, limit_ns};
  // every thread waits: the first to give up raises the flag, the others then leave quietly
  wir::mbar_wait(bar_addr, 0, ctx, wir::kRoleDrain, /*tag=*/77, /*detail=*/static_cast<int>(threadIdx.x));
  __syncthreads();
}

inline int selftest_bounded_wait_impl(int device, void* cuda_stream, int64_t limit_ns) {
  g_last_error[0] = 0;
  if (limit_ns <= 0 || limit_ns > 1000000000ll) return fail(WARPIR_EINVAL, "limit_ns must be in (0, 1e9]");
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      dev->status, static_cast<unsigned long long>(limit_ns));
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}

}  // namespace host
}  // namespace wir
