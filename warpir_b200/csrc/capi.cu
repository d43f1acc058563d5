// C-ABI entry points (see include/warpir_b200.h).  The work is in launch.cuh.
#include <dlfcn.h>

#include "launch.cuh"

using namespace wir::host;

extern "C" {

int warpir_abi_version(void) { return WARPIR_ABI_VERSION; }

const char* warpir_strerror(int code) {
  switch (code) {
    case WARPIR_OK: return "ok";
    case WARPIR_EINVAL: return "invalid argument";
    case WARPIR_EALIGN: return "pointer or pitch not 16-byte aligned";
    case WARPIR_ESHAPE: return "unsupported size";
    case WARPIR_ECUDA: return "CUDA runtime error";
    case WARPIR_EDRIVER: return "tensor-map encode unavailable or failed";
    case WARPIR_EKERNEL: return "kernel reported an error (bounded wait ran out)";
    case WARPIR_EDEVICE: return "wrong device or not device memory";
    case WARPIR_ENOMEM: return "scratch allocation failed";
    default: return "unknown error code";
  }
}

const char* warpir_last_error(void) { return g_last_error; }

int warpir_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int b_layout,
                     int device, void* cuda_stream) {
  return gemm_impl(A, B, C, M, N, K, b_layout, 0, 0, device, cuda_stream);
}

int warpir_gemm_bf16_ex(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int b_layout,
                        int block_n, int splits, int device, void* cuda_stream) {
  return gemm_impl(A, B, C, M, N, K, b_layout, block_n, splits, device, cuda_stream);
}

int warpir_gemm_bf16_allgather(const void* A, const void* B, void* const* C_dst, int n_dst, int64_t M, int64_t N,
                               int64_t K, int b_layout, int device, void* cuda_stream) {
  if (n_dst < 1) {
    g_last_error[0] = 0;
    return fail(WARPIR_EINVAL, "n_dst must be at least 1");
  }
  return gemm_impl(A, B, nullptr, M, N, K, b_layout, 0, 1, device, cuda_stream, nullptr, 1, C_dst, n_dst);
}

int warpir_attn_fwd_bf16(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B, int64_t Hq,
                         int64_t Hkv, int64_t S, int64_t D, float softmax_scale, int causal, int device,
                         void* cuda_stream) {
  return attn_impl(Q, K, V, O, LSE, B, Hq, Hkv, S, D, softmax_scale, causal, device, cuda_stream);
}

int warpir_attn_fwd_bf16_ex(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B, int64_t Hq,
                            int64_t Hkv, int64_t S, int64_t D, float softmax_scale, int causal, int variant,
                            int device, void* cuda_stream) {
  return attn_impl(Q, K, V, O, LSE, B, Hq, Hkv, S, D, softmax_scale, causal, device, cuda_stream, variant);
}

int warpir_attn_bwd_bf16(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* LSE,
                         float* dQ, float* dK, float* dV, float* delta_ws, int64_t B, int64_t Hq, int64_t Hkv,
                         int64_t S, int64_t D, float softmax_scale, int causal, int device, void* cuda_stream) {
  return attn_bwd_impl(Q, K, V, O, dO, LSE, dQ, dK, dV, delta_ws, B, Hq, Hkv, S, D, softmax_scale, causal, device,
                       cuda_stream);
}

int warpir_launch_generated(void* module_handle, const char* kernel_name, const void* const* tensor_ptrs,
                            const int64_t* dims, int n_tensors, const int64_t* scalars, int n_scalars, int device,
                            void* cuda_stream) {
  g_last_error[0] = 0;
  if (module_handle == nullptr || kernel_name == nullptr) return fail(WARPIR_EINVAL, "module handle or kernel name is NULL");
  if (n_tensors < 0 || n_scalars < 0 || (n_tensors > 0 && (tensor_ptrs == nullptr || dims == nullptr)))
    return fail(WARPIR_EINVAL, "tensor arrays missing");
  char symbol[256];
  const int len = snprintf(symbol, sizeof symbol, "%s_launch", kernel_name);
  if (len < 0 || len >= static_cast<int>(sizeof symbol)) return fail(WARPIR_EINVAL, "kernel name too long");
  using LaunchFn = int (*)(const void* const*, const int64_t*, const int64_t*, int, void*);
  dlerror();
  LaunchFn fn = reinterpret_cast<LaunchFn>(dlsym(module_handle, symbol));
  if (fn == nullptr) return fail(WARPIR_EINVAL, "%s not found in the module: %s", symbol, dlerror());
  // emitted launchers read a fixed number of entries; hand them zero-padded copies so that a short
  // caller array can never be over-read (one optional trailing tensor, four trailing scalars)
  constexpr int kMaxTensors = 16, kMaxScalars = 16;
  if (n_tensors >= kMaxTensors || n_scalars > kMaxScalars - 4) return fail(WARPIR_EINVAL, "too many tensors or scalars");
  const void* t[kMaxTensors] = {};
  int64_t d[4 * kMaxTensors] = {};
  int64_t sc[kMaxScalars] = {};
  for (int i = 0; i < n_tensors; ++i) {
    t[i] = tensor_ptrs[i];
    for (int k = 0; k < 4; ++k) d[4 * i + k] = dims[4 * i + k];
  }
  for (int i = 0; i < n_scalars; ++i) sc[i] = scalars[i];
  const int rc = fn(t, d, sc, device, cuda_stream);
  if (rc != WARPIR_OK) {
    // the text of the failure lives in the module's own copy of the error buffer
    snprintf(symbol, sizeof symbol, "%s_last_error", kernel_name);
    using ErrFn = const char* (*)(void);
    ErrFn err = reinterpret_cast<ErrFn>(dlsym(module_handle, symbol));
    return fail(rc, "%s", err ? err() : "launch failed");
  }
  return rc;
}

int warpir_read_status(int device, void* cuda_stream, int* code, int* detail) {
  return read_status_impl(device, cuda_stream, code, detail);
}

int warpir_plan_gemm(int64_t M, int64_t N, int64_t K, int sms, int* block_m, int* block_n, int* cta_group,
                     int* stream_k, int* a_rows) {
  g_last_error[0] = 0;
  if (M <= 0 || N <= 0 || K <= 0 || sms <= 0) return fail(WARPIR_EINVAL, "sizes and the SM count must be positive");
  const GemmChoice ch = plan_gemm_choice(M, N, K, sms, /*block_n=*/0, /*splits=*/0, /*n_dst=*/0, /*fixed=*/false);
  if (block_m) *block_m = 128 * ch.mt;
  if (block_n) *block_n = ch.block_n;
  if (cta_group) *cta_group = ch.pair ? 2 : 1;
  if (stream_k) *stream_k = ch.stream_k ? 1 : 0;
  if (a_rows) *a_rows = ch.a_rows;
  return WARPIR_OK;
}

}  // extern "C"

extern "C" int warpir_selftest_bounded_wait(int device, void* cuda_stream, int64_t limit_ns) {
  return selftest_bounded_wait_impl(device, cuda_stream, limit_ns);
}

#ifdef WIR_TRACE
// Debug builds only: hands the kernels a device buffer for their event trace.
extern "C" void warpir_debug_set_trace(void* device_buffer) {
  g_trace = static_cast<unsigned long long*>(device_buffer);
}
#endif

// ------------------------------------------------------------------------------------------
// Split-K GEMM without any allocation (see include/warpir_b200.h).
//
// For hosts that own all device memory themselves or cannot afford the implicit
// synchronisation of cudaMalloc/cudaFree: the fp32 partial sums of the K-splits and the
// kernel status words live in the array below, which is part of the library image, so
// each GPU that loads the library holds it (16 MiB + 256 B) until the process exits.
//
// `g_noalloc_scratch` is a DEVICE symbol.  In host code its name is only a host-side
// stand-in: passing `g_noalloc_scratch` itself to a kernel would hand the kernel a host
// address.  The device address is looked up once per device, with that device current,
// by cudaGetSymbolAddress in noalloc_device_ptr() below, and that pointer is what the
// kernels receive.
constexpr size_t kNoallocFloats = WARPIR_NOALLOC_SCRATCH_BYTES / sizeof(float);
constexpr size_t kNoallocStatusFloats = 64;   // status words live behind the partial sums
static __device__ __align__(256) float g_noalloc_scratch[kNoallocFloats + kNoallocStatusFloats];

namespace {

std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[kMaxDevices] = {};
int g_noalloc_sms[kMaxDevices] = {};

// Device address of g_noalloc_scratch on `device` (which must be current).  The first call
// per device does the lookup; it allocates nothing.
int noalloc_device_ptr(int device, float** out, int* sms) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[device] == nullptr) {
    int major = 0;
    WIR_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return fail(WARPIR_EDEVICE, "device %d has compute capability %d.x; sm_100a needed", device, major);
    WIR_CUDA(cudaDeviceGetAttribute(&g_noalloc_sms[device], cudaDevAttrMultiProcessorCount, device));
    void* ptr = nullptr;
    WIR_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return fail(WARPIR_ECUDA, "cudaGetSymbolAddress returned a null device address");
    g_noalloc_ptr[device] = static_cast<float*>(ptr);
  }
  if (int rc = ensure_encode()) return rc;
  *out = g_noalloc_ptr[device];
  *sms = g_noalloc_sms[device];
  return WARPIR_OK;
}

}  // namespace

// Status words of the allocation-free entry point: waits for the stream, copies the four words out of
// the static array (a plain cudaMemcpy into caller stack memory: nothing is allocated) and clears
// them when they hold an error.
extern "C" int warpir_noalloc_read_status(int device, void* cuda_stream, int* code, int* detail) {
  g_last_error[0] = 0;
  if (device < 0 || device >= kMaxDevices) return fail(WARPIR_EDEVICE, "device index %d out of range", device);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  float* scratch = nullptr;
  int sms = 0;
  if (int rc = noalloc_device_ptr(device, &scratch, &sms)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int host[4] = {0, 0, 0, 0};
  WIR_CUDA(cudaStreamSynchronize(stream));
  WIR_CUDA(cudaMemcpy(host, scratch + kNoallocFloats, sizeof host, cudaMemcpyDeviceToHost));
  if (host[0] != 0) WIR_CUDA(cudaMemset(scratch + kNoallocFloats, 0, sizeof host));
  if (code) *code = host[0];
  if (detail) *detail = host[2];
  if (host[0] != 0)
    return fail(WARPIR_EKERNEL, "kernel status %d: cta %d role %d tag %d detail %d", host[0], host[1], host[2] >> 16,
                host[2] & 0xffff, host[3]);
  return WARPIR_OK;
}

extern "C" int warpir_gemm_bf16_splitk_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N,
                                               int64_t K, int b_layout, int block_n, int splits, int device,
                                               void* cuda_stream) {
  g_last_error[0] = 0;
  if (M < 0 || N < 0 || K < 0) return fail(WARPIR_EINVAL, "negative size");
  if (b_layout != 0 && b_layout != 1) return fail(WARPIR_EINVAL, "b_layout must be 0 or 1");
  if (block_n != 0 && block_n != 64 && block_n != 128 && block_n != 256)
    return fail(WARPIR_EINVAL, "block_n must be 0, 64, 128 or 256");
  if (splits < 1 || splits > 64) return fail(WARPIR_EINVAL, "splits must be in [1, 64]");
  if (device < 0 || device >= kMaxDevices) return fail(WARPIR_EDEVICE, "device index %d out of range", device);
  if (M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2) return fail(WARPIR_ESHAPE, "size above 2^30");
  if (M == 0 || N == 0) return WARPIR_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  if (int rc = check_device_ptr(C, "C", device)) return rc;
  if (K == 0) {
    WIR_CUDA(cudaMemsetAsync(C, 0, static_cast<size_t>(M) * N * 2, stream));
    return WARPIR_OK;
  }
  if (int rc = check_device_ptr(A, "A", device)) return rc;
  if (int rc = check_device_ptr(B, "B", device)) return rc;
  if (K % 8 != 0) return fail(WARPIR_ESHAPE, "K = %lld: the row pitch of A must be a multiple of 16 bytes (K %% 8 == 0)", (long long)K);
  if (b_layout == 0 && N % 8 != 0) return fail(WARPIR_ESHAPE, "N = %lld: with B stored [K,N] its row pitch must be a multiple of 16 bytes (N %% 8 == 0)", (long long)N);

  float* scratch = nullptr;
  int sms = 0;
  if (int rc = noalloc_device_ptr(device, &scratch, &sms)) return rc;

  int bn = block_n != 0 ? block_n : choose_gemm(M, N, K, sms).block_n;
  const int num_kb = static_cast<int>((K + wir::kGemmBK - 1) / wir::kGemmBK);
  int want = splits > num_kb ? num_kb : splits;
  if (want > 1 && N % 4 != 0) want = 1;  // the reduce pass works on groups of four columns

  wir::GemmParams p;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.ldc = p.N;
  p.tiles_m = static_cast<int>((M + wir::kGemmBM - 1) / wir::kGemmBM);
  p.tiles_n = static_cast<int>((N + bn - 1) / bn);
  p.num_kb = num_kb;
  p.kb_per_split = (num_kb + want - 1) / want;
  p.splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.partial = scratch;
  p.status = reinterpret_cast<int*>(scratch + kNoallocFloats);
  p.trace = nullptr;
  if (p.splits > 1) {
    const size_t need = static_cast<size_t>(p.splits) * M * N;
    if (need > kNoallocFloats)
      return fail(WARPIR_ESHAPE,
                  "splits * M * N = %zu partial sums (%zu bytes) exceed the static scratch of %u bytes; "
                  "use fewer splits or warpir_gemm_bf16_ex",
                  need, need * sizeof(float), WARPIR_NOALLOC_SCRATCH_BYTES);
  }

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {wir::kGemmBK, wir::kGemmBM};
    if (int rc = make_tmap(&ta, A, 2, dims, strides, box)) return rc;
  }
  if (b_layout == 1) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {wir::kGemmBK, static_cast<uint32_t>(bn)};
    if (int rc = make_tmap(&tb, B, 2, dims, strides, box)) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, wir::kGemmBK};
    if (int rc = make_tmap(&tb, B, 2, dims, strides, box)) return rc;
  }
  const int64_t work = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.splits;
  const int grid = static_cast<int>(work < sms ? work : sms);
  const bool mn = (b_layout == 0);
  int rc;
  switch (bn) {
    case 256: rc = mn ? launch_gemm_cfg<256, 4, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<256, 4, false>(ta, tb, p, grid, stream); break;
    case 128: rc = mn ? launch_gemm_cfg<128, 6, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<128, 6, false>(ta, tb, p, grid, stream); break;
    default:  rc = mn ? launch_gemm_cfg<64, 8, true>(ta, tb, p, grid, stream) : launch_gemm_cfg<64, 8, false>(ta, tb, p, grid, stream); break;
  }
  if (rc) return rc;
  if (p.splits > 1) {
    const size_t total4 = (static_cast<size_t>(M) * N) >> 2;
    int blocks = static_cast<int>((total4 + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    wir::splitk_reduce_bf16<<<blocks, 256, 0, stream>>>(p.partial, p.C, p.M, p.N, p.ldc, p.splits);
    WIR_CUDA(cudaGetLastError());
  }
  return WARPIR_OK;
}
