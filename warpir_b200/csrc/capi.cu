// C-ABI entry points (see include/warpir_b200.h).  The work is in launch.cuh.
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

int warpir_attn_fwd_bf16(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B, int64_t Hq,
                         int64_t Hkv, int64_t S, int64_t D, float softmax_scale, int causal, int device,
                         void* cuda_stream) {
  return attn_impl(Q, K, V, O, LSE, B, Hq, Hkv, S, D, softmax_scale, causal, device, cuda_stream);
}

int warpir_read_status(int device, void* cuda_stream, int* code, int* detail) {
  return read_status_impl(device, cuda_stream, code, detail);
}

}  // extern "C"
