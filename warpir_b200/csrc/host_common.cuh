// Host-side plumbing shared by everything that launches an sm_100a kernel of this
// package: error text, per-device state (status words), argument validation, TMA tensor
// maps, the shared-memory opt-in and the status read-back.  Host code only touches CUDA
// through the runtime API; cuTensorMapEncodeTiled is fetched with cudaGetDriverEntryPoint,
// so nothing links against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../../include/warpir_b200.h"

namespace wir {
namespace host {

inline thread_local char g_last_error[256] = "";

inline int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
  va_end(ap);
  return code;
}

#define WIR_CUDA(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e_ = (expr);                                                                \
    if (e_ != cudaSuccess) return fail(WARPIR_ECUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

constexpr int kMaxDevices = 64;

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* status = nullptr;        // 4 ints
  // Scratch of the K-splitting GEMM paths (fp32 partial sums; stream-K arrival counters, zero
  // between launches), one set per CUDA stream: launches on one stream run one after the other,
  // launches on different streams may overlap and must not share it.  Grown on demand.
  struct Scratch {
    float* partial = nullptr;
    size_t partial_bytes = 0;
    int* counters = nullptr;    // kSkMaxTiles ints
  };
  std::unordered_map<void*, Scratch> scratch;   // keyed by stream handle
};
constexpr int kSkMaxTiles = 8192;

inline std::mutex g_mutex;
inline DeviceState g_dev[kMaxDevices];
inline PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
inline unsigned long long* g_trace = nullptr;   // event-trace buffer; only debug builds (-DWIR_TRACE) write to it

// Makes `device` current for the calling thread for the lifetime of the object.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      switched = (err == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// cuTensorMapEncodeTiled, fetched once per process (whichever entry point gets here first).
inline int ensure_encode() {
  static std::once_flag once;
  static int rc = WARPIR_OK;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) rc = WARPIR_EDRIVER;
    else g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  if (rc != WARPIR_OK) return fail(WARPIR_EDRIVER, "cuTensorMapEncodeTiled not available from this driver");
  return WARPIR_OK;
}

inline int get_device_state(int device, DeviceState** out) {
  if (device < 0 || device >= kMaxDevices) return fail(WARPIR_EDEVICE, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& d = g_dev[device];
  if (!d.ready) {
    int count = 0;
    WIR_CUDA(cudaGetDeviceCount(&count));
    if (device >= count) return fail(WARPIR_EDEVICE, "device index %d but %d devices", device, count);
    int major = 0;
    WIR_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return fail(WARPIR_EDEVICE, "device %d has compute capability %d.x; sm_100a needed", device, major);
    WIR_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    // the status words must live on `device`, whatever device the calling thread has current
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
    WIR_CUDA(cudaMalloc(&d.status, 4 * sizeof(int)));
    WIR_CUDA(cudaMemset(d.status, 0, 4 * sizeof(int)));
    d.ready = true;
  }
  if (int rc = ensure_encode()) return rc;
  *out = &d;
  return WARPIR_OK;
}

// The calling stream's scratch with at least `bytes` of partial-sum space (and the counters).
// May allocate, which synchronises: the first call of a given size on a stream does, later ones do not.
inline int stream_scratch(DeviceState* dev, cudaStream_t stream, size_t bytes, DeviceState::Scratch** out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState::Scratch& sc = dev->scratch[static_cast<void*>(stream)];
  if (sc.counters == nullptr) {
    if (cudaMalloc(&sc.counters, kSkMaxTiles * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      return fail(WARPIR_ENOMEM, "stream-K counters");
    }
    WIR_CUDA(cudaMemset(sc.counters, 0, kSkMaxTiles * sizeof(int)));
  }
  if (sc.partial_bytes < bytes) {
    if (sc.partial) {
      WIR_CUDA(cudaStreamSynchronize(stream));   // the buffer being replaced may still be in use there
      WIR_CUDA(cudaFree(sc.partial));
      sc.partial = nullptr;
      sc.partial_bytes = 0;
    }
    if (cudaMalloc(&sc.partial, bytes) != cudaSuccess) {
      cudaGetLastError();
      return fail(WARPIR_ENOMEM, "K-split scratch of %zu bytes", bytes);
    }
    sc.partial_bytes = bytes;
  }
  *out = &sc;
  return WARPIR_OK;
}

inline int check_device_ptr(const void* p, const char* name, int device) {
  if (p == nullptr) return fail(WARPIR_EINVAL, "%s is NULL", name);
  if (reinterpret_cast<uintptr_t>(p) & 15) return fail(WARPIR_EALIGN, "%s is not 16-byte aligned", name);
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(WARPIR_EDEVICE, "%s: cudaPointerGetAttributes failed", name);
  }
  if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)
    return fail(WARPIR_EDEVICE, "%s is not device memory", name);
  if (attr.type == cudaMemoryTypeDevice && attr.device != device)
    return fail(WARPIR_EDEVICE, "%s lives on device %d, not %d", name, attr.device, device);
  return WARPIR_OK;
}

// bf16 tensor map with 128-byte swizzle.  dims/box innermost first; strides in bytes
// for dims 1.. (dim 0 is contiguous).
inline int encode_tmap(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box);

// Encoding a tensor map costs a few microseconds of host time, which matters for small
// problems launched back to back; the last few maps of each thread are kept, keyed by
// everything that goes into the encoding.
inline int make_tmap(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box) {
  struct Entry {
    const void* base;
    int rank;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    CUtensorMap map;
  };
  constexpr int kEntries = 16;
  static thread_local Entry cache[kEntries];
  static thread_local int next = 0, used = 0;
  Entry key{};
  key.base = base;
  key.rank = rank;
  for (int i = 0; i < rank && i < 3; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
  }
  if (rank <= 3) {
    for (int i = 0; i < used; ++i) {
      const Entry& e = cache[i];
      if (e.base == key.base && e.rank == key.rank && !memcmp(e.dims, key.dims, sizeof key.dims) &&
          !memcmp(e.strides, key.strides, sizeof key.strides) && !memcmp(e.box, key.box, sizeof key.box)) {
        *map = e.map;
        return WARPIR_OK;
      }
    }
  }
  if (int rc = encode_tmap(map, base, rank, dims, strides_bytes, box)) return rc;
  if (rank <= 3) {
    key.map = *map;
    cache[next] = key;
    next = (next + 1) % kEntries;
    if (used < kEntries) ++used;
  }
  return WARPIR_OK;
}

inline int encode_tmap(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box) {
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdims, gstrides, gbox,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(WARPIR_EDRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return WARPIR_OK;
}

// Tensor map for the op-by-op tile programs (tile_program.cuh): a bf16 tensor of extents
// ext = (batch, depth, rows, cols), read as (cols, rows, batch * depth) in boxes of 64 columns
// by `tile_rows` rows.
inline int tile_program_tmap(CUtensorMap* map, const void* base, const int64_t* ext, int tile_rows) {
  if (ext[3] % 8 != 0)
    return fail(WARPIR_ESHAPE, "row pitch of %lld bf16 elements is not a multiple of 16 bytes", (long long)ext[3]);
  const uint64_t dims[3] = {static_cast<uint64_t>(ext[3]), static_cast<uint64_t>(ext[2]),
                            static_cast<uint64_t>(ext[0] * ext[1])};
  const uint64_t strides[2] = {static_cast<uint64_t>(ext[3]) * 2, static_cast<uint64_t>(ext[3]) * ext[2] * 2};
  const uint32_t box[3] = {64, static_cast<uint32_t>(tile_rows), 1};
  return make_tmap(map, base, 3, dims, strides, box);
}

// Raises a kernel's dynamic shared-memory limit, once per (kernel, device).
inline int opt_in_smem(const void* kernel, int bytes) {
  struct Seen { const void* fn; int device; };
  static thread_local Seen seen[32];
  static thread_local int n_seen = 0;
  int device = 0;
  WIR_CUDA(cudaGetDevice(&device));
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].fn == kernel && seen[i].device == device) return WARPIR_OK;
  WIR_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (n_seen < 32) seen[n_seen++] = Seen{kernel, device};
  return WARPIR_OK;
}

inline int read_status_impl(int device, void* cuda_stream, int* code, int* detail) {
  g_last_error[0] = 0;
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int host[4] = {0, 0, 0, 0};
  WIR_CUDA(cudaStreamSynchronize(stream));
  WIR_CUDA(cudaMemcpy(host, dev->status, sizeof host, cudaMemcpyDeviceToHost));
  if (host[0] != 0) {
    WIR_CUDA(cudaMemset(dev->status, 0, sizeof host));
    // a kernel that gave up may have left stream-K tickets behind
    std::lock_guard<std::mutex> lock(g_mutex);
    for (auto& kv : dev->scratch)
      if (kv.second.counters) WIR_CUDA(cudaMemset(kv.second.counters, 0, kSkMaxTiles * sizeof(int)));
  }
  if (code) *code = host[0];
  if (detail) *detail = host[2];
  if (host[0] != 0)
    return fail(WARPIR_EKERNEL, "kernel status %d: cta %d role %d tag %d detail %d", host[0], host[1], host[2] >> 16,
                host[2] & 0xffff, host[3]);
  return WARPIR_OK;
}

}  // namespace host
}  // namespace wir
