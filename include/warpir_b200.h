/*
 * C ABI of libwarpir_b200.so: the sm_100a launcher for WarpIR's hot path
 * (bf16 GEMM and attention forward).
 *
 * Each entry point replaces a run-time interface of the reference, which has no
 * library of its own: it JIT-builds a pybind module per generated kernel with
 * torch's load_inline and calls `launch_gemm(A, B, C)` / `launch_attention(Q, K, V, O)`
 * on torch tensors.  The citations below name the reference wrapper each entry
 * point stands in for.
 *
 * Conventions
 *  - plain pointers and sizes only; every pointer is DEVICE memory on `device`;
 *  - the caller owns every buffer, outputs included (as in the reference, which
 *    passes a pre-allocated C / O: tests/test_gemm_baseline.py:80);
 *  - calls enqueue work on `cuda_stream` (a cudaStream_t, NULL = legacy default
 *    stream, which is what the reference's wrappers launch on) and return without
 *    synchronising; results are ready when the stream reaches that point;
 *  - return value: 0 on success, a negative WARPIR_E* code otherwise; nothing is
 *    thrown across the boundary and the process is never terminated;
 *  - arguments are validated BEFORE anything is launched; a rejected call has no
 *    side effect;
 *  - the library keeps a few hundred bytes of state per device (status words) and,
 *    only when a GEMM is split along K, a scratch buffer it grows on demand;
 *  - thread-safe: calls may come from several host threads, for one or several
 *    devices.
 */
#ifndef WARPIR_B200_H_
#define WARPIR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WARPIR_ABI_VERSION 1

enum {
  WARPIR_OK = 0,
  WARPIR_EINVAL = -1,      /* NULL pointer, negative size, bad enum value            */
  WARPIR_EALIGN = -2,      /* a pointer or a row pitch is not 16-byte aligned        */
  WARPIR_ESHAPE = -3,      /* a size the kernels do not cover (see each function)    */
  WARPIR_ECUDA = -4,       /* a CUDA runtime call failed; see warpir_last_error()    */
  WARPIR_EDRIVER = -5,     /* cuTensorMapEncodeTiled missing or failed               */
  WARPIR_EKERNEL = -6,     /* a kernel reported an error in its status words         */
  WARPIR_EDEVICE = -7,     /* pointer does not live on `device`, or bad device index */
  WARPIR_ENOMEM = -8       /* scratch allocation failed                              */
};

/* ABI version of the loaded library (== WARPIR_ABI_VERSION it was built with). */
int warpir_abi_version(void);

/* Static, human-readable text for a WARPIR_E* code. */
const char* warpir_strerror(int code);

/* Text of the most recent failure on the calling thread (CUDA error string,
 * the argument that was rejected ...).  Valid until the thread's next call. */
const char* warpir_last_error(void);

/*
 * C[M,N] = A[M,K] * B, bf16 inputs, fp32 accumulation, bf16 output, all row-major
 * and densely packed.
 *   b_layout 0: B is stored [K,N] (the layout of the reference's GEMM tile program,
 *               tests/gemm_baseline_v2.py:78-79);
 *   b_layout 1: B is stored [N,K], i.e. C = A * B_stored^T ("K-major").
 * Replaces `launch_gemm(A, B, C)` (reference: tests/test_gemm_baseline.py:20-31,
 * tests/test_modal_gpu.py:24-50), which takes square N x N tensors only and requires
 * N to be a multiple of 64.  Here M, N, K are free, except that the row pitches TMA
 * reads must be multiples of 16 bytes: K % 8 == 0, and N % 8 == 0 for b_layout 0.
 * M, N or K equal to 0 is a valid no-op (K == 0 zero-fills C).
 */
int warpir_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                     int b_layout, int device, void* cuda_stream);

/*
 * Same as warpir_gemm_bf16 with the two launch parameters the scheduling pass may
 * choose made explicit: the tile width `block_n` (64, 128 or 256; 0 = choose) and
 * the number of K-splits per output tile `splits` (>= 1; 0 = choose).  With
 * splits > 1 the partial sums go through an fp32 scratch buffer owned by the
 * library and are reduced in a fixed order, so results do not depend on timing.
 * No counterpart in the reference, whose tile shape is a constant of the tile
 * program (tests/gemm_baseline_v2.py:32).
 */
int warpir_gemm_bf16_ex(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                        int b_layout, int block_n, int splits, int device, void* cuda_stream);

/*
 * Split-K GEMM for callers that must not allocate device memory.
 *
 * Some hosts cannot tolerate a cudaMalloc coming out of a library call: a serving process
 * that handed the whole GPU to its own memory pool at start-up (a later cudaMalloc simply
 * fails, or succeeds only by fragmenting what the pool left over), a latency-critical
 * loop where the implicit device synchronisation of cudaMalloc/cudaFree is not
 * acceptable, or code whose device-memory footprint is fixed at load time.
 * warpir_gemm_bf16_ex with splits > 1 grows a scratch buffer on demand and
 * warpir_gemm_bf16 allocates its status words on first use, so neither is usable there.
 *
 * With an explicit tile width (block_n = 64, 128 or 256) this entry point computes exactly what
 * warpir_gemm_bf16_ex(A, B, C, M, N, K, b_layout, block_n, splits, ...) computes -- same
 * kernels, same fixed reduction order, bit-identical C.  With block_n = 0 it picks the width
 * by the tile count alone (it never takes the few-rows kernels that load only part of an A
 * tile, nor stream-K, which warpir_gemm_bf16_ex may), so then the two agree to rounding, not
 * bit for bit.  It keeps the fp32 partial sums (and its kernel status words) in a statically
 * allocated device array that is part of the library image.  It calls no cudaMalloc,
 * cudaFree or any other allocating routine.  Consequences:
 *  - every GPU whose context loads this library holds WARPIR_NOALLOC_SCRATCH_BYTES
 *    (16 MiB) for that array until the process exits, whether or not this function is used;
 *  - splits * M * N * 4 bytes must fit in it; larger problems are rejected with
 *    WARPIR_ESHAPE and a message naming the limit (nothing is launched);
 *  - the first call on a device looks up the array's device address (one
 *    cudaGetSymbolAddress); make that first call before starting any stream capture;
 *  - all calls on a device share the one array and it keeps the previous call's
 *    contents.  Nothing in it needs clearing between calls (every partial sum that is
 *    read has been written by the same call), but two calls that overlap on the GPU --
 *    different streams, or different host threads -- race on it: serialise them;
 *  - a bounded wait that runs out inside these launches is recorded in status words inside
 *    the static array, not in the ones warpir_read_status reports: read (and clear) them
 *    with warpir_noalloc_read_status, which allocates nothing either.
 * block_n is 0 (choose), 64, 128 or 256; splits is >= 1.  Other arguments, size rules
 * and return codes are those of warpir_gemm_bf16.
 * This function has no counterpart in the reference.
 */
#define WARPIR_NOALLOC_SCRATCH_BYTES (16u << 20)
int warpir_gemm_bf16_splitk_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                    int b_layout, int block_n, int splits, int device, void* cuda_stream);

/* Status of the launches made by warpir_gemm_bf16_splitk_noalloc on `device`: same contract as
 * warpir_read_status (waits for `cuda_stream`, reports, clears on error), same guarantee as the
 * entry point it serves (no allocation).  No counterpart in the reference. */
int warpir_noalloc_read_status(int device, void* cuda_stream, int* code, int* detail);

/*
 * GEMM with the all-gather of its output fused into the epilogue.  In a job that splits the rows
 * of A (and of C) over GPUs, every GPU ends up with the whole C: each finished tile is stored to
 * n_dst destinations, C_dst[d] being the address of THIS GPU's row block inside GPU d's full C
 * (its own memory, or a peer's buffer mapped into this GPU's address space, e.g. through torch's
 * symmetric memory or CUDA IPC / virtual memory mappings).  The stores to peers cross NVLink while
 * the tensor cores work on the next tiles; nothing else is exchanged and nothing waits.  All
 * destinations have row pitch N.  The caller orders consumers after the kernel (stream
 * synchronisation plus a barrier between the processes).  n_dst is 1 .. 8.
 * Arguments, size rules and return codes otherwise as warpir_gemm_bf16; K is never split here.
 * No counterpart in the reference (which is single-GPU).
 */
int warpir_gemm_bf16_allgather(const void* A, const void* B, void* const* C_dst, int n_dst,
                               int64_t M, int64_t N, int64_t K, int b_layout, int device, void* cuda_stream);

/*
 * Attention forward: O[b,h] = softmax(softmax_scale * Q[b,h] K[b,hk]^T (+ causal mask)) V[b,hk],
 * LSE[b,h,i] = log sum_j exp(softmax_scale * q_i . k_j) (natural log), hk = h / (Hq / Hkv).
 *   Q, O: [B, Hq, S, D] bf16, contiguous;  K, V: [B, Hkv, S, D] bf16, contiguous;
 *   LSE: [B, Hq, S] fp32, or NULL to skip it;  D is 64 or 128;  Hq % Hkv == 0;
 *   causal != 0: key j is visible to query i iff j <= i.
 * Replaces `launch_attention(Q, K, V, O)` (reference: tests/test_modal_attention.py:25-39:
 * one head, [N, 64], non-causal, scale 1/8 fixed, N a multiple of 64, no LSE) and the
 * host wrapper `attention_forward` of the reference's hand-written target
 * (kernel_examples/attention/mha_h100.cu:651-797: 4-D, D in {64,128}, causal flag,
 * grouped KV heads, an L vector).  S is free (any S >= 1).
 */
int warpir_attn_fwd_bf16(const void* Q, const void* K, const void* V, void* O, float* LSE,
                         int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                         float softmax_scale, int causal, int device, void* cuda_stream);

/*
 * Same with the kernel variant spelled out: 0 lets the library choose, 1 is the kernel with 64-key
 * blocks and double-buffered scores (one MMA-issuing warp per 128-row Q tile), 4 the kernel with 128-key
 * blocks (one score tile per Q tile, the two Q tiles of a CTA taking turns on the tensor core).  Other
 * values are rejected (2 and 3 named experimental kernels that measured slower and were withdrawn).
 * Results agree to rounding.  The library's own choice (0) is 4 without a causal mask and 1 with one.
 * No counterpart in the reference; exists for tests and tuning.
 */
int warpir_attn_fwd_bf16_ex(const void* Q, const void* K, const void* V, void* O, float* LSE,
                            int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                            float softmax_scale, int causal, int variant, int device, void* cuda_stream);

/*
 * Attention backward: gradients of warpir_attn_fwd_bf16's O with respect to Q, K and V.
 *   Q, O, dO: [B, Hq, S, D] bf16;  K, V: [B, Hkv, S, D] bf16;  LSE: [B, Hq, S] fp32 as written
 *   by the forward (natural log);  dQ: [B, Hq, S, D] fp32;  dK, dV: [B, Hkv, S, D] fp32
 *   (summed over the query heads that share a K/V head);  delta_ws: [B, Hq, S] fp32
 *   workspace owned by the caller (receives rowsum(dO * O)).  All contiguous, 16-byte
 *   aligned; same size rules, scale and causal convention as the forward.
 * Two launches on `cuda_stream` (dQ, then dK and dV); no atomics, results repeat bit for bit.
 * Replaces the host wrapper `attention_backward(q, k, v, o, l_vec, og, causal)` of the
 * reference's hand-written target (kernel_examples/attention/mha_h100.cu:799-1010), which
 * likewise returns fp32 gradients and keeps a d_vec workspace; unlike it, LSE here is the
 * plain log-sum-exp, not the reference's negated and rescaled L vector (mha_h100.cu:216-221).
 */
int warpir_attn_bwd_bf16(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                         const float* LSE, float* dQ, float* dK, float* dV, float* delta_ws,
                         int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                         float softmax_scale, int causal, int device, void* cuda_stream);

/*
 * Launches a tile program that was lowered and compiled into its own shared object
 * (`Sm100Lowerer().lower(kernel)` -> nvcc -shared): looks `<kernel_name>_launch` up in
 * `module_handle` (a dlopen handle) and calls it.  `tensor_ptrs`: device pointers of the
 * program's global inputs then outputs, in signature order; `dims`: four extents (batch,
 * depth, rows, cols) per tensor; `scalars`: the program's int inputs in signature order.
 * Replaces the pybind module the reference builds per program with `load_inline` and its
 * f-string launch wrapper (tests/test_gemm_baseline.py:20-74, tests/test_modal_attention.py:25-99).
 */
int warpir_launch_generated(void* module_handle, const char* kernel_name, const void* const* tensor_ptrs,
                            const int64_t* dims, int n_tensors, const int64_t* scalars, int n_scalars,
                            int device, void* cuda_stream);

/*
 * What the launcher would run for C[M,N] = A[M,K] B on a device with `sms` SMs: CTA tile
 * (block_m x block_n), whether the tile is computed by a CTA pair (cta_group 2), whether the
 * k-blocks rather than the tiles are dealt out to the SMs (stream_k), and how many rows of A a
 * stage loads (a_rows < 128 for problems with few rows).  Host arithmetic only: touches no device.
 * The tile-planning pass of the Python front end (warpir_b200/passes/tile_planner.py) states the
 * same rules for tile programs; this export lets the two be checked against each other.  The
 * reference fixes its tile in the program text (tests/gemm_baseline_v2.py:32) and has no planner.
 * Any output pointer may be NULL.
 */
int warpir_plan_gemm(int64_t M, int64_t N, int64_t K, int sms, int* block_m, int* block_n, int* cta_group,
                     int* stream_k, int* a_rows);

/*
 * Waits for `cuda_stream`, then reports and clears the device's status words:
 * *code is 0 when every kernel launched so far on this device ran to completion,
 * otherwise the kernel-side error (1 = a bounded wait ran out); *detail packs
 * (role << 16 | tag).  Returns WARPIR_OK when *code == 0, WARPIR_EKERNEL otherwise.
 * Every wait inside the kernels is bounded, so a protocol failure surfaces here
 * rather than as a hung GPU.  The reference checks nothing after a launch
 * (tests/test_gemm_baseline.py:21-30).
 */
int warpir_read_status(int device, void* cuda_stream, int* code, int* detail);

/*
 * Exercises the kernels' failure path without failing anything: launches one small CTA that
 * waits, for at most `limit_ns` nanoseconds (1 .. 1e9), on a barrier nothing arrives on.  The
 * wait runs out, the kernel writes the same status words a GEMM or attention kernel would
 * write when one of its waits runs out, and exits normally; the next warpir_read_status
 * returns WARPIR_EKERNEL with code 1 and clears the words, after which the device is usable
 * as before.  Lets a host verify its error handling around warpir_read_status on a healthy
 * GPU.  No counterpart in the reference, which has no error path at all.
 */
int warpir_selftest_bounded_wait(int device, void* cuda_stream, int64_t limit_ns);

#ifdef __cplusplus
}
#endif
#endif /* WARPIR_B200_H_ */
