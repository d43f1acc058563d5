"""ctypes binding of the C-ABI launcher and torch-tensor convenience wrappers.

This replaces what the reference does at run time: JIT-build a pybind module per
generated kernel with ``load_inline`` and call ``launch_gemm(A, B, C)`` /
``launch_attention(Q, K, V, O)`` (reference: tests/test_gemm_baseline.py:52-74,
tests/test_modal_attention.py:80-99).  The callables here keep those call
shapes -- the caller allocates every tensor, outputs included; the call is
asynchronous on torch's current stream -- and raise instead of silently
continuing when something is wrong.  There is no fallback: without the compiled
library, or without an sm_100 GPU, every entry point raises.
"""
from __future__ import annotations

import ctypes
import os
import math
import threading
from pathlib import Path
from typing import Optional

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libwarpir_b200.so"
_lib = None
_lock = threading.Lock()

ABI_VERSION = 1

EXPORTS = (
    "warpir_abi_version", "warpir_strerror", "warpir_last_error", "warpir_gemm_bf16",
    "warpir_gemm_bf16_ex", "warpir_gemm_bf16_allgather", "warpir_attn_fwd_bf16", "warpir_attn_fwd_bf16_ex", "warpir_attn_bwd_bf16",
    "warpir_launch_generated", "warpir_read_status",
    "warpir_gemm_bf16_splitk_noalloc", "warpir_noalloc_read_status", "warpir_selftest_bounded_wait",
    "warpir_plan_gemm",
)


class WarpirError(RuntimeError):
    """A C-ABI call returned a negative code."""

    def __init__(self, code: int, what: str, detail: str):
        super().__init__(f"{what}: {detail}" if detail else what)
        self.code = code


def library_path() -> Path:
    return _LIB_PATH


def load_library() -> ctypes.CDLL:
    """Load ``libwarpir_b200.so`` (built by ``python -m warpir_b200.build``) and
    declare its prototypes.  Raises if the file is missing or its ABI differs."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        # WARPIR_B200_LIBRARY names another build of the same library (a debug build with event
        # traces, a measurement build); it must export the same ABI
        path = Path(os.environ["WARPIR_B200_LIBRARY"]).resolve() if os.environ.get("WARPIR_B200_LIBRARY") else _LIB_PATH
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -m warpir_b200.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(str(path))
        vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        lib.warpir_abi_version.restype = ci
        lib.warpir_abi_version.argtypes = []
        lib.warpir_strerror.restype = ctypes.c_char_p
        lib.warpir_strerror.argtypes = [ci]
        lib.warpir_last_error.restype = ctypes.c_char_p
        lib.warpir_last_error.argtypes = []
        lib.warpir_gemm_bf16.restype = ci
        lib.warpir_gemm_bf16.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, vp]
        lib.warpir_gemm_bf16_ex.restype = ci
        lib.warpir_gemm_bf16_ex.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, ci, vp]
        lib.warpir_gemm_bf16_splitk_noalloc.restype = ci
        lib.warpir_gemm_bf16_splitk_noalloc.argtypes = [vp, vp, vp, i64, i64, i64, ci, ci, ci, ci, vp]
        lib.warpir_attn_fwd_bf16.restype = ci
        lib.warpir_attn_fwd_bf16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, cf, ci, ci, vp]
        lib.warpir_attn_fwd_bf16_ex.restype = ci
        lib.warpir_attn_fwd_bf16_ex.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, cf, ci, ci, ci, vp]
        lib.warpir_gemm_bf16_allgather.restype = ci
        lib.warpir_gemm_bf16_allgather.argtypes = [vp, vp, ctypes.POINTER(vp), ci, i64, i64, i64, ci, ci, vp]
        lib.warpir_launch_generated.restype = ci
        lib.warpir_launch_generated.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(vp), ctypes.POINTER(i64), ci,
                                                ctypes.POINTER(i64), ci, ci, vp]
        lib.warpir_attn_bwd_bf16.restype = ci
        lib.warpir_attn_bwd_bf16.argtypes = [vp] * 10 + [i64] * 5 + [cf, ci, ci, vp]
        lib.warpir_selftest_bounded_wait.restype = ci
        lib.warpir_selftest_bounded_wait.argtypes = [ci, vp, i64]
        lib.warpir_read_status.restype = ci
        lib.warpir_read_status.argtypes = [ci, vp, ctypes.POINTER(ci), ctypes.POINTER(ci)]
        lib.warpir_noalloc_read_status.restype = ci
        lib.warpir_noalloc_read_status.argtypes = [ci, vp, ctypes.POINTER(ci), ctypes.POINTER(ci)]
        lib.warpir_plan_gemm.restype = ci
        lib.warpir_plan_gemm.argtypes = [i64, i64, i64, ci] + [ctypes.POINTER(ci)] * 5
        if lib.warpir_abi_version() != ABI_VERSION:
            raise RuntimeError(f"ABI {lib.warpir_abi_version()} != expected {ABI_VERSION}: rebuild the library")
        _lib = lib
        return lib


def _check(rc: int) -> None:
    if rc != 0:
        lib = load_library()
        raise WarpirError(rc, lib.warpir_strerror(rc).decode(), lib.warpir_last_error().decode())


def _stream_of(t) -> int:
    import torch
    return torch.cuda.current_stream(t.device).cuda_stream


def _require(t, name: str, dtype, ndim: Optional[int] = None):
    import torch
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dimensions, got {t.dim()}")


def launch_gemm(A, B, C, b_layout: int = 0, block_n: int = 0, splits: int = 0) -> None:
    """``C = A @ B`` (``b_layout=0``, B stored ``[K,N]``) or ``C = A @ B.T``
    (``b_layout=1``, B stored ``[N,K]``) on torch's current stream.

    Same call shape as the reference's ``launch_gemm(A, B, C)``
    (tests/test_gemm_baseline.py:20-31): bf16 CUDA tensors, C pre-allocated,
    asynchronous.  Sizes need not be square nor tile multiples.
    """
    import torch
    lib = load_library()
    for t, n in ((A, "A"), (B, "B"), (C, "C")):
        _require(t, n, torch.bfloat16, 2)
    M, K = A.shape
    if b_layout == 1:
        N, Kb = B.shape
    elif b_layout == 0:
        Kb, N = B.shape
    else:
        raise ValueError("b_layout must be 0 or 1")
    if Kb != K or tuple(C.shape) != (M, N):
        raise ValueError(f"shape mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}, C {tuple(C.shape)}")
    if not (A.device == B.device == C.device):
        raise ValueError("A, B and C must be on one device")
    _check(lib.warpir_gemm_bf16_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, b_layout,
                                   block_n, splits, A.device.index, _stream_of(A)))


def launch_gemm_allgather(A, B, dst_ptrs, N: int, b_layout: int = 1) -> None:
    """``A @ B`` for this GPU's rows of A, every finished tile stored to each address in
    ``dst_ptrs``: the place of this row block inside every GPU's copy of the full output (own
    buffer and peers' buffers mapped into this GPU's address space; see
    ``warpir_b200.sharding.GatheredOutput``).  Asynchronous on torch's current stream; the caller
    synchronises the GPUs before reading the gathered output."""
    import torch
    lib = load_library()
    _require(A, "A", torch.bfloat16, 2)
    _require(B, "B", torch.bfloat16, 2)
    M, K = A.shape
    Nb, Kb = (B.shape if b_layout == 1 else B.shape[::-1])
    if Kb != K or Nb != N:
        raise ValueError(f"shape mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}, N {N}")
    ptrs = (ctypes.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    _check(lib.warpir_gemm_bf16_allgather(A.data_ptr(), B.data_ptr(), ptrs, len(dst_ptrs), M, N, K, b_layout,
                                          A.device.index, _stream_of(A)))


def launch_attention(Q, K, V, O, LSE=None, softmax_scale: Optional[float] = None,
                     causal: bool = False, variant: int = 0) -> None:
    """Attention forward on torch's current stream.

    Accepts the reference's single-head call ``launch_attention(Q, K, V, O)``
    with ``[N, D]`` tensors (tests/test_modal_attention.py:25-39) as well as
    ``[B, H, S, D]`` tensors with grouped KV heads; ``LSE`` (fp32 ``[B, H, S]``
    or ``[N]``) is filled when given.  Scale defaults to ``1/sqrt(D)``.
    ``variant``: 0 lets the library choose, 1 forces the kernel with 64-key blocks, 4 the kernel with
    128-key blocks (the library's own choice without a causal mask; with one it is 1).
    """
    import torch
    lib = load_library()
    if Q.dim() == 2:
        Bz, Hq, Hkv = 1, 1, 1
        S, D = Q.shape
    else:
        for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (O, "O")):
            _require(t, n, torch.bfloat16, 4)
        Bz, Hq, S, D = Q.shape
        Hkv = K.shape[1]
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (O, "O")):
        _require(t, n, torch.bfloat16)
    if K.shape != V.shape or K.shape[-2:] != Q.shape[-2:] or O.shape != Q.shape:
        raise ValueError(f"shape mismatch: Q {tuple(Q.shape)}, K {tuple(K.shape)}, V {tuple(V.shape)}, O {tuple(O.shape)}")
    lse_ptr = None
    if LSE is not None:
        _require(LSE, "LSE", torch.float32)
        if LSE.numel() != Bz * Hq * S:
            raise ValueError("LSE must hold B*H*S elements")
        lse_ptr = LSE.data_ptr()
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    _check(lib.warpir_attn_fwd_bf16_ex(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), lse_ptr,
                                       Bz, Hq, Hkv, S, D, float(softmax_scale), int(bool(causal)), int(variant),
                                       Q.device.index, _stream_of(Q)))


def launch_attention_backward(Q, K, V, O, dO, LSE, dQ, dK, dV, delta=None, softmax_scale: Optional[float] = None,
                              causal: bool = False) -> None:
    """Gradients of ``launch_attention``'s output: fills ``dQ`` (shape of Q), ``dK`` and
    ``dV`` (shape of K), all fp32, from ``dO`` and the forward's ``O`` and ``LSE``.

    Mirrors the reference's ``attention_backward(q, k, v, o, l_vec, og, causal)``
    (kernel_examples/attention/mha_h100.cu:799-1010) with caller-allocated outputs.
    ``delta`` is an fp32 ``[B, Hq, S]`` workspace; one is allocated with torch when omitted.
    Asynchronous on torch's current stream."""
    import torch
    lib = load_library()
    if Q.dim() == 2:
        Bz, Hq, Hkv = 1, 1, 1
        S, D = Q.shape
    else:
        Bz, Hq, S, D = Q.shape
        Hkv = K.shape[1]
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (O, "O"), (dO, "dO")):
        _require(t, n, torch.bfloat16, Q.dim())
    for t, n in ((LSE, "LSE"), (dQ, "dQ"), (dK, "dK"), (dV, "dV")):
        _require(t, n, torch.float32)
    if K.shape != V.shape or O.shape != Q.shape or dO.shape != Q.shape or K.shape[-2:] != Q.shape[-2:]:
        raise ValueError("shape mismatch between Q, K, V, O and dO")
    if dQ.shape != Q.shape or dK.shape != K.shape or dV.shape != V.shape:
        raise ValueError("dQ, dK, dV must have the shapes of Q, K, V")
    if LSE.numel() != Bz * Hq * S:
        raise ValueError("LSE must hold B*H*S elements")
    if delta is None:
        delta = torch.empty(Bz * Hq * S, dtype=torch.float32, device=Q.device)
    _require(delta, "delta", torch.float32)
    if delta.numel() < Bz * Hq * S:
        raise ValueError("delta must hold B*H*S elements")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    _check(lib.warpir_attn_bwd_bf16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), dO.data_ptr(),
                                    LSE.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), delta.data_ptr(),
                                    Bz, Hq, Hkv, S, D, float(softmax_scale), int(bool(causal)),
                                    Q.device.index, _stream_of(Q)))


def read_status(device=None) -> None:
    """Synchronise torch's current stream on ``device`` and raise ``WarpirError``
    if any kernel launched so far reported a failed (bounded) wait."""
    import torch
    lib = load_library()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code, detail = ctypes.c_int(0), ctypes.c_int(0)
    rc = lib.warpir_read_status(dev.index, torch.cuda.current_stream(dev).cuda_stream,
                                ctypes.byref(code), ctypes.byref(detail))
    _check(rc)


# --------------------------------------------------------------------------- lowered programs
_JIT_DIR = Path(__file__).resolve().parent / "_jit"


class LoadedKernel:
    """A compiled translation unit emitted by ``Sm100Lowerer``, callable on torch tensors.

    Stands in for the module the reference gets from ``load_inline`` plus its
    hand-written launch wrapper: ``mod.launch_gemm(A, B, C)`` /
    ``mod.launch_attention(Q, K, V, O)`` work as there (tensors in kernel-signature
    order, outputs pre-allocated, asynchronous on the current stream).
    """

    def __init__(self, so_path: Path, name: str):
        self.path = so_path
        self.name = name
        self._dll = ctypes.CDLL(str(so_path))
        vp, ci = ctypes.c_void_p, ctypes.c_int
        self._launch = getattr(self._dll, f"{name}_launch")
        self._launch.restype = ci
        self._launch.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_int64),
                                 ctypes.POINTER(ctypes.c_int64), ci, vp]
        self._err = getattr(self._dll, f"{name}_last_error")
        self._err.restype = ctypes.c_char_p
        kind = getattr(self._dll, f"{name}_kind")
        kind.restype = ctypes.c_char_p
        self.kind = kind().decode()
        self._status = getattr(self._dll, f"{name}_read_status")
        self._status.restype = ci
        self._status.argtypes = [ci, vp, ctypes.POINTER(ci), ctypes.POINTER(ci)]
        if self.kind == "gemm":
            self.launch_gemm = self.__call__
        elif self.kind == "attention":
            self.launch_attention = self.__call__
        # every kind also answers to the name the reference's wrappers would have
        # (``launch_<kernel name>``, tests/test_gemm_baseline.py:33-36)
        setattr(self, f"launch_{name}", self.__call__)

    def __call__(self, *tensors, causal: bool = False, LSE=None, ints=None) -> None:
        """Launch on torch's current stream.  ``tensors``: the global inputs then outputs in
        signature order.  ``ints``: the program's int inputs in signature order; programs
        emitted op by op (kind ``tile_program``) need them spelled out, the two recognised
        kinds derive their loop extent from the tensor shapes."""
        import torch
        for i, t in enumerate(tensors):
            _require(t, f"tensor {i}", torch.bfloat16)
        dev = tensors[0].device
        if any(t.device != dev for t in tensors):
            raise ValueError("all tensors must be on one device")
        n = len(tensors)
        ptrs = (ctypes.c_void_p * (n + 1))(*[t.data_ptr() for t in tensors], None)
        if LSE is not None:
            _require(LSE, "LSE", torch.float32)
            ptrs[n] = LSE.data_ptr()
        flat = []
        for t in tensors:
            shape = list(t.shape)
            if len(shape) > 4:
                raise ValueError("tensors have at most four dimensions")
            flat += [1] * (4 - len(shape)) + shape
        dims = (ctypes.c_int64 * len(flat))(*flat)
        # the program's int inputs (its loop extent) are implied by the tensor shapes
        if self.kind == "tile_program":
            if causal or LSE is not None:
                raise ValueError("causal= and LSE= belong to the recognised attention kernel")
            vals = [int(v) for v in (ints or ())]
            scalars = (ctypes.c_int64 * max(4, len(vals) + 1))(*vals)
        else:
            scalars = (ctypes.c_int64 * 4)(int(tensors[0].shape[-1]), int(bool(causal)), 0, 0)
            if self.kind == "attention":
                scalars[0] = int(tensors[0].shape[-2])
        rc = self._launch(ptrs, dims, scalars, dev.index, _stream_of(tensors[0]))
        if rc != 0:
            raise WarpirError(rc, load_library().warpir_strerror(rc).decode(), self._err().decode())

    def read_status(self, device=None) -> None:
        import torch
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        code, detail = ctypes.c_int(0), ctypes.c_int(0)
        rc = self._status(dev.index, torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(code),
                          ctypes.byref(detail))
        if rc != 0:
            raise WarpirError(rc, load_library().warpir_strerror(rc).decode(), self._err().decode())


def _included_text(source: str, repo_root: Path) -> str:
    """Text of every header of this package that ``source`` includes, directly or not (the
    cache key of a compiled translation unit covers exactly what it is built from)."""
    import re
    csrc = repo_root / "warpir_b200" / "csrc"
    seen, todo = {}, re.findall(r'#include "warpir_b200/csrc/([\w.]+)"', source)
    while todo:
        name = todo.pop()
        path = csrc / name
        if name in seen or not path.exists():
            continue
        seen[name] = path.read_text()
        todo += re.findall(r'#include "([\w.]+)"', seen[name])
    seen["warpir_b200.h"] = (repo_root / "include" / "warpir_b200.h").read_text()
    return "".join(seen[k] for k in sorted(seen))


def compile_source(source: str, name: str) -> Path:
    """nvcc the emitted translation unit for sm_100a into ``warpir_b200/_jit`` (cached by
    content hash, in-tree so the built file travels with the checkout)."""
    import hashlib
    import subprocess
    from . import build as _build
    repo_root = Path(__file__).resolve().parent.parent
    deps = _included_text(source, repo_root)
    digest = hashlib.sha256((source + deps).encode()).hexdigest()[:16]
    _JIT_DIR.mkdir(exist_ok=True)
    so = _JIT_DIR / f"{name}_{digest}.so"
    if so.exists():
        return so
    cu = _JIT_DIR / f"{name}_{digest}.cu"
    cu.write_text(source)
    cmd = [_build.find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-I", str(repo_root), "-o", str(so), str(cu)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on the emitted source:\n{proc.stdout}{proc.stderr}")
    return so


def load(kernel_or_source, name: Optional[str] = None, op_by_op: bool = False) -> LoadedKernel:
    """Lower (if given a ``Kernel``), compile and load a tile program.

    Replaces the reference's ``lower`` + ``load_inline`` + launch-wrapper sequence
    (tests/test_gemm_baseline.py:52-74).  ``op_by_op=True`` emits even the two recognised
    programs one helper call per op instead of instantiating their hand-written kernels."""
    if isinstance(kernel_or_source, str):
        if name is None:
            raise ValueError("name= is needed when loading emitted source text")
        source = kernel_or_source
    else:
        from .lowering import Sm100Lowerer
        source = Sm100Lowerer(op_by_op=op_by_op).lower(kernel_or_source)
        name = kernel_or_source.name
    return LoadedKernel(compile_source(source, name), name)
