"""ctypes wrapper of ``tile_oracle.c``.  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "libtile_oracle.so"
_lib = None


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    return LIB


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
    return _lib


def _bits(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.contiguous().view(torch.int16).numpy().view(np.uint16))


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def tile_gemm(A: torch.Tensor, B: torch.Tensor, b_layout: int = 1, tile: int = 64) -> torch.Tensor:
    lib = _load()
    M, K = A.shape
    N = B.shape[0] if b_layout == 1 else B.shape[1]
    a, b = _bits(A), _bits(B)
    c = np.zeros((M, N), dtype=np.uint16)
    vp = ctypes.c_void_p
    lib.tile_gemm(vp(a.ctypes.data), vp(b.ctypes.data), vp(c.ctypes.data), M, N, K, b_layout, tile)
    return _bf16(c)


def tile_attention(Q, K, V, scale: float, causal: bool, block_q: int = 64, block_kv: int = 64):
    """One head: Q, K, V ``[S, D]`` bf16 -> (O ``[S, D]`` bf16, LSE ``[S]`` fp32)."""
    lib = _load()
    S, D = Q.shape
    q, k, v = _bits(Q), _bits(K), _bits(V)
    o = np.zeros((S, D), dtype=np.uint16)
    lse = np.zeros(S, dtype=np.float32)
    vp = ctypes.c_void_p
    lib.tile_attention(vp(q.ctypes.data), vp(k.ctypes.data), vp(v.ctypes.data), vp(o.ctypes.data),
                       vp(lse.ctypes.data), S, D, ctypes.c_float(scale), int(causal), block_q, block_kv)
    return _bf16(o), torch.from_numpy(lse)
