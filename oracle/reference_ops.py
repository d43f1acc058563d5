"""CPU restatement of the reference's numerical oracles.  TEST INFRASTRUCTURE ONLY.

The reference checks its generated kernels against two torch expressions:

* GEMM: ``torch.mm(A.float(), B.float())`` (reference: tests/test_gemm_baseline.py:85,
  tests/test_modal_gpu.py:115);
* attention forward: ``softmax(q @ k.T / sqrt(d)) @ v`` in fp32
  (reference: tests/test_modal_attention.py:92-98).

They are restated here to run on CPU tensors, extended with what the measured
workloads need and the reference's scripts lack: a batch x head loop, a
lower-triangular (causal) mask, an explicit ``softmax_scale`` and the natural
log-sum-exp of the scaled scores.  Parity pin: ``tests/test_oracle.py`` checks
these functions against fixtures produced by the reference's own
``_ref_attention`` and ``torch.mm`` expression (``tests/golden/make_golden.py``).

Also here: the seeded input generators for the five measured workloads and the
error metrics the parity tests gate on.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import torch

# ---------------------------------------------------------------------------
# seeded inputs
# ---------------------------------------------------------------------------


def randn_bf16(shape, gen: torch.Generator, std: float = 1.0) -> torch.Tensor:
    """fp32 normal draws from ``gen`` (CPU), scaled, rounded to bf16."""
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    if std != 1.0:
        x = x * std
    return x.to(torch.bfloat16)


def gemm_inputs(M: int, N: int, K: int, seed: int = 0, std: float = 1.0,
                b_layout: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """A ``[M,K]`` row-major and B as stored: ``[N,K]`` (K-major, ``b_layout=1``)
    or ``[K,N]`` (row-major, ``b_layout=0``, the layout of the reference's GEMM
    tile program, tests/gemm_baseline_v2.py:78-79).  A is drawn first."""
    g = torch.Generator().manual_seed(seed)
    A = randn_bf16((M, K), g, std)
    B = randn_bf16((N, K) if b_layout == 1 else (K, N), g, std)
    return A, B


def attention_inputs(B: int, H: int, S: int, D: int, seed: int = 0,
                     Hkv: Optional[int] = None):
    """Q ``[B,H,S,D]``, K and V ``[B,Hkv,S,D]`` contiguous bf16, drawn in that order."""
    g = torch.Generator().manual_seed(seed)
    Hkv = H if Hkv is None else Hkv
    Q = randn_bf16((B, H, S, D), g)
    K = randn_bf16((B, Hkv, S, D), g)
    V = randn_bf16((B, Hkv, S, D), g)
    return Q, K, V


# ---------------------------------------------------------------------------
# the two reference computations
# ---------------------------------------------------------------------------


def gemm_ref(A: torch.Tensor, B_store: torch.Tensor, b_layout: int = 1) -> torch.Tensor:
    """fp32 ``A @ B`` on CPU (tests/test_gemm_baseline.py:85), not re-rounded to bf16."""
    A32 = A.float()
    B32 = B_store.float()
    return torch.mm(A32, B32.t() if b_layout == 1 else B32)


def attention_slice_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                        scale: Optional[float] = None, causal: bool = False):
    """One head: the reference's ``_ref_attention`` (tests/test_modal_attention.py:92-98)
    kept in fp32, plus the causal mask and the log-sum-exp.  Returns ``(O[S,D], LSE[S])``."""
    q, k, v = q.float(), k.float(), v.float()
    if scale is None:
        scores = q @ k.T / math.sqrt(q.size(-1))   # the reference's own spelling
    else:
        scores = (q @ k.T) * scale
    if causal:
        Sq, Sk = scores.shape
        keep = torch.ones(Sq, Sk, dtype=torch.bool).tril(diagonal=Sk - Sq)
        scores = scores.masked_fill(~keep, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    P = torch.softmax(scores, dim=-1)
    return P @ v, lse


def attention_ref(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                  scale: Optional[float] = None, causal: bool = False,
                  slices: Optional[range] = None):
    """Batched: loops the one-head computation over ``batch x head`` (one slice at
    a time so the score matrix stays small).  ``slices`` restricts the loop to a
    subset of flat ``b*H+h`` indices; untouched slices are returned as NaN."""
    Bz, H, S, D = Q.shape
    Hkv = K.shape[1]
    O = torch.full((Bz, H, S, D), float("nan"), dtype=torch.float32)
    L = torch.full((Bz, H, S), float("nan"), dtype=torch.float32)
    idx = range(Bz * H) if slices is None else slices
    for flat in idx:
        b, h = divmod(flat, H)
        hk = h // (H // Hkv)
        O[b, h], L[b, h] = attention_slice_ref(Q[b, h], K[b, hk], V[b, hk], scale, causal)
    return O, L


def attention_backward_ref(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, dO: torch.Tensor,
                           scale: Optional[float] = None, causal: bool = False):
    """Gradients of ``attention_ref``'s output by torch autograd on fp32 CPU tensors (the
    definition the reference's own backward, kernel_examples/attention/mha_h100.cu:483-642,
    is meant to match; the reference ships no test of it).  With grouped K/V heads the
    gradients of K and V are summed over the query heads of a group.  Returns
    ``(dQ, dK, dV)`` in fp32."""
    Bz, H, S, D = Q.shape
    Hkv = K.shape[1]
    q = Q.float().clone().requires_grad_(True)
    k = K.float().clone().requires_grad_(True)
    v = V.float().clone().requires_grad_(True)
    total = None
    for b in range(Bz):
        for h in range(H):
            hk = h // (H // Hkv)
            o, _ = attention_slice_ref(q[b, h], k[b, hk], v[b, hk], scale, causal)
            term = (o * dO[b, h].float()).sum()
            total = term if total is None else total + term
    total.backward()
    return q.grad, k.grad, v.grad


ATTN_GRAD_REL_TOL = 1e-2  # max |grad - ref| / max |ref|, attention backward (P and dS are rounded to bf16)


# ---------------------------------------------------------------------------
# error metrics
# ---------------------------------------------------------------------------


def gemm_errors(C: torch.Tensor, ref: torch.Tensor) -> Dict[str, float]:
    """Two relative-error figures for a GEMM result against the fp32 oracle:

    * ``normalised``: ``max|C - ref| / max|ref|``;
    * ``elementwise``: ``max(|C - ref| / max(|ref|, tau))`` with the floor
      ``tau = 2**-7 * rms(ref)`` -- a plain element-wise ratio is ill-defined at
      outputs that cancel to nearly zero, where fp32 summation-order noise of
      the large terms dominates.

    Both are gated at 1e-2 (the tolerance the workload definition states).
    """
    C = C.float()
    ref = ref.float()
    diff = (C - ref).abs()
    if ref.numel() == 0:
        return {"normalised": 0.0, "elementwise": 0.0, "max_abs": 0.0}
    peak = ref.abs().max().item()
    rms = ref.pow(2).mean().sqrt().item()
    tau = max(rms * 2.0 ** -7, 1e-30)
    return {
        "normalised": (diff.max().item() / peak) if peak > 0 else diff.max().item(),
        "elementwise": (diff / ref.abs().clamp_min(tau)).max().item(),
        "max_abs": diff.max().item(),
    }


GEMM_REL_TOL = 1e-2      # max relative error, GEMM
ATTN_O_ABS_TOL = 2e-2    # max absolute error, attention output
ATTN_LSE_ABS_TOL = 1e-3  # max absolute error, log-sum-exp


def attention_errors(O, L, O_ref, L_ref) -> Dict[str, float]:
    mask = ~torch.isnan(O_ref)
    o = (O.float() - O_ref)[mask].abs().max().item() if mask.any() else 0.0
    lm = ~torch.isnan(L_ref)
    l = (L.float() - L_ref)[lm].abs().max().item() if lm.any() else 0.0
    return {"o_max_abs": o, "lse_max_abs": l}


def host_threads() -> int:
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    return n
