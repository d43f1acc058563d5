"""Parity at the exact shapes the benchmark times, through the C ABI.

The reference checks every size it times (reference: tests/test_modal_gpu.py:184-196,
tests/test_modal_attention.py:178-187).  At these sizes the CPU oracle cannot finish the whole
problem in seconds, so each case checks

* the oracle on sampled row blocks (GEMM) or on whole batch x head slices spread over the grid,
  first and last included (attention);
* sampled query rows of EVERY batch x head slice with the oracle's row-wise expression
  (softmax(q K^T scale) V and its log-sum-exp in fp32 on the CPU, keys past the row masked when
  causal), so that no slice of the grid goes unchecked;
* a size-independent identity over the whole output (linearity in A, or in V).

Inputs are the seeded CPU draws of ``oracle.reference_ops`` (N(0,1), or N(0,1) * 0.02 for the
rectangular GEMM).  Tolerances are the workload's: GEMM max relative error 1e-2, attention
|O - O_ref| <= 2e-2 and |LSE - LSE_ref| <= 1e-3.
"""
import math

import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def _gemm_case(M, N, K, std, seed):
    A, B = R.gemm_inputs(M, N, K, seed=seed, std=std)
    Ad, Bd = A.cuda(), B.cuda()
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    C2 = torch.empty_like(C)
    runtime.launch_gemm(Ad, Bd, C, 1)
    runtime.launch_gemm(Ad * 2, Bd, C2, 1)
    runtime.read_status()
    assert not torch.isnan(C.float()).any()
    # linearity over the whole output: doubling A doubles every fp32 sum exactly
    assert torch.equal((C.float() * 2).bfloat16(), C2)
    # oracle on row blocks spread over M: first, last, and blocks straddling tile boundaries
    starts = sorted({0, 96, M // 2 - 32, M // 2 + 224, M - 64} | {(M // 7) * i + 17 for i in range(1, 7)})
    rows = torch.cat([torch.arange(s, min(s + 64, M)) for s in starts])
    ref = R.gemm_ref(A[rows], B, 1)
    e = R.gemm_errors(C[rows.cuda()].cpu(), ref)
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


def test_gemm_4096_cubed(lib):
    _gemm_case(4096, 4096, 4096, 1.0, seed=4096)


def test_gemm_16384x4096x8192(lib):
    _gemm_case(16384, 4096, 8192, 0.02, seed=3)


@pytest.mark.parametrize("block", [0, 3, 7])
def test_gemm_8192_row_block_of_the_eight_way_split(block, lib):
    """The 8-GPU run gives each GPU 1024 rows of A and the whole B; the shard's result is checked
    against the oracle on its own."""
    g = torch.Generator().manual_seed(0)
    A_full_rows = R.randn_bf16((8192, 8192), g)[block * 1024:(block + 1) * 1024]
    B = R.randn_bf16((8192, 8192), g)
    C = torch.full((1024, 8192), float("nan"), dtype=torch.bfloat16, device="cuda")
    runtime.launch_gemm(A_full_rows.cuda(), B.cuda(), C, 1)
    runtime.read_status()
    rows = torch.cat([torch.arange(s, s + 32) for s in (0, 240, 500, 992)])
    e = R.gemm_errors(C[rows.cuda()].cpu(), R.gemm_ref(A_full_rows[rows], B, 1))
    assert not torch.isnan(C.float()).any()
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


def _attention_case(B, H, S, D, causal, seed):
    Q, K, V = R.attention_inputs(B, H, S, D, seed=seed)
    Qd, Kd, Vd = Q.cuda(), K.cuda(), V.cuda()
    O = torch.full_like(Qd, float("nan"))
    L = torch.full((B, H, S), float("nan"), device="cuda")
    O2 = torch.empty_like(Qd)
    runtime.launch_attention(Qd, Kd, Vd, O, L, None, causal)
    runtime.launch_attention(Qd, Kd, Vd * 2, O2, None, None, causal)
    runtime.read_status()
    assert not torch.isnan(O.float()).any() and not torch.isnan(L).any()
    # linear in V over the whole grid
    assert torch.equal((O.float() * 2).bfloat16(), O2)
    Oc, Lc = O.cpu(), L.cpu()
    # whole slices: first, last and two in between
    n = B * H
    slices = sorted({0, n // 3, (2 * n) // 3 + 1, n - 1})
    O_ref, L_ref = R.attention_ref(Q, K, V, None, causal, slices=slices)
    e = R.attention_errors(Oc, Lc, O_ref, L_ref)
    assert e["o_max_abs"] <= R.ATTN_O_ABS_TOL and e["lse_max_abs"] <= R.ATTN_LSE_ABS_TOL, e
    # sampled rows of every slice (a row's output depends on that row of Q only)
    gen = torch.Generator().manual_seed(S + D)
    rows = torch.cat([torch.tensor([0, 127, 128, S - 1]), torch.randint(0, S, (8,), generator=gen)])
    worst_o = worst_l = 0.0
    for b in range(B):                                     # one batch entry at a time keeps the scores small
        scores = (Q[b][:, rows].float() @ K[b].float().transpose(-1, -2)) / math.sqrt(D)      # [H, rows, S]
        if causal:
            visible = torch.arange(S).view(1, 1, S) <= rows.view(1, -1, 1)
            scores = scores.masked_fill(~visible, float("-inf"))
        o_ref = torch.softmax(scores, -1) @ V[b].float()
        l_ref = torch.logsumexp(scores, -1)
        worst_o = max(worst_o, (Oc[b][:, rows].float() - o_ref).abs().max().item())
        worst_l = max(worst_l, (Lc[b][:, rows] - l_ref).abs().max().item())
    assert worst_o <= R.ATTN_O_ABS_TOL and worst_l <= R.ATTN_LSE_ABS_TOL, (worst_o, worst_l)


def test_attention_noncausal_b16_h16_s4096_d128(lib):
    _attention_case(16, 16, 4096, 128, False, seed=0)


@pytest.mark.parametrize("D", [64, 128])
def test_attention_causal_b4_h32_s8192(D, lib):
    _attention_case(4, 32, 8192, D, True, seed=D)


def _backward_case(B, H, S, D, causal, seed, slices):
    """Attention backward at a benchmark shape: exactly linear in dO over the whole grid (doubling dO is
    exact in bf16 and in every fp32 accumulation), and whole batch x head slices against autograd of the
    CPU oracle."""
    Q, K, V = R.attention_inputs(B, H, S, D, seed=seed)
    dO = R.randn_bf16((B, H, S, D), torch.Generator().manual_seed(seed + 1000))
    Qd, Kd, Vd, dOd = (t.cuda() for t in (Q, K, V, dO))
    O = torch.empty_like(Qd)
    LSE = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    runtime.launch_attention(Qd, Kd, Vd, O, LSE, None, causal)

    def grads(g):
        out = [torch.full(t.shape, float("nan"), dtype=torch.float32, device="cuda") for t in (Qd, Kd, Vd)]
        runtime.launch_attention_backward(Qd, Kd, Vd, O, g, LSE, *out, causal=causal)
        runtime.read_status()
        return out

    once = grads(dOd)
    twice = grads(dOd * 2)
    for name, a, b in zip(("dQ", "dK", "dV"), once, twice):
        assert not torch.isnan(a).any(), name
        assert torch.equal(a * 2, b), name
    for b, h in slices:
        ref = R.attention_backward_ref(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1],
                                       dO[b:b + 1, h:h + 1], None, causal)
        for name, got, want in zip(("dQ", "dK", "dV"), once, ref):
            err = ((got[b, h].cpu() - want[0, 0]).abs().max() / want.abs().max()).item()
            assert err <= R.ATTN_GRAD_REL_TOL, (name, b, h, err)


def test_attention_backward_noncausal_b16_h16_s4096_d128(lib):
    _backward_case(16, 16, 4096, 128, False, seed=3, slices=[(0, 0), (9, 7), (15, 15)])


@pytest.mark.parametrize("D", [64, 128])
def test_attention_backward_causal_b4_h32_s8192(D, lib):
    _backward_case(4, 32, 8192, D, True, seed=4 + D, slices=[(0, 0), (3, 31)])
