"""Attention backward on a B200 through the C ABI against torch autograd of the CPU oracle.

Tolerance: for each of dQ, dK, dV the largest error is at most 1e-2 of the largest
reference magnitude (P and dS go through bf16 before their matrix products, as in the
forward).  The reference ships no test for its backward kernel; the oracle here is the
derivative of the forward oracle, which is pinned to the reference's own torch
computation."""
import math

import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def run_case(B, H, Hkv, S, D, causal, seed=0, scale=None):
    Q, K, V = R.attention_inputs(B, H, S, D, seed=seed, Hkv=Hkv)
    gen = torch.Generator().manual_seed(seed + 1000)
    dO = R.randn_bf16((B, H, S, D), gen)
    Qd, Kd, Vd, dOd = (t.cuda() for t in (Q, K, V, dO))
    O = torch.empty_like(Qd)
    LSE = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    runtime.launch_attention(Qd, Kd, Vd, O, LSE, scale, causal)
    nan = float("nan")
    dQ = torch.full(Qd.shape, nan, dtype=torch.float32, device="cuda")
    dK = torch.full(Kd.shape, nan, dtype=torch.float32, device="cuda")
    dV = torch.full(Vd.shape, nan, dtype=torch.float32, device="cuda")
    runtime.launch_attention_backward(Qd, Kd, Vd, O, dOd, LSE, dQ, dK, dV, softmax_scale=scale, causal=causal)
    runtime.read_status()
    ref = R.attention_backward_ref(Q, K, V, dO, scale, causal)
    out = {}
    for name, got, want in zip(("dQ", "dK", "dV"), (dQ, dK, dV), ref):
        got = got.cpu()
        assert not torch.isnan(got).any(), name
        out[name] = ((got - want).abs().max() / want.abs().max()).item()
    return out, (dQ, dK, dV)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [64, 128, 200, 384])
def test_backward_matches_autograd(D, causal, S, lib):
    err, _ = run_case(1, 2, 2, S, D, causal, seed=S + D)
    assert max(err.values()) <= R.ATTN_GRAD_REL_TOL, err


@pytest.mark.parametrize("causal", [False, True])
def test_backward_grouped_heads_and_batch(causal, lib):
    err, _ = run_case(2, 4, 2, 320, 128, causal, seed=5)
    assert max(err.values()) <= R.ATTN_GRAD_REL_TOL, err
    err, _ = run_case(1, 8, 1, 192, 64, causal, seed=6)
    assert max(err.values()) <= R.ATTN_GRAD_REL_TOL, err


def test_backward_custom_scale_and_longer_sequence(lib):
    err, _ = run_case(1, 1, 1, 1024, 128, True, seed=7, scale=0.05)
    assert max(err.values()) <= R.ATTN_GRAD_REL_TOL, err


def test_backward_repeats_bit_for_bit(lib):
    _, first = run_case(1, 2, 1, 512, 128, True, seed=8)
    _, second = run_case(1, 2, 1, 512, 128, True, seed=8)
    for a, b in zip(first, second):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_backward_rejections(lib):
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device="cuda")
    Q, K, V, O, dO = (z(1, 2, 64, 64) for _ in range(5))
    L = z(1, 2, 64, dt=torch.float32)
    dQ, dK, dV = (z(1, 2, 64, 64, dt=torch.float32) for _ in range(3))
    with pytest.raises(TypeError):
        runtime.launch_attention_backward(Q, K, V, O, dO, L, dQ.bfloat16(), dK, dV)
    with pytest.raises(ValueError):
        runtime.launch_attention_backward(Q, K, V, O, dO, L, dQ, dK, z(1, 1, 64, 64, dt=torch.float32))
    Q96 = z(1, 2, 64, 96)
    with pytest.raises(runtime.WarpirError):
        runtime.launch_attention_backward(Q96, Q96, Q96, Q96, Q96, L, z(1, 2, 64, 96, dt=torch.float32),
                                          z(1, 2, 64, 96, dt=torch.float32), z(1, 2, 64, 96, dt=torch.float32))


def test_the_64_row_kernel_stays_correct():
    """The library runs the backward in steps of 128 streamed rows; the kernel that streams 64 rows per step
    remains selectable (WARPIR_ATTN_BWD_ROWS=64, read once per process, hence the child process) and must keep
    passing the same comparison."""
    import os
    import subprocess
    import sys
    import textwrap
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    script = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        sys.path.insert(0, %r)
        import test_attention_backward_gpu as t
        from oracle import reference_ops as R
        for (B, H, Hkv, S, D, causal) in [(1, 2, 2, 200, 128, True), (2, 4, 2, 320, 128, False), (1, 8, 1, 192, 64, True)]:
            err, _ = t.run_case(B, H, Hkv, S, D, causal, seed=S + D)
            assert max(err.values()) <= R.ATTN_GRAD_REL_TOL, err
        print("OK")
    """ % (str(root), str(root / "tests")))
    env = dict(os.environ, WARPIR_ATTN_BWD_ROWS="64")
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and proc.stdout.strip().endswith("OK"), proc.stdout + proc.stderr
