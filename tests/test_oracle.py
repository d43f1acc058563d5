"""The CPU oracle against fixtures produced by the reference itself (CPU only)."""
import math

import numpy as np
import pytest
import torch

from oracle import reference_ops as R


def bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_gemm_oracle_matches_reference_expression(golden_dir):
    z = np.load(golden_dir / "gemm_small.npz")
    A, B = bf16(z["A"]), bf16(z["B"])
    ref = torch.from_numpy(z["ref"])
    assert torch.equal(R.gemm_ref(A, B, b_layout=0), ref)
    # K-major storage of the same B gives the same product
    assert torch.allclose(R.gemm_ref(A, B.t().contiguous(), b_layout=1), ref, rtol=0, atol=1e-4)


@pytest.mark.parametrize("tag", ["n256_d64", "n128_d128"])
def test_attention_oracle_matches_reference_ref_attention(golden_dir, tag):
    z = np.load(golden_dir / "attention_small.npz")
    Q, K, V, O = (bf16(z[f"{tag}_{n}"]) for n in "QKVO")
    o, lse = R.attention_slice_ref(Q, K, V)            # default scale 1/sqrt(D), non-causal
    assert torch.equal(o.bfloat16(), O)               # bit-equal after the reference's final rounding
    scores = Q.float() @ K.float().T / math.sqrt(Q.shape[-1])
    assert torch.allclose(lse, torch.logsumexp(scores, -1))


def test_batched_attention_and_causal_mask():
    Q, K, V = R.attention_inputs(2, 4, 96, 64, seed=3, Hkv=2)
    O, L = R.attention_ref(Q, K, V, causal=True)
    assert O.shape == (2, 4, 96, 64) and L.shape == (2, 4, 96)
    # first query sees only key 0: output is V[0], LSE is the single score
    assert torch.allclose(O[1, 3, 0], V[1, 1, 0].float(), atol=1e-6)
    s00 = (Q[1, 3, 0].float() @ K[1, 1, 0].float()) / 8.0
    assert abs(L[1, 3, 0].item() - s00.item()) < 1e-5
    # slices= restricts the work; untouched slices stay NaN
    O2, _ = R.attention_ref(Q, K, V, causal=True, slices=range(2, 3))
    assert torch.isnan(O2[0, 0]).all() and torch.equal(O2[0, 2], O[0, 2])


def test_inputs_are_seeded_and_ordered():
    A1, B1 = R.gemm_inputs(8, 16, 24, seed=5)
    A2, B2 = R.gemm_inputs(8, 16, 24, seed=5)
    assert torch.equal(A1, A2) and torch.equal(B1, B2) and B1.shape == (16, 24)
    assert R.gemm_inputs(8, 16, 24, seed=5, b_layout=0)[1].shape == (24, 16)
    assert float(R.gemm_inputs(64, 64, 64, std=0.02)[0].float().std()) < 0.03


def test_error_metrics():
    ref = torch.tensor([[1.0, -2.0], [0.0, 4.0]])
    e = R.gemm_errors(ref.clone(), ref)
    assert e["normalised"] == 0 and e["elementwise"] == 0
    e = R.gemm_errors(ref + 0.04, ref)
    assert abs(e["normalised"] - 0.01) < 1e-6
    assert R.gemm_errors(torch.zeros(0, 4), torch.zeros(0, 4))["normalised"] == 0.0
    # bf16 rounding of an exact product stays far inside the gate
    A, B = R.gemm_inputs(64, 64, 256, seed=1)
    r = R.gemm_ref(A, B)
    e = R.gemm_errors(r.bfloat16(), r)
    assert e["normalised"] < 4e-3 and e["elementwise"] < 4.1e-3 < R.GEMM_REL_TOL


# ---- the C restatement of the tile programs against the torch oracle -------------------
def test_tile_gemm_c_restatement_matches_torch_oracle():
    from oracle import tile_oracle as T
    for b_layout in (0, 1):
        A, B = R.gemm_inputs(48, 40, 200, seed=4, b_layout=b_layout)
        C = T.tile_gemm(A, B, b_layout, tile=64)
        e = R.gemm_errors(C, R.gemm_ref(A, B, b_layout))
        assert e["normalised"] < 4e-3 and e["elementwise"] < R.GEMM_REL_TOL


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D,blk", [(64, 64), (128, 128)])
def test_tile_attention_c_restatement_matches_torch_oracle(D, blk, causal):
    from oracle import tile_oracle as T
    Q, K, V = R.attention_inputs(1, 1, 200, D, seed=8)
    O, L = T.tile_attention(Q[0, 0], K[0, 0], V[0, 0], 1.0 / math.sqrt(D), causal, blk, blk)
    O_ref, L_ref = R.attention_slice_ref(Q[0, 0], K[0, 0], V[0, 0], None, causal)
    assert (O.float() - O_ref).abs().max().item() <= R.ATTN_O_ABS_TOL
    assert (L - L_ref).abs().max().item() <= R.ATTN_LSE_ABS_TOL


def test_tile_attention_reproduces_reference_golden(golden_dir):
    """The reference's own program shape: one head, D = 64, 64-wide tiles, scale 1/8."""
    from oracle import tile_oracle as T
    z = np.load(golden_dir / "attention_small.npz")
    Q, K, V, O = (bf16(z[f"n256_d64_{n}"]) for n in "QKVO")
    O_c, _ = T.tile_attention(Q, K, V, 0.125, False, 64, 64)
    assert (O_c.float() - O.float()).abs().max().item() <= R.ATTN_O_ABS_TOL


@pytest.mark.parametrize("causal", [False, True])
def test_backward_oracle_matches_the_closed_form(causal):
    """The autograd oracle of the attention backward against the textbook expressions
    dV = P^T dO, dP = dO V^T, dS = P * (dP - rowsum(dO * O)) * scale, dQ = dS K, dK = dS^T Q,
    with grouped K/V heads summed over their query heads."""
    B, H, Hkv, S, D = 1, 4, 2, 96, 64
    Q, K, V = R.attention_inputs(B, H, S, D, seed=21, Hkv=Hkv)
    dO = R.randn_bf16((B, H, S, D), torch.Generator().manual_seed(22))
    dQ, dK, dV = R.attention_backward_ref(Q, K, V, dO, None, causal)
    scale = 1.0 / math.sqrt(D)
    dK2, dV2 = torch.zeros_like(dK), torch.zeros_like(dV)
    for h in range(H):
        hk = h // (H // Hkv)
        q, k, v, g = Q[0, h].double(), K[0, hk].double(), V[0, hk].double(), dO[0, h].double()
        s = q @ k.T * scale
        if causal:
            s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = p @ v
        ds = p * (g @ v.T - (g * o).sum(-1, keepdim=True)) * scale
        assert torch.allclose(dQ[0, h].double(), ds @ k, atol=1e-4, rtol=1e-4)
        dK2[0, hk] += (ds.T @ q).float()
        dV2[0, hk] += (p.T @ g).float()
    assert torch.allclose(dK, dK2, atol=1e-4, rtol=1e-4)
    assert torch.allclose(dV, dV2, atol=1e-4, rtol=1e-4)
