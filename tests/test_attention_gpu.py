"""Attention-forward parity on a B200 vs the CPU oracle.

Tolerances (stated by the workload definition): max |O - O_ref| <= 2e-2 with
O_ref kept in fp32, max |LSE - LSE_ref| <= 1e-3.
"""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def run_attn(Q, K, V, causal, scale=None, want_lse=True, variant=0):
    Qd = Q.cuda()
    O = torch.full_like(Qd, float("nan"))
    L = torch.full(Q.shape[:-1], float("nan"), device="cuda") if want_lse else None
    runtime.launch_attention(Qd, K.cuda(), V.cuda(), O, L, scale, causal, variant)
    runtime.read_status()
    return O.cpu(), (L.cpu() if want_lse else None)


def check(O, L, O_ref, L_ref):
    assert not torch.isnan(O.float()).any() and not torch.isnan(L).any()
    e = R.attention_errors(O, L, O_ref, L_ref)
    assert e["o_max_abs"] <= R.ATTN_O_ABS_TOL and e["lse_max_abs"] <= R.ATTN_LSE_ABS_TOL, e


@pytest.mark.parametrize("tag", ["n256_d64", "n128_d128"])
def test_reference_golden_vectors(golden_dir, tag, lib):
    """Single-head [N, D] call, as the reference's launch_attention is used."""
    z = np.load(golden_dir / "attention_small.npz")
    Q, K, V, O_gold = (torch.from_numpy(z[f"{tag}_{n}"].view(np.int16).copy()).view(torch.bfloat16) for n in "QKVO")
    O, _ = run_attn(Q, K, V, False)
    assert (O.float() - O_gold.float()).abs().max().item() <= R.ATTN_O_ABS_TOL


# the reference's sweep: one head, D = 64, N in {64 .. 1024} (tests/test_modal_attention.py:178)
@pytest.mark.parametrize("n", [64, 128, 256, 512, 1024])
def test_reference_sweep_single_head(n, lib):
    Q, K, V = R.attention_inputs(1, 1, n, 64, seed=n)
    O, L = run_attn(Q, K, V, False)
    check(O, L, *R.attention_ref(Q, K, V))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [1, 100, 128, 129, 384, 1000])
def test_ragged_lengths(S, D, causal, lib):
    Q, K, V = R.attention_inputs(2, 3, S, D, seed=S + D)
    O, L = run_attn(Q, K, V, causal)
    check(O, L, *R.attention_ref(Q, K, V, None, causal))


@pytest.mark.parametrize("variant", [1, 4])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1, 129, 512, 700, 1100, 2048])
def test_every_kernel_variant_at_d128(S, causal, variant, lib):
    """Both forward kernels (64-key blocks: 1, 128-key blocks: 4) against the oracle, with grouped K/V heads,
    across lengths that leave tiles partly or wholly past the end of the sequence."""
    Q, K, V = R.attention_inputs(2, 4, S, 128, seed=S + variant, Hkv=2)
    O, L = run_attn(Q, K, V, causal, variant=variant)
    check(O, L, *R.attention_ref(Q, K, V, None, causal))


@pytest.mark.parametrize("variant", [1, 4])
def test_rescale_path_in_every_variant(variant, lib):
    Q, K, V = R.attention_inputs(1, 2, 1024, 128, seed=2)
    ramp = torch.linspace(0.2, 6.0, 1024).view(1, 1, 1024, 1)
    K = (K.float() * ramp).bfloat16()
    O, L = run_attn(Q, K, V, True, variant=variant)
    check(O, L, *R.attention_ref(Q, K, V, None, True))


@pytest.mark.parametrize("variant", [1, 4])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1, 100, 384, 1000, 2048])
def test_kernel_variants_at_d64(S, causal, variant, lib):
    Q, K, V = R.attention_inputs(2, 4, S, 64, seed=S + variant, Hkv=4)
    O, L = run_attn(Q, K, V, causal, variant=variant)
    check(O, L, *R.attention_ref(Q, K, V, None, causal))
    if S == 1000:      # steep score growth: the lazy rescale fires in both column halves
        ramp = torch.linspace(0.2, 6.0, S).view(1, 1, S, 1)
        K2 = (K.float() * ramp).bfloat16()
        O, L = run_attn(Q, K2, V, causal, variant=variant)
        check(O, L, *R.attention_ref(Q, K2, V, None, causal))


def test_variant_rejections(lib):
    Q, K, V = (t.cuda() for t in R.attention_inputs(1, 1, 64, 64, seed=1))
    O = torch.empty_like(Q)
    for bad in (2, 3, 5, -1):                     # only 0 (choose), 1 and 4 name a kernel
        with pytest.raises(runtime.WarpirError):
            runtime.launch_attention(Q, K, V, O, None, None, False, bad)


def test_grouped_kv_heads_and_custom_scale(lib):
    Q, K, V = R.attention_inputs(2, 8, 640, 128, seed=5, Hkv=2)
    O, L = run_attn(Q, K, V, True, scale=0.05)
    check(O, L, *R.attention_ref(Q, K, V, 0.05, True))


def test_lse_optional(lib):
    Q, K, V = R.attention_inputs(1, 2, 256, 64, seed=9)
    O, _ = run_attn(Q, K, V, False, want_lse=False)
    O_ref, _ = R.attention_ref(Q, K, V)
    assert (O.float() - O_ref).abs().max().item() <= R.ATTN_O_ABS_TOL


def test_large_magnitude_scores_exercise_the_rescale_path(lib):
    """Scores grow along the sequence so the running max keeps moving by more than
    the lazy-rescale threshold."""
    Q, K, V = R.attention_inputs(1, 2, 1024, 128, seed=2)
    ramp = torch.linspace(0.2, 6.0, 1024).view(1, 1, 1024, 1)
    K = (K.float() * ramp).bfloat16()
    O, L = run_attn(Q, K, V, False)
    check(O, L, *R.attention_ref(Q, K, V))


@pytest.mark.parametrize("cfg", [(1, 4, 4096, 128, False), (1, 4, 8192, 128, True), (1, 2, 8192, 64, True)])
def test_benchmark_shapes_on_sampled_slices(cfg, lib):
    """Full sequence lengths of the measured workloads, a few batch x head slices
    checked against the oracle."""
    B, H, S, D, causal = cfg
    Q, K, V = R.attention_inputs(B, H, S, D, seed=S)
    O, L = run_attn(Q, K, V, causal)
    O_ref, L_ref = R.attention_ref(Q, K, V, None, causal, slices=range(0, B * H, max(1, B * H // 2)))
    check(O, L, O_ref, L_ref)


def test_full_size_property_v_linearity(lib):
    """Config-4 sized call; softmax rows sum to one, so with V == 1 every output is 1,
    and the output is linear in V: attn(Q,K,2V) == 2 attn(Q,K,V) exactly in bf16."""
    B, H, S, D = 4, 16, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    Q = torch.randn(B, H, S, D, generator=g, device="cuda").bfloat16()
    K = torch.randn(B, H, S, D, generator=g, device="cuda").bfloat16()
    V = torch.randn(B, H, S, D, generator=g, device="cuda").bfloat16()
    O1, O2, O3 = torch.empty_like(Q), torch.empty_like(Q), torch.empty_like(Q)
    runtime.launch_attention(Q, K, V, O1)
    runtime.launch_attention(Q, K, V * 2, O2)
    runtime.launch_attention(Q, K, torch.ones_like(V), O3)
    runtime.read_status()
    assert torch.equal((O1.float() * 2).bfloat16(), O2)
    assert (O3.float() - 1).abs().max().item() <= 8e-3


@pytest.mark.parametrize("cfg", [(1, 4, 16384, 128), (1, 2, 20000, 128), (1, 2, 32768, 64)])
def test_long_sequences_on_sampled_rows(cfg, lib):
    """Hundreds of K/V blocks per Q tile (every barrier parity wraps many times) and a ragged
    last block.  Without a causal mask a query row's output depends on that row of Q only, so
    sampled rows are checked with the oracle's expression (softmax(q K^T / sqrt(D)) V in fp32 on
    the CPU) instead of the full S x S problem."""
    B, H, S, D = cfg
    Q, K, V = R.attention_inputs(B, H, S, D, seed=S)
    O, L = run_attn(Q, K, V, False)
    assert not torch.isnan(O.float()).any() and not torch.isnan(L).any()   # every row was written
    rows = torch.randint(0, S, (96,), generator=torch.Generator().manual_seed(S))
    scores = Q[:, :, rows].float() @ K.float().transpose(-1, -2) / D ** 0.5
    O_ref = torch.softmax(scores, -1) @ V.float()
    L_ref = torch.logsumexp(scores, -1)
    assert (O[:, :, rows].float() - O_ref).abs().max().item() <= R.ATTN_O_ABS_TOL
    assert (L[:, :, rows] - L_ref).abs().max().item() <= R.ATTN_LSE_ABS_TOL


def test_rejections(lib):
    Q = torch.zeros(1, 1, 128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(runtime.WarpirError) as ei:
        runtime.launch_attention(Q, Q, Q, torch.empty_like(Q))
    assert ei.value.code == -3


def test_three_score_tiles_give_the_same_bits_every_launch(lib):
    """D = 64 runs the 128-key kernel with three score tiles rotating between the two Q tiles, so a Q
    tile's softmax can be a block ahead of the warp that issues the MMAs.  Its hand-offs must not
    depend on who is ahead: the same inputs give the same bits, launch after launch, and no wait
    runs into its limit (which would raise)."""
    for S, causal in ((2048, True), (1000, False)):
        Q, K, V = (t.cuda() for t in R.attention_inputs(2, 4, S, 64, seed=S))
        first = None
        for _ in range(40):
            O = torch.empty_like(Q)
            L = torch.empty(2, 4, S, device="cuda")
            runtime.launch_attention(Q, K, V, O, L, None, causal, 4)
            runtime.read_status()
            if first is None:
                first = (O, L)
            else:
                assert torch.equal(O, first[0]) and torch.equal(L, first[1])
