"""The CPU interpreter of the tile IR against torch, and the op-by-op emitter's text.

The interpreter is the checker for programs that have no closed-form oracle of their own;
here it is itself pinned: the reference's two tile programs, run through it, must agree
with the reference's torch oracles, and each extra program with its definition in torch.
"""
import math

import pytest
import torch

from oracle import ir_interp
from oracle import reference_ops as R
from warpir_b200.lowering import Sm100Lowerer
from warpir_b200.lowering.generic import emit_tile_program
from warpir_b200.passes.modulo_scheduler import REFERENCE_MODEL, kernel_pass
from warpir_b200.programs import build_attention_kernel, build_gemm_kernel

import tile_programs as TP


def rnd(gen, *shape, std=1.0):
    return (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)


def bf16_close(out, ref, rel=1e-2):
    """Output rounded to bf16: error at most `rel` of the largest reference magnitude."""
    err = (out.float() - ref).abs().max().item()
    return err <= rel * max(ref.abs().max().item(), 1e-6)


def test_reference_gemm_program_matches_the_reference_oracle():
    gen = torch.Generator().manual_seed(0)
    A, B = rnd(gen, 128, 256), rnd(gen, 256, 192)
    C = torch.zeros(128, 192, dtype=torch.bfloat16)
    ir_interp.run_kernel(build_gemm_kernel(), {"A": A, "B": B, "C_global": C}, {"N": 256})
    err = R.gemm_errors(C, R.gemm_ref(A, B, 0))
    assert err["normalised"] <= R.GEMM_REL_TOL and err["elementwise"] <= R.GEMM_REL_TOL, err


@pytest.mark.parametrize("k_extent", [64, 128, 192, 448])
def test_pipelined_form_computes_the_same_product(k_extent):
    gen = torch.Generator().manual_seed(1)
    A, B = rnd(gen, 64, k_extent), rnd(gen, k_extent, 64)
    plain, piped = (torch.zeros(64, 64, dtype=torch.bfloat16) for _ in range(2))
    kernel = build_gemm_kernel()
    ir_interp.run_kernel(kernel, {"A": A, "B": B, "C_global": plain}, {"N": k_extent})
    ir_interp.run_kernel(kernel_pass(kernel, REFERENCE_MODEL), {"A": A, "B": B, "C_global": piped}, {"N": k_extent})
    assert bf16_close(piped, plain.float(), rel=4e-3)
    assert bf16_close(plain, A.float() @ B.float(), rel=4e-3)


def test_pipelined_k_major_form():
    gen = torch.Generator().manual_seed(2)
    A, Bt = rnd(gen, 64, 256), rnd(gen, 128, 256)
    C = torch.zeros(64, 128, dtype=torch.bfloat16)
    kernel = kernel_pass(build_gemm_kernel(block_n=64, b_k_major=True), REFERENCE_MODEL)
    ir_interp.run_kernel(kernel, {"A": A, "B": Bt, "C_global": C}, {"N": 256})
    assert bf16_close(C, A.float() @ Bt.float().t(), rel=4e-3)


@pytest.mark.parametrize("head_dim", [64, 128])
def test_reference_attention_program_matches_the_reference_oracle(head_dim):
    gen = torch.Generator().manual_seed(3)
    Q, K, V = (rnd(gen, 256, head_dim) for _ in range(3))
    O = torch.zeros(256, head_dim, dtype=torch.bfloat16)
    ir_interp.run_kernel(build_attention_kernel(head_dim=head_dim), {"Q": Q, "K": K, "V": V, "O": O}, {"N": 256})
    ref, _ = R.attention_slice_ref(Q, K, V, causal=False)
    assert (O.float() - ref).abs().max().item() <= R.ATTN_O_ABS_TOL


def test_extra_programs_match_their_definitions():
    gen = torch.Generator().manual_seed(4)
    A, B = rnd(gen, 128, 192), rnd(gen, 192, 128)
    C = torch.zeros(128, 128, dtype=torch.bfloat16)
    kernel, ref = TP.scaled_gemm()
    ir_interp.run_kernel(kernel, {"A": A, "B": B, "C": C}, {"K_extent": 192})
    assert bf16_close(C, ref(A, B), rel=4e-3)

    kernel, ref = TP.square_minus()
    ir_interp.run_kernel(kernel, {"A": A, "B": B, "C": C}, {"K_extent": 192})
    assert bf16_close(C, ref(A, B), rel=4e-3)

    Q, K = rnd(gen, 256, 128), rnd(gen, 64, 128)
    P = torch.zeros(256, 64, dtype=torch.bfloat16)
    kernel, ref = TP.row_softmax()
    ir_interp.run_kernel(kernel, {"Q": Q, "K": K, "P": P})
    assert (P.float() - ref(Q, K)).abs().max().item() <= 4e-3

    A, B, W = rnd(gen, 128, 128, std=0.3), rnd(gen, 128, 64, std=0.3), rnd(gen, 64, 256, std=0.3)
    D = torch.zeros(128, 256, dtype=torch.bfloat16)
    kernel, ref = TP.chained_gemm()
    ir_interp.run_kernel(kernel, {"A": A, "B": B, "W": W, "D": D}, {"K_extent": 128})
    assert bf16_close(D, ref(A, B, W), rel=4e-3)


def test_batched_program_and_ragged_edges():
    gen = torch.Generator().manual_seed(5)
    A, B = rnd(gen, 3, 1, 100, 200), rnd(gen, 3, 1, 200, 72)
    C = torch.zeros(3, 1, 100, 72, dtype=torch.bfloat16)
    kernel, _ = TP.scaled_gemm(batched=True)
    assert ir_interp.grid_of(kernel, {"A": A, "B": B, "C": C}) == (2, 2, 3)
    ir_interp.run_kernel(kernel, {"A": A, "B": B, "C": C}, {"K_extent": 200})
    assert bf16_close(C, 0.5 * (A.float() @ B.float()), rel=4e-3)


# ------------------------------------------------------------------ emitter text (no GPU needed)
def test_unrecognised_programs_are_emitted_op_by_op():
    low = Sm100Lowerer()
    src = low.lower(TP.scaled_gemm()[0])
    assert low.plan.kind == "tile_program"
    assert 'scaled_gemm_kind(void) { return "tile_program"; }' in src
    assert "wir::tp::mma_smem<64, 64, true>" in src and "wir::tp::mul_scalar" in src
    assert "emitted op by op because" in src
    # the two programs of the hot path keep their hand-written kernels ...
    assert Sm100Lowerer().lower(build_gemm_kernel()).count("wir::tp::") == 0
    # ... unless asked otherwise
    low = Sm100Lowerer(op_by_op=True)
    src = low.lower(build_attention_kernel())
    assert low.plan.kind == "tile_program" and low.plan.n_mma == 2
    assert "wir::tp::mma_regs<64, 64, true," in src and "wir::tp::mma_smem<64, 64, false>" in src


def test_plan_of_the_op_by_op_emitter():
    plan, _ = emit_tile_program(TP.row_softmax()[0])
    assert plan.rows == 64 and plan.tensors == ["Q", "K", "P"] and plan.ints == []
    assert [(t.rows, t.cols, t.count) for t in plan.tiles.values()] == [(64, 128, 1), (64, 128, 1)]
    assert plan.barriers == 3 and plan.smem_bytes == 4 * 16384 + 1024
    assert plan.grid == ("((dims[10] + 63) / 64)", "1", "1")
    plan, _ = emit_tile_program(kernel_pass(build_gemm_kernel(), REFERENCE_MODEL))
    assert [t.count for t in plan.tiles.values()] == [3, 3] and plan.barriers == 7
    plan, _ = emit_tile_program(TP.chained_gemm()[0])
    assert plan.a_col == 128 and plan.tmem_cols == 256      # accumulator 128 wide, packed A operand behind it


def test_what_the_emitter_refuses():
    from warpir_b200 import ir as _ir
    from warpir_b200.ir import GPUType, RegTileType, SharedTileType, Value
    with pytest.raises(NotImplementedError, match="does not accumulate"):
        Sm100Lowerer(op_by_op=True).lower(build_gemm_kernel(b_k_major=True))
    kernel, _ = TP.scaled_gemm(bm=64, bn=64, bk=32)       # a 32-wide shared tile is half a swizzle row
    with pytest.raises(NotImplementedError, match="multiple of 64"):
        Sm100Lowerer().lower(kernel)
    kernel, _ = TP.scaled_gemm(bm=256, bn=64, bk=64)
    with pytest.raises(NotImplementedError):
        Sm100Lowerer().lower(kernel)
