"""Programs emitted op by op (``lowering/generic.py`` over ``csrc/tile_program.cuh``) on a
B200, against the CPU interpreter of the IR on the same inputs.  Covers the op table of
the reference's lowering (warpir/lowering/lowering.py:427-570): both MMA forms and operand
layouts, ring buffers with prologue / steady state / drain, every elementwise and
row-wise op, ragged edges, batch indices."""
import math

import pytest
import torch

from oracle import ir_interp
from oracle import reference_ops as R
from warpir_b200 import runtime

import tile_programs as TP

pytestmark = pytest.mark.gpu

CASES = TP.op_by_op_cases()


def rnd(gen, *shape, std=1.0):
    return (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)


def run_both(case, inputs, out_name, out_shape, ints):
    """Run the program on the GPU and in the interpreter; returns (gpu, oracle) as fp32 on CPU."""
    kernel, force = CASES[case]
    mod = runtime.load(kernel, op_by_op=force)
    assert mod.kind == "tile_program"
    order = [v.name for v in (*kernel.inputs, *kernel.outputs) if type(v.type).__name__ == "GlobalType"]
    int_order = [v.name for v in kernel.inputs if type(v.type).__name__ == "IntType"]
    expect = torch.zeros(*out_shape, dtype=torch.bfloat16)
    ir_interp.run_kernel(kernel, {**inputs, out_name: expect}, ints)
    got = torch.full(out_shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    dev = {**{k: v.cuda() for k, v in inputs.items()}, out_name: got}
    mod(*[dev[n] for n in order], ints=[ints[n] for n in int_order])
    mod.read_status()
    return got.cpu().float(), expect.float()


def assert_gemm_close(got, expect):
    e = R.gemm_errors(got, expect)
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= 2 * R.GEMM_REL_TOL, e


@pytest.mark.parametrize("case,bm,bn", [("scaled_gemm_64", 64, 64), ("scaled_gemm_128x128", 128, 128),
                                        ("scaled_gemm_128x256", 128, 256), ("square_minus", 64, 64)])
@pytest.mark.parametrize("shape", [(128, 256, 192), (100, 72, 200), (256, 512, 64)])
def test_gemm_with_epilogue(case, bm, bn, shape, lib):
    M, N, K = shape
    gen = torch.Generator().manual_seed(M + N + K)
    std = 0.25 if case == "square_minus" else 1.0
    A, B = rnd(gen, M, K, std=std), rnd(gen, K, N, std=std)
    got, expect = run_both(case, {"A": A, "B": B}, "C", (M, N), {"K_extent": K})
    assert_gemm_close(got, expect)


def test_batched_gemm_with_epilogue(lib):
    gen = torch.Generator().manual_seed(11)
    A, B = rnd(gen, 3, 1, 100, 200), rnd(gen, 3, 1, 200, 72)
    got, expect = run_both("scaled_gemm_batched", {"A": A, "B": B}, "C", (3, 1, 100, 72), {"K_extent": 200})
    assert_gemm_close(got, expect)


@pytest.mark.parametrize("case,bq,bkv,d", [("row_softmax_d128", 64, 64, 128), ("row_softmax_q128_kv128", 128, 128, 64)])
def test_row_softmax(case, bq, bkv, d, lib):
    gen = torch.Generator().manual_seed(12)
    Q, K = rnd(gen, 320, d), rnd(gen, bkv, d)
    got, expect = run_both(case, {"Q": Q, "K": K}, "P", (320, bkv), {})
    assert (got - expect).abs().max().item() <= 4e-3
    assert (got.sum(dim=1) - 1).abs().max().item() <= 2e-2      # rows of a softmax sum to one (bf16 outputs)


def test_chained_gemm_register_operand(lib):
    gen = torch.Generator().manual_seed(13)
    A, B, W = rnd(gen, 192, 256, std=0.3), rnd(gen, 256, 64, std=0.3), rnd(gen, 64, 384, std=0.3)
    got, expect = run_both("chained_gemm", {"A": A, "B": B, "W": W}, "D", (192, 384), {"K_extent": 256})
    assert_gemm_close(got, expect)


@pytest.mark.parametrize("case", ["reference_gemm", "reference_gemm_pipelined"])
@pytest.mark.parametrize("n", [64, 128, 448])
def test_reference_gemm_program_op_by_op(case, n, lib):
    gen = torch.Generator().manual_seed(n)
    A, B = rnd(gen, n, n), rnd(gen, n, n)
    got, expect = run_both(case, {"A": A, "B": B}, "C_global", (n, n), {"N": n})
    assert_gemm_close(got, expect)
    assert_gemm_close(got, A.float() @ B.float())


def test_k_major_ring_op_by_op(lib):
    gen = torch.Generator().manual_seed(14)
    A, Bt = rnd(gen, 128, 320), rnd(gen, 192, 320)
    got, expect = run_both("k_major_gemm_pipelined", {"A": A, "B": Bt}, "C_global", (128, 192), {"N": 320})
    assert_gemm_close(got, expect)
    assert_gemm_close(got, A.float() @ Bt.float().t())


@pytest.mark.parametrize("case,d", [("reference_attention", 64), ("attention_d128", 128)])
@pytest.mark.parametrize("n", [64, 256, 1024])
def test_reference_attention_program_op_by_op(case, d, n, lib):
    gen = torch.Generator().manual_seed(n + d)
    Q, K, V = (rnd(gen, n, d) for _ in range(3))
    got, expect = run_both(case, {"Q": Q, "K": K, "V": V}, "O", (n, d), {"N": n})
    assert (got - expect).abs().max().item() <= R.ATTN_O_ABS_TOL
    ref, _ = R.attention_slice_ref(Q, K, V, causal=False)
    assert (got - ref).abs().max().item() <= R.ATTN_O_ABS_TOL


def test_emitted_kernel_rejects_bad_arguments(lib):
    kernel, force = CASES["scaled_gemm_64"]
    mod = runtime.load(kernel, op_by_op=force)
    A = torch.zeros(64, 68, dtype=torch.bfloat16, device="cuda")     # row pitch not a multiple of 16 bytes
    B = torch.zeros(68, 64, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(runtime.WarpirError):
        mod(A, B, C, ints=[68])
    with pytest.raises(ValueError):
        mod(A.cpu(), B, C, ints=[68])
