"""IR value semantics and printer goldens (CPU only).

Goldens were produced by the reference's own ``format_kernel`` on its own tile
programs (tests/golden/make_golden.py); the programs here are rebuilt with this
repo's IR and must print identically.
"""
import dataclasses

import pytest

from warpir_b200 import ir
from warpir_b200.ir import (BufSlotExpr, ColVecType, ForOp, GPUType, GlobalType, IntType, IterArg,
                            Kernel, MMAOp, RegTileType, SharedBufferType, SharedTileType, TileLayout,
                            TMALoadBufOp, TMALoadOp, Value, WaitBufOp, ZeroOp)
from warpir_b200.printing import format_kernel, print_kernel
from warpir_b200.programs import build_attention_kernel, build_gemm_kernel


def test_type_strings():
    st = SharedTileType(GPUType.bf16, 64, 64)
    assert str(st) == "shared_tile<bf16, 64x64, row_major>"
    assert str(RegTileType(GPUType.fp32, 16, 64, TileLayout.col_major)) == "reg_tile<fp32, 16x64, col_major>"
    assert str(GlobalType(GPUType.bf16, st, 1, 1)) == "global<bf16, 1, 1, -1, -1>"
    assert str(SharedBufferType(st, 3)) == "shared_buffer<shared_tile<bf16, 64x64, row_major>, count=3>"
    assert str(ColVecType(GPUType.fp32, 16, 64)) == "col_vec<fp32, 16x64>"
    assert str(IntType()) == "int"


def test_types_are_values():
    a, b = SharedTileType(GPUType.bf16, 64, 64), SharedTileType(GPUType.bf16, 64, 64)
    assert a == b and hash(a) == hash(b)
    assert IntType() == IntType() and hash(IntType()) == hash(IntType())
    assert Value("x", a) == Value("x", b)
    assert len({Value("x", a), Value("x", b), Value("y", a)}) == 2
    with pytest.raises(dataclasses.FrozenInstanceError):
        a.rows = 3


def test_value_repr_and_op_repr():
    v = Value("c", RegTileType(GPUType.fp32, 16, 64))
    assert repr(v) == "%c: reg_tile<fp32, 16x64, row_major>"
    assert repr(ZeroOp(result=v)) == "ZeroOp(result=%c: reg_tile<fp32, 16x64, row_major>)"
    assert ZeroOp(result=v) == ZeroOp(v)


def test_op_defaults_and_fields():
    t = SharedTileType(GPUType.bf16, 64, 64)
    r = RegTileType(GPUType.fp32, 16, 64)
    op = MMAOp(result=Value("c", r), a=Value("a", t), b=Value("b", t), accum=Value("z", r))
    assert op.transpose_b is False
    assert [f.name for f in dataclasses.fields(op)] == ["result", "a", "b", "accum", "transpose_b"]
    assert set(ir.__all__) >= {"ZeroOp", "TMALoadOp", "WaitOp", "MMAOp", "TMAStoreOp", "NegInftyOp", "CopyOp",
                               "MulScalarOp", "SubOp", "MulOp", "Exp2Op", "RowMaxOp", "RowSumOp", "SubRowOp",
                               "MulRowOp", "DivRowOp", "AllocSharedOp", "TMALoadBufOp", "WaitBufOp", "MMABufOp",
                               "YieldOp", "IterArg", "ForOp", "Kernel", "BufSlotExpr", "BufIdx", "Op", "Value"}


def test_substitute():
    t = SharedTileType(GPUType.bf16, 64, 64)
    g = GlobalType(GPUType.bf16, t, 1, 1)
    i, by = Value("i", IntType()), Value("blockIdx.y", IntType())
    ld = TMALoadOp(result=Value("a", t), source=Value("A", g), coords=(0, 0, by, i))
    assert ld.substitute({i: 3}).coords == (0, 0, by, 3)
    buf = Value("a_bufs", SharedBufferType(t, 3))
    lb = TMALoadBufOp(buf=buf, slot=BufSlotExpr(i, -2, 3), source=Value("A", g), coords=(0, 0, by, i))
    j = Value("j", IntType())
    sub = lb.substitute({i: j})
    assert sub.slot == BufSlotExpr(j, -2, 3) and sub.coords[-1] == j
    assert WaitBufOp(bufs=(buf,), slot=BufSlotExpr(None, 1, 3)).substitute({i: j}).slot.value is None


@pytest.mark.parametrize("builder,golden", [(build_gemm_kernel, "printer_gemm.txt"),
                                            (build_attention_kernel, "printer_attention.txt")])
def test_printer_matches_reference_golden(builder, golden, golden_dir):
    assert format_kernel(builder()) + "\n" == (golden_dir / golden).read_text()


def test_print_kernel_writes_stdout(capsys):
    k = build_gemm_kernel()
    print_kernel(k)
    assert capsys.readouterr().out == format_kernel(k) + "\n"


def test_alias_package_is_the_same_objects():
    import warpir.ir
    import warpir.ir.ops
    import warpir.printing
    from warpir.ir import Kernel as K2
    assert K2 is Kernel and warpir.printing.format_kernel is format_kernel
    assert warpir.ir.ops.ForOp is ForOp


def test_generalised_programs_print():
    txt = format_kernel(build_gemm_kernel(128, 256, 64, b_k_major=True))
    assert "transpose_b=True" in txt and "shared_tile<bf16, 256x64, row_major>" in txt
    txt = format_kernel(build_attention_kernel(head_dim=128, block_q=128, block_kv=128))
    assert "mul_scalar(%att: reg_tile<fp32, 32x128, row_major>, 0.1275" in txt
