"""Lowering: program recognition, parameters read off the IR, emitted text (CPU only)."""
import dataclasses

import pytest

from warpir_b200 import ir
from warpir_b200.ir import ForOp, Kernel
from warpir_b200.lowering import Sm100Lowerer, ThunderKittensLowerer
from warpir_b200.lowering.lowering import AttentionPlan, GemmPlan, analyze
from warpir_b200.passes.modulo_scheduler import REFERENCE_MODEL, kernel_pass
from warpir_b200.programs import build_attention_kernel, build_gemm_kernel


def test_alias_and_statelessness():
    assert ThunderKittensLowerer is Sm100Lowerer
    import warpir.lowering
    assert warpir.lowering.ThunderKittensLowerer is Sm100Lowerer
    L = Sm100Lowerer()
    a = L.lower(build_gemm_kernel())
    L.lower(build_attention_kernel())
    assert L.lower(build_gemm_kernel()) == a


def test_reference_gemm_program_is_retiled():
    p = analyze(build_gemm_kernel())
    assert isinstance(p, GemmPlan) and p.tile_as_written == (64, 64, 64) and p.b_row_major
    assert p.block_n == 0 and (p.a, p.b, p.c) == ("A", "B", "C_global")
    assert (p.row_builtin, p.col_builtin) == ("blockIdx.y", "blockIdx.x")
    src = Sm100Lowerer().lower(build_gemm_kernel())
    assert 'extern "C" int gemm_launch(' in src and "/*b_layout=*/0" in src
    assert "%c_new: reg_tile<fp32, 16x64, row_major> = mma(" in src      # the IR is quoted in the header comment


def test_reference_pipelined_program_lowers_too():
    p = analyze(kernel_pass(build_gemm_kernel(), REFERENCE_MODEL))
    assert p.pipelined_in_ir and p.b_row_major and p.block_n == 0


@pytest.mark.parametrize("bm,bn,stages", [(128, 256, 4), (128, 128, 6), (128, 64, 7), (256, 256, 5)])
@pytest.mark.parametrize("pipelined", [False, True])
def test_hardware_tiles_are_instantiated_as_written(bm, bn, stages, pipelined):
    k = build_gemm_kernel(bm, bn, 64, b_k_major=True)
    if pipelined:
        k = kernel_pass(k)
    L = Sm100Lowerer()
    src = L.lower(k)
    assert (L.plan.block_m, L.plan.block_n, L.plan.stages) == (bm, bn, stages) and not L.plan.b_row_major
    inst = f"launch_gemm_pair_cfg<{stages}, false>" if (bm, bn) == (256, 256) else \
        f"launch_gemm_cfg<{bn}, {stages}, false, {bm // 128}>"
    assert inst in src and "/*b_layout=*/1" in src


@pytest.mark.parametrize("bm,bn,floor", [(128, 64, 5), (128, 128, 4), (128, 256, 3)])
def test_ring_shallower_than_one_cta_per_sm_is_deepened(bm, bn, floor):
    """A program pipelined for another machine may ask for a ring so shallow that two CTAs would fit on
    an SM (each allocates all of tensor memory); the instantiation is deepened to the floor, which the
    program's semantics cannot see."""
    k = kernel_pass(build_gemm_kernel(bm, bn, 64, b_k_major=True), REFERENCE_MODEL)     # 3 stages
    L = Sm100Lowerer()
    src = L.lower(k)
    assert L.plan.stages == floor and f"launch_gemm_cfg<{bn}, {floor}, false, 1>" in src


def test_ring_too_deep_for_shared_memory_is_rejected():
    from warpir_b200.passes.modulo_scheduler import MachineModel
    deep = MachineModel("too-deep", 15, 4, 15, {"tma": 16, "tc": 1}, max_cycles=400, depth=10, max_stages=8)
    k = kernel_pass(build_gemm_kernel(128, 256, 64, b_k_major=True), deep)   # 8 stages of 48 KB
    with pytest.raises(NotImplementedError, match="do not fit"):
        analyze(k)


def test_attention_parameters():
    p = analyze(build_attention_kernel())
    assert isinstance(p, AttentionPlan) and p.head_dim == 64 and p.tile_as_written == (64, 64)
    assert abs(p.softmax_scale - 0.125) < 1e-9
    p = analyze(build_attention_kernel(128, 128, 128, scale=0.3))
    assert p.head_dim == 128 and p.exp2_scale == 0.3
    src = Sm100Lowerer().lower(build_attention_kernel())
    assert 'extern "C" int attention_fwd_launch(' in src and "attn_impl(" in src


def _replace_loop_body(k: Kernel, fn) -> Kernel:
    body = []
    for o in k.body:
        if isinstance(o, ForOp):
            o = dataclasses.replace(o, body=tuple(fn(list(o.body))))
        body.append(o)
    return dataclasses.replace(k, body=tuple(body))


def test_unknown_programs_are_rejected_not_guessed():
    g = build_gemm_kernel()
    with pytest.raises(NotImplementedError):                 # no loop at all
        analyze(Kernel("k", g.inputs, g.outputs, tuple(o for o in g.body if not isinstance(o, ForOp))))
    with pytest.raises(NotImplementedError, match="zero-initialised"):
        analyze(dataclasses.replace(g, body=g.body[1:]))
    with pytest.raises(NotImplementedError, match="transpose_b"):
        analyze(_replace_loop_body(g, lambda b: [dataclasses.replace(o, transpose_b=True)
                                                  if isinstance(o, ir.MMAOp) else o for o in b]))
    # a GEMM loop with anything besides loads, waits and the MMA must not be taken for a plain GEMM: the
    # hand-written kernel would drop the extra op.  It lowers op by op instead.
    def scaled(body):
        out = []
        for o in body:
            if isinstance(o, ir.YieldOp):
                mma = next(x for x in body if isinstance(x, ir.MMAOp))
                half = ir.Value("c_half", mma.result.type)
                out.append(ir.MulScalarOp(result=half, input=mma.result, scalar=0.5))
                o = dataclasses.replace(o, values=(half,))
            out.append(o)
        return out
    k_scaled = _replace_loop_body(g, scaled)
    with pytest.raises(NotImplementedError, match="MulScalarOp"):
        analyze(k_scaled)
    L = Sm100Lowerer()
    src = L.lower(k_scaled)
    assert L.plan.kind == "tile_program" and "wir::tp::" in src
    # ... and an op between the loop and the store (an epilogue on the accumulator) likewise
    body = list(g.body)
    st = next(o for o in body if isinstance(o, ir.TMAStoreOp))
    scaled_out = ir.Value("c_scaled", st.source.type)
    body[body.index(st):body.index(st) + 1] = [ir.MulScalarOp(result=scaled_out, input=st.source, scalar=2.0),
                                              dataclasses.replace(st, source=scaled_out)]
    with pytest.raises(NotImplementedError):
        analyze(dataclasses.replace(g, body=tuple(body)))
    a = build_attention_kernel()
    with pytest.raises(NotImplementedError, match="row sum"):
        analyze(_replace_loop_body(a, lambda b: [o for o in b if not isinstance(o, ir.RowSumOp)]))
    with pytest.raises(NotImplementedError, match="head dimension"):
        analyze(build_attention_kernel(head_dim=32))


def test_emitted_source_compiles_for_sm100a():
    from warpir_b200 import runtime
    k = runtime.load(build_gemm_kernel())
    assert k.kind == "gemm" and k.path.exists() and hasattr(k, "launch_gemm")
    k = runtime.load(build_attention_kernel())
    assert k.kind == "attention" and hasattr(k, "launch_attention")
