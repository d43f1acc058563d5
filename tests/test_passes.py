"""Scheduling passes (CPU only)."""
import pytest

from warpir_b200.ir import ForOp
from warpir_b200.passes import modulo_scheduler as ms
from warpir_b200.passes import warp_assigner as wa
from warpir_b200.printing import format_kernel
from warpir_b200.programs import build_attention_kernel, build_gemm_kernel


def test_reference_model_reproduces_reference_pipelined_ir(golden_dir):
    """Golden made by the reference's own kernel_pass (CP-SAT stood in for by an exact
    enumerator, see tests/golden/make_golden.py)."""
    out = format_kernel(ms.kernel_pass(build_gemm_kernel(), ms.REFERENCE_MODEL)) + "\n"
    assert out == (golden_dir / "printer_gemm_pipelined.txt").read_text()


def test_reference_demo_model_solves_to_ii6_three_stages():
    # the model at the bottom of the reference file (modulo_scheduler.py:360-388)
    la, lb = ms.MSInstruction("tma", 12, "load_a", []), ms.MSInstruction("tma", 12, "load_b", [])
    mac = ms.MSInstruction("tc", 4, "mac", [])
    mac.parent_edges += [ms.MSInstructionEdge(la, mac, 0), ms.MSInstructionEdge(lb, mac, 0),
                         ms.MSInstructionEdge(mac, mac, 1)]
    mgr = ms.MSInstructionManager()
    for i in (la, lb, mac):
        mgr.add_instruction(i)
    pro, steady, epi, ii, stages, stage_of = mgr.solve(100, 5, {"tma": 4, "tc": 1})
    assert (ii, stages) == (6, 3) and stage_of == {"load_a": 0, "load_b": 0, "mac": 2}
    assert len(pro) == 2 and len(epi) == 2 and len(steady) == 3
    assert mgr.solve(10, 5, {"tma": 4, "tc": 1}) == (None,) * 6   # does not fit


@pytest.mark.parametrize("shape,stages", [((128, 256, 64), 4), ((128, 128, 64), 6), ((128, 64, 64), 8),
                                          ((256, 256, 64), 3)])
def test_sm100_model_picks_the_ring_depths_the_kernels_use(shape, stages):
    k = build_gemm_kernel(*shape, b_k_major=True)
    loop = next(o for o in k.body if isinstance(o, ForOp))
    s = ms.schedule_loop(loop)
    assert s.num_stages == stages
    piped = ms.kernel_pass(k)
    txt = format_kernel(piped)
    assert f"count={stages}> = alloc_shared" in txt and f"for %i: int = {stages - 1} to" in txt
    assert txt.count("drain(+") == 3 * (stages - 1)


def test_attention_loop_is_left_alone():
    k = build_attention_kernel()
    assert ms.kernel_pass(k) == k


def test_generic_warp_assigner_on_reference_demo():
    sched = wa.check_roles_with_solver(wa.assign_roles(build_gemm_kernel()), ii=6, load_latency=12, mma_latency=4)
    assert sched.type_to_warp["load_a"] == 0
    # six MMAs, one every II after the first loads land
    macs = sorted(v for k, v in sched.start_of.items() if k.startswith("mac_"))
    assert macs[0] >= 12 and all(b - a >= 4 for a, b in zip(macs, macs[1:]))
    assert sched.makespan <= 60


def test_sync_cost_is_paid_only_across_warps():
    a = wa.WAInstruction("a", 0, [], [], False, 1, 5, 0)
    b = wa.WAInstruction("b", 0, [a], [], False, 1, 5, 0)
    m = wa.WAInstructionManager()
    m.add_instruction(a)
    m.add_instruction(b)
    assert m.solve(1000, 2, 80, ["a", "b"]).makespan == 10            # same warp is best
    s = m._schedule({"a": 0, "b": 1}, 2, 80, 1000)
    assert s.start_of["b_0"] == 85


def test_role_tables():
    g = wa.assign_roles(build_gemm_kernel())
    assert g.kind == "gemm" and g.threads == 192 and g.warp_of("mma") == (1,) and g.warp_of("tma_load") == (0,)
    assert wa.assign_roles(ms.kernel_pass(build_gemm_kernel(128, 256, 64, True))).kind == "gemm"
    a = wa.assign_roles(build_attention_kernel())
    assert a.kind == "attention" and a.threads == 320 and len(a.warp_of("exp2")) == 8
