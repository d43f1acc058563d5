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


@pytest.mark.parametrize("shape,stages", [((128, 256, 64), 4), ((128, 128, 64), 6), ((128, 64, 64), 7),
                                          ((256, 256, 64), 5)])
def test_sm100_model_ring_depth_is_what_the_schedule_needs(shape, stages):
    """The ring depth is the lifetime of a slot (load issue to the end of the MMA that reads it) over the
    initiation interval, with the interval raised until the slots fit in shared memory: an output of the
    solved schedule, not a constant.  (256 x 256 runs on a CTA pair: 32 KB of stage per CTA.)"""
    k = build_gemm_kernel(*shape, b_k_major=True)
    loop = next(o for o in k.body if isinstance(o, ForOp))
    s = ms.schedule_loop(loop)
    lifetime = max(s.start_of[n] + s.machine.mma_latency for n in s.start_of if n.startswith("MMAOp"))
    assert s.num_stages == stages == -(-lifetime // s.ii) and stages <= s.machine.max_stages
    assert -(-lifetime // (s.ii - 1)) > s.machine.max_stages or s.ii == s.machine.mma_latency   # II is minimal
    piped = ms.kernel_pass(k)
    txt = format_kernel(piped)
    assert f"count={stages}> = alloc_shared" in txt and f"for %i: int = {stages - 1} to" in txt
    assert txt.count("drain(+") == 3 * (stages - 1)


def test_changing_the_machine_model_changes_schedule_and_emitted_instantiation():
    """A machine whose loads land sooner needs a shallower ring, one with less shared memory gets a
    shallower ring and a longer interval, and the lowering instantiates the kernel with what the
    schedule says (never shallower than what keeps one CTA per SM)."""
    from warpir_b200.lowering import Sm100Lowerer
    k = build_gemm_kernel(128, 256, 64, b_k_major=True)
    loop = next(o for o in k.body if isinstance(o, ForOp))
    base = ms.schedule_loop(loop)
    fast = ms.sm100_model(128, 256, 64, tma_latency_clk=600)
    small = ms.sm100_model(128, 256, 64, ring_budget=150 * 1024)
    s_fast, s_small = ms.schedule_loop(loop, fast), ms.schedule_loop(loop, small)
    assert (base.ii, base.num_stages) == (5, 4)
    assert (s_fast.ii, s_fast.num_stages) == (4, 3)          # tensor-core bound, three slots cover the latency
    assert s_small.num_stages == 3 and s_small.ii > base.ii   # three slots fit: the loop waits on loads
    assert "launch_gemm_cfg<256, 4, false, 1>" in Sm100Lowerer().lower(k)
    assert "launch_gemm_cfg<256, 3, false, 1>" in Sm100Lowerer(machine=fast).lower(k)
    assert "count=3> = alloc_shared" in format_kernel(ms.kernel_pass(k, fast))


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


def test_role_tables_match_the_kernel_headers():
    """The role tables carry the thread counts and warp numbers of the kernels they describe; the
    constants are read out of the kernel headers here, and the emitted translation units check the same
    thing again at compile time (static_asserts written by the lowering)."""
    import re
    from pathlib import Path
    csrc = Path(wa.__file__).resolve().parent.parent / "csrc"

    def const(header, name):
        m = re.search(rf"constexpr int {name} = (\d+);", (csrc / header).read_text())
        assert m, (header, name)
        return int(m.group(1))

    g = wa.assign_roles(build_gemm_kernel())
    assert g.kind == "gemm" and g.threads == 192 == const("gemm_sm100.cuh", "kGemmThreads")
    assert g.warp_of("mma") == (1,) and g.warp_of("tma_load") == (0,) and g.cxx == "GemmRoles<1>"
    g2 = wa.assign_roles(build_gemm_kernel(), tile_rows=256)
    assert g2.threads == 320 and g2.role("epilogue").warps == tuple(range(2, 10))
    gp = wa.assign_roles(build_gemm_kernel(), tile_rows=256, cta_group=2)
    assert gp.threads == const("gemm_pair_sm100.cuh", "kPairThreads") and gp.ctas_per_tile == 2
    assert wa.assign_roles(ms.kernel_pass(build_gemm_kernel(128, 256, 64, True))).kind == "gemm"
    a = wa.assign_roles(build_attention_kernel())
    assert a.kind == "attention" and a.threads == const("attn_fwd_sm100.cuh", "kAttnThreads") == 352
    assert a.warp_of("mma") == (8, 9) and a.role("producer").warps == (const("attn_fwd_sm100.cuh", "kAttnMmaWarp") + 2,)
    assert len(a.warp_of("exp2")) == 8
    w = wa.assign_roles(build_attention_kernel(), keys_per_block=128)
    assert w.threads == const("attn_fwd_wide_sm100.cuh", "kWideThreads") == 384
    assert w.warp_of("mma") == (const("attn_fwd_wide_sm100.cuh", "kWideMmaWarp"),) and w.role("idle").warps == (9, 11)
    for table in (g, g2, gp, a, w):
        text = table.static_asserts()
        assert f"wir::{table.cxx}::kThreads == {table.threads}" in text


def test_emitted_translation_units_check_their_role_tables():
    from warpir_b200.lowering import Sm100Lowerer
    src = Sm100Lowerer().lower(build_attention_kernel())
    assert "wir::AttnRoles::kThreads == 352" in src and "wir::AttnWideRoles::kThreads == 384" in src
    src = Sm100Lowerer().lower(ms.kernel_pass(build_gemm_kernel(256, 256, 64, b_k_major=True)))
    assert "wir::GemmPairRoles::kCtasPerTile == 2" in src and "launch_gemm_pair_cfg<5, false>" in src


def test_tile_planner_agrees_with_the_launcher(lib):
    """passes/tile_planner.py and the C launcher's plan_gemm_choice state the same rules."""
    import ctypes
    from warpir_b200.passes.tile_planner import plan_gemm
    shapes = [(8192, 8192, 8192), (4096, 4096, 4096), (2048, 2048, 2048), (1024, 1024, 1024), (16384, 4096, 8192),
              (16, 8192, 8192), (64, 8192, 8192), (128, 8192, 8192), (48, 5000, 4096), (1, 4096, 8192),
              (520, 8192, 2048), (2000, 4104, 2056), (256, 512, 2048), (5, 1000, 24), (64, 8192, 2048)]
    for M, N, K in shapes:
        out = [ctypes.c_int() for _ in range(5)]
        assert lib.warpir_plan_gemm(M, N, K, 148, *[ctypes.byref(o) for o in out]) == 0
        bm, bn, group, sk, a_rows = (o.value for o in out)
        p = plan_gemm(M, N, K, 148)
        assert (p.block_m, p.block_n, p.cta_group, int(p.stream_k), p.a_rows) == (bm, bn, group, sk, a_rows), (M, N, K)


def test_planned_tile_is_pinned_in_the_emitted_kernel():
    """With the problem size known the lowering re-tiles the (64 x 64 x 64) reference program with the
    planner's tile, pipelines it and pins the instantiation; the decision shows in the plan it prints."""
    from warpir_b200.lowering import Sm100Lowerer
    L = Sm100Lowerer(problem=(8192, 8192, 8192))
    src = L.lower(build_gemm_kernel())
    assert L.tile_plan.cta_group == 2 and (L.plan.block_m, L.plan.block_n) == (256, 256)
    assert "launch_gemm_pair_cfg<5, true>" in src and "re-tiled for M, N, K = (8192, 8192, 8192)" in src
    assert "shared_buffer<shared_tile<bf16, 256x64, row_major>, count=5> = alloc_shared" in src
    L = Sm100Lowerer(problem=(2048, 2048, 2048))
    assert "launch_gemm_cfg<256, 4, true, 1>" in L.lower(build_gemm_kernel())
    L = Sm100Lowerer(problem=(16, 8192, 8192))           # stream-K lives in the launcher
    src = L.lower(build_gemm_kernel())
    assert L.tile_plan.stream_k and "left to the launcher" in src and "/*block_n: per launch*/0" in src
