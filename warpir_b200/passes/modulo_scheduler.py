"""Modulo scheduling of a tile program's main loop, retargeted to sm_100a.

Public surface as in the reference (``warpir/passes/modulo_scheduler.py``):
``MSInstruction``, ``MSInstructionEdge``, ``MSInstructionManager.solve`` and
``kernel_pass(kernel) -> Kernel``, which rewrites the first-level ``for`` loops of
a kernel into prologue / steady-state loop / drain over shared-memory rings
(``AllocSharedOp``, ``TMALoadBufOp``, ``WaitBufOp``, ``MMABufOp``).

What differs:

* the reference hands its model to OR-tools CP-SAT (modulo_scheduler.py:51-166);
  this module carries its own exact solver for that model class.  The model has
  one start per instruction for iteration 0, every later iteration is a copy
  shifted by the initiation interval II, so the solver walks II upward and, for
  each II, places instructions as early as the dependences (with their iteration
  distances) and the cumulative resource caps allow;
* the machine model is a parameter.  ``REFERENCE_MODEL`` holds the reference's
  symbolic numbers (TMA latency 12, MMA latency 4, four TMA slots, one tensor
  core: modulo_scheduler.py:169,186-190) and reproduces its schedule (II = 6,
  three stages for the GEMM program).  ``sm100_model`` derives latencies from the
  tile shape on a B200: a ``tcgen05.mma`` over a 128 x N x 64 stage occupies the
  tensor core for 128*N*64*2/8192 clocks, a TMA load takes about a microsecond
  to land, and the number of loads in flight is bounded by how many stages fit
  in the 227 KB of shared memory rather than by a fixed slot count;
* the ring depth is an OUTPUT of the schedule on such a machine (``_ring_plan``): the
  lifetime of a slot (load issue to the end of the MMA that reads it) divided by the
  initiation interval, with the interval raised until that many slots fit in shared
  memory.  A machine with a shorter load latency or more shared memory gets a
  different depth, and the lowering instantiates the kernel with whatever comes out.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..ir import ops as _ops
from ..ir.ops import BufSlotExpr, ForOp, Kernel, Op, Value
from ..ir.types import SharedBufferType, SharedTileType

TMALoadOp, MMAOp, TMAStoreOp = _ops.TMALoadOp, _ops.MMAOp, _ops.TMAStoreOp
WaitOp, YieldOp = _ops.WaitOp, _ops.YieldOp
AllocSharedOp, TMALoadBufOp, WaitBufOp, MMABufOp = (
    _ops.AllocSharedOp, _ops.TMALoadBufOp, _ops.WaitBufOp, _ops.MMABufOp)


# --------------------------------------------------------------------------- model
@dataclass
class MSInstructionEdge:
    source: "MSInstruction"
    dest: "MSInstruction"
    distance: int  # iterations between producer and consumer (1 = loop-carried)


@dataclass
class MSInstruction:
    resource: str
    latency: int
    name: str
    parent_edges: List[MSInstructionEdge]


@dataclass(frozen=True)
class MachineModel:
    """Latencies (in model cycles) and resource caps the scheduler plans against."""

    name: str
    tma_load_latency: int
    mma_latency: int
    tma_store_latency: int
    resources: Dict[str, int] = field(default_factory=dict)
    max_cycles: int = 100
    depth: int = 5                     # unrolled copies the schedule is checked over
    max_stages: Optional[int] = None   # ring depth that fits in shared memory (None: no bound)
    cycle_clocks: int = 1              # SM clocks per model cycle (documentation)


REFERENCE_MODEL = MachineModel("reference-h100", 12, 4, 12, {"tma": 4, "tc": 1})

SM100_SMEM_BYTES = 227 * 1024
SM100_RING_BUDGET = 192 * 1024         # what the kernels give the operand ring
SM100_MMA_FLOP_PER_CLK = 8192          # dense bf16 per SM
SM100_TMA_LATENCY_CLK = 1800           # about a microsecond from issue to landed tile


def sm100_model(block_m: int, block_n: int, block_k: int, cycle_clocks: int = 128, cta_group: int = 1,
                tma_latency_clk: int = SM100_TMA_LATENCY_CLK, ring_budget: int = SM100_RING_BUDGET) -> MachineModel:
    """Machine model for one pipeline stage of a ``block_m x block_n x block_k`` GEMM tile.
    ``cta_group = 2``: the tile is computed by a CTA pair, each CTA holding half of A's and half of
    B's rows (half the stage bytes per CTA, both tensor cores working on the stage)."""
    mma_clk = 2 * block_m * block_n * block_k / (SM100_MMA_FLOP_PER_CLK * cta_group)
    stage_bytes = 2 * block_k * (block_m + block_n) // cta_group
    max_stages = max(2, ring_budget // stage_bytes)
    return MachineModel(
        name=f"sm100-{block_m}x{block_n}x{block_k}" + ("-pair" if cta_group == 2 else ""),
        tma_load_latency=math.ceil(tma_latency_clk / cycle_clocks),
        mma_latency=max(1, math.ceil(mma_clk / cycle_clocks)),
        tma_store_latency=math.ceil(tma_latency_clk / cycle_clocks),
        resources={"tma": 2 * max_stages, "tc": 1},
        max_cycles=400, depth=max_stages + 2, max_stages=max_stages, cycle_clocks=cycle_clocks)


def default_cta_group(block_m: int, block_n: int) -> int:
    """The 256 x 256 tile runs on a CTA pair (``csrc/gemm_pair_sm100.cuh``); every other tile on one CTA."""
    return 2 if (block_m, block_n) == (256, 256) else 1


# --------------------------------------------------------------------------- solver
class MSInstructionManager:
    """Collects the loop's instructions and solves the modulo-scheduling model."""

    def __init__(self) -> None:
        self.instructions: List[MSInstruction] = []
        self.child_edges: Dict[str, List[MSInstructionEdge]] = {}
        self.start_of: Dict[str, int] = {}

    def add_instruction(self, instruction: MSInstruction) -> None:
        self.instructions.append(instruction)
        for e in instruction.parent_edges:
            self.child_edges.setdefault(e.source.name, []).append(e)

    # -- one II ---------------------------------------------------------------
    def _place(self, ii: int, depth: int, caps: Dict[str, int], horizon: int) -> Optional[Dict[str, int]]:
        """Earliest starts for iteration 0 under dependences and resource caps, or None."""
        instrs = self.instructions
        start = {i.name: 0 for i in instrs}
        # dependence lower bounds: start[v] >= start[u] + lat[u] - distance * ii
        for _ in range(len(instrs) + 1):
            moved = False
            for v in instrs:
                for e in v.parent_edges:
                    lo = start[e.source.name] + e.source.latency - e.distance * ii
                    if lo > start[v.name]:
                        start[v.name] = lo
                        moved = True
            if not moved:
                break
        else:
            return None  # a recurrence cannot be met at this II

        def usage_ok(placed: List[Tuple[MSInstruction, int]]) -> bool:
            for res, cap in caps.items():
                events = []
                for ins, s in placed:
                    if ins.resource != res:
                        continue
                    for k in range(depth):
                        events.append((s + k * ii, 1))
                        events.append((s + k * ii + ins.latency, -1))
                load = 0
                for _, d in sorted(events, key=lambda ev: (ev[0], ev[1])):
                    load += d
                    if load > cap:
                        return False
            return True

        placed: List[Tuple[MSInstruction, int]] = []
        for ins in sorted(instrs, key=lambda x: (start[x.name], instrs.index(x))):
            s = start[ins.name]
            for e in ins.parent_edges:  # parents may have been pushed later by resources
                if e.source.name in {p.name for p, _ in placed} or e.source is ins:
                    s = max(s, start[e.source.name] + e.source.latency - e.distance * ii)
            while s + (depth - 1) * ii + ins.latency <= horizon:
                if usage_ok(placed + [(ins, s)]):
                    break
                s += 1
            else:
                return None
            start[ins.name] = s
            placed.append((ins, s))
        # final check of every dependence (resource pushes may have broken an earlier bound)
        for v in instrs:
            for e in v.parent_edges:
                if start[v.name] < start[e.source.name] + e.source.latency - e.distance * ii:
                    return None
        return start

    def solve(self, max_cycles: int, depth: int, resource_counts: Dict[str, int], use_verbose: bool = False):
        """Returns ``(prologue, steady_state, epilogue, ii, num_stages, stage_of)`` in the
        reference's format (modulo_scheduler.py:122-160), or six ``None`` if no schedule fits
        in ``max_cycles``."""
        if not self.instructions:
            return (None,) * 6
        best = None
        for ii in range(1, max_cycles):
            if best is not None and (depth - 1) * ii >= best[0]:
                break
            limit = (best[0] - 1) if best is not None else max_cycles - 1
            start = self._place(ii, depth, resource_counts, limit)
            if start is None:
                continue
            span = max(start[i.name] + (depth - 1) * ii + i.latency for i in self.instructions)
            if use_verbose:
                print(f"[modulo] II={ii} makespan={span} starts={start}")
            if best is None or span < best[0]:
                best = (span, ii, start)
        if best is None:
            return (None,) * 6
        _, ii, start = best
        self.start_of = dict(start)
        stage_of = {i.name: start[i.name] // ii for i in self.instructions}
        num_stages = max(stage_of.values()) + 1
        names = [i.name for i in self.instructions]
        prologue = [[(step - stage_of[n], n) for n in names if stage_of[n] <= step]
                    for step in range(num_stages - 1)]
        steady = [[(n, k - stage_of[n]) for n in names] for k in range(num_stages - 1, depth)]
        epilogue = [[(n, stage_of[n] - step) for n in names if stage_of[n] >= step]
                    for step in range(1, num_stages)]
        return prologue, steady, epilogue, ii, num_stages, stage_of


# --------------------------------------------------------------------------- IR rewrite
@dataclass
class LoopSchedule:
    """What the scheduler decided for one loop (kept for the lowering and for tests)."""

    ii: int
    num_stages: int
    stage_of: Dict[str, int]
    start_of: Dict[str, int]
    machine: MachineModel


def _gemm_tile_shape(loop: ForOp) -> Optional[Tuple[int, int, int]]:
    """(block_m, block_n, block_k) of a loads + MMA loop, from the shared-tile types."""
    mma = next((o for o in loop.body if isinstance(o, MMAOp)), None)
    if mma is None or not isinstance(mma.a.type, SharedTileType) or not isinstance(mma.b.type, SharedTileType):
        return None
    a, b = mma.a.type, mma.b.type
    return (a.rows, b.rows, a.cols) if mma.transpose_b else (a.rows, b.cols, a.cols)


def _schedulable(loop: ForOp) -> bool:
    """Only loops made of TMA loads, waits, MMAs and the yield are rewritten; a loop with
    other ops (the attention body) is left as it is rather than silently losing them."""
    allowed = (TMALoadOp, WaitOp, MMAOp, YieldOp, TMAStoreOp)
    return (loop.step == 1 and all(isinstance(o, allowed) for o in loop.body)
            and any(isinstance(o, MMAOp) for o in loop.body)
            and any(isinstance(o, TMALoadOp) for o in loop.body))


def schedule_loop(loop: ForOp, machine: Optional[MachineModel] = None) -> Optional[LoopSchedule]:
    """Build the dependence graph of ``loop`` and solve it on ``machine``."""
    if machine is None:
        shape = _gemm_tile_shape(loop)
        machine = sm100_model(*shape, cta_group=default_cta_group(shape[0], shape[1])) if shape else REFERENCE_MODEL
    latency = {TMALoadOp: ("tma", machine.tma_load_latency), MMAOp: ("tc", machine.mma_latency),
               TMAStoreOp: ("tma", machine.tma_store_latency)}
    nodes: Dict[str, MSInstruction] = {}
    producer: Dict[Value, MSInstruction] = {}
    for o in loop.body:
        if type(o) in latency:
            res, lat = latency[type(o)]
            nodes[str(o)] = MSInstruction(resource=res, latency=lat, name=str(o), parent_edges=[])
            if hasattr(o, "result"):
                producer[o.result] = nodes[str(o)]
    yielded = next((o for o in loop.body if isinstance(o, YieldOp)), None)
    carried = {ia.block_arg: yielded.values[k] for k, ia in enumerate(loop.iter_args)} if yielded else {}
    for o in loop.body:
        node = nodes.get(str(o))
        if node is None:
            continue
        for fname, role in o.roles:
            if role != "use":
                continue
            operand = getattr(o, fname)
            distance = 1 if operand in carried else 0
            src = producer.get(carried.get(operand, operand))
            if src is not None:
                node.parent_edges.append(MSInstructionEdge(source=src, dest=node, distance=distance))
    mgr = MSInstructionManager()
    for n in nodes.values():
        mgr.add_instruction(n)
    _, _, _, ii, stages, stage_of = mgr.solve(machine.max_cycles, machine.depth, machine.resources)
    if ii is None:
        return None
    if machine.max_stages is not None:
        ii, stages, stage_of = _ring_plan(mgr, nodes, ii, machine)
    return LoopSchedule(ii=ii, num_stages=stages, stage_of=stage_of, start_of=mgr.start_of, machine=machine)


def _ring_plan(mgr: "MSInstructionManager", nodes: Dict[str, MSInstruction], ii: int,
               machine: MachineModel) -> Tuple[int, int, Dict[str, int]]:
    """Ring depth from the solved schedule, for machines whose shared memory bounds it.

    The reference counts stages as ``start // II`` of the last instruction, plus one.  That is the
    number of iterations in flight at an instant, but a ring slot is occupied from the moment its
    load is issued until the MMA that reads it has FINISHED, which is ``start(mma) + latency(mma)``
    later: the slots a schedule needs are that lifetime divided by II, rounded up.  (The reference's
    own model gives 3 either way: loads at 0, MMA at 12 for 4 cycles, II = 6.)  If shared memory
    holds fewer slots than that, the loop cannot run at the solver's II: II is raised until the
    slots fit, which is the model's statement that the loop is then bound by load latency rather
    than by the tensor core.  Loads are placed at stage 0 and the MMAs at the last stage.
    """
    start = mgr.start_of
    loads = [n for n in nodes.values() if n.resource == "tma"]
    mmas = [n for n in nodes.values() if n.resource == "tc"]
    first_load = min(start[n.name] for n in loads)
    lifetime = max(start[n.name] + n.latency for n in mmas) - first_load
    ii_fit = ii
    while -(-lifetime // ii_fit) > machine.max_stages:
        ii_fit += 1
    stages = max(2, -(-lifetime // ii_fit))
    stage_of = {k: (stages - 1 if n.resource == "tc" else 0) for k, n in nodes.items()}
    return ii_fit, stages, stage_of


def _pipeline(loop: ForOp, sched: LoopSchedule) -> List[Op]:
    """Prologue loads, steady-state loop and drain steps for ``loop`` under ``sched``."""
    S = sched.num_stages
    depth = S - 1
    loads = [o for o in loop.body if isinstance(o, TMALoadOp)]
    mmas = [o for o in loop.body if isinstance(o, MMAOp)]
    yield_op = next(o for o in loop.body if isinstance(o, YieldOp))
    iv = loop.induction_var
    out: List[Op] = []

    ring: Dict[Value, Value] = {}
    for ld in loads:
        ring[ld.result] = Value(f"{ld.source.name.lower()}_bufs", SharedBufferType(tile_type=ld.result.type, count=S))
        out.append(AllocSharedOp(result=ring[ld.result]))
    all_rings = tuple(ring[ld.result] for ld in loads)

    # prologue: step s issues every load whose stage has been reached, for iteration s - stage
    for step in range(depth):
        for ld in loads:
            st = sched.stage_of[str(ld)]
            if st <= step:
                coords = ld.substitute({iv: step - st}).coords
                out.append(TMALoadBufOp(buf=ring[ld.result], slot=step, source=ld.source, coords=coords))

    def slot_for(op: Op) -> BufSlotExpr:
        return BufSlotExpr(value=iv, offset=-sched.stage_of[str(op)], modulus=S)

    body: List[Op] = [WaitBufOp(bufs=all_rings, slot=slot_for(mmas[0]))]
    for o in loop.body:
        if isinstance(o, TMALoadOp):
            body.append(TMALoadBufOp(buf=ring[o.result], slot=slot_for(o), source=o.source, coords=o.coords))
        elif isinstance(o, MMAOp):
            sl = slot_for(o)
            body.append(MMABufOp(result=o.result, a_buf=ring[o.a], a_slot=sl, b_buf=ring[o.b], b_slot=sl,
                                 accum=o.accum))
    body.append(yield_op)
    out.append(ForOp(induction_var=iv, start=depth, stop=loop.stop, step=loop.step, tile_size=loop.tile_size,
                     iter_args=loop.iter_args, body=tuple(body), results=loop.results))

    # drain: the iterations whose loads were issued but whose MMA has not run yet
    for step in range(depth):
        drain = BufSlotExpr(value=None, offset=step, modulus=S)
        out.append(WaitBufOp(bufs=all_rings, slot=drain))
        for o in mmas:
            if sched.stage_of[str(o)] >= step + 1:
                carried_idx = next(k for k, ia in enumerate(loop.iter_args) if ia.block_arg == o.accum)
                out.append(MMABufOp(result=Value(f"{o.result.name}_ep{step}", o.result.type),
                                    a_buf=ring[o.a], a_slot=drain, b_buf=ring[o.b], b_slot=drain,
                                    accum=loop.results[carried_idx]))
    return out


def kernel_pass(kernel: Kernel, machine: Optional[MachineModel] = None) -> Kernel:
    """Software-pipeline every top-level loads + MMA loop of ``kernel``.

    Same contract as the reference's ``kernel_pass`` (modulo_scheduler.py:168-358): loops it
    cannot schedule come back unchanged.  ``machine=None`` plans for sm_100a from the loop's
    tile shape; ``machine=REFERENCE_MODEL`` reproduces the reference's output.
    """
    body: List[Op] = []
    for o in kernel.body:
        if isinstance(o, ForOp) and _schedulable(o):
            sched = schedule_loop(o, machine)
            if sched is not None and sched.num_stages >= 2:
                body.extend(_pipeline(o, sched))
                continue
        body.append(o)
    return Kernel(name=kernel.name, inputs=kernel.inputs, outputs=kernel.outputs, body=tuple(body))
