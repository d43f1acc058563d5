"""Warp specialisation: which warp issues which instruction stream.

Two layers:

* ``WAInstruction`` / ``WAInstructionManager.solve`` keep the interface of the
  reference's prototype (``warpir/passes/warp_assigner.py:7-143``): unrolled
  instruction instances with data and ordering dependences, instruction *types*
  pinned to one warp each, a cross-warp synchronisation cost on synchronous data
  dependences, one issue slot per warp, minimise the makespan.  The reference gives
  the model to OR-tools CP-SAT; here the type-to-warp maps are enumerated (there
  are ``num_warps ** len(types)`` of them, a handful) and each is list-scheduled in
  dependence order, which is exact for this model because, once the map is fixed,
  every constraint is a lower bound on a start time plus per-warp non-overlap of
  unit issue slots.
* ``assign_roles`` is what the sm_100a lowering uses.  On Blackwell the answer is
  structural rather than searched: TMA loads and ``tcgen05.mma`` are each issued
  by ONE elected thread, so loads get a producer warp, MMAs get an issuer warp,
  and everything that touches accumulator rows (tensor-memory loads, softmax,
  conversion, stores) goes to warpgroups of four warps, because a warp can only
  reach the 32 tensor-memory lanes ``32 * (warp_id % 4)``...  It returns the role
  table of the kernel the program is instantiated as; ``RoleTable.static_asserts``
  turns the table into compile-time checks against the constants that kernel's
  header exports, which the lowering writes into every translation unit.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..ir import ops as _ops
from ..ir.ops import ForOp, Kernel


@dataclass
class WAInstruction:
    name: str
    version: int
    parent_instructions: List["WAInstruction"]     # data dependences: pay the sync cost across warps
    ordering_instructions: List["WAInstruction"]   # sequencing only: never pay it
    is_async: bool
    cuda_latency: int       # issue-slot occupancy on the issuing warp
    total_latency: int      # issue to result available
    modulo_issue_cycle: int

    def __str__(self) -> str:
        return f"{self.name}_{self.version}"


@dataclass
class WarpSchedule:
    makespan: int
    type_to_warp: Dict[str, int]
    warp_of: Dict[str, int]
    start_of: Dict[str, int]

    def per_warp(self, num_warps: int) -> List[List[Tuple[str, int]]]:
        rows: List[List[Tuple[str, int]]] = [[] for _ in range(num_warps)]
        for key, w in self.warp_of.items():
            rows[w].append((key, self.start_of[key]))
        for r in rows:
            r.sort(key=lambda kv: kv[1])
        return rows


class WAInstructionManager:
    def __init__(self) -> None:
        self.instructions: List[WAInstruction] = []

    def add_instruction(self, instruction: WAInstruction) -> None:
        self.instructions.append(instruction)

    @staticmethod
    def _separation(child: WAInstruction, parent: WAInstruction) -> int:
        gap = child.modulo_issue_cycle - parent.modulo_issue_cycle
        return max(gap, parent.total_latency) if gap > 0 else parent.total_latency

    def _schedule(self, pin: Dict[str, int], num_warps: int, sync_cost: int, max_cycles: int) -> Optional[WarpSchedule]:
        order = sorted(self.instructions, key=lambda i: (i.modulo_issue_cycle, self.instructions.index(i)))
        done: Dict[str, int] = {}
        warp_of: Dict[str, int] = {}
        busy: List[List[Tuple[int, int]]] = [[] for _ in range(num_warps)]
        pending = list(order)
        while pending:
            progressed = False
            for ins in list(pending):
                deps = ins.parent_instructions + ins.ordering_instructions
                if any(str(d) not in done for d in deps):
                    continue
                candidates = [pin[ins.name]] if ins.name in pin else list(range(num_warps))
                best = None
                for w in candidates:
                    lo = 0
                    for par in ins.parent_instructions:
                        extra = 0 if (par.is_async or warp_of[str(par)] == w) else sync_cost
                        lo = max(lo, done[str(par)] + self._separation(ins, par) + extra)
                    for par in ins.ordering_instructions:
                        lo = max(lo, done[str(par)] + self._separation(ins, par))
                    s = lo
                    while any(s < e and b < s + ins.cuda_latency for b, e in busy[w]):
                        s = min(e for b, e in busy[w] if s < e and b < s + ins.cuda_latency)
                    if best is None or s < best[1]:
                        best = (w, s)
                w, s = best
                if s + max(ins.cuda_latency, ins.total_latency) > max_cycles - 1:
                    return None
                done[str(ins)] = s
                warp_of[str(ins)] = w
                busy[w].append((s, s + ins.cuda_latency))
                pending.remove(ins)
                progressed = True
            if not progressed:
                return None  # dependence cycle
        makespan = max(done[str(i)] + i.total_latency for i in self.instructions)
        return WarpSchedule(makespan, dict(pin), warp_of, done)

    def solve(self, max_cycles: int, num_warps: int, synchronization_cost: int, instruction_types: List[str],
              use_verbose: bool = False) -> Optional[WarpSchedule]:
        """Best schedule over all type-to-warp maps, or None if nothing fits in ``max_cycles``.
        With ``use_verbose`` the per-warp listing is printed, as the reference does."""
        best: Optional[WarpSchedule] = None
        for combo in itertools.product(range(num_warps), repeat=len(instruction_types)):
            if combo and combo[0] != 0:
                break  # warps are interchangeable: fix the first type on warp 0
            sched = self._schedule(dict(zip(instruction_types, combo)), num_warps, synchronization_cost, max_cycles)
            if sched is not None and (best is None or sched.makespan < best.makespan):
                best = sched
        if use_verbose:
            if best is None:
                print("INFEASIBLE!")
            else:
                for w, row in enumerate(best.per_warp(num_warps)):
                    print(f"warp {w}:")
                    for entry in row:
                        print("\t", entry)
        return best


# --------------------------------------------------------------------------- sm_100a roles
@dataclass(frozen=True)
class Role:
    name: str            # "producer", "mma", "epilogue", "softmax", "idle"
    warps: Tuple[int, ...]
    issues: Tuple[str, ...]   # op mnemonics this role executes
    single_thread: bool       # one elected lane does the issuing


@dataclass(frozen=True)
class RoleTable:
    """Who issues what in the kernel a tile program is instantiated as.

    The table is not commentary: ``static_asserts()`` renders it as C++ checks against the
    constants the kernel header exports (``csrc/*_sm100.cuh``: ``GemmRoles<MT>``, ``GemmPairRoles``,
    ``AttnRoles``, ``AttnWideRoles``), and the lowering writes those into every translation unit
    it emits, so a table that disagrees with the kernel does not compile."""

    kind: str                 # "gemm" or "attention"
    roles: Tuple[Role, ...]
    threads: int              # per CTA
    cxx: str                  # the header's constants this table mirrors
    ctas_per_tile: int = 1    # 2: a CTA pair (cta_group::2) computes one tile

    def warp_of(self, mnemonic: str) -> Tuple[int, ...]:
        for r in self.roles:
            if mnemonic in r.issues:
                return r.warps
        raise KeyError(mnemonic)

    def role(self, name: str) -> Role:
        return next(r for r in self.roles if r.name == name)

    def static_asserts(self) -> str:
        c = f"wir::{self.cxx}"
        checks = [f"{c}::kThreads == {self.threads}", f"{c}::kProducerWarp == {self.role('producer').warps[0]}"]
        if self.kind == "gemm":
            epi = self.role("epilogue").warps
            checks += [f"{c}::kMmaWarp == {self.role('mma').warps[0]}", f"{c}::kFirstEpilogueWarp == {epi[0]}",
                       f"{c}::kEpilogueWarps == {len(epi)}"]
            if self.ctas_per_tile > 1:
                checks.append(f"{c}::kCtasPerTile == {self.ctas_per_tile}")
        else:
            mma = self.role("mma").warps
            checks += [f"{c}::kSoftmaxWarps == {len(self.role('softmax').warps)}", f"{c}::kFirstMmaWarp == {mma[0]}",
                       f"{c}::kMmaWarps == {len(mma)}"]
        body = " &&\n              ".join(checks)
        return (f'static_assert({body},\n              "the role table the lowering planned with disagrees '
                f'with the kernel ({self.cxx})");')


_ROW_OPS = ("zero", "neg_infty", "copy", "mul_scalar", "sub", "mul", "exp2", "row_max", "row_sum",
            "sub_row", "mul_row", "div_row", "tma_store")


def _loop_ops(kernel: Kernel):
    for o in kernel.body:
        if isinstance(o, ForOp):
            return o.body
    return ()


def gemm_roles(tile_rows: int = 128, cta_group: int = 1) -> RoleTable:
    """Role table of the GEMM kernels: ``tile_rows`` = 128 or 256 rows per CTA tile
    (``gemm_bf16_sm100<.., MT>``), ``cta_group`` = 2 for the 256-row tile on a CTA pair
    (``gemm_pair_sm100``)."""
    if cta_group == 2:
        return RoleTable("gemm", (
            Role("producer", (0,), ("tma_load", "tma_load_buf"), True),
            Role("mma", (1,), ("mma", "mma_buf", "wait", "wait_buf"), True),      # issues in the pair's leader only
            Role("epilogue", (2, 3, 4, 5), ("tma_store", "zero"), False),
        ), threads=192, cxx="GemmPairRoles", ctas_per_tile=2)
    mt = tile_rows // 128
    return RoleTable("gemm", (
        Role("producer", (0,), ("tma_load", "tma_load_buf"), True),
        Role("mma", (1,), ("mma", "mma_buf", "wait", "wait_buf"), True),
        Role("epilogue", tuple(range(2, 2 + 4 * mt)), ("tma_store", "zero"), False),   # a warpgroup per 128 rows
    ), threads=32 * (2 + 4 * mt), cxx=f"GemmRoles<{mt}>")


def attention_roles(keys_per_block: int = 64) -> RoleTable:
    """Role table of the attention-forward kernels: two softmax warpgroups (warps 0-3 and 4-7, one per
    128-row Q tile, also doing the O rescale and the final store); with 64-key blocks one MMA-issuing
    warp per Q tile (8, 9) and the producer at warp 10 (352 threads); with 128-key blocks ONE issuer
    (warp 8) serving both tiles in turn, the producer at warp 10 and two idle warps (9, 11) that only
    complete the warpgroup whose registers move to the softmax warps (384 threads)."""
    if keys_per_block == 128:
        return RoleTable("attention", (
            Role("softmax", tuple(range(8)), _ROW_OPS, False),
            Role("mma", (8,), ("mma", "wait"), True),
            Role("producer", (10,), ("tma_load",), True),
            Role("idle", (9, 11), (), False),
        ), threads=384, cxx="AttnWideRoles")
    return RoleTable("attention", (
        Role("softmax", tuple(range(8)), _ROW_OPS, False),
        Role("mma", (8, 9), ("mma", "wait"), True),
        Role("producer", (10,), ("tma_load",), True),
    ), threads=352, cxx="AttnRoles")


def assign_roles(kernel: Kernel, tile_rows: int = 128, cta_group: int = 1, keys_per_block: int = 64) -> RoleTable:
    """Role table for a GEMM-shaped or attention-shaped tile program on sm_100a.

    On Blackwell the split is structural rather than searched: TMA loads and ``tcgen05.mma`` are
    each issued by one elected thread, so loads get a producer warp and MMAs an issuer warp, and
    everything that touches accumulator rows goes to warpgroups of four warps, because a warp
    reaches only the 32 tensor-memory lanes ``32 * (warp_id % 4)``.  What varies is which kernel
    the program is instantiated as (tile height, CTA pairs, keys per block): the keyword arguments.
    """
    body = _loop_ops(kernel)
    n_mma = sum(isinstance(o, (_ops.MMAOp, _ops.MMABufOp)) for o in body)
    has_rows = any(isinstance(o, (_ops.RowMaxOp, _ops.Exp2Op, _ops.RowSumOp)) for o in body)
    if n_mma == 1 and not has_rows:
        return gemm_roles(tile_rows, cta_group)
    if n_mma == 2 and has_rows:
        return attention_roles(keys_per_block)
    raise NotImplementedError(
        f"kernel {kernel.name!r} is neither a loads+MMA loop nor an online-softmax attention loop")


def check_roles_with_solver(table: RoleTable, ii: int, load_latency: int, mma_latency: int, iterations: int = 6,
                            synchronization_cost: int = 1) -> WarpSchedule:
    """Runs the generic assigner on an unrolled loads -> MMA chain with the role table's
    producer / MMA split pinned, and returns the schedule (used by tests to confirm that
    splitting loads and MMAs over two warps sustains the initiation interval)."""
    mgr = WAInstructionManager()
    loads_a, loads_b, macs = {}, {}, {}
    stages = -(-load_latency // ii)
    for k in range(iterations):
        for name, bag in (("load_a", loads_a), ("load_b", loads_b)):
            bag[k] = WAInstruction(name, k, [], [], True, 1, load_latency, k * ii)
    for k in range(iterations):
        parents = [loads_a[k], loads_b[k]] + ([macs[k - 1]] if k else [])
        macs[k] = WAInstruction("mac", k, parents, [], False, 1, mma_latency, (k + stages) * ii)
        if k + stages < iterations:   # back-pressure: a ring slot is reused after its MMA
            loads_a[k + stages].ordering_instructions.append(macs[k])
            loads_b[k + stages].ordering_instructions.append(macs[k])
    for bag in (loads_a, loads_b, macs):
        for k in sorted(bag):
            mgr.add_instruction(bag[k])
    sched = mgr.solve(10_000, 2, synchronization_cost, ["load_a", "load_b", "mac"])
    assert sched is not None
    return sched
