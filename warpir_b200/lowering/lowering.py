"""Lowering of tile programs to sm_100a.

``Sm100Lowerer().lower(kernel) -> str`` has the contract of the reference's
``ThunderKittensLowerer().lower`` (warpir/lowering/lowering.py:67-81): a ``Kernel``
in, the text of a CUDA C++ translation unit out, stateless between calls.  The
name ``ThunderKittensLowerer`` is kept as an alias so existing drivers
(``from warpir.lowering import ThunderKittensLowerer``, reference
tests/test_gemm_baseline.py:12,54) pick up the new backend unchanged.

The reference walks the ops and prints one ThunderKittens call per op, which on
Hopper yields a 64x64 tile per CTA with every step fenced by block barriers.
On Blackwell a tile program does not map op-by-op onto the hardware: MMAs are
issued by one thread into tensor memory, loads by another, and the row-wise ops
run in warpgroups that own tensor-memory lanes.  So this lowerer

1. recognises the program from its *dataflow* (not its name): a loads -> MMA ->
   yield loop followed by a store is a GEMM; Q load, then a loop of K/V loads,
   ``mma(transpose_b)``, running row max, ``exp2``, row sum, ``mul_row``, second MMA,
   then ``div_row`` and a store is attention forward with an online softmax;
2. reads the parameters off the IR -- tile shapes from the shared-tile types,
   operand layout from which coordinate carries the induction variable, ring
   depth from ``AllocSharedOp`` (or from the modulo scheduler when the program is
   not pipelined yet), the softmax scale from the ``mul_scalar`` constant, the
   grid mapping from the ``blockIdx`` builtins in the coordinates;
3. emits a translation unit that instantiates the hand-written warp-specialised
   kernel templates (``csrc/gemm_sm100.cuh``, ``csrc/attn_fwd_sm100.cuh``) with
   those parameters and exports one ``extern "C"`` launch function.

Tile shapes that ``tcgen05.mma`` cannot run as written (the reference's programs
use 64x64x64; the MMA here is 128 rows tall) are re-tiled: the emitted kernel
computes the same function with the hardware tile, and the launch grid follows
from the re-tiled shape exactly as the reference's wrapper derives ``N / 64``.
Anything that is neither of the two shapes is emitted op by op
(``lowering/generic.py``): one CTA per block index, one helper call per op, ``mma`` on
the tensor core through tensor memory.  That path is general, not fast.  Programs it
cannot express either raise ``NotImplementedError``; there is no CPU path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, Union

from ..ir import ops as _ops
from ..ir.ops import ForOp, Kernel, Op, Value
from ..ir.types import GlobalType, IntType, SharedBufferType, SharedTileType
from ..passes import modulo_scheduler as _ms
from ..passes.warp_assigner import RoleTable, assign_roles
from ..printing import format_kernel

LOG2E = 1.4426950408889634
HW_BLOCK_M = (128, 256)                   # 256: two 128-row MMAs per k-step share one B tile
HW_BLOCK_K = 64
HW_BLOCK_N = (64, 128, 256)
HW_TILES = ((128, 256), (128, 128), (128, 64), (256, 256))     # CTA tiles the GEMM kernels are instantiated with
ONE_CTA_PER_SM_BYTES = 116 * 1024      # a kernel holding more shared memory than this runs one CTA per SM


def min_stages(block_m: int, block_n: int, block_k: int = HW_BLOCK_K, cta_group: int = 1) -> int:
    """Shallowest ring a GEMM kernel may be instantiated with: every CTA allocates all of tensor memory,
    so two CTAs must never share an SM, which the kernels guarantee by holding more than half of its
    shared memory.  A ring deeper than the schedule asks for does not change what the program
    computes, only how far the loads run ahead."""
    stage = 2 * block_k * (block_m + block_n) // cta_group
    return max(2, ONE_CTA_PER_SM_BYTES // stage + 1)


@dataclass(frozen=True)
class GemmPlan:
    name: str
    a: str
    b: str
    c: str
    tile_as_written: Tuple[int, int, int]      # (block_m, block_n, block_k) in the IR
    b_row_major: bool                          # True: B stored [K,N]; False: B stored [N,K]
    block_n: int                               # hardware tile width, 0 = chosen per launch
    block_m: int                               # hardware tile height (128 or 256) when block_n is fixed
    cta_group: int                             # 2: the tile is computed by a CTA pair (cta_group::2)
    stages: int                                # ring depth of the instantiated kernel
    pipelined_in_ir: bool
    row_builtin: str
    col_builtin: str
    roles: RoleTable

    @property
    def kind(self) -> str:
        return "gemm"


@dataclass(frozen=True)
class AttentionPlan:
    name: str
    q: str
    k: str
    v: str
    o: str
    head_dim: int
    tile_as_written: Tuple[int, int]           # (block_q, block_kv) in the IR
    exp2_scale: float                          # constant applied inside exp2 (scale * log2 e)
    roles: RoleTable                           # of the 64-key kernel (what a causal launch runs)
    roles_wide: RoleTable                      # of the 128-key kernel (what a launch without a mask runs)

    @property
    def kind(self) -> str:
        return "attention"

    @property
    def softmax_scale(self) -> float:
        return self.exp2_scale / LOG2E


Plan = Union[GemmPlan, AttentionPlan]


def _is_builtin(v, axis: Optional[str] = None) -> bool:
    return isinstance(v, Value) and v.name.startswith("blockIdx.") and (axis is None or v.name.endswith(axis))


def _top_loop(kernel: Kernel) -> ForOp:
    loops = [o for o in kernel.body if isinstance(o, ForOp)]
    if len(loops) != 1:
        raise NotImplementedError(f"{kernel.name}: expected exactly one top-level loop, found {len(loops)}")
    return loops[0]


def _reject(kernel: Kernel, why: str):
    raise NotImplementedError(
        f"tile program {kernel.name!r} is not a GEMM or an attention forward this backend knows: {why}")


# --------------------------------------------------------------------------- analysis
def _analyze_gemm(kernel: Kernel, loop: ForOp, machine: Optional["_ms.MachineModel"] = None) -> GemmPlan:
    iv = loop.induction_var
    mmas = [o for o in loop.body if isinstance(o, (_ops.MMAOp, _ops.MMABufOp))]
    mma = mmas[0]
    pre_loop = [o for o in kernel.body if o is not loop]
    pipelined = isinstance(mma, _ops.MMABufOp)
    # The hand-written kernel computes loads -> MMA -> store and nothing else.  Any other op in the loop
    # (a scale, an epilogue on the accumulator) or a yield of something other than the MMA's result would
    # be silently dropped, so such programs are not a GEMM for this purpose: they go op by op.
    loop_ok = (_ops.TMALoadOp, _ops.TMALoadBufOp, _ops.WaitOp, _ops.WaitBufOp, _ops.MMAOp, _ops.MMABufOp, _ops.YieldOp)
    extra = [o for o in loop.body if not isinstance(o, loop_ok)]
    if extra:
        _reject(kernel, f"the loop body holds {type(extra[0]).__name__} besides loads, waits and the MMA")
    yields = [o for o in loop.body if isinstance(o, _ops.YieldOp)]
    if len(yields) != 1 or len(loop.iter_args) != 1 or tuple(yields[0].values) != (mma.result,):
        _reject(kernel, "the loop does not yield exactly the MMA's result")

    if pipelined:
        loads = {o.buf: o for o in loop.body if isinstance(o, _ops.TMALoadBufOp)}
        ld_a, ld_b = loads.get(mma.a_buf), loads.get(mma.b_buf)
        if ld_a is None or ld_b is None:
            _reject(kernel, "an MMA operand ring is never loaded inside the loop")
        a_tile, b_tile = mma.a_buf.type.tile_type, mma.b_buf.type.tile_type
        stages = max(mma.a_buf.type.count, mma.b_buf.type.count)
        transpose_b = None
    else:
        loads = {o.result: o for o in loop.body if isinstance(o, _ops.TMALoadOp)}
        ld_a, ld_b = loads.get(mma.a), loads.get(mma.b)
        if ld_a is None or ld_b is None:
            _reject(kernel, "an MMA operand is not produced by a TMA load inside the loop")
        a_tile, b_tile = mma.a.type, mma.b.type
        stages = 0
        transpose_b = mma.transpose_b

    # accumulate chain: accum is a loop-carried value seeded by a zero tile
    carried = {ia.block_arg: ia for ia in loop.iter_args}
    if mma.accum not in carried:
        _reject(kernel, "the MMA does not accumulate into a loop-carried value")
    init = carried[mma.accum].init
    if not any(isinstance(o, _ops.ZeroOp) and o.result == init for o in pre_loop):
        _reject(kernel, "the accumulator is not zero-initialised")

    # layouts from the coordinates: A(.., row, i); B(.., i, col) row-major or B(.., col, i) K-major
    ca, cb = ld_a.coords, ld_b.coords
    if len(ca) != 4 or len(cb) != 4 or ca[3] != iv or not _is_builtin(ca[2]):
        _reject(kernel, "A must be fetched at (0, 0, blockIdx.*, i)")
    if cb[2] == iv and _is_builtin(cb[3]):
        b_row_major, col = True, cb[3]
    elif cb[3] == iv and _is_builtin(cb[2]):
        b_row_major, col = False, cb[2]
    else:
        _reject(kernel, "B must be fetched at (0, 0, i, blockIdx.*) or (0, 0, blockIdx.*, i)")
    if transpose_b is not None and transpose_b == b_row_major:
        _reject(kernel, "transpose_b disagrees with the coordinates B is fetched at")

    block_m, block_k = a_tile.rows, a_tile.cols
    if b_row_major:
        bk2, block_n = b_tile.rows, b_tile.cols
    else:
        block_n, bk2 = b_tile.rows, b_tile.cols
    if bk2 != block_k:
        _reject(kernel, f"A and B tiles disagree on the K extent ({block_k} vs {bk2})")
    if loop.tile_size not in (None, block_k):
        _reject(kernel, "loop tile_size differs from the K extent of the tiles")

    stores = [o for o in pre_loop if isinstance(o, _ops.TMAStoreOp)]
    after_ok = (_ops.TMAStoreOp, _ops.WaitBufOp, _ops.MMABufOp) if pipelined else (_ops.TMAStoreOp,)
    after = kernel.body[list(kernel.body).index(loop) + 1:]
    stray = [o for o in after if not isinstance(o, after_ok)]
    if stray:
        _reject(kernel, f"{type(stray[0]).__name__} follows the loop: the accumulator is not stored as it is")
    result_of = {r: ia.block_arg for r, ia in zip(loop.results, loop.iter_args)}
    if len(stores) != 1 or result_of.get(stores[0].source) != mma.accum:
        _reject(kernel, "the loop result is not stored exactly once")
    st = stores[0]
    if tuple(st.coords[2:]) != (ca[2], col):
        _reject(kernel, "the store coordinates do not match the operands' grid mapping")

    hw_legal = (block_k == HW_BLOCK_K and (block_m, block_n) in HW_TILES)
    fixed_n = block_n if hw_legal else 0
    cta_group = _ms.default_cta_group(block_m, block_n) if hw_legal else 1
    if fixed_n and not stages:
        sched = _ms.schedule_loop(loop, machine)
        if sched is None:
            _reject(kernel, "the loop cannot be scheduled on this machine model")
        stages = sched.num_stages
    if fixed_n:
        # the depth the program (or the scheduler) asks for, but never so shallow that two CTAs fit on an SM
        stages = max(stages, min_stages(block_m, block_n, block_k, cta_group))
        if stages * 2 * block_k * (block_m + block_n) // cta_group > _ms.SM100_RING_BUDGET:
            _reject(kernel, f"{stages} stages of a {block_m}x{block_n}x{block_k} tile do not fit in shared memory")
    else:
        stages = 0   # re-tiled: width and ring depth are picked per launch from the problem size
    return GemmPlan(name=kernel.name, a=ld_a.source.name, b=ld_b.source.name, c=st.dest.name,
                    tile_as_written=(block_m, block_n, block_k), b_row_major=b_row_major, block_n=fixed_n,
                    block_m=block_m if fixed_n else 0, cta_group=cta_group, stages=stages, pipelined_in_ir=pipelined,
                    row_builtin=ca[2].name, col_builtin=col.name,
                    roles=assign_roles(kernel, tile_rows=block_m if fixed_n else 128, cta_group=cta_group))


def _analyze_attention(kernel: Kernel, loop: ForOp) -> AttentionPlan:
    iv = loop.induction_var
    body = loop.body
    mmas = [o for o in body if isinstance(o, _ops.MMAOp)]
    qk, pv = mmas
    if not qk.transpose_b or pv.transpose_b:
        _reject(kernel, "expected S = Q K^T (transpose_b) followed by O += P V")
    loads = {o.result: o for o in body if isinstance(o, _ops.TMALoadOp)}
    pre = {o.result: o for o in kernel.body if isinstance(o, _ops.TMALoadOp)}
    if qk.a not in pre or qk.b not in loads or pv.b not in loads:
        _reject(kernel, "Q must be loaded before the loop, K and V inside it")
    ld_q, ld_k, ld_v = pre[qk.a], loads[qk.b], loads[pv.b]
    if ld_k.coords[2] != iv or ld_v.coords[2] != iv or not _is_builtin(ld_q.coords[2]):
        _reject(kernel, "K/V tiles must advance with the loop, the Q tile with blockIdx")

    def producer(v: Value) -> Optional[Op]:
        return next((o for o in body if getattr(o, "result", None) == v), None)

    # P = exp2(scale * S - scale * rowmax): walk back from the PV operand
    cast = producer(pv.a)
    ex = producer(cast.input) if isinstance(cast, _ops.CopyOp) else None
    shifted = producer(ex.input) if isinstance(ex, _ops.Exp2Op) else None
    scaled = producer(shifted.tile) if isinstance(shifted, _ops.SubRowOp) else None
    if not isinstance(scaled, _ops.MulScalarOp) or scaled.input != qk.result:
        _reject(kernel, "P is not exp2(scale * S - row offset) of the score tile")
    vec = producer(shifted.vec)
    rmax = producer(vec.input) if isinstance(vec, _ops.MulScalarOp) else None
    if not isinstance(rmax, _ops.RowMaxOp) or rmax.tile != qk.result or vec.scalar != scaled.scalar:
        _reject(kernel, "the row offset is not the scaled running row max of S")
    if not any(isinstance(o, _ops.RowSumOp) and o.tile == ex.result for o in body):
        _reject(kernel, "the normaliser is not the running row sum of P")
    resc = producer(pv.accum)
    if not isinstance(resc, _ops.MulRowOp):
        _reject(kernel, "O is not rescaled by the correction factor before accumulation")
    post = [o for o in kernel.body if isinstance(o, (_ops.DivRowOp, _ops.TMAStoreOp))]
    if [type(o) for o in post] != [_ops.DivRowOp, _ops.TMAStoreOp] or post[1].source != post[0].result:
        _reject(kernel, "expected O / l followed by one store")
    q_tile, kv_tile = ld_q.result.type, ld_k.result.type
    if q_tile.cols != kv_tile.cols or q_tile.cols not in (64, 128):
        _reject(kernel, f"head dimension {q_tile.cols} (the kernels cover 64 and 128)")
    if not scaled.scalar > 0:
        _reject(kernel, "the exp2 scale must be positive")
    return AttentionPlan(name=kernel.name, q=ld_q.source.name, k=ld_k.source.name, v=ld_v.source.name,
                         o=post[1].dest.name, head_dim=q_tile.cols, tile_as_written=(q_tile.rows, kv_tile.rows),
                         exp2_scale=float(scaled.scalar), roles=assign_roles(kernel, keys_per_block=64),
                         roles_wide=assign_roles(kernel, keys_per_block=128))


def analyze(kernel: Kernel, machine: Optional["_ms.MachineModel"] = None) -> Plan:
    """Recognise ``kernel`` and extract the parameters its sm_100a kernel is instantiated with.
    ``machine``: the model an un-pipelined GEMM loop is scheduled on for its ring depth (default: the
    sm_100a model of its tile shape)."""
    loop = _top_loop(kernel)
    n_mma = sum(isinstance(o, (_ops.MMAOp, _ops.MMABufOp)) for o in loop.body)
    for v in (*kernel.inputs, *kernel.outputs):
        if not isinstance(v.type, (GlobalType, IntType)):
            raise TypeError(f"Cannot lower kernel argument {v!r}")
    if n_mma == 1:
        return _analyze_gemm(kernel, loop, machine)
    if n_mma == 2:
        return _analyze_attention(kernel, loop)
    _reject(kernel, f"{n_mma} MMAs in the loop")


# --------------------------------------------------------------------------- emission
_PREAMBLE = """\
// Translation unit emitted by warpir_b200.lowering.Sm100Lowerer for sm_100a.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -shared -Xcompiler -fPIC -I <repo root>
//
// Tile program:
{ir}
//
// Plan:
{plan}
{includes}

// Arguments follow the kernel signature: `tensors` holds the device pointers of the
// global inputs, then the global outputs, in declaration order; `dims` holds four
// extents (batch, depth, rows, cols) per tensor in the same order; `scalars` holds the
// int inputs in declaration order.  Returns 0 or a negative WARPIR_E* code; the text of
// a failure is available from {name}_last_error().
extern "C" const char* {name}_last_error(void) {{ return wir::host::g_last_error; }}
extern "C" const char* {name}_kind(void) {{ return "{kind}"; }}
extern "C" int {name}_read_status(int device, void* stream, int* code, int* detail) {{
  return wir::host::read_status_impl(device, stream, code, detail);
}}
"""


_INCLUDES_KERNELS = '#include "warpir_b200/csrc/launch.cuh"'
_INCLUDES_OP_BY_OP = '#include "warpir_b200/csrc/host_common.cuh"\n#include "warpir_b200/csrc/tile_program.cuh"'


def _comment(text: str) -> str:
    return "\n".join("//   " + line for line in text.splitlines())


def _tensor_index(kernel: Kernel, name: str) -> int:
    tensors = [v.name for v in (*kernel.inputs, *kernel.outputs) if isinstance(v.type, GlobalType)]
    return tensors.index(name)


def _emit_gemm(kernel: Kernel, plan: GemmPlan) -> str:
    ia, ib, ic = (_tensor_index(kernel, n) for n in (plan.a, plan.b, plan.c))
    b_layout = 0 if plan.b_row_major else 1
    b_mn = 'true' if plan.b_row_major else 'false'
    if plan.block_n and plan.cta_group == 2:
        inst = f"&wir::host::launch_gemm_pair_cfg<{plan.stages}, {b_mn}>"
        fixed = (f"{plan.block_n}, /*splits=*/1, device, stream, {inst}, /*tile rows / 128=*/{plan.block_m // 128}, "
                 f"nullptr, 0, /*CTA pair=*/true")
    elif plan.block_n:
        inst = f"&wir::host::launch_gemm_cfg<{plan.block_n}, {plan.stages}, {b_mn}, {plan.block_m // 128}>"
        fixed = f"{plan.block_n}, /*splits=*/1, device, stream, {inst}, /*tile rows / 128=*/{plan.block_m // 128}"
    else:
        fixed = "/*block_n: per launch*/0, /*splits: per launch*/0, device, stream"
    n_dim = "dims[4 * {i} + 3]".format(i=ic)
    return f"""
// who issues what in the instantiated kernel, as planned by the warp-assignment pass
{plan.roles.static_asserts()}

extern "C" int {plan.name}_launch(const void* const* tensors, const int64_t* dims, const int64_t* scalars,
                                  int device, void* stream) {{
  (void)scalars;  // the K extent is taken from the A tensor, as the loop bound of the program is
  const int64_t M = dims[4 * {ia} + 2], K = dims[4 * {ia} + 3], N = {n_dim};
  const int64_t Kb = dims[4 * {ib} + {2 if plan.b_row_major else 3}], Nb = dims[4 * {ib} + {3 if plan.b_row_major else 2}];
  if (Kb != K || Nb != N || dims[4 * {ic} + 2] != M)
    return wir::host::fail(WARPIR_ESHAPE, "{plan.name}: operand extents disagree");
  return wir::host::gemm_impl(tensors[{ia}], tensors[{ib}], const_cast<void*>(tensors[{ic}]), M, N, K,
                              /*b_layout=*/{b_layout}, {fixed});
}}
"""


def _emit_attention(kernel: Kernel, plan: AttentionPlan) -> str:
    iq, ik, iv_, io = (_tensor_index(kernel, n) for n in (plan.q, plan.k, plan.v, plan.o))
    return f"""
// who issues what in the two kernels a launch may run (64-key blocks with a causal mask, 128-key blocks
// without), as planned by the warp-assignment pass
{plan.roles.static_asserts()}
{plan.roles_wide.static_asserts()}

// `scalars` may carry two optional trailing values after the program's own ints:
// scalars[n_ints] != 0 selects the causal variant, and a non-NULL tensors[n_tensors] is an
// fp32 [B, H, S] buffer that receives the log-sum-exp.  (The tile program as written is
// non-causal and has no such output; both are launcher-level extensions.)
extern "C" int {plan.name}_launch(const void* const* tensors, const int64_t* dims, const int64_t* scalars,
                                  int device, void* stream) {{
  constexpr int kTensors = {len([v for v in (*kernel.inputs, *kernel.outputs) if isinstance(v.type, GlobalType)])};
  constexpr int kInts = {len([v for v in kernel.inputs if isinstance(v.type, IntType)])};
  const int64_t B = dims[4 * {iq} + 0], H = dims[4 * {iq} + 1], S = dims[4 * {iq} + 2], D = dims[4 * {iq} + 3];
  const int64_t Hkv = dims[4 * {ik} + 1];
  if (D != {plan.head_dim})
    return wir::host::fail(WARPIR_ESHAPE, "{plan.name}: head dimension %lld, program was built for {plan.head_dim}", (long long)D);
  if (dims[4 * {ik} + 2] != S || dims[4 * {iv_} + 2] != S || dims[4 * {io} + 2] != S)
    return wir::host::fail(WARPIR_ESHAPE, "{plan.name}: sequence extents disagree");
  const int causal = scalars[kInts] != 0;
  float* lse = static_cast<float*>(const_cast<void*>(tensors[kTensors]));
  // exp2 constant of the program {plan.exp2_scale!r} = softmax scale * log2(e)
  return wir::host::attn_impl(tensors[{iq}], tensors[{ik}], tensors[{iv_}], const_cast<void*>(tensors[{io}]), lse,
                              B, H, Hkv, S, D, {plan.softmax_scale!r}f, causal, device, stream);
}}
"""


class Sm100Lowerer:
    """Tile program -> sm_100a translation unit (see the module docstring).

    ``op_by_op=True`` skips the recognition step and emits every program, the GEMM and
    the attention forward included, one helper call per op (``lowering/generic.py``)."""

    def __init__(self, op_by_op: bool = False, problem: Optional[Tuple[int, int, int]] = None,
                 machine: Optional["_ms.MachineModel"] = None) -> None:
        """``problem = (M, N, K)``: a GEMM program is re-tiled for that problem by the tile planner
        (``passes/tile_planner.py``), pipelined by ``kernel_pass`` and pinned to the resulting
        instantiation, instead of leaving the tile to the launcher.  ``machine``: the model the ring depth
        of a not yet pipelined GEMM loop is solved on (default: the sm_100a model of its tile)."""
        self.op_by_op = op_by_op
        self.problem = problem
        self.machine = machine
        self.plan = None
        self.tile_plan = None

    def lower(self, kernel: Kernel) -> str:
        from .generic import emit_tile_program
        self.plan = None
        self.tile_plan = None
        plan, body, why = None, None, ""
        planned_note = ""
        if not self.op_by_op:
            try:
                plan = analyze(kernel, self.machine)
                if isinstance(plan, GemmPlan) and self.problem is not None:
                    from ..passes.tile_planner import plan_gemm, retile
                    tp = plan_gemm(*self.problem)
                    self.tile_plan = tp
                    if not tp.stream_k and tp.a_rows == 128:
                        kernel = _ms.kernel_pass(retile(kernel, tp), self.machine)
                        plan = analyze(kernel, self.machine)
                        planned_note = f"re-tiled for M, N, K = {self.problem}: {tp.describe()}"
                    else:
                        planned_note = (f"for M, N, K = {self.problem} the planner asks for {tp.describe()}: "
                                        "left to the launcher, which implements that path")
            except NotImplementedError as exc:     # not one of the two recognised programs
                why = str(exc)
        if plan is None:
            plan, body = emit_tile_program(kernel)
            shown = {k: v for k, v in vars(plan).items() if k != "tiles"}
            shown["tiles"] = {t.name: f"{t.count} x {t.rows}x{t.cols} at byte {t.offset}, barrier {t.bar}"
                              for t in plan.tiles.values()}
            if why:
                shown["emitted op by op because"] = why
        else:
            shown = {k: v for k, v in vars(plan).items() if k not in ("roles", "roles_wide")}
            shown["warps"] = {r.name: r.warps for r in plan.roles.roles}
            if planned_note:
                shown["tile planner"] = planned_note
            body = _emit_gemm(kernel, plan) if isinstance(plan, GemmPlan) else _emit_attention(kernel, plan)
        self.plan = plan
        head = _PREAMBLE.format(ir=_comment(format_kernel(kernel)),
                                plan=_comment("\n".join(f"{k} = {v}" for k, v in shown.items())),
                                name=kernel.name, kind=plan.kind,
                                includes=_INCLUDES_OP_BY_OP if plan.kind == "tile_program" else _INCLUDES_KERNELS)
        return head + body


# Existing drivers import the lowerer under the reference's class name.
ThunderKittensLowerer = Sm100Lowerer
