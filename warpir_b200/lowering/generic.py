"""Op-by-op emission of tile programs for sm_100a.

The reference's lowerer prints one ThunderKittens call per op
(warpir/lowering/lowering.py:427-570).  Programs that are neither the GEMM nor the
attention forward of the hot path get the same treatment here, against the helpers of
``csrc/tile_program.cuh`` instead of ThunderKittens: one CTA of 128 threads per block
index, one row of every register tile per thread, shared tiles filled by TMA, ``mma``
on the tensor core through tensor memory.  Semantics follow the op docstrings of the
reference (warpir/ir/ops.py:57-230):

* ``mma`` computes ``a @ b + accum``; with ``transpose_b`` it computes ``a @ b^T`` and,
  like the reference's ``mm_ABt`` (lowering.py:462), does not add ``accum``;
* ``mma_buf`` accumulates in place into its ``accum`` value (lowering.py:474-480);
* ``copy`` converts when the element types differ (fp32 -> bf16 rounds to nearest even);
* ``row_max`` / ``row_sum`` fold the previous vector in; ``*_row`` ops broadcast one
  scalar per row;
* loads past the end of a tensor read zeros, stores past the end are dropped;
* the drain counter ``drain(+k, %S)`` names the slot ``k`` after the last one the
  steady-state loop consumed.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple, Union

from ..ir import ops as _ops
from ..ir.ops import BufSlotExpr, ForOp, Kernel, Op, Value
from ..ir.types import (ColVecType, GlobalType, GPUType, IntType, RegTileType, SharedBufferType,
                        SharedTileType)

CHUNK_BYTES = 128 * 128          # one 64-column chunk of a shared tile, padded to 128 rows
SMEM_BUDGET = 200 * 1024
MAX_BARRIERS = 32


def _reject(kernel: Kernel, why: str):
    raise NotImplementedError(f"tile program {kernel.name!r} cannot be emitted op by op: {why}")


def _ident(name: str) -> str:
    return "v_" + re.sub(r"\W", "_", name)


@dataclass
class _Tile:
    """A shared tile or a ring of them."""
    name: str
    rows: int
    cols: int
    count: int
    offset: int = 0
    bar: int = 0

    @property
    def bytes_per_slot(self) -> int:
        return (self.cols // 64) * CHUNK_BYTES


@dataclass
class TileProgramPlan:
    name: str
    rows: int                                   # rows of the CTA tile (4 x the per-warp rows)
    tensors: List[str]                          # global tensors in signature order
    ints: List[str]                             # int inputs in signature order
    tiles: Dict[str, _Tile] = field(default_factory=dict)
    maps: List[Tuple[int, int]] = field(default_factory=list)   # (tensor index, box rows)
    stored: List[int] = field(default_factory=list)             # tensor indices written by stores
    smem_bytes: int = 0
    tmem_cols: int = 32
    a_col: int = 0                              # tensor-memory column of register-tile A operands
    barriers: int = 1
    grid: Tuple[str, str, str] = ("1", "1", "1")
    n_mma: int = 0

    @property
    def kind(self) -> str:
        return "tile_program"


class _Emitter:
    def __init__(self, kernel: Kernel):
        self.k = kernel
        self.lines: List[str] = []
        self.depth = 1
        self.loop_depth = 0
        self.producers: Dict[Value, Op] = {}
        self.loop_ivs: List[Value] = []
        tensors = [v for v in (*kernel.inputs, *kernel.outputs) if isinstance(v.type, GlobalType)]
        ints = [v for v in kernel.inputs if isinstance(v.type, IntType)]
        for v in (*kernel.inputs, *kernel.outputs):
            if not isinstance(v.type, (GlobalType, IntType)):
                raise TypeError(f"Cannot lower kernel argument {v!r}")
        for v in tensors:
            if v.type.data_type != GPUType.bf16:
                _reject(kernel, f"global tensor {v.name} is not bf16")
        self.tensor_index = {v.name: i for i, v in enumerate(tensors)}
        self.int_index = {v.name: i for i, v in enumerate(ints)}
        self.plan = TileProgramPlan(name=kernel.name, rows=0, tensors=[v.name for v in tensors],
                                    ints=[v.name for v in ints])
        self.values: Dict[str, Value] = {}       # register values to declare
        self.all_ops: List[Tuple[Op, int]] = []
        self._walk(kernel.body, 0)

    # ------------------------------------------------------------------ analysis
    def _walk(self, ops, depth):
        for op in ops:
            self.all_ops.append((op, depth))
            res = getattr(op, "result", None)
            if isinstance(res, Value):
                self.producers[res] = op
            if isinstance(op, ForOp):
                self.loop_ivs.append(op.induction_var)
                self._walk(op.body, depth + 1)

    def _note_value(self, v: Value):
        if isinstance(v.type, (RegTileType, ColVecType)):
            rows = 4 * v.type.rows
            if self.plan.rows == 0:
                self.plan.rows = rows
            elif self.plan.rows != rows:
                _reject(self.k, f"register values disagree on the tile height ({self.plan.rows} vs {rows} rows)")
            if isinstance(v.type, RegTileType) and v.type.cols % 16 != 0:
                _reject(self.k, f"{v.name}: register tile width {v.type.cols} is not a multiple of 16")
            self.values.setdefault(v.name, v)

    def analyze(self):
        k, plan = self.k, self.plan
        for op, _ in self.all_ops:
            if isinstance(op, ForOp):
                for ia in op.iter_args:
                    self._note_value(ia.block_arg)
                    self._note_value(ia.init)
                for r in op.results:
                    self._note_value(r)
                continue
            for fname, role in op.roles:
                x = getattr(op, fname)
                if role in ("result", "use") and isinstance(x, Value):
                    self._note_value(x)
                elif role == "uses":
                    for v in x:
                        self._note_value(v)
        if plan.rows == 0:
            _reject(k, "the program holds no register tile")
        if plan.rows > 128:
            _reject(k, f"tile height {plan.rows} exceeds the 128 rows of one CTA")

        # shared tiles and rings
        for op, _ in self.all_ops:
            if isinstance(op, _ops.TMALoadOp):
                t = op.result.type
                if not isinstance(t, SharedTileType):
                    _reject(k, f"tma_load result {op.result.name} is not a shared tile")
                self._add_tile(op.result.name, t, 1)
            elif isinstance(op, _ops.AllocSharedOp):
                t = op.result.type
                if not isinstance(t, SharedBufferType):
                    _reject(k, f"alloc_shared result {op.result.name} is not a shared buffer")
                self._add_tile(op.result.name, t.tile_type, t.count)
        offset, bar = 0, 1
        for t in plan.tiles.values():
            t.offset, t.bar = offset, bar
            offset += t.count * t.bytes_per_slot
            bar += t.count
        plan.smem_bytes = offset + 1024          # slack for aligning the data area to 1024 bytes
        plan.barriers = bar
        if offset > SMEM_BUDGET:
            _reject(k, f"shared tiles need {offset} bytes (padded), more than the {SMEM_BUDGET} available")
        if bar > MAX_BARRIERS:
            _reject(k, f"{bar} barriers needed, at most {MAX_BARRIERS} supported")

        # tensor memory: accumulator at column 0, register-tile A operands behind it
        max_n, max_ka = 16, 0
        for op, _ in self.all_ops:
            if isinstance(op, (_ops.MMAOp, _ops.MMABufOp)):
                plan.n_mma += 1
                max_n = max(max_n, op.result.type.cols)
                if isinstance(op, _ops.MMAOp) and isinstance(op.a.type, RegTileType):
                    max_ka = max(max_ka, op.a.type.cols)
        plan.a_col = (max_n + 31) // 32 * 32
        need = plan.a_col + max_ka // 2
        plan.tmem_cols = 32
        while plan.tmem_cols < need:
            plan.tmem_cols *= 2
        if plan.tmem_cols > 512:
            _reject(k, f"{need} tensor-memory columns needed, 512 available")

        # launch grid: one CTA per tile of what the stores (else the loads) address with blockIdx
        grid = {"x": None, "y": None, "z": None}
        def scan(op, tensor: Value, tile_rows: int, tile_cols: int):
            t = self.tensor_index[tensor.name]
            for pos, c in enumerate(op.coords):
                if isinstance(c, Value) and c.name.startswith("blockIdx.") and grid.get(c.name[-1]) is None:
                    ext = f"dims[{4 * t + pos}]"
                    unit = {0: 1, 1: 1, 2: tile_rows, 3: tile_cols}[pos]
                    grid[c.name[-1]] = f"(({ext} + {unit - 1}) / {unit})"
        for op, _ in self.all_ops:
            if isinstance(op, _ops.TMAStoreOp):
                rows, cols = self._store_unit(op)
                scan(op, op.dest, rows, cols)
        for op, _ in self.all_ops:
            if isinstance(op, (_ops.TMALoadOp, _ops.TMALoadBufOp)):
                tile = plan.tiles[op.result.name if isinstance(op, _ops.TMALoadOp) else op.buf.name]
                scan(op, op.source, tile.rows, tile.cols)
        plan.grid = tuple(grid[a] or "1" for a in "xyz")
        return plan

    def _add_tile(self, name: str, t: SharedTileType, count: int):
        if t.data_type != GPUType.bf16:
            _reject(self.k, f"shared tile {name} is not bf16")
        if t.cols % 64 != 0 or t.rows % 8 != 0 or not (8 <= t.rows <= 128) or t.cols > 256:
            _reject(self.k, f"shared tile {name} is {t.rows}x{t.cols}; rows must be a multiple of 8 up to 128, "
                            f"columns a multiple of 64 up to 256")
        if name in self.plan.tiles:
            _reject(self.k, f"shared tile {name} is defined twice")
        self.plan.tiles[name] = _Tile(name=name, rows=t.rows, cols=t.cols, count=count)

    def _store_unit(self, op) -> Tuple[int, int]:
        sub = getattr(op.dest.type, "sub_tile_type", None)
        if isinstance(sub, SharedTileType):
            return sub.rows, sub.cols
        return self.plan.rows, op.source.type.cols

    def _map_index(self, tensor: Value, box_rows: int) -> int:
        key = (self.tensor_index[tensor.name], box_rows)
        if key not in self.plan.maps:
            self.plan.maps.append(key)
        return self.plan.maps.index(key)

    # ------------------------------------------------------------------ emission helpers
    def _emit(self, text: str):
        self.lines.append("  " * self.depth + text)

    def _int_expr(self, x: Union[Value, int]) -> str:
        if isinstance(x, int):
            return str(x)
        if x.name.startswith("blockIdx."):
            return f"static_cast<int>({x.name})"
        if x.name in self.int_index:
            return f"args.scalar[{self.int_index[x.name]}]"
        if x in self.loop_ivs:
            return _ident(x.name)
        _reject(self.k, f"integer value {x.name} is neither an input, a block index nor a loop counter")

    def _slot_expr(self, slot) -> str:
        if isinstance(slot, int):
            return str(slot)
        if slot.value is None:
            return f"wir::tp::slot_of(ctx.consumed + ({slot.offset}), {slot.modulus})"
        return f"wir::tp::slot_of({self._int_expr(slot.value)} + ({slot.offset}), {slot.modulus})"

    def _tile_addr(self, tile: _Tile, slot: Optional[str] = None) -> str:
        base = f"ctx.smem + {tile.offset}u"
        return base if slot is None else f"{base} + {tile.bytes_per_slot}u * static_cast<uint32_t>({slot})"

    def _tile_bar(self, tile: _Tile, slot: Optional[str] = None) -> str:
        return str(tile.bar) if slot is None else f"{tile.bar} + ({slot})"

    def _is_tile(self, v: Value) -> bool:
        return isinstance(v.type, RegTileType)

    def _known_zero(self, v: Value) -> bool:
        return isinstance(self.producers.get(v), _ops.ZeroOp)

    def _load(self, tile: _Tile, slot: Optional[str], source: Value, coords):
        if len(coords) != 4:
            _reject(self.k, "tile coordinates are (batch, depth, row, col)")
        t = self.tensor_index[source.name]
        m = self._map_index(source, tile.rows)
        b, d, r, c = (self._int_expr(x) for x in coords)
        plane = f"({b}) * static_cast<int>(args.ext[{t}][1]) + ({d})"
        self._emit(f"wir::tp::load_tile<{tile.rows}, {tile.cols}>(ctx, &args.maps[{m}], {self._tile_addr(tile, slot)}, "
                   f"{self._tile_bar(tile, slot)}, ({c}) * {tile.cols}, ({r}) * {tile.rows}, {plane});")

    def _b_is_mn(self, ring: Value) -> bool:
        """Layout of a ring used as the B operand of ``mma_buf``: the loads that fill it tell
        whether the loop counter walks its rows ([K, N], N contiguous) or its columns."""
        for op, _ in self.all_ops:
            if isinstance(op, _ops.TMALoadBufOp) and op.buf == ring:
                if isinstance(op.coords[3], Value) and op.coords[3] in self.loop_ivs:
                    return False
                if isinstance(op.coords[2], Value) and op.coords[2] in self.loop_ivs:
                    return True
        return True

    def _mma_shapes(self, n: int, a_rows_cols: Tuple[int, int], b: Tuple[int, int], b_mn: bool, what: str):
        k = a_rows_cols[1]
        want = (k, n) if b_mn else (n, k)
        if b != want:
            _reject(self.k, f"{what}: B tile is {b[0]}x{b[1]}, expected {want[0]}x{want[1]}")
        if k % 16 != 0 or n % 16 != 0 or n > 256:
            _reject(self.k, f"{what}: unsupported MMA shape N={n}, K={k}")
        return k

    # ------------------------------------------------------------------ ops
    def _op(self, op: Op):
        T = _ops
        name = lambda v: _ident(v.name)
        if isinstance(op, ForOp):
            return self._for(op)
        if isinstance(op, T.AllocSharedOp) or isinstance(op, T.YieldOp):
            return
        if isinstance(op, T.ZeroOp) or isinstance(op, T.NegInftyOp):
            val = "0.f" if isinstance(op, T.ZeroOp) else "-INFINITY"
            if self._is_tile(op.result):
                self._emit(f"{name(op.result)} = wir::tp::fill<{op.result.type.cols}>({val});")
            else:
                self._emit(f"{name(op.result)} = {val};")
            return
        if isinstance(op, T.TMALoadOp):
            return self._load(self.plan.tiles[op.result.name], None, op.source, op.coords)
        if isinstance(op, T.TMALoadBufOp):
            return self._load(self.plan.tiles[op.buf.name], self._slot_expr(op.slot), op.source, op.coords)
        if isinstance(op, T.WaitOp):
            for v in op.values:
                self._emit(f"wir::tp::ensure_loaded(ctx, {self.plan.tiles[v.name].bar});")
            return
        if isinstance(op, T.WaitBufOp):
            slot = self._slot_expr(op.slot)
            for ring in op.bufs:
                self._emit(f"wir::tp::ensure_loaded(ctx, {self._tile_bar(self.plan.tiles[ring.name], slot)});")
            return
        if isinstance(op, T.MMAOp):
            return self._mma(op)
        if isinstance(op, T.MMABufOp):
            return self._mma_buf(op)
        if isinstance(op, T.TMAStoreOp):
            return self._store(op)
        if isinstance(op, T.CopyOp):
            narrow = op.result.type.data_type == GPUType.bf16 and op.input.type.data_type != GPUType.bf16
            fn = "to_bf16" if narrow else "copy"
            self._emit(f"{name(op.result)} = wir::tp::{fn}({name(op.input)});")
            return
        if isinstance(op, T.MulScalarOp):
            self._emit(f"{name(op.result)} = wir::tp::mul_scalar({name(op.input)}, {float(op.scalar)!r}f);")
            return
        if isinstance(op, T.Exp2Op):
            self._emit(f"{name(op.result)} = wir::tp::exp2({name(op.input)});")
            return
        if isinstance(op, (T.SubOp, T.MulOp)):
            if self._is_tile(op.a) != self._is_tile(op.b):
                _reject(self.k, f"{op.mnemonic} mixes a tile with a vector; use the *_row ops")
            self._emit(f"{name(op.result)} = wir::tp::{op.mnemonic}({name(op.a)}, {name(op.b)});")
            return
        if isinstance(op, (T.RowMaxOp, T.RowSumOp)):
            self._emit(f"{name(op.result)} = wir::tp::{op.mnemonic}({name(op.tile)}, {name(op.prev)});")
            return
        if isinstance(op, (T.SubRowOp, T.MulRowOp, T.DivRowOp)):
            self._emit(f"{name(op.result)} = wir::tp::{op.mnemonic}({name(op.tile)}, {name(op.vec)});")
            return
        _reject(self.k, f"no emission rule for op {type(op).__name__}")

    def _mma(self, op):
        name = lambda v: _ident(v.name)
        n = op.result.type.cols
        b_mn = not op.transpose_b
        bt = op.b.type
        if not isinstance(bt, SharedTileType):
            _reject(self.k, "the B operand of mma must be a shared tile")
        if op.transpose_b and not self._known_zero(op.accum):
            _reject(self.k, f"mma -> {op.result.name}: with transpose_b the reference's mma does not accumulate "
                            f"(mm_ABt); pass a zero tile as accum")
        accumulate = b_mn and not self._known_zero(op.accum)
        if accumulate:
            self._emit(f"{name(op.result)} = {name(op.accum)};")
        b_tile = self.plan.tiles[op.b.name]
        self._emit(f"wir::tp::ensure_loaded(ctx, {b_tile.bar});")
        acc = "true" if accumulate else "false"
        if isinstance(op.a.type, SharedTileType):
            k = self._mma_shapes(n, (op.a.type.rows, op.a.type.cols), (bt.rows, bt.cols), b_mn, f"mma -> {op.result.name}")
            a_tile = self.plan.tiles[op.a.name]
            self._emit(f"wir::tp::ensure_loaded(ctx, {a_tile.bar});")
            self._emit(f"wir::tp::mma_smem<{n}, {k}, {str(b_mn).lower()}>(ctx, {self._tile_addr(a_tile)}, "
                       f"{self._tile_addr(b_tile)}, {name(op.result)}, {acc});")
        elif isinstance(op.a.type, RegTileType):
            if op.a.type.data_type != GPUType.bf16:
                _reject(self.k, f"register-tile A operand {op.a.name} must be bf16 (convert it with copy)")
            k = self._mma_shapes(n, (self.plan.rows, op.a.type.cols), (bt.rows, bt.cols), b_mn, f"mma -> {op.result.name}")
            if k % 32 != 0:
                _reject(self.k, f"register-tile A operand needs K a multiple of 32, got {k}")
            self._emit(f"wir::tp::mma_regs<{n}, {k}, {str(b_mn).lower()}, {self.plan.a_col}>(ctx, {name(op.a)}, "
                       f"{self._tile_addr(b_tile)}, {name(op.result)}, {acc});")
        else:
            _reject(self.k, f"A operand {op.a.name} is neither a shared tile nor a register tile")

    def _mma_buf(self, op):
        name = lambda v: _ident(v.name)
        n = op.result.type.cols
        a_ring, b_ring = self.plan.tiles[op.a_buf.name], self.plan.tiles[op.b_buf.name]
        b_mn = self._b_is_mn(op.b_buf)
        k = self._mma_shapes(n, (a_ring.rows, a_ring.cols), (b_ring.rows, b_ring.cols), b_mn, f"mma_buf -> {op.result.name}")
        sa, sb = self._slot_expr(op.a_slot), self._slot_expr(op.b_slot)
        self._emit(f"wir::tp::ensure_loaded(ctx, {self._tile_bar(a_ring, sa)});")
        self._emit(f"wir::tp::ensure_loaded(ctx, {self._tile_bar(b_ring, sb)});")
        self._emit(f"wir::tp::mma_smem<{n}, {k}, {str(b_mn).lower()}>(ctx, {self._tile_addr(a_ring, sa)}, "
                   f"{self._tile_addr(b_ring, sb)}, {name(op.accum)}, true);")
        self._emit(f"{name(op.result)} = {name(op.accum)};")
        if self.loop_depth > 0:
            self._emit("++ctx.consumed;")

    def _store(self, op):
        t = self.tensor_index[op.dest.name]
        if t not in self.plan.stored:
            self.plan.stored.append(t)
        if not self._is_tile(op.source):
            _reject(self.k, "only register tiles can be stored")
        rows, cols = self._store_unit(op)
        b, d, r, c = (self._int_expr(x) for x in op.coords)
        n = op.source.type.cols
        self._emit(f"wir::tp::store_tile<{n}>(ctx, {_ident(op.source.name)}, args.out[{self.plan.stored.index(t)}], "
                   f"args.ext[{t}][2], args.ext[{t}][3], ({b}) * args.ext[{t}][1] + ({d}), "
                   f"static_cast<long long>({r}) * {rows}, static_cast<long long>({c}) * {cols}, {self.plan.rows});")

    def _for(self, op: ForOp):
        iv = _ident(op.induction_var.name)
        for ia in op.iter_args:
            self._emit(f"{_ident(ia.block_arg.name)} = {_ident(ia.init.name)};")
        stop = self._int_expr(op.stop)
        if op.tile_size is not None:
            stop = f"(({stop}) + {op.tile_size - 1}) / {op.tile_size}"
        self._emit("#pragma unroll 1")
        self._emit(f"for (int {iv} = {self._int_expr(op.start)}; {iv} < {stop}; {iv} += {self._int_expr(op.step)}) {{")
        self.depth += 1
        self.loop_depth += 1
        for inner in op.body:
            self._op(inner)
        yields = [o for o in op.body if isinstance(o, _ops.YieldOp)]
        if op.iter_args:
            if len(yields) != 1 or len(yields[0].values) != len(op.iter_args):
                _reject(self.k, "a loop with iter_args needs one yield with as many values")
            # all yielded values are read before any block argument is overwritten
            for i, v in enumerate(yields[0].values):
                self._emit(f"const auto y{i}_{iv} = {_ident(v.name)};")
            for i, ia in enumerate(op.iter_args):
                self._emit(f"{_ident(ia.block_arg.name)} = y{i}_{iv};")
        self.loop_depth -= 1
        self.depth -= 1
        self._emit("}")
        for r, ia in zip(op.results, op.iter_args):
            self._emit(f"{_ident(r.name)} = {_ident(ia.block_arg.name)};")

    def body(self) -> str:
        for op in self.k.body:
            self._op(op)
        return "\n".join(self.lines)


def emit_tile_program(kernel: Kernel) -> Tuple[TileProgramPlan, str]:
    """Plan and CUDA text (kernel plus ``<name>_launch``) for ``kernel``; the caller puts the
    shared preamble of emitted translation units in front."""
    em = _Emitter(kernel)
    plan = em.analyze()
    body = em.body()          # also fills plan.maps and plan.stored
    if not plan.stored:
        _reject(kernel, "the program stores nothing")
    name = kernel.name
    decls = []
    for v in em.values.values():
        if isinstance(v.type, RegTileType):
            decls.append(f"  wir::tp::Tile<{v.type.cols}> {_ident(v.name)} = wir::tp::fill<{v.type.cols}>(0.f);")
        else:
            decls.append(f"  float {_ident(v.name)} = 0.f;")
    n_t, n_i = len(plan.tensors), max(1, len(plan.ints))
    maps = "\n".join(
        f"  if (int rc = tile_program_tmap(&args.maps[{m}], tensors[{t}], dims + {4 * t}, {rows})) return rc;"
        for m, (t, rows) in enumerate(plan.maps))
    outs = "\n".join(
        f"  args.out[{i}] = static_cast<__nv_bfloat16*>(const_cast<void*>(tensors[{t}]));"
        for i, t in enumerate(plan.stored))
    names = ", ".join(f'"{t}"' for t in plan.tensors)
    text = f"""
namespace {{

struct {name}_Args {{
  CUtensorMap maps[{max(1, len(plan.maps))}];
  __nv_bfloat16* out[{len(plan.stored)}];
  long long ext[{n_t}][4];     // (batch, depth, rows, cols) of every tensor, signature order
  int scalar[{n_i}];
  int* status;
}};

__global__ void __launch_bounds__(wir::tp::kThreads) {name}_kernel(const __grid_constant__ {name}_Args args) {{
  __shared__ wir::tp::Control<{plan.barriers}> ctl;
  extern __shared__ uint8_t dyn_smem[];
  wir::tp::Ctx ctx;
  wir::tp::begin(ctx, ctl, dyn_smem, args.status, {plan.tmem_cols}u);
{chr(10).join(decls)}
{body}
  wir::tp::end(ctx);
}}

}}  // namespace

// `tensors`: device pointers of the global inputs, then outputs, in signature order
// ({', '.join(plan.tensors)}); `dims`: four extents per tensor; `scalars`: the int inputs
// ({', '.join(plan.ints) or 'none'}).
extern "C" int {name}_launch(const void* const* tensors, const int64_t* dims, const int64_t* scalars,
                             int device, void* stream_) {{
  using namespace wir::host;
  static const char* const kNames[] = {{{names}}};
  g_last_error[0] = 0;
  DeviceState* dev = nullptr;
  if (int rc = get_device_state(device, &dev)) return rc;
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return fail(WARPIR_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(guard.err));
  {name}_Args args{{}};
  for (int t = 0; t < {n_t}; ++t) {{
    for (int d = 0; d < 4; ++d) {{
      if (dims[4 * t + d] < 0 || dims[4 * t + d] > INT32_MAX / 2)
        return fail(WARPIR_ESHAPE, "{name}: extent %d of %s out of range", d, kNames[t]);
      args.ext[t][d] = dims[4 * t + d];
    }}
    if (dims[4 * t] * dims[4 * t + 1] * dims[4 * t + 2] * dims[4 * t + 3] == 0) return WARPIR_OK;  // nothing to do
    if (int rc = check_device_ptr(tensors[t], kNames[t], device)) return rc;
  }}
  for (int i = 0; i < {len(plan.ints)}; ++i) {{
    if (scalars[i] < 0 || scalars[i] > INT32_MAX / 2) return fail(WARPIR_EINVAL, "{name}: int input %d out of range", i);
    args.scalar[i] = static_cast<int>(scalars[i]);
  }}
{maps}
{outs}
  args.status = dev->status;
  const int64_t gx = {plan.grid[0]}, gy = {plan.grid[1]}, gz = {plan.grid[2]};
  if (gx <= 0 || gy <= 0 || gz <= 0) return WARPIR_OK;
  if (gy > 65535 || gz > 65535) return fail(WARPIR_ESHAPE, "{name}: grid %lld x %lld x %lld", (long long)gx, (long long)gy, (long long)gz);
  if (int rc = opt_in_smem(reinterpret_cast<const void*>(&{name}_kernel), {plan.smem_bytes})) return rc;
  {name}_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(gz)),
                  wir::tp::kThreads, {plan.smem_bytes}, static_cast<cudaStream_t>(stream_)>>>(args);
  WIR_CUDA(cudaGetLastError());
  return WARPIR_OK;
}}
"""
    return plan, text
