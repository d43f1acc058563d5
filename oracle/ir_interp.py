"""CPU interpreter of the tile IR.  TEST INFRASTRUCTURE: the product never imports it.

Executes a ``Kernel`` block index by block index on torch CPU tensors, one op at a
time, with the semantics the reference documents for each op
(warpir/ir/ops.py:57-230) and implements in its lowering
(warpir/lowering/lowering.py:427-570):

* ``tma_load`` copies the sub-tile at ``(batch, depth, row, col)`` (in units of the
  destination tile) into a shared tile; elements past the tensor read as zero;
* ``mma`` is ``a @ b + accum`` in fp32 on bf16 operands; with ``transpose_b`` it is
  ``a @ b^T`` without ``accum`` (the reference emits ``mm_ABt``, lowering.py:462);
* ``mma_buf`` accumulates in place into ``accum`` (lowering.py:474-480);
* ``copy`` rounds to bf16 when the result type is bf16;
* ``row_max``/``row_sum`` fold ``prev`` in; ``sub_row``/``mul_row``/``div_row`` broadcast
  a per-row scalar;
* ``tma_store`` rounds to bf16 and drops what falls outside the tensor;
* a loop's ``iter_args`` start from their ``init`` and take the yielded values after each
  trip; with ``tile_size`` the trip count is ``ceil(stop / tile_size)``;
* ``drain(+k, %S)`` is slot ``(consumed + k) % S`` with ``consumed`` the number of
  ``mma_buf`` executed inside loops.

The reference has no interpreter; this one is pinned by running the reference's own two
tile programs through it and comparing with the reference's torch oracles
(tests/test_gemm_baseline.py:85, tests/test_modal_attention.py:92-98) in
tests/test_ir_interp.py.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch


def _as4d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape((1,) * (4 - t.dim()) + tuple(t.shape))


def _tname(x) -> str:
    return type(x).__name__


class _Block:
    def __init__(self, kernel, tensors: Dict[str, torch.Tensor], ints: Dict[str, int], block: Tuple[int, int, int]):
        self.kernel = kernel
        self.tensors = tensors
        self.env: Dict[str, object] = {}
        self.rings: Dict[str, list] = {}
        self.ints = dict(ints)
        self.ints.update({"blockIdx.x": block[0], "blockIdx.y": block[1], "blockIdx.z": block[2]})
        self.consumed = 0
        self.loop_depth = 0

    # -- helpers
    def int_of(self, x) -> int:
        return x if isinstance(x, int) else int(self.ints[x.name])

    def slot_of(self, slot) -> int:
        if isinstance(slot, int):
            return slot
        base = self.consumed if slot.value is None else self.int_of(slot.value)
        return (base + slot.offset) % slot.modulus

    def rows_of(self, v) -> int:
        return 4 * v.type.rows

    def load(self, source, coords, rows: int, cols: int) -> torch.Tensor:
        src = _as4d(self.tensors[source.name])
        b, d, r, c = (self.int_of(x) for x in coords)
        out = torch.zeros(rows, cols, dtype=torch.float32)
        if b < src.shape[0] and d < src.shape[1]:
            r0, c0 = r * rows, c * cols
            part = src[b, d, r0:r0 + rows, c0:c0 + cols].float()
            out[:part.shape[0], :part.shape[1]] = part
        return out

    def store(self, value: torch.Tensor, dest, coords, unit_rows: int, unit_cols: int):
        dst = _as4d(self.tensors[dest.name])
        b, d, r, c = (self.int_of(x) for x in coords)
        r0, c0 = r * unit_rows, c * unit_cols
        nr = max(0, min(value.shape[0], dst.shape[2] - r0))
        nc = max(0, min(value.shape[1], dst.shape[3] - c0))
        if nr and nc:
            dst[b, d, r0:r0 + nr, c0:c0 + nc] = value[:nr, :nc].to(dst.dtype)

    def mma(self, a: torch.Tensor, b: torch.Tensor, accum: Optional[torch.Tensor], transpose_b: bool) -> torch.Tensor:
        a = a.to(torch.bfloat16).float()          # operands are bf16 by type; idempotent on loaded tiles
        b = b.to(torch.bfloat16).float()
        if transpose_b:
            return a @ b.t()
        return a @ b + accum

    # -- execution
    def run(self, ops: Sequence[object]):
        for op in ops:
            self.step(op)

    def step(self, op):
        E, kind = self.env, _tname(op)
        if kind == "ForOp":
            return self.loop(op)
        if kind in ("AllocSharedOp",):
            t = op.result.type
            self.rings[op.result.name] = [torch.zeros(t.tile_type.rows, t.tile_type.cols) for _ in range(t.count)]
            return
        if kind in ("WaitOp", "WaitBufOp", "YieldOp"):
            return
        if kind in ("ZeroOp", "NegInftyOp"):
            fill = 0.0 if kind == "ZeroOp" else float("-inf")
            t = op.result.type
            shape = (self.rows_of(op.result), t.cols) if _tname(t) == "RegTileType" else (self.rows_of(op.result),)
            E[op.result.name] = torch.full(shape, fill, dtype=torch.float32)
            return
        if kind == "TMALoadOp":
            t = op.result.type
            E[op.result.name] = self.load(op.source, op.coords, t.rows, t.cols)
            return
        if kind == "TMALoadBufOp":
            t = op.buf.type.tile_type
            self.rings[op.buf.name][self.slot_of(op.slot)] = self.load(op.source, op.coords, t.rows, t.cols)
            return
        if kind == "MMAOp":
            E[op.result.name] = self.mma(E[op.a.name], E[op.b.name], E.get(op.accum.name), op.transpose_b)
            return
        if kind == "MMABufOp":
            a = self.rings[op.a_buf.name][self.slot_of(op.a_slot)]
            b = self.rings[op.b_buf.name][self.slot_of(op.b_slot)]
            k, n = a.shape[1], op.result.type.cols
            if k != n:
                transposed = tuple(b.shape) == (n, k)
            else:                      # square tile: the loads that fill the ring tell its layout
                transposed = self.b_k_major(op.b_buf)
            out = E[op.accum.name] + self.mma(a, b, None, True) if transposed else self.mma(a, b, E[op.accum.name], False)
            E[op.accum.name] = out
            E[op.result.name] = out
            if self.loop_depth > 0:
                self.consumed += 1
            return
        if kind == "TMAStoreOp":
            sub = getattr(op.dest.type, "sub_tile_type", None)
            val = E[op.source.name]
            ur, uc = (sub.rows, sub.cols) if sub is not None else val.shape
            return self.store(val, op.dest, op.coords, ur, uc)
        if kind == "CopyOp":
            x = E[op.input.name]
            narrow = op.result.type.data_type.value == "bf16" and op.input.type.data_type.value != "bf16"
            E[op.result.name] = x.to(torch.bfloat16).float() if narrow else x.clone()
            return
        if kind == "MulScalarOp":
            E[op.result.name] = E[op.input.name] * torch.tensor(op.scalar, dtype=torch.float32)
            return
        if kind == "Exp2Op":
            E[op.result.name] = torch.exp2(E[op.input.name])
            return
        if kind == "SubOp":
            E[op.result.name] = E[op.a.name] - E[op.b.name]
            return
        if kind == "MulOp":
            E[op.result.name] = E[op.a.name] * E[op.b.name]
            return
        if kind == "RowMaxOp":
            E[op.result.name] = torch.maximum(E[op.tile.name].max(dim=1).values, E[op.prev.name])
            return
        if kind == "RowSumOp":
            E[op.result.name] = E[op.tile.name].sum(dim=1) + E[op.prev.name]
            return
        if kind == "SubRowOp":
            E[op.result.name] = E[op.tile.name] - E[op.vec.name][:, None]
            return
        if kind == "MulRowOp":
            E[op.result.name] = E[op.tile.name] * E[op.vec.name][:, None]
            return
        if kind == "DivRowOp":
            E[op.result.name] = E[op.tile.name] / E[op.vec.name][:, None]
            return
        raise NotImplementedError(f"no interpretation for {kind}")

    def b_k_major(self, ring) -> bool:
        """A square B ring is [N, K] when the loads that fill it advance the loop counter along
        its columns (coordinate 3), [K, N] when along its rows."""
        def walk(ops):
            for op in ops:
                if _tname(op) == "ForOp":
                    r = walk(op.body)
                    if r is not None:
                        return r
                elif _tname(op) == "TMALoadBufOp" and op.buf == ring:
                    for pos in (3, 2):
                        c = op.coords[pos]
                        if not isinstance(c, int) and c.name in self.loop_vars:
                            return pos == 3
            return None
        r = walk(self.kernel.body)
        return bool(r)

    @property
    def loop_vars(self):
        names = set()
        def walk(ops):
            for op in ops:
                if _tname(op) == "ForOp":
                    names.add(op.induction_var.name)
                    walk(op.body)
        walk(self.kernel.body)
        return names

    def loop(self, op):
        E = self.env
        for ia in op.iter_args:
            E[ia.block_arg.name] = E[ia.init.name]
        start, stop, step = self.int_of(op.start), self.int_of(op.stop), self.int_of(op.step)
        if op.tile_size is not None:
            stop = (stop + op.tile_size - 1) // op.tile_size
        self.loop_depth += 1
        i = start
        while i < stop:
            self.ints[op.induction_var.name] = i
            self.run(op.body)
            yields = [o for o in op.body if _tname(o) == "YieldOp"]
            if op.iter_args:
                vals = [E[v.name] for v in yields[0].values]
                for ia, v in zip(op.iter_args, vals):
                    E[ia.block_arg.name] = v
            i += step
        self.loop_depth -= 1
        for r, ia in zip(op.results, op.iter_args):
            E[r.name] = E[ia.block_arg.name]


def grid_of(kernel, tensors: Dict[str, torch.Tensor]) -> Tuple[int, int, int]:
    """One block per tile of what the stores (else the loads) address with ``blockIdx``."""
    grid = {"x": None, "y": None, "z": None}

    def scan(coords, tensor, unit):
        shape = _as4d(tensors[tensor.name]).shape
        for pos, c in enumerate(coords):
            if not isinstance(c, int) and c.name.startswith("blockIdx.") and grid[c.name[-1]] is None:
                grid[c.name[-1]] = -(-shape[pos] // unit[pos])

    def walk(ops, stores: bool):
        for op in ops:
            kind = _tname(op)
            if kind == "ForOp":
                walk(op.body, stores)
            elif stores and kind == "TMAStoreOp":
                sub = op.dest.type.sub_tile_type
                scan(op.coords, op.dest, (1, 1, sub.rows, sub.cols))
            elif not stores and kind == "TMALoadOp":
                scan(op.coords, op.source, (1, 1, op.result.type.rows, op.result.type.cols))
            elif not stores and kind == "TMALoadBufOp":
                t = op.buf.type.tile_type
                scan(op.coords, op.source, (1, 1, t.rows, t.cols))

    walk(kernel.body, True)
    walk(kernel.body, False)
    return tuple(grid[a] or 1 for a in "xyz")


def run_kernel(kernel, tensors: Dict[str, torch.Tensor], ints: Optional[Dict[str, int]] = None,
               grid: Optional[Tuple[int, int, int]] = None) -> None:
    """Execute ``kernel`` on CPU tensors (bf16, up to four dimensions, keyed by value name);
    output tensors are written in place."""
    ints = ints or {}
    gx, gy, gz = grid or grid_of(kernel, tensors)
    for bz in range(gz):
        for by in range(gy):
            for bx in range(gx):
                _Block(kernel, tensors, ints, (bx, by, bz)).run(kernel.body)
