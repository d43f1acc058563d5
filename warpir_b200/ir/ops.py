"""Operations of the tile IR.

The public surface (class names, constructor fields and their order, defaults,
frozen value semantics, ``Op.substitute``) mirrors the reference's
``warpir/ir/ops.py:9-285`` so tile programs written for the reference build
unchanged.  Unlike the reference, which spells every op out as its own class
body and teaches the printer about each one in a long ``elif`` chain, the ops
here are generated from one table (``_OP_TABLE``).  Each row carries, next to
the fields, the op's text mnemonic and the role each field plays (result,
operand, coordinate list, buffer slot ...), and the printer and the sm_100a
lowerer both walk that metadata instead of switching on the class.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple, Union

from .types import TypeRef


@dataclass(frozen=True)
class Value:
    """An SSA value: a unique name and a type (reference: ops.py:9-16).
    ``repr`` gives the ``%name: type`` spelling the printer uses."""

    name: str
    type: TypeRef

    def __repr__(self) -> str:
        return f"%{self.name}: {self.type}"


@dataclass(frozen=True)
class BufSlotExpr:
    """Slot index ``(value + offset) % modulus`` into a shared-memory ring.
    ``value is None`` names the drain-phase counter that the backend keeps
    after the steady-state loop has ended (reference: ops.py:19-28)."""

    value: Optional[Value]
    offset: int = 0
    modulus: int = 1


BufIdx = Union[int, BufSlotExpr]


class Op:
    """Base of every operation (reference: ops.py:34-50)."""

    #: text mnemonic, filled in per class from the op table
    mnemonic: str = ""
    #: role of each field, in field order: see ``_OP_TABLE``
    roles: Tuple[Tuple[str, str], ...] = ()

    def __repr__(self) -> str:  # dataclass subclasses generate an equal form
        inner = ", ".join(f"{k}={v}" for k, v in vars(self).items())
        return f"{type(self).__name__}({inner})"

    def substitute(self, replacements: Dict[Value, Union[Value, int]]) -> "Op":
        """A copy of the op with every ``Value`` that is a key of
        ``replacements`` swapped for its image; looks inside tuples and slot
        expressions, leaves everything else alone."""

        def swap(x):
            if isinstance(x, Value):
                return replacements.get(x, x)
            if isinstance(x, tuple):
                return tuple(swap(e) for e in x)
            if isinstance(x, BufSlotExpr):
                inner = None if x.value is None else swap(x.value)
                return BufSlotExpr(value=inner, offset=x.offset, modulus=x.modulus)
            return x

        return type(self)(**{k: swap(v) for k, v in vars(self).items()})


# Field roles understood by the printer and the lowerer:
#   result  - SSA value defined by the op
#   use     - SSA value read by the op
#   uses    - tuple of SSA values read by the op
#   coords  - tuple of tile coordinates (Value or int)
#   buf     - shared ring buffer (printed by bare name)
#   bufs    - tuple of ring buffers
#   slot    - BufIdx
#   attr    - compile-time attribute (float, bool)
_R, _U, _US, _C, _B, _BS, _S, _A = (
    "result", "use", "uses", "coords", "buf", "bufs", "slot", "attr")

_Coords = Tuple[Union[Value, int], ...]

# name, mnemonic, doc, ((field, type, role[, default]), ...)
_OP_TABLE = (
    # ---- SSA tile ops (pre-pipelining form), reference ops.py:57-96
    ("ZeroOp", "zero", "Zero-fill a register tile or column vector.",
     (("result", Value, _R),)),
    ("TMALoadOp", "tma_load",
     "Asynchronous bulk-tensor load of one global sub-tile into shared memory.",
     (("result", Value, _R), ("source", Value, _U), ("coords", _Coords, _C))),
    ("WaitOp", "wait", "Block until the named loads have landed.",
     (("values", Tuple[Value, ...], _US),)),
    ("MMAOp", "mma",
     "Tile matrix multiply-accumulate: ``a @ b + accum``; with "
     "``transpose_b`` the product is ``a @ b^T`` (the reference's form ignores "
     "``accum`` there; it only ever passes a zero tile).",
     (("result", Value, _R), ("a", Value, _U), ("b", Value, _U),
      ("accum", Value, _U), ("transpose_b", bool, _A, False))),
    ("TMAStoreOp", "tma_store", "Store a tile to global memory.",
     (("source", Value, _U), ("dest", Value, _U), ("coords", _Coords, _C))),
    # ---- elementwise / row reductions, reference ops.py:103-190
    ("NegInftyOp", "neg_infty", "Fill with -inf.", (("result", Value, _R),)),
    ("CopyOp", "copy", "Copy, converting the element type if the types differ.",
     (("result", Value, _R), ("input", Value, _U))),
    ("MulScalarOp", "mul_scalar", "``input * scalar`` with a compile-time scalar.",
     (("result", Value, _R), ("input", Value, _U), ("scalar", float, _A))),
    ("SubOp", "sub", "Elementwise ``a - b``.",
     (("result", Value, _R), ("a", Value, _U), ("b", Value, _U))),
    ("MulOp", "mul", "Elementwise ``a * b``.",
     (("result", Value, _R), ("a", Value, _U), ("b", Value, _U))),
    ("Exp2Op", "exp2", "Elementwise ``2 ** input``.",
     (("result", Value, _R), ("input", Value, _U))),
    ("RowMaxOp", "row_max", "``max(rowmax(tile), prev)`` per row.",
     (("result", Value, _R), ("tile", Value, _U), ("prev", Value, _U))),
    ("RowSumOp", "row_sum", "``rowsum(tile) + prev`` per row.",
     (("result", Value, _R), ("tile", Value, _U), ("prev", Value, _U))),
    ("SubRowOp", "sub_row", "``tile[r, c] - vec[r]``.",
     (("result", Value, _R), ("tile", Value, _U), ("vec", Value, _U))),
    ("MulRowOp", "mul_row", "``tile[r, c] * vec[r]``.",
     (("result", Value, _R), ("tile", Value, _U), ("vec", Value, _U))),
    ("DivRowOp", "div_row", "``tile[r, c] / vec[r]``.",
     (("result", Value, _R), ("tile", Value, _U), ("vec", Value, _U))),
    # ---- ring-buffer ops (post-pipelining form), reference ops.py:197-230
    ("AllocSharedOp", "alloc_shared", "Reserve a ring of shared tiles.",
     (("result", Value, _R),)),
    ("TMALoadBufOp", "tma_load_buf", "Load a sub-tile into one slot of a ring.",
     (("buf", Value, _B), ("slot", BufIdx, _S), ("source", Value, _U),
      ("coords", _Coords, _C))),
    ("WaitBufOp", "wait_buf", "Wait until one slot of the named rings is full.",
     (("bufs", Tuple[Value, ...], _BS), ("slot", BufIdx, _S))),
    ("MMABufOp", "mma_buf", "MMA whose operands are ring slots.",
     (("result", Value, _R), ("a_buf", Value, _B), ("a_slot", BufIdx, _S),
      ("b_buf", Value, _B), ("b_slot", BufIdx, _S), ("accum", Value, _U))),
    # ---- control flow, reference ops.py:237-245
    ("YieldOp", "yield", "End of a loop body; hands values to the next trip.",
     (("values", Tuple[Value, ...], _US),)),
)


def _make_op(name, mnemonic, doc, rows):
    fields = []
    for row in rows:
        fname, ftype = row[0], row[1]
        if len(row) == 4:
            fields.append((fname, ftype, field(default=row[3])))
        else:
            fields.append((fname, ftype))
    cls = dataclasses.make_dataclass(name, fields, bases=(Op,), frozen=True)
    cls.__doc__ = doc
    cls.__module__ = __name__
    cls.mnemonic = mnemonic
    cls.roles = tuple((row[0], row[2]) for row in rows)
    return cls


for _row in _OP_TABLE:
    globals()[_row[0]] = _make_op(*_row)
del _row

# Names for static readers; the objects are the generated classes above.
ZeroOp = globals()["ZeroOp"]
TMALoadOp = globals()["TMALoadOp"]
WaitOp = globals()["WaitOp"]
MMAOp = globals()["MMAOp"]
TMAStoreOp = globals()["TMAStoreOp"]
NegInftyOp = globals()["NegInftyOp"]
CopyOp = globals()["CopyOp"]
MulScalarOp = globals()["MulScalarOp"]
SubOp = globals()["SubOp"]
MulOp = globals()["MulOp"]
Exp2Op = globals()["Exp2Op"]
RowMaxOp = globals()["RowMaxOp"]
RowSumOp = globals()["RowSumOp"]
SubRowOp = globals()["SubRowOp"]
MulRowOp = globals()["MulRowOp"]
DivRowOp = globals()["DivRowOp"]
AllocSharedOp = globals()["AllocSharedOp"]
TMALoadBufOp = globals()["TMALoadBufOp"]
WaitBufOp = globals()["WaitBufOp"]
MMABufOp = globals()["MMABufOp"]
YieldOp = globals()["YieldOp"]


@dataclass(frozen=True)
class IterArg:
    """A loop-carried value: ``block_arg`` is ``init`` on the first trip and
    the matching yielded value afterwards (reference: ops.py:248-256)."""

    block_arg: Value
    init: Value


@dataclass(frozen=True)
class ForOp(Op):
    """Counted loop with loop-carried values, in the style of ``scf.for``
    (reference: ops.py:259-273).  ``results[i]`` is the last value yielded for
    ``iter_args[i]``.  With ``tile_size`` set, ``stop`` is an element extent
    and the trip count is ``ceil(stop / tile_size)``."""

    induction_var: Value
    start: Union[Value, int]
    stop: Union[Value, int]
    step: Union[Value, int]
    iter_args: Tuple[IterArg, ...]
    body: Tuple[Op, ...]
    results: Tuple[Value, ...]
    tile_size: Optional[int] = None

    mnemonic = "for"


@dataclass(frozen=True)
class Kernel:
    """A named tile program (reference: ops.py:280-285)."""

    name: str
    inputs: Tuple[Value, ...] = field(default_factory=tuple)
    outputs: Tuple[Value, ...] = field(default_factory=tuple)
    body: Tuple[Op, ...] = field(default_factory=tuple)
