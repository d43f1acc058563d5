"""Tile IR: types and operations (API of the reference's ``warpir/ir/__init__.py:1-82``)."""
from . import ops as _ops
from . import types as _types
from .ops import BufIdx, BufSlotExpr, ForOp, IterArg, Kernel, Op, Value
from .types import (ColVecType, GPUType, GlobalType, IntType, RegTileType, ScalarType,
                    SharedBufferType, SharedTileType, TileLayout, TypeRef)

# the table-generated op classes
for _name in [row[0] for row in _ops._OP_TABLE]:
    globals()[_name] = getattr(_ops, _name)
del _name

__all__ = sorted(
    [row[0] for row in _ops._OP_TABLE]
    + ["BufIdx", "BufSlotExpr", "ForOp", "IterArg", "Kernel", "Op", "Value",
       "ColVecType", "GPUType", "GlobalType", "IntType", "RegTileType", "ScalarType",
       "SharedBufferType", "SharedTileType", "TileLayout", "TypeRef"])
