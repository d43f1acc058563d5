"""Type vocabulary of the tile IR.

The constructors, field names, defaults, equality/hash behaviour and the
``str()`` spellings mirror the reference's ``warpir/ir/types.py:8-87`` so that
tile programs written against the reference build unchanged and print the same
text.  Every type is an immutable value object: two types with equal fields
are equal and hash alike, which the passes rely on when they key dictionaries
by ``Value``.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Union


class GPUType(str, enum.Enum):
    """Element type of a tile (reference: warpir/ir/types.py:8-10)."""

    bf16 = "bf16"
    fp32 = "fp32"

    @property
    def nbytes(self) -> int:
        return 2 if self is GPUType.bf16 else 4


class TileLayout(str, enum.Enum):
    """Major-ness of a tile (reference: warpir/ir/types.py:13-15)."""

    row_major = "row_major"
    col_major = "col_major"


def _tile_text(kind: str, t) -> str:
    return f"{kind}<{t.data_type.value}, {t.rows}x{t.cols}, {t.layout.value}>"


@dataclass(frozen=True)
class SharedTileType:
    """A tile resident in shared memory (reference: types.py:18-26)."""

    data_type: GPUType
    rows: int
    cols: int
    layout: TileLayout = TileLayout.row_major

    def __str__(self) -> str:
        return _tile_text("shared_tile", self)

    @property
    def nbytes(self) -> int:
        return self.rows * self.cols * self.data_type.nbytes


@dataclass(frozen=True)
class RegTileType:
    """A per-warp register tile (reference: types.py:29-37).

    ``rows`` follows the reference's convention of *rows held by one warp* of
    a four-warp group: a 16-row register tile describes a 64-row CTA tile.
    On sm_100a the fp32 accumulators it names live in tensor memory.
    """

    data_type: GPUType
    rows: int
    cols: int
    layout: TileLayout = TileLayout.row_major

    def __str__(self) -> str:
        return _tile_text("reg_tile", self)


@dataclass(frozen=True)
class GlobalType:
    """A 4-D global tensor ``[batch, depth, rows, cols]`` addressed in units of
    ``sub_tile_type`` tiles; ``-1`` marks a run-time extent (types.py:40-50).
    The printed form leaves the sub-tile out, as the reference's does."""

    data_type: GPUType
    sub_tile_type: SharedTileType
    batch: int = -1
    depth: int = -1
    rows: int = -1
    cols: int = -1

    def __str__(self) -> str:
        dims = ", ".join(str(d) for d in (self.batch, self.depth, self.rows, self.cols))
        return f"global<{self.data_type.value}, {dims}>"


@dataclass(frozen=True)
class SharedBufferType:
    """A ring of ``count`` shared tiles; a mutable buffer, not an SSA value
    (types.py:53-60)."""

    tile_type: SharedTileType
    count: int

    def __str__(self) -> str:
        return f"shared_buffer<{self.tile_type}, count={self.count}>"


@dataclass(frozen=True)
class ColVecType:
    """One fp32/bf16 scalar per row of a ``rows x cols`` register tile
    (types.py:63-71)."""

    data_type: GPUType
    rows: int
    cols: int

    def __str__(self) -> str:
        return f"col_vec<{self.data_type.value}, {self.rows}x{self.cols}>"


@dataclass(frozen=True)
class ScalarType:
    """A named scalar type (types.py:74-79)."""

    name: str

    def __str__(self) -> str:
        return self.name


class IntType(ScalarType):
    """The ``int`` scalar; built without arguments (types.py:82-84)."""

    def __init__(self) -> None:
        ScalarType.__init__(self, "int")


TypeRef = Union[GlobalType, IntType, SharedTileType, RegTileType, SharedBufferType, ColVecType]
