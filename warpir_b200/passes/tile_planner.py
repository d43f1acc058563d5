"""Tile planning for a GEMM of known extents on sm_100a: tile shape, CTA group and K decomposition.

The reference fixes the tile in the program text (64 x 64 x 64, tests/gemm_baseline_v2.py:31-60) and
leaves "which tile" to whoever writes the program.  On a B200 the right tile depends on the problem:
the widest MMA keeps the tensor core busiest per byte of shared-memory traffic, but the tile count has
to fill 148 SMs, a 256-row tile only pays when the k-loop is long, and problems with a handful of rows
are bound by streaming B from HBM, not by the tensor core.  ``plan_gemm`` makes that choice from a
small cost model, ``retile`` rewrites a GEMM tile program to the planned tile, and the lowering pins
the emitted kernel to it (``Sm100Lowerer(problem=(M, N, K))``), so the decision is visible in the
printed IR (tile types, ring depth after ``kernel_pass``) and in the emitted translation unit instead
of being taken inside the launcher.  The C launcher (``csrc/launch.cuh: choose_gemm``) applies the same
rules for callers of the plain C ABI, which have no tile program; ``tests/test_passes.py`` checks the
two against each other through ``warpir_plan_gemm``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..ir.ops import Kernel

SM_COUNT = 148
# relative tensor-core efficiency of a 128-row MMA by tile width: a 128 x N x 16 MMA from shared memory
# reads (128 + N) * 32 bytes at 128 bytes per clock, so N = 64 takes 48 clocks for 32 clocks of arithmetic,
# N = 128 and 256 run at the arithmetic rate but narrower tiles pay more per-stage barrier and commit cost
WIDTH_EFFICIENCY = {256: 1.0, 128: 0.65, 64: 0.40}


@dataclass(frozen=True)
class GemmTilePlan:
    block_m: int          # rows of the CTA tile (128 or 256)
    block_n: int          # columns of the tile = MMA N (64, 128 or 256)
    block_k: int          # K extent of a pipeline stage
    cta_group: int        # 2: the 256-row tile is computed by a CTA pair with 256-row MMAs
    stream_k: bool        # k-blocks, not tiles, dealt out to the SMs (few rows, many columns)
    a_rows: int           # rows of A loaded per stage (fewer than 128 for problems with few rows)
    tiles: int
    waves: float          # tiles / (SMs or SM pairs)

    def describe(self) -> str:
        how = "CTA pair, cta_group::2" if self.cta_group == 2 else "one CTA"
        tail = ", stream-K" if self.stream_k else ""
        return f"{self.block_m}x{self.block_n}x{self.block_k} tiles ({how}{tail}), {self.tiles} tiles = {self.waves:.2f} waves"


def _fill(tiles: int, slots: int) -> float:
    waves = -(-tiles // slots)
    return tiles / (waves * slots)


def plan_gemm(M: int, N: int, K: int, sms: int = SM_COUNT) -> GemmTilePlan:
    """Tile plan for ``C[M,N] = A[M,K] B`` on ``sms`` SMs."""
    tm = -(-M // 128)
    best, block_n = -1.0, 256
    for bn in (256, 128, 64):
        score = WIDTH_EFFICIENCY[bn] * _fill(tm * -(-N // bn), sms)
        if score > best + 1e-9:
            best, block_n = score, bn
    block_m, cta_group = 128, 1
    # 256-row tiles (two 128-row halves sharing B) when the k-loop is long enough to amortise the tile
    # switch and the tile count still fills the SMs as well; they run on CTA pairs
    if block_n == 256 and M >= 512 and K >= 2048:
        tn = -(-N // 256)
        if _fill(-(-M // 256) * tn, sms) >= 0.97 * _fill(tm * tn, sms):
            block_m, cta_group = 256, 2
    stream_k, a_rows = False, 128
    if M <= 64 and N >= 64 * 64:
        # few rows: HBM-bound on B; only the existing rows of A are loaded
        block_n, block_m, cta_group = 64, 128, 1
        a_rows = 16 if M <= 16 else 64
        tiles64 = -(-N // 64)
        if N % 4 == 0 and (M <= 32 or _fill(tiles64, sms) < 0.7):
            tiles = -(-N // 128)
            if tiles <= 8192 and tiles * -(-K // 64) >= 4 * sms:
                block_n, stream_k = 128, True
    tiles = -(-M // block_m) * -(-N // block_n)
    slots = sms // 2 if cta_group == 2 else sms
    return GemmTilePlan(block_m, block_n, 64, cta_group, stream_k, a_rows, tiles, tiles / slots)


def retile(kernel: Kernel, plan: GemmTilePlan) -> Kernel:
    """The GEMM tile program ``kernel`` rebuilt with the planned tile shape (same name, operands,
    B layout and grid mapping).  Anything that is not a plain GEMM program is rejected by the
    lowering's analysis, which this uses to read the program."""
    from ..lowering.lowering import GemmPlan, analyze
    from ..programs import build_gemm_kernel
    p = analyze(kernel)
    if not isinstance(p, GemmPlan):
        raise NotImplementedError(f"{kernel.name}: only GEMM tile programs can be re-tiled")
    out = build_gemm_kernel(plan.block_m, plan.block_n, plan.block_k, b_k_major=not p.b_row_major)
    if (out.name, [v.name for v in out.inputs], [v.name for v in out.outputs]) != \
            (kernel.name, [v.name for v in kernel.inputs], [v.name for v in kernel.outputs]):
        raise NotImplementedError(f"{kernel.name}: operands differ from the canonical GEMM program")
    return out
