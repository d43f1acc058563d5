"""Tensor-core instruction-rate probe: clocks per ``tcgen05.mma`` by shape, operand source and CTA group.

    python -m warpir_b200.probe            # prints a markdown table (needs a B200)

The kernel is ``csrc/probe_mma_rate.cu``; it is a measurement aid, not part of the GEMM / attention path.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List

from . import build

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build.build_probe()))
        _lib.warpir_probe_mma_rate.restype = ctypes.c_int
        _lib.warpir_probe_mma_rate.argtypes = [ctypes.c_int] * 11 + [ctypes.c_void_p, ctypes.c_int,
                                                                     ctypes.POINTER(ctypes.c_double)]
        _lib.warpir_probe_mma_rate_ex.restype = ctypes.c_int
        _lib.warpir_probe_mma_rate_ex.argtypes = [ctypes.c_int] * 12 + [ctypes.c_void_p, ctypes.c_int,
                                                                        ctypes.POINTER(ctypes.c_double)]
        _lib.warpir_probe_mma_pattern.restype = ctypes.c_int
        _lib.warpir_probe_mma_pattern.argtypes = [ctypes.POINTER(ctypes.c_int)] + [ctypes.c_int] * 7 + [ctypes.POINTER(ctypes.c_double)]
        _lib.warpir_probe_issue_loop.restype = ctypes.c_int
        _lib.warpir_probe_issue_loop.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_double)]
        _lib.warpir_probe_last_error.restype = ctypes.c_char_p
    return _lib


def mma_rate(n: int, ts: bool, pair: bool, batches: int = 512, bg_tmem: bool = False, bg_tma: bool = False,
             b_mn: bool = False, single: bool = False, random_data: bool = True, bg_alu: bool = False,
             commit_every: int = 0, issuers: int = 1, device: int = 0) -> Dict[str, float]:
    """Clocks per MMA (median over SMs) for one configuration.  With ``issuers=2`` a second warp issues the same
    stream into a second accumulator; ``clocks_per_mma`` then counts both streams' MMAs."""
    import torch
    lib = load()
    buf = torch.zeros(64 * 128 * 64, dtype=torch.bfloat16, device=f"cuda:{device}") if bg_tma else None
    out = (ctypes.c_double * 2)()
    rc = lib.warpir_probe_mma_rate_ex(n, int(ts), int(pair), batches, int(bg_tmem), int(bg_tma), int(b_mn), int(single),
                                      int(random_data), int(bg_alu), commit_every, issuers,
                                      buf.data_ptr() if buf is not None else None, device, out)
    if rc != 0:
        raise RuntimeError(f"probe failed ({rc}): {lib.warpir_probe_last_error().decode()}")
    mmas = 4 * batches * issuers
    commits = batches // commit_every if commit_every > 0 else 0
    m = 256 if pair else 128
    ideal = m * n * 16 / 4096 / (2 if pair else 1)   # clocks the arithmetic needs (4096 FMA per clock per SM)
    n_local = n // 2 if pair else n
    return {"m": m, "n": n, "form": "TS" if ts else "SS", "cta_group": 2 if pair else 1,
            "bg_tmem": bg_tmem, "bg_tma": bg_tma, "bg_alu": bg_alu, "commit_every": commit_every, "b_major": "N" if b_mn else "K",
            "issue": "one by one" if single else "blocks of four", "data": "random" if random_data else "zeros",
            "issuers": issuers, "commits": commits,
            "issue_clocks_per_mma": out[0] / (4 * batches), "clocks_per_mma": out[1] / mmas, "arithmetic_clocks": ideal,
            "rate_fraction": ideal / (out[1] / mmas),
            "smem_bytes_per_mma_per_sm": (0 if ts else 128 * 32) + n_local * 32}


def sweep(device: int = 0) -> List[Dict[str, float]]:
    rows = []
    for pair in (False, True):
        for ts in (False, True):
            for n in (64, 128, 256):
                for bg_tmem, bg_tma in ((False, False), (True, True)):
                    rows.append(mma_rate(n, ts, pair, bg_tmem=bg_tmem, bg_tma=bg_tma, device=device))
                rows.append(mma_rate(n, ts, pair, b_mn=True, device=device))
                rows.append(mma_rate(n, ts, pair, random_data=False, device=device))
                rows.append(mma_rate(n, ts, pair, bg_alu=True, device=device))
                rows.append(mma_rate(n, ts, pair, bg_alu=True, bg_tmem=True, bg_tma=True, commit_every=2, device=device))
                rows.append(mma_rate(n, ts, pair, commit_every=1, device=device))
                if not pair:
                    rows.append(mma_rate(n, ts, pair, single=True, device=device))
    return rows


def format_table(rows: List[Dict[str, float]]) -> str:
    lines = ["| shape (M x N x K) | form | cta_group | B major | issue | data | background | clocks / MMA | arithmetic | "
             "fraction of rate | issue clocks / MMA | smem B / MMA / SM |", "|---|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in rows:
        bg = "+".join(x for x, on in (("tmem ld/st", r["bg_tmem"]), ("TMA loads", r["bg_tma"]), ("arithmetic", r["bg_alu"]),
                                       (f"commit every {r['commit_every']}", r["commit_every"] > 0)) if on) or "none"
        lines.append(f"| {r['m']} x {r['n']} x 16 | {r['form']} | {r['cta_group']} | {r['b_major']} | {r['issue']} | {r['data']} | {bg} | "
                     f"{r['clocks_per_mma']:.1f} | "
                     f"{r['arithmetic_clocks']:.0f} | {r['rate_fraction']:.2f} | {r['issue_clocks_per_mma']:.1f} | "
                     f"{r['smem_bytes_per_mma_per_sm']} |")
    return "\n".join(lines)


def factor_matrix(device: int = 0) -> str:
    """What slows a stream of MMAs down: every combination of the three kinds of background load and a
    tcgen05.commit after every eight MMAs, for the two narrow widths, shared- and tensor-memory A."""
    import itertools
    lines = ["| form | N | tmem ld/st | TMA loads | arithmetic | commit every 8 MMAs | clocks / MMA |", "|---|---|---|---|---|---|---|"]
    for ts in (False, True):
        for n in (128, 64):
            for tmem, tma, alu, com in itertools.product((False, True), repeat=4):
                r = mma_rate(n, ts, False, bg_tmem=tmem, bg_tma=tma, bg_alu=alu, commit_every=2 if com else 0, device=device)
                yn = lambda b: "yes" if b else "-"
                lines.append(f"| {'TS' if ts else 'SS'} | {n} | {yn(tmem)} | {yn(tma)} | {yn(alu)} | {yn(com)} | {r['clocks_per_mma']:.1f} |")
    return "\n".join(lines)


def commit_study(device: int = 0) -> str:
    """Clocks per MMA against the number of MMAs between commits, on an idle SM and under tensor-memory traffic
    plus arithmetic, with one issuing warp and with two (each its own stream, accumulator and commits)."""
    lines = ["| form | N | background | MMAs per commit | issuing warps | clocks / MMA | lost per commit |",
             "|---|---|---|---|---|---|---|"]
    for ts, n in ((True, 64), (False, 64), (True, 128), (False, 128)):
        for busy in (False, True):
            for issuers in (1, 2):
                base = None
                for every in (0, 1, 2, 4, 8):
                    r = mma_rate(n, ts, False, bg_tmem=busy, bg_alu=busy, commit_every=every, issuers=issuers, device=device)
                    if every == 0:
                        base = r["clocks_per_mma"]
                    lost = (r["clocks_per_mma"] - base) * 4 * every * issuers if every else 0.0
                    lines.append(f"| {'TS' if ts else 'SS'} | {n} | {'tmem ld/st + arithmetic' if busy else 'none'} | "
                                 f"{4 * every if every else '-'} | {issuers} | {r['clocks_per_mma']:.1f} | {lost:.0f} |")
    return "\n".join(lines)


def mma_pattern(blocks, steps: int = 256, ts: bool = True, b_mn: bool = True, busy: bool = False, device: int = 0) -> float:
    """Clocks per step (median over SMs) of a replayed issue order: ``blocks`` is a list of
    (N, accumulator column, first MMA overwrites, commit after) tuples, four MMAs each."""
    lib = load()
    flat = (ctypes.c_int * (4 * len(blocks)))(*[int(v) for b in blocks for v in b])
    out = (ctypes.c_double * 2)()
    rc = lib.warpir_probe_mma_pattern(flat, len(blocks), steps, int(ts), int(b_mn), int(busy), int(busy), device, out)
    if rc != 0:
        raise RuntimeError(f"probe failed ({rc}): {lib.warpir_probe_last_error().decode()}")
    return out[1] / steps


# Issue orders of one 64-key step of the attention backward's dQ kernel (16 narrow MMAs for T0 = Q K^T and
# T1 = dO V^T, 4 wide ones for dQ += dS K), and variations that separate the suspects.
PATTERNS = {
    "dQ step as issued: T0,T1,T0,T1 (4 MMAs each), commit, dQ (4 wide), commit":
        [(64, 0, 1, 0), (64, 128, 1, 0), (64, 0, 0, 0), (64, 128, 0, 1), (128, 320, 0, 1)],
    "same, one commit per step":
        [(64, 0, 1, 0), (64, 128, 1, 0), (64, 0, 0, 0), (64, 128, 0, 1), (128, 320, 0, 0)],
    "same, no commits":
        [(64, 0, 1, 0), (64, 128, 1, 0), (64, 0, 0, 0), (64, 128, 0, 0), (128, 320, 0, 0)],
    "T0 x8 then T1 x8 (two accumulator changes fewer), commits as issued":
        [(64, 0, 1, 0), (64, 0, 0, 0), (64, 128, 1, 0), (64, 128, 0, 1), (128, 320, 0, 1)],
    "all narrow MMAs into one accumulator, accumulating, commits as issued":
        [(64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 1), (128, 320, 0, 1)],
    "all narrow MMAs into one accumulator, accumulating, no commits":
        [(64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 0), (128, 320, 0, 0)],
    "narrow MMAs only, two accumulators alternating, no commits":
        [(64, 0, 0, 0), (64, 128, 0, 0), (64, 0, 0, 0), (64, 128, 0, 0)],
    "narrow MMAs only, one accumulator, no commits":
        [(64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 0), (64, 0, 0, 0)],
    "narrow MMAs only, one accumulator, first of every four overwrites, no commits":
        [(64, 0, 1, 0), (64, 0, 1, 0), (64, 0, 1, 0), (64, 0, 1, 0)],
    "wide MMAs only, one accumulator, no commits":
        [(128, 320, 0, 0), (128, 320, 0, 0)],
    "wide MMAs only, two accumulators alternating, no commits":
        [(128, 0, 0, 0), (128, 128, 0, 0)],
    "narrow and wide alternating into the same columns, no commits":
        [(64, 0, 0, 0), (128, 0, 0, 0), (64, 0, 0, 0), (128, 0, 0, 0)],
}


LOOP_SHAPES = {
    1: "as the kernels wrote it: loop ends early when a bounded wait fails",
    2: "fixed trip count, a failed wait switches the rest off",
    3: "no waits, no fences",
    4: "waits that cannot fail, fixed trip count",
    5: "as 1, ring slot in a counter instead of step % 6",
    6: "as 3, all of a step's operand addresses computed before its blocks",
    7: "as 1 without the tcgen05 fences after the waits",
    8: "as 3 plus the two fences per step",
    9: "as 1, every lane waits for itself, no vote",
    10: "as 1, ring-slot barrier tested before stage 2 is issued",
    11: "as 1, stage 1 in two blocks of eight MMAs",
    12: "10 and 11 together",
    13: "as 1, one elected lane issues the whole step from inside one branch",
}


def issue_loop(shape: int, steps: int = 256, busy: int = 0, device: int = 0):
    """(clocks until the last MMA was issued, clocks until all completed) per step for one loop shape.
    ``busy``: 0 idle SM, 1 tensor-memory traffic and arithmetic on every scheduler, 2 on every scheduler but the
    issuing warp's, 3 eight warps polling a barrier that never completes."""
    lib = load()
    out = (ctypes.c_double * 2)()
    rc = lib.warpir_probe_issue_loop(shape, steps, 0 if busy == 3 else int(busy), int(busy), device, out)
    if rc != 0:
        raise RuntimeError(f"probe failed ({rc}): {lib.warpir_probe_last_error().decode()}")
    return out[0] / steps, out[1] / steps


def loop_shape_study(device: int = 0) -> str:
    lines = ["| loop shape | background | clocks per step (768 of arithmetic) | issue clocks per step |", "|---|---|---|---|"]
    for shape, name in LOOP_SHAPES.items():
        for busy in (0, 1, 2, 3):
            i, c = issue_loop(shape, busy=busy, device=device)
            bg = ("none", "tmem ld/st + arithmetic", "tmem ld/st + arithmetic, not on the issuing warp's scheduler",
                  "eight warps polling a barrier")[busy]
            lines.append(f"| {shape}: {name} | {bg} | {c:.0f} | {i:.0f} |")
    return "\n".join(lines)


def pattern_study(device: int = 0) -> str:
    lines = ["| issue order | A from | background | MMAs per step | arithmetic clocks | clocks per step |", "|---|---|---|---|---|---|"]
    for name, blocks in PATTERNS.items():
        arith = sum(4 * (32 if n == 64 else 64) for n, _, _, _ in blocks)
        for ts in (True, False):
            for busy in (False, True):
                c = mma_pattern(blocks, ts=ts, busy=busy, device=device)
                lines.append(f"| {name} | {'tensor memory' if ts else 'shared memory'} | {'tmem ld/st + arithmetic' if busy else 'none'} | "
                             f"{4 * len(blocks)} | {arith} | {c:.0f} |")
    return "\n".join(lines)


if __name__ == "__main__":
    import sys
    if "--commits" in sys.argv:
        print(commit_study())
    elif "--loops" in sys.argv:
        print(loop_shape_study())
    elif "--patterns" in sys.argv:
        print(pattern_study())
    else:
        print(factor_matrix() if "--matrix" in sys.argv else format_table(sweep()))
