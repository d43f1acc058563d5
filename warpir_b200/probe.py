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
        _lib.warpir_probe_last_error.restype = ctypes.c_char_p
    return _lib


def mma_rate(n: int, ts: bool, pair: bool, batches: int = 512, bg_tmem: bool = False, bg_tma: bool = False,
             b_mn: bool = False, single: bool = False, random_data: bool = True, bg_alu: bool = False,
             commit_every: int = 0, device: int = 0) -> Dict[str, float]:
    """Clocks per MMA (median over SMs) for one configuration."""
    import torch
    lib = load()
    buf = torch.zeros(64 * 128 * 64, dtype=torch.bfloat16, device=f"cuda:{device}") if bg_tma else None
    out = (ctypes.c_double * 2)()
    rc = lib.warpir_probe_mma_rate(n, int(ts), int(pair), batches, int(bg_tmem), int(bg_tma), int(b_mn), int(single), int(random_data), int(bg_alu), commit_every,
                                   buf.data_ptr() if buf is not None else None, device, out)
    if rc != 0:
        raise RuntimeError(f"probe failed ({rc}): {lib.warpir_probe_last_error().decode()}")
    mmas = 4 * batches
    m = 256 if pair else 128
    ideal = m * n * 16 / 4096 / (2 if pair else 1)   # clocks the arithmetic needs (4096 FMA per clock per SM)
    n_local = n // 2 if pair else n
    return {"m": m, "n": n, "form": "TS" if ts else "SS", "cta_group": 2 if pair else 1,
            "bg_tmem": bg_tmem, "bg_tma": bg_tma, "bg_alu": bg_alu, "commit_every": commit_every, "b_major": "N" if b_mn else "K",
            "issue": "one by one" if single else "blocks of four", "data": "random" if random_data else "zeros",
            "issue_clocks_per_mma": out[0] / mmas, "clocks_per_mma": out[1] / mmas, "arithmetic_clocks": ideal,
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


if __name__ == "__main__":
    import sys
    print(factor_matrix() if "--matrix" in sys.argv else format_table(sweep()))
