"""The GEMM kernel's work decomposition (static tiles x K-splits, and stream-K runs) checked on
the host: `tests/host/work_check.cu` compiles the kernel header's own `work_begin` / `work_next`
for the CPU and verifies coverage and segment numbering for a sweep of shapes."""
import itertools
import subprocess
from pathlib import Path

import pytest

from warpir_b200 import build as wb

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = tmp_path_factory.mktemp("work_check") / "work_check"
    cmd = [wb.find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1",
           "-o", str(exe), str(ROOT / "tests" / "host" / "work_check.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    return exe


def run(checker, cases):
    text = "".join(" ".join(map(str, c)) + "\n" for c in cases)
    out = subprocess.run([str(checker)], input=text, capture_output=True, text=True, check=True).stdout.split("\n")
    return [(c, o) for c, o in zip(cases, out) if o != "ok"]


def test_static_tiles_and_k_splits(checker):
    cases = []
    for tm, tn, kb, splits, grid in itertools.product((1, 3, 17, 40), (1, 5, 32), (1, 7, 128), (1, 2, 3, 8), (1, 7, 148)):
        if splits <= kb:
            cases.append((tm, tn, kb, splits, grid, 0))
    assert run(checker, cases) == []


def test_stream_k_runs(checker):
    cases = []
    for tn, kb, grid in itertools.product((1, 2, 32, 64, 65, 148, 300), (1, 4, 56, 128, 129, 256), (1, 2, 37, 147, 148)):
        units = tn * kb
        per = -(-units // grid)
        if per >= 1:
            cases.append((1, tn, kb, 1, -(-units // per), per))
    # several row blocks too (the band rasterisation), and unit counts that leave the last CTA short
    for tm, tn, kb, per in itertools.product((2, 17, 33), (3, 16), (5, 64), (1, 3, 50, 1000)):
        units = tm * tn * kb
        cases.append((tm, tn, kb, 1, -(-units // per), per))
    assert run(checker, cases) == []
