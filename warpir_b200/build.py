"""Builds ``libwarpir_b200.so`` (sm_100a only) in-tree with nvcc.

    python -m warpir_b200.build [--force]

The library lands in ``warpir_b200/lib/``; it is what ``warpir_b200.runtime``
loads through ``ctypes``.  nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libwarpir_b200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-ldl",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")))


def source_digest() -> str:
    h = hashlib.sha256()
    for f in _sources():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def is_current() -> bool:
    stamp = LIB_DIR / "build.stamp"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == source_digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile if the sources changed since the last build; return the library path."""
    if not force and is_current():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(LIB_PATH), str(CSRC / "capi.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (LIB_DIR / "ptxas.log").write_text(proc.stdout + proc.stderr)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    (LIB_DIR / "build.stamp").write_text(source_digest() + "\n")
    return LIB_PATH


def build_variant(tag: str, defines) -> Path:
    """Another build of the library with extra -D flags (``-DWIR_TRACE`` event traces,
    ``-DWIR_ABLATE=n`` measurement builds): ``lib/libwarpir_b200_<tag>.so``.  Load it by pointing
    ``WARPIR_B200_LIBRARY`` at it."""
    LIB_DIR.mkdir(exist_ok=True)
    out = LIB_DIR / f"libwarpir_b200_{tag}.so"
    flags = [f for f in NVCC_FLAGS if f not in ("-Xptxas", "-v")]
    cmd = [find_nvcc(), *flags, *[f"-D{d}" for d in defines], "-I", str(INCLUDE), "-o", str(out), str(CSRC / "capi.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return out


PROBE_PATH = LIB_DIR / "libwarpir_probe.so"


def build_probe(force: bool = False) -> Path:
    """The tensor-core instruction-rate probe (csrc/probe_mma_rate.cu), a library of its own."""
    stamp = LIB_DIR / "probe.stamp"
    if not force and PROBE_PATH.exists() and stamp.exists() and stamp.read_text().strip() == source_digest():
        return PROBE_PATH
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(PROBE_PATH), str(CSRC / "probe_mma_rate.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    stamp.write_text(source_digest() + "\n")
    return PROBE_PATH


if __name__ == "__main__":
    if "--variant" in sys.argv:      # python -m warpir_b200.build --variant trace WIR_TRACE
        i = sys.argv.index("--variant")
        print(build_variant(sys.argv[i + 1], sys.argv[i + 2:]))
    else:
        path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
        print(path)
