"""The C-ABI library: loads, exports every symbol the header declares, and rejects
bad arguments before launching anything (CPU only: no compute call is made)."""
import ctypes
import re
from pathlib import Path

from warpir_b200 import runtime

HEADER = Path(__file__).resolve().parent.parent / "include" / "warpir_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(warpir_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    syms = declared_symbols()
    assert set(syms) == set(runtime.EXPORTS)
    for s in syms:
        assert hasattr(lib, s), s


def test_abi_version_and_strerror(lib):
    assert lib.warpir_abi_version() == runtime.ABI_VERSION == 1
    assert lib.warpir_strerror(0) == b"ok"
    seen = {lib.warpir_strerror(-c) for c in range(1, 9)}
    assert len(seen) == 8 and b"unknown error code" not in seen
    assert lib.warpir_strerror(-99) == b"unknown error code"


def test_argument_validation_happens_before_any_cuda_call(lib):
    # these return before the device is touched, so they work without a GPU
    assert lib.warpir_gemm_bf16(None, None, None, -1, 8, 8, 0, 0, None) == -1
    assert b"negative" in lib.warpir_last_error()
    assert lib.warpir_gemm_bf16(None, None, None, 8, 8, 8, 2, 0, None) == -1
    assert lib.warpir_gemm_bf16_ex(None, None, None, 8, 8, 8, 0, 96, 1, 0, None) == -1
    assert lib.warpir_gemm_bf16_ex(None, None, None, 8, 8, 8, 0, 64, 65, 0, None) == -1
    assert lib.warpir_gemm_bf16(None, None, None, 0, 8, 8, 0, 0, None) == 0      # empty: no-op
    assert lib.warpir_attn_fwd_bf16(None, None, None, None, None, 1, 1, 1, 128, 96, 0.1, 0, 0, None) == -3
    assert b"64 or 128" in lib.warpir_last_error()
    assert lib.warpir_attn_fwd_bf16(None, None, None, None, None, 1, 3, 2, 128, 64, 0.1, 0, 0, None) == -3
    assert lib.warpir_attn_fwd_bf16(None, None, None, None, None, 1, 1, 1, 128, 64, -1.0, 0, 0, None) == -1
    assert lib.warpir_attn_fwd_bf16(None, None, None, None, None, 0, 1, 1, 128, 64, 0.1, 0, 0, None) == 0


def test_runtime_wrappers_refuse_cpu_tensors():
    import pytest
    import torch
    a = torch.zeros(8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        runtime.launch_gemm(a, a, a)
    with pytest.raises(ValueError, match="CUDA"):
        runtime.launch_attention(a, a, a, a)


def test_header_and_library_from_plain_c(tmp_path):
    """`include/warpir_b200.h` compiles as C, the library links from a C program, and argument
    checks answer without a GPU (`tests/host/cabi_c_check.c`)."""
    import subprocess
    from pathlib import Path
    from warpir_b200 import build as wb
    root = Path(__file__).resolve().parent.parent
    lib = wb.build_library()
    exe = tmp_path / "cabi_c_check"
    cmd = ["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(root / "include"), str(root / "tests" / "host" / "cabi_c_check.c"),
           "-o", str(exe), "-L", str(lib.parent), "-lwarpir_b200", f"-Wl,-rpath,{lib.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), run.stdout + run.stderr
