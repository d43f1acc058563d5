"""The allocation-free split-K GEMM entry point, through the C ABI, on a B200.

`warpir_gemm_bf16_splitk_noalloc` exists for hosts that cannot have a library call
cudaMalloc behind their back -- a server that gave the whole GPU to its own memory pool,
or a loop that cannot take the implicit synchronisation of cudaMalloc/cudaFree.  It keeps
the fp32 partial sums of the K-splits in a 16 MiB array that is part of the library image
instead of a buffer grown on demand.  It must produce the very bits the allocating entry
point (`warpir_gemm_bf16_ex`) produces, on two calls in a row (the array keeps the first
call's contents, so the second call -- different data, different shape -- would show a stale
partial sum if one were ever read), and it must refuse problems whose partial sums do not
fit.  Collected last (file name) so that a failure here cannot hide the other tests; passes
alone in a fresh process as well as after them.
"""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from oracle import reference_ops as R

pytestmark = pytest.mark.gpu


def _gemm(lib, fn_name, A, B, M, N, K, block_n, splits):
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = getattr(lib, fn_name)(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, 1, block_n, splits,
                               torch.cuda.current_device(), stream)
    assert rc == 0, lib.warpir_last_error()
    torch.cuda.synchronize()
    return C


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(lib):
    for (M, N, K, block_n, splits, seed) in [(128, 2048, 4096, 64, 4, 21), (96, 1024, 2048, 128, 3, 22)]:
        A, B = R.gemm_inputs(M, N, K, seed=seed, std=0.05)
        A, B = A.cuda(), B.cuda()
        got = _gemm(lib, "warpir_gemm_bf16_splitk_noalloc", A, B, M, N, K, block_n, splits)
        want = _gemm(lib, "warpir_gemm_bf16_ex", A, B, M, N, K, block_n, splits)
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))       # same kernels, same order
        e = R.gemm_errors(got.cpu(), R.gemm_ref(A.cpu(), B.cpu(), 1))
        assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e
    # its own status words (inside the static array) stayed clean, and reading them allocates nothing either
    import ctypes
    code, detail = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.warpir_noalloc_read_status(torch.cuda.current_device(), None, ctypes.byref(code), ctypes.byref(detail)) == 0
    assert code.value == 0


def test_noalloc_with_the_width_left_to_the_library_agrees_to_rounding(lib):
    """block_n = 0 with few rows: the allocating entry point takes its few-rows kernels (part of an A tile
    per stage, or stream-K), this one the plain tiles; same sums in another order, so the two agree to
    rounding and both with the oracle."""
    M, N, K = 48, 4096, 2048
    A, B = R.gemm_inputs(M, N, K, seed=5, std=0.05)
    got = _gemm(lib, "warpir_gemm_bf16_splitk_noalloc", A.cuda(), B.cuda(), M, N, K, 0, 2)
    want = _gemm(lib, "warpir_gemm_bf16_ex", A.cuda(), B.cuda(), M, N, K, 0, 0)
    ref = R.gemm_ref(A, B, 1)
    for C in (got, want):
        e = R.gemm_errors(C.cpu(), ref)
        assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


def test_noalloc_really_allocates_nothing():
    """The one property the entry point exists for, measured: in a fresh process (so that nothing else
    has touched the library), free device memory as the driver reports it (cudaMemGetInfo) does not
    drop across the first GEMM call, the second call, or the status read.  The caller's buffers are
    allocated and the library image is loaded (one status read, which also does the one-off
    symbol-address lookup) before the first reading."""
    root = Path(__file__).resolve().parent.parent
    script = textwrap.dedent("""
        import ctypes, sys
        sys.path.insert(0, %r)
        import torch
        from warpir_b200 import runtime
        lib = runtime.load_library()
        torch.cuda.set_device(0)
        M, N, K = 128, 2048, 4096
        A = torch.randn(M, K, device="cuda").bfloat16(); B = torch.randn(N, K, device="cuda").bfloat16()
        C = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        # the library image (code and the static array) is resident once the module is loaded: make sure
        # it is before the first reading, so that only what the CALLS do is measured
        assert lib.warpir_noalloc_read_status(0, None, None, None) == 0
        torch.cuda.synchronize()
        free = [torch.cuda.mem_get_info()[0]]
        for _ in range(2):
            rc = lib.warpir_gemm_bf16_splitk_noalloc(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, 1, 64, 4, 0, None)
            assert rc == 0, lib.warpir_last_error()
            torch.cuda.synchronize()
            free.append(torch.cuda.mem_get_info()[0])
        code = ctypes.c_int(-1)
        assert lib.warpir_noalloc_read_status(0, None, ctypes.byref(code), None) == 0 and code.value == 0
        free.append(torch.cuda.mem_get_info()[0])
        print("FREE", *free)
        assert min(free[1:]) >= free[0], free
        ref = (A.float() @ B.float().t())
        assert (C.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
        print("OK")
    """ % str(root))
    import os
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")     # no lazily loaded kernel images during the calls
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0 and proc.stdout.strip().endswith("OK"), proc.stdout + proc.stderr


def test_noalloc_rejects_what_does_not_fit_and_bad_arguments(lib):
    A = torch.zeros(2048, 64, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(2048, 64, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(2048, 2048, dtype=torch.bfloat16, device="cuda")
    # 2 * 2048 * 2048 partial sums = 32 MiB > 16 MiB (K = 128 gives two k-blocks, so two splits survive)
    A2 = torch.zeros(2048, 128, dtype=torch.bfloat16, device="cuda")
    B2 = torch.zeros(2048, 128, dtype=torch.bfloat16, device="cuda")
    rc = lib.warpir_gemm_bf16_splitk_noalloc(A2.data_ptr(), B2.data_ptr(), C.data_ptr(), 2048, 2048, 128, 1, 0, 2,
                                             0, None)
    assert rc == -3 and b"static scratch" in lib.warpir_last_error()
    # a single split needs no scratch at all, whatever the size
    rc = lib.warpir_gemm_bf16_splitk_noalloc(A.data_ptr(), B.data_ptr(), C.data_ptr(), 2048, 2048, 64, 1, 0, 1, 0, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.warpir_gemm_bf16_splitk_noalloc(A.data_ptr(), B.data_ptr(), C.data_ptr(), 8, 8, 8, 1, 0, 0, 0, None) == -1
    assert lib.warpir_gemm_bf16_splitk_noalloc(None, B.data_ptr(), C.data_ptr(), 8, 8, 8, 1, 0, 2, 0, None) == -1
