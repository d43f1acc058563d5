"""The kernels' failure path, exercised on a healthy GPU without faulting or hanging anything:
a self-test kernel waits (bounded, 2 ms) on a barrier nothing arrives on; the wait runs out, the
status words are written as a GEMM / attention kernel would write them, the kernel exits normally,
`warpir_read_status` reports it once, and the device keeps working."""
import ctypes

import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_the_device_stays_usable(lib):
    stream = torch.cuda.current_stream().cuda_stream
    runtime.read_status()                                   # clean slate
    assert lib.warpir_selftest_bounded_wait(0, stream, 2_000_000) == 0
    code, detail = ctypes.c_int(0), ctypes.c_int(0)
    rc = lib.warpir_read_status(0, stream, ctypes.byref(code), ctypes.byref(detail))
    assert rc == -6 and code.value == 1                     # WARPIR_EKERNEL, "a bounded wait ran out"
    assert detail.value >> 16 == 5 and detail.value & 0xffff == 77    # role and tag of the self-test
    assert b"kernel status 1" in lib.warpir_last_error()
    # reported once, then cleared
    assert lib.warpir_read_status(0, stream, ctypes.byref(code), ctypes.byref(detail)) == 0 and code.value == 0
    # the Python wrapper raises on it
    assert lib.warpir_selftest_bounded_wait(0, stream, 1_000_000) == 0
    with pytest.raises(runtime.WarpirError) as ei:
        runtime.read_status()
    assert ei.value.code == -6
    # and the next ordinary launch is unaffected
    A, B = R.gemm_inputs(128, 128, 256, seed=1)
    C = torch.empty(128, 128, dtype=torch.bfloat16, device="cuda")
    runtime.launch_gemm(A.cuda(), B.cuda(), C, 1)
    runtime.read_status()
    e = R.gemm_errors(C.cpu(), R.gemm_ref(A, B, 1))
    assert e["normalised"] <= R.GEMM_REL_TOL


def test_selftest_argument_check(lib):
    assert lib.warpir_selftest_bounded_wait(0, None, 0) == -1
    assert lib.warpir_selftest_bounded_wait(0, None, 5_000_000_000) == -1
