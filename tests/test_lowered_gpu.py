"""End to end as the reference's drivers do it: build IR -> (pipeline) -> lower -> compile ->
launch -> compare with torch (reference: tests/test_gemm_baseline.py:52-105,
tests/test_modal_gpu.py:159-201, tests/test_modal_attention.py:158-191), on a B200 and
against the CPU oracle with the workload tolerances instead of the reference's 1.0."""
import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime
from warpir_b200.passes.modulo_scheduler import REFERENCE_MODEL, kernel_pass
from warpir_b200.programs import build_attention_kernel, build_gemm_kernel

pytestmark = pytest.mark.gpu


def _check_gemm(mod, n, b_layout):
    A, B = R.gemm_inputs(n, n, n, seed=n, b_layout=b_layout)
    C = torch.zeros(n, n, device="cuda", dtype=torch.bfloat16)
    mod.launch_gemm(A.cuda(), B.cuda(), C)
    mod.read_status()
    e = R.gemm_errors(C.cpu(), R.gemm_ref(A, B, b_layout))
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, (n, e)


def test_reference_gemm_program_baseline_and_pipelined(lib):
    base = runtime.load(build_gemm_kernel())
    piped = runtime.load(kernel_pass(build_gemm_kernel(), REFERENCE_MODEL))
    for n in (64, 128, 256, 512, 1024):
        _check_gemm(base, n, 0)
        _check_gemm(piped, n, 0)


@pytest.mark.parametrize("bm,bn", [(128, 64), (128, 128), (128, 256), (256, 256)])
def test_hardware_tile_programs(bm, bn, lib):
    mod = runtime.load(kernel_pass(build_gemm_kernel(bm, bn, 64, b_k_major=True)))
    for n in (128, 1024):
        _check_gemm(mod, n, 1)


def test_reference_attention_program(lib):
    mod = runtime.load(build_attention_kernel())
    for n in (64, 128, 256, 512, 1024):
        Q, K, V = R.attention_inputs(1, 1, n, 64, seed=n)
        O = torch.zeros(n, 64, device="cuda", dtype=torch.bfloat16)
        mod.launch_attention(Q[0, 0].cuda(), K[0, 0].cuda(), V[0, 0].cuda(), O)
        mod.read_status()
        O_ref, _ = R.attention_ref(Q, K, V)
        assert (O.cpu().float() - O_ref[0, 0]).abs().max().item() <= R.ATTN_O_ABS_TOL


def test_attention_program_d128_batched_causal_with_lse(lib):
    mod = runtime.load(build_attention_kernel(128, 128, 128))
    Q, K, V = R.attention_inputs(2, 4, 512, 128, seed=3)
    O = torch.zeros_like(Q, device="cuda")
    L = torch.zeros(2, 4, 512, device="cuda")
    mod.launch_attention(Q.cuda(), K.cuda(), V.cuda(), O, causal=True, LSE=L)
    mod.read_status()
    O_ref, L_ref = R.attention_ref(Q, K, V, None, True)
    e = R.attention_errors(O.cpu(), L.cpu(), O_ref, L_ref)
    assert e["o_max_abs"] <= R.ATTN_O_ABS_TOL and e["lse_max_abs"] <= R.ATTN_LSE_ABS_TOL


def test_launch_by_name_through_the_c_abi(lib):
    """`warpir_launch_generated`: the C-ABI way to launch a lowered program from its shared object."""
    import ctypes
    mod = runtime.load(kernel_pass(build_gemm_kernel(), REFERENCE_MODEL))
    n = 256
    A, B = R.gemm_inputs(n, n, n, seed=3, b_layout=0)
    Ad, Bd = A.cuda(), B.cuda()
    C = torch.zeros(n, n, device="cuda", dtype=torch.bfloat16)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    ptrs = (vp * 3)(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr())
    dims = (i64 * 12)(1, 1, n, n, 1, 1, n, n, 1, 1, n, n)
    scalars = (i64 * 1)(n)
    handle = vp(mod._dll._handle)
    stream = vp(torch.cuda.current_stream().cuda_stream)
    rc = lib.warpir_launch_generated(handle, b"gemm", ptrs, dims, 3, scalars, 1, 0, stream)
    assert rc == 0, lib.warpir_last_error()
    runtime.read_status()
    e = R.gemm_errors(C.cpu(), R.gemm_ref(A, B, 0))
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e
    assert lib.warpir_launch_generated(handle, b"no_such_kernel", ptrs, dims, 3, scalars, 1, 0, stream) == -1
    assert b"not found" in lib.warpir_last_error()
