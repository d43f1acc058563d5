"""GEMM parity on a B200: the CUDA path through the C ABI vs the CPU oracle.

Tolerance (stated by the workload definition): max relative error <= 1e-2, in
both forms computed by ``oracle.reference_ops.gemm_errors``.
"""
import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def run_gemm(A, B, b_layout, block_n=0, splits=0):
    M = A.shape[0]
    N = B.shape[0] if b_layout == 1 else B.shape[1]
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    runtime.launch_gemm(A.cuda(), B.cuda(), C, b_layout, block_n, splits)
    runtime.read_status()
    return C.cpu()


def check(C, ref):
    assert not torch.isnan(C.float()).any()
    e = R.gemm_errors(C, ref)
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


def test_reference_golden_vector(golden_dir, lib):
    z = np.load(golden_dir / "gemm_small.npz")
    A = torch.from_numpy(z["A"].view(np.int16).copy()).view(torch.bfloat16)
    B = torch.from_numpy(z["B"].view(np.int16).copy()).view(torch.bfloat16)
    check(run_gemm(A, B, 0), torch.from_numpy(z["ref"]))


# the sizes the reference's own drivers sweep (tests/test_gemm_baseline.py:97,
# tests/test_modal_gpu.py:184), in the reference's layout (B stored [K,N])
@pytest.mark.parametrize("n", [64, 128, 256, 512, 1024])
def test_reference_sweep_square_row_major_b(n, lib):
    A, B = R.gemm_inputs(n, n, n, seed=n, b_layout=0)
    check(run_gemm(A, B, 0), R.gemm_ref(A, B, 0))


@pytest.mark.parametrize("block_n", [0, 64, 128, 256])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_config1_1024_cubed_every_tile_width(block_n, b_layout, lib):
    A, B = R.gemm_inputs(1024, 1024, 1024, seed=0, b_layout=b_layout)
    check(run_gemm(A, B, b_layout, block_n), R.gemm_ref(A, B, b_layout))


@pytest.mark.parametrize("shape", [(1, 8, 8), (16, 64, 64), (128, 64, 16), (200, 136, 72), (129, 264, 520),
                                   (384, 40, 1000), (5, 1000, 24)])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_ragged_shapes(shape, b_layout, lib):
    M, N, K = shape
    A, B = R.gemm_inputs(M, N, K, seed=7, b_layout=b_layout)
    check(run_gemm(A, B, b_layout), R.gemm_ref(A, B, b_layout))


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_split_k_is_exact_and_deterministic(splits, lib):
    A, B = R.gemm_inputs(256, 512, 2048, seed=11)
    ref = R.gemm_ref(A, B)
    C1 = run_gemm(A, B, 1, 64, splits)
    C2 = run_gemm(A, B, 1, 64, splits)
    check(C1, ref)
    assert torch.equal(C1.view(torch.int16), C2.view(torch.int16))


@pytest.mark.parametrize("m", [16, 64, 128])
def test_config3_skinny(m, lib):
    A, B = R.gemm_inputs(m, 8192, 8192, seed=m, std=0.02)
    check(run_gemm(A, B, 1), R.gemm_ref(A, B))


@pytest.mark.parametrize("shape", [(1, 4096, 8192), (16, 4096, 520), (17, 4100, 1024), (48, 5000, 4096),
                                   (64, 8192, 2048), (16, 8192, 16384)])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_few_rows_stream_k(shape, b_layout, lib):
    """Few rows, many columns: k-blocks (not tiles) are dealt out to the SMs, tiles shared between
    CTAs are finished by whoever arrives last.  Exact against the oracle, bit-identical from run to
    run (the partial sums are added in a fixed order), and repeatable (the arrival counters are
    back at zero after every launch)."""
    M, N, K = shape
    if b_layout == 0 and N % 8 != 0:
        N = (N + 7) // 8 * 8
    A, B = R.gemm_inputs(M, N, K, seed=M + K, std=0.05, b_layout=b_layout)
    ref = R.gemm_ref(A, B, b_layout)
    runs = [run_gemm(A, B, b_layout) for _ in range(3)]
    check(runs[0], ref)
    for other in runs[1:]:
        assert torch.equal(runs[0].view(torch.int16), other.view(torch.int16))
    # the statically tiled path (explicit tile width) must agree to rounding
    check(run_gemm(A, B, b_layout, 64, 1), ref)


def test_k_split_paths_on_two_streams_at_once(lib):
    """The K-splitting paths keep fp32 partial sums and arrival counters in library scratch; every
    CUDA stream has its own, so launches that overlap on different streams do not disturb each other."""
    shapes = [(16, 8192, 4096), (8, 4096, 8192)]
    streams = [torch.cuda.Stream() for _ in shapes]
    data = []
    for (M, N, K), st in zip(shapes, streams):
        A, B = R.gemm_inputs(M, N, K, seed=M, std=0.05)
        with torch.cuda.stream(st):
            Ad, Bd = A.cuda(), B.cuda()
            C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        data.append((A, B, Ad, Bd, C))
    torch.cuda.synchronize()
    for _ in range(20):                      # interleaved launches, both streams busy
        for (A, B, Ad, Bd, C), st in zip(data, streams):
            with torch.cuda.stream(st):
                runtime.launch_gemm(Ad, Bd, C, 1)             # stream-K
                runtime.launch_gemm(Ad, Bd, C, 1, 64, 4)      # split-K with the reduce pass
                runtime.launch_gemm(Ad, Bd, C, 1)
    torch.cuda.synchronize()
    runtime.read_status()
    for A, B, Ad, Bd, C in data:
        check(C.cpu(), R.gemm_ref(A, B))


@pytest.mark.parametrize("shape", [(2048, 4096, 2048), (2000, 4104, 2056), (4096, 2048, 4096), (520, 8192, 2048)])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_large_tiles_on_cta_pairs(shape, b_layout, lib):
    """Shapes for which the library picks the 256 x 256 tile, computed by a pair of CTAs (cta_group::2
    MMAs, each CTA holding half of the tile's rows of A and of B), in both storage layouts of B and with
    ragged edges in every dimension; sampled row blocks against the oracle plus linearity over the whole
    output."""
    M, N, K = shape
    A, B = R.gemm_inputs(M, N, K, seed=M + N, b_layout=b_layout)
    C = run_gemm(A, B, b_layout)
    C2 = run_gemm((A.float() * 2).bfloat16(), B, b_layout)
    assert torch.equal((C.float() * 2).bfloat16(), C2)
    rows = torch.cat([torch.arange(s, min(s + 40, M)) for s in (0, 100, 236, M // 2 - 20, M - 40)])
    ref = R.gemm_ref(A[rows], B, b_layout)
    e = R.gemm_errors(C[rows], ref)
    assert not torch.isnan(C.float()).any()
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


def test_config2_2048_against_oracle(lib):
    A, B = R.gemm_inputs(2048, 2048, 2048, seed=1)
    check(run_gemm(A, B, 1), R.gemm_ref(A, B))


def test_empty_and_zero_k(lib):
    A = torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(0, 32, dtype=torch.bfloat16, device="cuda")
    runtime.launch_gemm(A, B, C, 1)          # M = 0: no-op
    A = torch.zeros(16, 0, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(32, 0, dtype=torch.bfloat16, device="cuda")
    C = torch.full((16, 32), 3.0, dtype=torch.bfloat16, device="cuda")
    runtime.launch_gemm(A, B, C, 1)          # K = 0: C = 0
    runtime.read_status()
    assert (C == 0).all()


def test_rejections(lib):
    A = torch.zeros(16, 12, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(32, 12, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(16, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(runtime.WarpirError) as ei:
        runtime.launch_gemm(A, B, C, 1)      # K % 8 != 0
    assert ei.value.code == -3
    host = torch.zeros(16, 16, dtype=torch.bfloat16).pin_memory()
    dev = torch.zeros(16, 16, dtype=torch.bfloat16, device="cuda")
    rc = lib.warpir_gemm_bf16(host.data_ptr(), dev.data_ptr(), dev.data_ptr(), 16, 16, 16, 1, 0, None)
    assert rc == -7                           # A is not device memory
    rc = lib.warpir_gemm_bf16(dev.data_ptr() + 2, dev.data_ptr(), dev.data_ptr(), 8, 8, 8, 1, 0, None)
    assert rc == -2                           # misaligned


def test_full_size_properties_8192(lib):
    """At the benchmark's full size the oracle is checked on sampled rows, and the
    whole product through linearity: (2A) B == 2 (A B) exactly in bf16."""
    g = torch.Generator(device="cuda").manual_seed(0)
    N = 8192
    A = torch.randn(N, N, generator=g, device="cuda").bfloat16()
    B = torch.randn(N, N, generator=g, device="cuda").bfloat16()
    C = torch.empty(N, N, dtype=torch.bfloat16, device="cuda")
    C2 = torch.empty_like(C)
    runtime.launch_gemm(A, B, C, 1)
    runtime.launch_gemm(A * 2, B, C2, 1)
    runtime.read_status()
    assert torch.equal((C.float() * 2).bfloat16(), C2)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191])
    ref = R.gemm_ref(A[rows.cuda()].cpu(), B.cpu(), 1)
    check(C[rows.cuda()].cpu(), ref)
