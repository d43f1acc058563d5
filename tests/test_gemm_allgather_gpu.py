"""GEMM with the all-gather of its output fused into the epilogue.

On one GPU the destinations are several buffers of that GPU (the store loop itself); with two or
more GPUs in the box, one process per GPU is spawned, every rank computes its row block and
writes it into every rank's copy of the output over peer mappings, and every copy must equal the
CPU oracle."""
import ctypes
import os
import socket
import sys

import pytest
import torch

from oracle import reference_ops as R
from warpir_b200 import runtime

pytestmark = pytest.mark.gpu


def check(C, ref):
    e = R.gemm_errors(C, ref)
    assert e["normalised"] <= R.GEMM_REL_TOL and e["elementwise"] <= R.GEMM_REL_TOL, e


@pytest.mark.parametrize("shape", [(256, 512, 320), (129, 264, 520), (16, 4096, 512), (1024, 1024, 1024)])
@pytest.mark.parametrize("n_dst", [1, 3])
def test_several_destinations_on_one_gpu(shape, n_dst, lib):
    M, N, K = shape
    A, B = R.gemm_inputs(M, N, K, seed=M + n_dst)
    outs = [torch.full((M + 8, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(n_dst)]
    # each destination is row 5 of a taller buffer: the address arithmetic a gathered output needs
    ptrs = [o.data_ptr() + 5 * N * 2 for o in outs]
    runtime.launch_gemm_allgather(A.cuda(), B.cuda(), ptrs, N, 1)
    runtime.read_status()
    ref = R.gemm_ref(A, B, 1)
    for o in outs:
        check(o[5:5 + M].cpu(), ref)
        assert torch.isnan(o[:5].float()).all() and torch.isnan(o[5 + M:].float()).all()   # nothing outside the block
    for o in outs[1:]:
        assert torch.equal(o[5:5 + M].view(torch.int16), outs[0][5:5 + M].view(torch.int16))


def test_allgather_rejections(lib):
    A = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(runtime.WarpirError):
        runtime.launch_gemm_allgather(A, A, [], 64, 1)
    with pytest.raises(runtime.WarpirError):
        runtime.launch_gemm_allgather(A, A, [C.data_ptr() + 2], 64, 1)          # misaligned
    with pytest.raises(runtime.WarpirError):
        runtime.launch_gemm_allgather(A, A, [C.data_ptr()] * 9, 64, 1)          # too many
    host = torch.zeros(64, 64, dtype=torch.bfloat16)
    with pytest.raises(runtime.WarpirError):
        runtime.launch_gemm_allgather(A, A, [host.data_ptr()], 64, 1)           # not device memory


def _rank_main(rank, world, port, m_per_rank, N, K, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    from warpir_b200 import sharding
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        A, B = R.gemm_inputs(world * m_per_rank, N, K, seed=7)
        out = sharding.GatheredOutput(world * m_per_rank, N)
        out.tensor.fill_(float("nan"))
        out.wait_all()
        r0 = rank * m_per_rank
        sharding.gemm_allgather(A[r0:r0 + m_per_rank].cuda(), B.cuda(), out, r0)
        out.wait_all()
        runtime.read_status()
        torch.save(out.tensor.cpu(), os.path.join(result_dir, f"c{rank}.pt"))
        out.wait_all()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one box")
def test_every_rank_ends_up_with_the_whole_output(lib, tmp_path):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    m_per_rank, N, K = 384, 1024, 512
    mp.spawn(_rank_main, args=(world, port, m_per_rank, N, K, str(tmp_path)), nprocs=world, join=True)
    A, B = R.gemm_inputs(world * m_per_rank, N, K, seed=7)
    ref = R.gemm_ref(A, B, 1)
    copies = [torch.load(tmp_path / f"c{r}.pt") for r in range(world)]
    for c in copies:
        check(c, ref)
        assert torch.equal(c.view(torch.int16), copies[0].view(torch.int16))
