"""Multi-GPU host logic on CPU: partition arithmetic and a world_size-2 gloo run in which
each rank computes its shard (the oracle stands in for the kernel) and the optional
all-gather reassembles the full result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reference_ops as R
from warpir_b200 import sharding as S


def test_split_range_covers_everything_once():
    for total in (0, 1, 127, 128, 1000, 8192):
        for world in (1, 2, 3, 8):
            for mult in (1, 64, 128):
                spans = [S.split_range(total, world, r, mult) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == total
                assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
                sizes = [e - b for b, e in spans]
                assert max(sizes) - min(sizes) < 2 * mult
    with pytest.raises(ValueError):
        S.split_range(10, 2, 2)


def test_gemm_and_attention_shards():
    assert S.gemm_shard(8192, 8192, 8, 3) == {"axis": "rows", "rows": (3072, 4096), "cols": (0, 8192)}
    assert S.gemm_shard(16, 8192, 8, 7) == {"axis": "cols", "rows": (0, 16), "cols": (7168, 8192)}
    assert S.attention_shard(4, 32, 8, 1) == (16, 32)
    assert [S.attention_shard(1, 6, 2, r, Hkv=2) for r in range(2)] == [(0, 3), (3, 6)]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 384, 256, 192
        A, B = R.gemm_inputs(M, N, K, seed=0)
        sh = S.gemm_shard(M, N, world, rank)
        r0, r1 = sh["rows"]
        C_shard = R.gemm_ref(A[r0:r1], B, 1).bfloat16()          # kernel stand-in on CPU
        sizes = [e - b for b, e in (S.gemm_shard(M, N, world, r)["rows"] for r in range(world))]
        C = S.all_gather_outputs(C_shard, sizes, dim=0)
        ok_gemm = torch.equal(C, R.gemm_ref(A, B, 1).bfloat16())

        Q, Kt, V = R.attention_inputs(1, 6, 128, 64, seed=1)
        b, e = S.attention_shard(1, 6, world, rank)
        O, _ = R.attention_ref(Q, Kt, V, slices=range(b, e))
        O_shard = O.view(6, 128, 64)[b:e].bfloat16()
        O_all = S.all_gather_outputs(O_shard, [3, 3], dim=0)
        O_ref, _ = R.attention_ref(Q, Kt, V)
        ok_attn = torch.equal(O_all, O_ref.view(6, 128, 64).bfloat16())
        if rank == 0:
            out.put((ok_gemm, ok_attn))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo_shard_and_gather():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) == (True, True)
