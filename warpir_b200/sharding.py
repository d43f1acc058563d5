"""Multi-GPU partitioning of the hot path: one process per GPU, no data-path collective.

The reference is single-GPU throughout (its drivers rent one H100:
tests/test_modal_gpu.py:155).  Both ops shard without any exchange:

* GEMM: contiguous row blocks of A and C per rank, B replicated (skinny problems,
  M <= 128, shard the columns of B / C instead);
* attention: the flat ``batch x head`` slices, contiguous per rank (with grouped KV
  heads a rank's query heads stay whole KV groups when the counts divide).

The only collective is the optional all-gather of the output shards.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


def split_range(total: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """[begin, end) of rank's contiguous share of ``total`` units; shares are multiples of
    ``multiple`` (except the last, which takes the ragged tail) and differ by less than two multiples; empty shares are
    possible when ``total`` is small."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if total < 0 or multiple < 1:
        raise ValueError("total must be >= 0 and multiple >= 1")
    chunks = -(-total // multiple)
    base, extra = divmod(chunks, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(first * multiple, total), min((first + count) * multiple, total)


def gemm_shard(M: int, N: int, world: int, rank: int) -> dict:
    """Which block of C this rank computes: row blocks (multiples of the 128-row tile) or,
    for skinny M, column blocks (multiples of 64)."""
    if M > 128 or world == 1:
        r0, r1 = split_range(M, world, rank, 128)
        return {"axis": "rows", "rows": (r0, r1), "cols": (0, N)}
    c0, c1 = split_range(N, world, rank, 64)
    return {"axis": "cols", "rows": (0, M), "cols": (c0, c1)}


def attention_shard(B: int, H: int, world: int, rank: int, Hkv: Optional[int] = None) -> Tuple[int, int]:
    """[begin, end) of flat ``b * H + h`` slices for this rank; with grouped KV heads the
    boundaries fall on whole KV groups."""
    group = H // Hkv if Hkv else 1
    return split_range(B * H, world, rank, group)


def all_gather_outputs(shard, sizes: List[int], dim: int = 0, group=None):
    """Optional collective: concatenates every rank's output shard along ``dim``.
    ``sizes[r]`` is rank r's extent along ``dim`` (shards may be ragged)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if len(sizes) != world:
        raise ValueError("one size per rank")
    biggest = max(sizes)
    shape = list(shard.shape)
    shape[dim] = biggest
    padded = shard.new_zeros(shape)
    padded.narrow(dim, 0, shard.shape[dim]).copy_(shard)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p.narrow(dim, 0, n) for p, n in zip(parts, sizes)], dim=dim)


class GatheredOutput:
    """The full output ``C [M_total, N]`` (bf16) of a row-sharded GEMM, one copy per GPU, that
    every rank's GEMM writes into directly: the fused form of ``all_gather_outputs``.

    The copies live in torch symmetric memory, which maps every rank's buffer into every
    other rank's address space; ``runtime.launch_gemm_allgather`` then stores each finished
    tile of this rank's row block to all of them from the GEMM epilogue, the peer stores
    crossing NVLink while the next tiles are computed.  No NVLink multicast object is
    involved (plain peer stores), and multicast binding is switched off for the allocation.
    """

    def __init__(self, m_total: int, n: int, group=None):
        import os
        # plain peer mappings only: on shared hosts a rank that dies while bound to a multicast
        # object can disturb its peers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.m_total, self.n = int(m_total), int(n)
        self.tensor = symm.empty((self.m_total, self.n), dtype=torch.bfloat16,
                                 device=torch.device("cuda", torch.cuda.current_device()))
        handle = symm.rendezvous(self.tensor, self.group)
        self.rank, self.world = handle.rank, handle.world_size
        self.ptrs = [int(p) for p in handle.buffer_ptrs]
        if self.ptrs[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe this tensor")

    def dst_ptrs(self, row_start: int) -> List[int]:
        """Addresses of row ``row_start`` in every rank's copy, this rank's own copy first."""
        if not 0 <= row_start <= self.m_total:
            raise ValueError("row_start outside the output")
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.ptrs[r] + row_start * self.n * 2 for r in order]

    def wait_all(self) -> None:
        """Every rank's stores have landed in every copy once all ranks return from here."""
        import torch
        import torch.distributed as dist
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)


def gemm_allgather(A_block, B, out: GatheredOutput, row_start: int, b_layout: int = 1) -> None:
    """This rank's rows of ``A @ B`` stored straight into every rank's copy of ``out``."""
    from . import runtime
    if row_start + A_block.shape[0] > out.m_total:
        raise ValueError("row block does not fit the gathered output")
    runtime.launch_gemm_allgather(A_block, B, out.dst_ptrs(row_start), out.n, b_layout)
