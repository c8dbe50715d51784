"""Partitioning of the hot path across the GPUs of one box.

Both paths shard into independent units, so there is no collective on the data
path: attention by (batch x head) slices -- the reference's work item is
(m_block, batch*head) with no coupling between heads
(test/gpu/blackwell/flash_attention_defs.jl:269-272) -- and the GEMM by contiguous
blocks of output columns with A replicated; the row-wise kernels by blocks of rows.
Collectives (torch.distributed: NCCL
on GPUs, gloo in the CPU tests) are used only to agree on timings and to gather
results for verification.
"""
from __future__ import annotations

from typing import List, Tuple


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [begin, end) of `total` units for `rank`; the first
    `total % world` ranks take one extra unit."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def attention_shard(B: int, H: int, rank: int, world: int) -> Tuple[int, int]:
    """(first, last+1) flattened batch*head index owned by `rank`."""
    return shard_range(B * H, rank, world)


def gemm_column_shard(N: int, rank: int, world: int, granule: int = 128) -> Tuple[int, int]:
    """Contiguous column block of C / row block of B^T owned by `rank`, in
    multiples of `granule` columns (the kernel's N granularity)."""
    if N % granule != 0:
        raise ValueError("N must be a multiple of the column granule")
    b, e = shard_range(N // granule, rank, world)
    return b * granule, e * granule


def row_shard(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block of rows of a row-wise op (softmax, norms, SwiGLU) owned by
    `rank`: rows are independent, so the shards need no exchange either."""
    return shard_range(rows, rank, world)


def all_shards(total: int, world: int) -> List[Tuple[int, int]]:
    return [shard_range(total, r, world) for r in range(world)]


def gather_checksums(local_sum: float, local_abs_sum: float, dist) -> Tuple[float, float]:
    """Sum two scalars over all ranks (verification only, outside any timed region)."""
    import torch
    t = torch.tensor([local_sum, local_abs_sum], dtype=torch.float64)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t)
    return float(t[0]), float(t[1])
