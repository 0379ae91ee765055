"""(batch, head) sharding across the GPUs of one node.

Every (batch, head) pair of the attention path is independent and the ACSR metadata is shared,
so multi-GPU execution is a partition of the flat batch*head axis into contiguous chunks, one per
rank, with no collective on the data path.  (The reference is single-device; its kernels index the
flat batch*head axis as a grid dimension: SPLAT/r_sddmm.py:23-26, SPLAT/r_spmm.py:27-30.)
"""
from __future__ import annotations


def shard_range(total: int, world_size: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the flat batch*head indices owned by ``rank``.  Chunks are contiguous, differ
    in size by at most one, and cover [0, total) exactly once."""
    if world_size < 1 or not 0 <= rank < world_size or total < 0:
        raise ValueError("bad sharding arguments")
    base, extra = divmod(total, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_heads(batch: int, heads: int, world_size: int, rank: int):
    """Flat (batch*head) range of ``rank`` plus the shape (1, n_local, ...) helpers need."""
    begin, end = shard_range(batch * heads, world_size, rank)
    return begin, end, end - begin
