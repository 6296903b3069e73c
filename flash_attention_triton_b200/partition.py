"""Sharding of the independent (batch, head) problems over the GPUs of one node.

Every (batch, head) pair is a separate attention problem in forward and backward (the
reference indexes everything by ``offset_batch_head``, ``_triton_kernels_v2.py:79-81,448-464``),
so multi-GPU execution is a partition of the flattened ``b*H + h`` range with no data-path
collective.  A contiguous range of that index is a contiguous slab of a ``[B, H, N, D]`` tensor,
viewed on the owning GPU as ``[1, count, N, D]``.
"""

from __future__ import annotations

import torch


def shard_range(num_batch_heads: int, world_size: int, rank: int) -> tuple[int, int]:
    """Half-open range ``[start, stop)`` of flattened (batch, head) indices owned by ``rank``.

    Ranges are contiguous, ordered by rank, differ in size by at most one and cover
    ``[0, num_batch_heads)`` exactly once.
    """
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"invalid rank {rank} for world size {world_size}")
    if num_batch_heads < 0:
        raise ValueError("num_batch_heads must be >= 0")
    base, extra = divmod(num_batch_heads, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_slab(t: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """The slab of a contiguous ``[B, H, N, D]`` tensor owned by ``rank``, as ``[1, count, N, D]``."""
    if t.dim() != 4:
        raise ValueError("expected a [B, H, N, D] tensor")
    b, h, n, d = t.shape
    start, stop = shard_range(b * h, world_size, rank)
    return t.contiguous().view(1, b * h, n, d)[:, start:stop]
