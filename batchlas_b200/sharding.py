"""Contiguous batch sharding across the GPUs of one box.

Batch items are independent, so GPU g of G owns the contiguous item range
[floor(g*B/G), floor((g+1)*B/G)) of A, B and C (pointer offset b0*stride, same ld/stride) and no
collective is needed on the data path.  The reference has no multi-GPU code; it addresses one GPU
per Queue (BatchLAS include/util/sycl-device-queue.hh:75), which is what one rank here does.
"""
from __future__ import annotations


def shard_range(batch: int, rank: int, world: int) -> tuple[int, int]:
    """First item and item count of `rank`'s shard."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank/world out of range")
    if batch < 0:
        raise ValueError("negative batch")
    b0 = (batch * rank) // world
    b1 = (batch * (rank + 1)) // world
    return b0, b1 - b0
