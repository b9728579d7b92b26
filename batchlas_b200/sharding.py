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


def shard_desc(desc, rank: int, world: int, elem_bytes: int):
    """Copy of a descriptor (GemmDesc, EwiseDesc or GemvDesc) restricted to `rank`'s contiguous batch
    range: every base pointer advances by b0*stride elements of its own operand, ld/inc/stride are
    unchanged, batch becomes the shard's item count."""
    import ctypes
    b0, nb = shard_range(desc.batch, rank, world)
    sub = type(desc)()
    ctypes.memmove(ctypes.byref(sub), ctypes.byref(desc), ctypes.sizeof(desc))
    names = {f[0] for f in desc._fields_}
    for ptr in ("a", "b", "c", "x", "y"):
        if ptr in names:
            setattr(sub, ptr, (getattr(desc, ptr) or 0) + b0 * getattr(desc, "stride_" + ptr) * elem_bytes)
    sub.batch = nb
    return sub


def max_over_ranks(value: float, device=None) -> float:
    """Slowest rank's value (the time that bounds a sharded step); identity without a process group."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
