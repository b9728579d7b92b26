"""The multi-GPU path's host logic on CPU: two gloo ranks shard a batch by contiguous ranges
(no data-path collective), each runs its shard, and the union equals the unsharded result.  The
per-shard compute is the CPU oracle here (test infrastructure); on GPUs each rank launches the
same sub-descriptor through the C ABI."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from batchlas_b200 import _lib
from batchlas_b200.sharding import max_over_ranks, shard_desc, shard_range
from oracle import oracle
from tests._cases import make_inputs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        p = oracle.make_problem("d", "T", "N", 12, 10, 8, 7, ldc=15, alpha=2.0, beta=0.5)
        A, B, C = make_inputs(p)
        d = _lib.GemmDesc()
        d.a, d.b, d.c = A.ctypes.data, B.ctypes.data, C.ctypes.data
        d.batch, d.stride_a, d.stride_b, d.stride_c = p.batch, p.stride_a, p.stride_b, p.stride_c
        sub = shard_desc(d, rank, world, 8)
        b0, nb = shard_range(p.batch, rank, world)
        assert sub.batch == nb and sub.c == C.ctypes.data + b0 * p.stride_c * 8
        # run the shard in place on this rank's copy, through the sub-descriptor's pointers
        ps = oracle.make_problem("d", "T", "N", 12, 10, 8, nb, ldc=15, alpha=2.0, beta=0.5)
        ps.stride_a, ps.stride_b, ps.stride_c = p.stride_a, p.stride_b, p.stride_c
        def view(ptr, base):
            off = (ptr - base.ctypes.data) // 8
            return base[off:]
        assert oracle.gemm_netlib(ps, view(sub.a, A), view(sub.b, B), view(sub.c, C)) == 0
        # gather only the final result (host-visible), rank 0 checks it against the unsharded run
        mine = torch.from_numpy(C[b0 * p.stride_c:(b0 + nb) * p.stride_c].copy())
        sizes = [shard_range(p.batch, r, world)[1] * p.stride_c for r in range(world)]
        parts = [torch.empty(s, dtype=torch.float64) for s in sizes]
        if world > 1:
            # all_gather needs equal sizes: pad to the largest shard
            mx = max(sizes)
            padded = torch.zeros(mx, dtype=torch.float64)
            padded[: mine.numel()] = mine
            bufs = [torch.empty(mx, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(bufs, padded)
            parts = [b[:s] for b, s in zip(bufs, sizes)]
        slowest = max_over_ranks(1.0 + rank)
        assert slowest == float(world)
        if rank == 0:
            A2, B2, C2 = make_inputs(p)
            assert oracle.gemm_netlib(p, A2, B2, C2) == 0
            got = torch.cat(parts).numpy()
            np.save(out_path, np.array([np.array_equal(got, C2[: got.size])]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_contiguous_batch_sharding_over_gloo(world, tmp_path):
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert np.load(out)[0]


def test_c_shard_rule_matches_the_python_one(lib):
    """blb200_shard_range (what the one-call multi-GPU host entry cuts the batch with) against
    sharding.shard_range: contiguous, disjoint, complete, for awkward batch / shard counts."""
    first, count = ctypes.c_int64(0), ctypes.c_int64(0)
    for batch in (0, 1, 7, 64, 1000, 10_000, 1_000_000, 2**31 - 1):
        for world in (1, 2, 3, 4, 8, 13):
            covered = 0
            for g in range(world):
                lib.blb200_shard_range(batch, g, world, ctypes.byref(first), ctypes.byref(count))
                assert (first.value, count.value) == shard_range(batch, g, world)
                assert first.value == covered
                covered += count.value
            assert covered == batch
    lib.blb200_shard_range(10, 5, 4, ctypes.byref(first), ctypes.byref(count))  # shard out of range: empty
    assert (first.value, count.value) == (0, 0)


def test_multi_gpu_host_entry_rejects_bad_device_lists(lib):
    d = _lib.GemmDesc()
    d.m = d.n = d.k = 4
    d.batch = 2
    d.lda = d.ldb = d.ldc = 4
    d.stride_a = d.stride_b = d.stride_c = 16
    buf = np.zeros(64)
    d.a = d.b = d.c = buf.ctypes.data
    two_same = (ctypes.c_int32 * 2)(0, 0)
    assert lib.blb200_gemm_strided_batched_host_multi(d, None, 1, 0) == _lib.E_NULL
    assert lib.blb200_gemm_strided_batched_host_multi(d, two_same, 0, 0) == _lib.E_NULL
    assert lib.blb200_gemm_strided_batched_host_multi(d, two_same, 2, 0) == _lib.E_UNSUPPORTED
    d.stride_c = 3  # overlapping C items
    assert lib.blb200_gemm_strided_batched_host_multi(d, two_same, 1, 0) == _lib.E_SHAPE
