"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol the header
declares, validates descriptors the way the reference validates views, and the workspace arena
keeps the reference's lease semantics (BatchLAS tests/mempool_tests.cc:829-1078).  No compute call
is made here — those need a GPU."""
import ctypes
import os
import re

import pytest

from batchlas_b200 import _lib, shard_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "blb200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(blb200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 15
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.blb200_version().decode().count(".") == 1


def test_descriptor_layout_matches_header(lib):
    # 3 pointers, 4 int32, 6 int64, 4 doubles, 4 int32
    assert ctypes.sizeof(_lib.GemmDesc) == 3 * 8 + 4 * 4 + 6 * 8 + 4 * 8 + 4 * 4


def _desc(**kw):
    d = _lib.GemmDesc()
    base = dict(a=0x1000, b=0x2000, c=0x3000, m=4, n=4, k=4, batch=1, lda=4, ldb=4, ldc=4, stride_a=16,
                stride_b=16, stride_c=16, dtype=0, op_a=0, op_b=0, kernel_hint=0)
    base.update(kw)
    for k, v in base.items():
        setattr(d, k, v)
    d.alpha[0] = 1.0
    return d


def test_validate_follows_reference_shape_rules(lib):
    v = lib.blb200_gemm_validate
    assert v(_desc()) == 0
    assert v(None) == _lib.E_NULL
    assert v(_desc(m=-1)) == _lib.E_SHAPE
    assert v(_desc(lda=3)) == _lib.E_SHAPE
    assert v(_desc(op_a=1, k=8, lda=4)) == _lib.E_SHAPE      # A stored k x m: lda >= k
    assert v(_desc(op_b=1, n=8, ldb=4, ldc=4)) == _lib.E_SHAPE  # B stored n x k: ldb >= n
    assert v(_desc(ldc=3)) == _lib.E_SHAPE
    assert v(_desc(dtype=4)) == _lib.E_DTYPE
    assert v(_desc(op_a=3)) == _lib.E_DTYPE
    assert v(_desc(c=0)) == _lib.E_NULL
    assert v(_desc(a=0, k=0)) == 0                 # k == 0 never touches A or B
    assert v(_desc(a=0, b=0, c=0, m=0)) == 0       # empty output is a no-op
    assert v(_desc(kernel_hint=99)) == _lib.E_UNSUPPORTED
    assert v(_desc(kernel_hint=_lib.K_SGEMM128)) == 0
    assert lib.blb200_status_string(_lib.E_SHAPE).decode() == "GEMM: incompatible matrix dimensions"


def test_empty_problems_return_ok_without_a_device(lib):
    assert lib.blb200_gemm_strided_batched(_desc(m=0), None) == 0
    assert lib.blb200_gemm_strided_batched(_desc(batch=0), None) == 0
    assert lib.blb200_gemm_strided_batched(_desc(lda=1), None) == _lib.E_SHAPE
    assert lib.blb200_gemm_strided_batched_host(_desc(n=0), 0, 0) == 0


# ---- arena: host-backed instance, same bookkeeping as the device-backed one ----------------------
class Arena:
    def __init__(self, lib):
        self.lib = lib
        h = ctypes.c_void_p()
        assert lib.blb200_arena_create(-1, None, ctypes.byref(h)) == 0
        self.h = h

    def acquire(self, n):
        ls = _lib.Lease()
        assert self.lib.blb200_arena_acquire(self.h, n, ctypes.byref(ls)) == 0
        return ls

    def release(self, ls):
        assert self.lib.blb200_arena_release(self.h, ctypes.byref(ls)) == 0

    def capacity(self):
        return self.lib.blb200_arena_capacity(self.h)

    def blocks(self):
        return self.lib.blb200_arena_block_count(self.h)

    def trim(self):
        return self.lib.blb200_arena_trim(self.h)

    def close(self):
        self.lib.blb200_arena_destroy(self.h)


@pytest.fixture
def arena(lib):
    a = Arena(lib)
    yield a
    a.close()


def test_lease_is_aligned_and_usable(arena):
    ls = arena.acquire(1000)
    al = arena.lib.blb200_arena_alignment(arena.h)
    assert al >= 16 and ls.ptr % al == 0 and ls.bytes == 1000
    ctypes.memset(ls.ptr, 0xAB, 1000)
    arena.release(ls)


def test_released_bytes_are_reused_without_new_allocation(arena):
    a = arena.acquire(4096)
    p, cap = a.ptr, arena.capacity()
    arena.release(a)
    for _ in range(50):
        b = arena.acquire(4096)
        assert b.ptr == p
        arena.release(b)
    assert arena.capacity() == cap and arena.blocks() == 1
    assert cap >= 64 * 1024  # first block is at least 64 KiB


def test_nested_leases_are_disjoint_and_outer_pointer_survives_growth(arena):
    outer = arena.acquire(10_000)
    inner = arena.acquire(1_000_000)  # does not fit: opens a new block, outer must not move
    assert arena.blocks() == 2
    lo, hi = outer.ptr, outer.ptr + outer.bytes
    assert inner.ptr + inner.bytes <= lo or inner.ptr >= hi
    ctypes.memset(outer.ptr, 1, outer.bytes)
    ctypes.memset(inner.ptr, 2, inner.bytes)
    arena.release(inner)
    arena.release(outer)


def test_growth_is_geometric(arena):
    size, held = 1024, []
    for _ in range(40):  # ratcheting request, each larger than the last
        ls = arena.acquire(size)
        arena.release(ls)
        size = int(size * 1.5)
    assert arena.blocks() < 20


def test_out_of_order_release_never_aliases_a_live_lease(arena):
    a = arena.acquire(1000)
    b = arena.acquire(1000)
    arena.release(a)              # out of order: only marked
    c = arena.acquire(1000)       # must not be served from a's bytes while b is live above it
    assert c.ptr != a.ptr and c.ptr != b.ptr
    assert not (b.ptr <= c.ptr < b.ptr + 1000)
    arena.release(c)
    arena.release(b)              # b innermost now -> reclaims b and the already-returned a
    d = arena.acquire(1000)
    assert d.ptr == a.ptr         # LIFO reuse from the bottom again
    arena.release(d)


def test_trim_refuses_while_leased_and_frees_otherwise(arena):
    a = arena.acquire(5000)
    assert arena.trim() == 0 and arena.capacity() > 0
    arena.release(a)
    assert arena.trim() == 1 and arena.capacity() == 0 and arena.blocks() == 0
    b = arena.acquire(100)        # usable again after a trim
    arena.release(b)
    arena.release(b)              # releasing twice is harmless (stale sequence number)
    assert arena.trim() == 1


def test_shard_ranges_partition_the_batch():
    for batch in (0, 1, 7, 512, 10_000, 1_000_000):
        for world in (1, 2, 3, 4, 8):
            got, nxt = 0, 0
            for r in range(world):
                b0, nb = shard_range(batch, r, world)
                assert b0 == nxt and nb >= 0
                nxt = b0 + nb
                got += nb
            assert got == batch
    assert shard_range(512, 3, 8) == (192, 64)
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def test_shard_desc_advances_every_operand_of_every_descriptor():
    from batchlas_b200.sharding import shard_desc
    g = _lib.GemmDesc()
    g.a, g.b, g.c, g.batch, g.stride_a, g.stride_b, g.stride_c = 1000, 2000, 3000, 10, 6, 8, 12
    sub = shard_desc(g, 1, 4, 8)   # items [2, 5)
    assert (sub.a, sub.b, sub.c, sub.batch) == (1000 + 2 * 6 * 8, 2000 + 2 * 8 * 8, 3000 + 2 * 12 * 8, 3)
    v = _lib.GemvDesc()
    v.a, v.x, v.y, v.batch, v.stride_a, v.stride_x, v.stride_y, v.incx = 1000, 2000, 3000, 9, 20, 5, 4, 2
    sub = shard_desc(v, 2, 3, 4)   # items [6, 9)
    assert (sub.a, sub.x, sub.y, sub.batch, sub.incx) == (1000 + 6 * 20 * 4, 2000 + 6 * 5 * 4, 3000 + 6 * 4 * 4, 3, 2)
    e = _lib.EwiseDesc()
    e.a, e.b, e.c, e.batch, e.stride_a, e.stride_b, e.stride_c = 16, 32, 48, 4, 100, 100, 200
    sub = shard_desc(e, 3, 4, 16)  # item 3
    assert (sub.a, sub.b, sub.c, sub.batch) == (16 + 3 * 100 * 16, 32 + 3 * 100 * 16, 48 + 3 * 200 * 16, 1)
