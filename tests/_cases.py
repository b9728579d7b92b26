"""Shared helpers for the parity tests: seeded problems with canary padding, and the case lists
taken from the reference's own gemm tests (BatchLAS tests/gemm_tests.cc)."""
from __future__ import annotations

import numpy as np

from oracle import oracle

CANARY = {0: np.float32(-777.25), 1: np.float64(-777.25), 2: np.complex64(-777.25 + 3.5j),
          3: np.complex128(-777.25 + 3.5j)}


def make_inputs(p: oracle.Problem, seed: int = 42, dist_ab: str = "uniform", dist_c: str = "uniform",
                scale: float = 1.0, tail: int = 7):
    """Flat A, B, C buffers for `p`.  Every element outside the stored matrices (ld padding, stride
    gaps, a short tail) holds a canary; C inside the m x n windows holds seeded data."""
    npdt = oracle.NP_DTYPES[p.dtype]
    out = []
    for tid, which, dist in ((1, "a", dist_ab), (2, "b", dist_ab), (3, "c", dist_c)):
        n = p.alloc_len(which) + tail
        buf = np.full(n, CANARY[p.dtype], dtype=npdt)
        rows, cols = {"a": p.a_shape, "b": p.b_shape, "c": (p.m, p.n)}[which]
        ld, st = {"a": (p.lda, p.stride_a), "b": (p.ldb, p.stride_b), "c": (p.ldc, p.stride_c)}[which]
        if rows > 0 and cols > 0 and p.batch > 0:
            vals = oracle.fill(p.dtype, p.batch * rows * cols, seed, tid, dist, scale).reshape(p.batch, cols, rows)
            idx = (np.arange(p.batch, dtype=np.int64)[:, None, None] * st
                   + np.arange(cols, dtype=np.int64)[None, :, None] * ld
                   + np.arange(rows, dtype=np.int64)[None, None, :])
            buf[idx.ravel()] = vals.ravel()
        out.append(buf)
    return out


# (m, n, k, batch, opA, opB, alpha, beta) — shapes the reference's tests exercise:
#   identity-sized 10x10 b1/b3 (gemm_tests.cc:355-396); 32^3 b4 beta=0 and 128^3 b2 alpha=beta=1
#   (:674-739); T/T 24x20x16 b3 and 96x80x64 (:1276-1351); C.N 18x14x12 b2 (:2035-2071);
#   aligned 256^3 and ragged 200x130x70 alpha=2 beta=-1 b3 (:1964-2033); API cases 16^3/12^3/8^3
#   (backend_dispatch_tests.cc:96-142); python 2x2 and 3x3x3 (python/tests/test_batchlas.py:33-44).
REFERENCE_SHAPES = [
    (10, 10, 10, 1, "N", "N", 1.0, 0.0),
    (10, 10, 10, 3, "N", "N", 1.0, 0.0),
    (32, 32, 32, 4, "N", "N", 1.0, 0.0),
    (128, 128, 128, 2, "N", "N", 1.0, 1.0),
    (24, 20, 16, 3, "T", "T", 1.0, 0.0),
    (96, 80, 64, 1, "T", "T", 1.0, 0.0),
    (18, 14, 12, 2, "C", "N", 1.0, 0.0),
    (256, 256, 256, 1, "N", "N", 1.0, 0.0),
    (200, 130, 70, 3, "N", "N", 2.0, -1.0),
    (16, 16, 16, 2, "N", "N", 1.0, 0.0),
    (12, 12, 12, 1, "N", "T", 1.0, 0.0),
    (8, 8, 8, 1, "T", "N", 1.0, 0.0),
    (2, 2, 2, 1, "N", "N", 2.0, 0.5),
    (3, 3, 3, 3, "N", "N", 2.0, 0.5),
]

# Extra edges: unit dims, ragged everything, k == 0, batch == 1 with large-ish dims.
EDGE_SHAPES = [
    (1, 1, 1, 1, "N", "N", 1.0, 0.0),
    (1, 37, 5, 2, "N", "T", -1.0, 2.0),
    (41, 1, 9, 2, "T", "N", 0.5, 0.0),
    (33, 31, 1, 3, "N", "N", 1.0, 1.0),
    (17, 19, 0, 2, "N", "N", 1.0, 0.5),
    (17, 19, 0, 2, "T", "C", 1.0, 0.0),
    (65, 63, 67, 2, "C", "C", 1.25, -0.75),
    (130, 70, 33, 1, "N", "C", 1.0, 0.0),
]

DTYPE_NAMES = ["s", "d", "c", "z"]


def scalar_for(dtype_code: int, value: float) -> complex:
    """Complex dtypes get a genuinely complex scalar so the imaginary paths are exercised."""
    if dtype_code >= 2 and value != 0.0:
        return complex(value, 0.5 * value)
    return complex(value, 0.0)
