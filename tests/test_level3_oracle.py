"""The level-3 oracle pinned on the CPU: its extended-precision restatement of symm / hemm / trmm /
syrk / herk against the BLAS routines themselves (the OpenBLAS SciPy ships — the routines the
reference's host backend calls per batch item, BatchLAS src/backends/netlib_lapack.cc:333-760), on the
shapes the reference's own tests use (tests/symm_tests.cc:52-58, hemm_tests.cc, trmm_tests.cc:58-73,
syrk_tests.cc, herk_tests.cc:238-345), scaled down where they are large."""
import numpy as np
import pytest

from oracle import level3 as L

DTYPES = [np.float32, np.float64, np.complex64, np.complex128]


def rnd(rng, shape, dtype):
    x = rng.uniform(-1, 1, shape)
    if np.issubdtype(dtype, np.complexfloating):
        x = x + 1j * rng.uniform(-1, 1, shape)
    return x.astype(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("side", [0, 1])
@pytest.mark.parametrize("uplo", [0, 1])
def test_symm_restatement_matches_blas(dtype, side, uplo):
    rng = np.random.default_rng(5)
    n, m, batch = 96, 64, 3  # tests/symm_tests.cc:52-56
    k = n
    rows, cols = (n, m) if side == 0 else (m, n)
    a, b, c = rnd(rng, (batch, k, k), dtype), rnd(rng, (batch, rows, cols), dtype), rnd(rng, (batch, rows, cols), dtype)
    alpha, beta = dtype(1.25), dtype(-0.5)
    for herm in ([False, True] if np.issubdtype(dtype, np.complexfloating) else [False]):
        exact, bound = L.symm_exact(a, b, c, alpha, beta, side, uplo, herm)
        ok, worst = L.within(L.symm_blas(a, b, c, alpha, beta, side, uplo, herm), exact, bound, k, dtype)
        assert ok, worst


@pytest.mark.parametrize("dtype", DTYPES)
def test_trmm_restatement_matches_blas(dtype):
    rng = np.random.default_rng(6)
    batch = 2
    for m, n in [(48, 32), (17, 33)]:
        for side in (0, 1):
            k = m if side == 0 else n
            a, b = rnd(rng, (batch, k, k), dtype), rnd(rng, (batch, m, n), dtype)
            for uplo in (0, 1):
                for op in (0, 1, 2):
                    for unit in (False, True):
                        exact, bound = L.trmm_exact(a, b, dtype(0.9), side, uplo, op, unit)
                        got = L.trmm_blas(a, b, dtype(0.9), side, uplo, op, unit)
                        ok, worst = L.within(got, exact, bound, k, dtype)
                        assert ok, (side, uplo, op, unit, worst)


@pytest.mark.parametrize("dtype", DTYPES)
def test_syrk_herk_restatement_matches_blas(dtype):
    rng = np.random.default_rng(7)
    n, k, batch = 65, 40, 4  # tests/herk_tests.cc:242-244
    cplx = np.issubdtype(dtype, np.complexfloating)
    for herm in ([False, True] if cplx else [False]):
        for op in ((0, 2) if herm else (0, 1)):
            a = rnd(rng, (batch, n, k) if op == 0 else (batch, k, n), dtype)
            c = rnd(rng, (batch, n, n), dtype)
            for uplo in (0, 1):
                for alpha, beta in [(0.9, -0.35), (1.0, 0.0)]:
                    al, be = (alpha, beta) if herm else (dtype(alpha), dtype(beta))
                    exact, bound, mask = L.syrk_exact(a, c, al, be, uplo, op, herm)
                    got = L.syrk_blas(a, c, al, be, uplo, op, herm)
                    ok, worst = L.within(got, exact, bound, k, dtype, mask)
                    assert ok, (herm, op, uplo, worst)
                    if herm:
                        idx = np.arange(n)
                        assert np.all(got[:, idx, idx].imag == 0) and np.all(exact[:, idx, idx].imag == 0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_syr2k_her2k_restatement_matches_blas(dtype):
    rng = np.random.default_rng(8)
    n, k, batch = 48, 20, 3
    cplx = np.issubdtype(dtype, np.complexfloating)
    for herm in ([False, True] if cplx else [False]):
        for op in ((0, 2) if herm else (0, 1)):
            shape = (batch, n, k) if op == 0 else (batch, k, n)
            a, b, c = rnd(rng, shape, dtype), rnd(rng, shape, dtype), rnd(rng, (batch, n, n), dtype)
            for uplo in (0, 1):
                alpha = dtype(0.9 - 0.4j) if cplx else dtype(0.9)
                beta = -0.35 if herm else dtype(-0.35)
                exact, bound, mask = L.syr2k_exact(a, b, c, alpha, beta, uplo, op, herm)
                got = L.syr2k_blas(a, b, c, alpha, beta, uplo, op, herm)
                ok, worst = L.within(got, exact, bound, 2 * k, dtype, mask)
                assert ok, (herm, op, uplo, worst)


def test_expansions():
    a = np.arange(1, 10, dtype=np.complex128).reshape(1, 3, 3) * (1 + 1j)
    full = L.expand_full(a, 1, hermitian=True)[0]
    assert np.allclose(full, full.conj().T) and np.all(full.diagonal().imag == 0)
    assert full[2, 0] == a[0, 2, 0] and full[0, 2] == np.conj(a[0, 2, 0])
    sym = L.expand_full(a, 0)[0]
    assert np.array_equal(sym, sym.T) and sym[0, 2] == a[0, 0, 2]
    tri = L.expand_triangular(a, 0, True)[0]
    assert tri[1, 0] == 0 and tri[0, 1] == a[0, 0, 1] and np.all(tri.diagonal() == 1)
