"""The gemv / elementwise oracle pinned on the CPU: extended-precision restatement against the BLAS
routine (SciPy's OpenBLAS ?gemv, what the reference's host backend calls per item,
BatchLAS src/backends/netlib_lapack.cc:174-215) and against the known answers of the reference's
tests (tests/gemv_tests.cc:60-105: triple-loop expectation, alpha/beta cases)."""
import numpy as np
import pytest

from oracle import linalg as LA

DTYPES = [np.float32, np.float64, np.complex64, np.complex128]


def rnd(rng, shape, dtype):
    x = rng.uniform(-1, 1, shape)
    if np.issubdtype(dtype, np.complexfloating):
        x = x + 1j * rng.uniform(-1, 1, shape)
    return x.astype(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", [0, 1, 2])
def test_gemv_restatement_matches_blas(dtype, op):
    rng = np.random.default_rng(9)
    m, n, batch = 37, 23, 4
    a = rnd(rng, (batch, m, n), dtype)
    x = rnd(rng, (batch, n if op == 0 else m), dtype)
    y = rnd(rng, (batch, m if op == 0 else n), dtype)
    for alpha, beta in [(1.0, 0.0), (2.5, 0.0), (1.5, 0.8)]:  # tests/gemv_tests.cc:131,159,221,263
        exact, bound = LA.gemv_exact(a, x, y, dtype(alpha), dtype(beta), op)
        got = LA.gemv_blas(a, x, y, dtype(alpha), dtype(beta), op)
        ok, worst = LA.gemv_within(got, exact, bound, x.shape[1], dtype)
        assert ok, worst


def test_gemv_known_answer():
    a = np.array([[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]])  # 2 x 3
    x = np.array([[1.0, 0.5, -1.0]])
    y = np.array([[10.0, 20.0]])
    exact, _ = LA.gemv_exact(a, x, y, 2.0, 0.5, 0)
    assert np.allclose(np.asarray(exact, float), [[2 * (1 + 1 - 3) + 5, 2 * (4 + 2.5 - 6) + 10]])
    exact_t, _ = LA.gemv_exact(a, np.array([[1.0, -1.0]]), np.array([[0.0, 0.0, 0.0]]), 1.0, 0.0, 1)
    assert np.allclose(np.asarray(exact_t, float), [[-3.0, -3.0, -3.0]])


@pytest.mark.parametrize("dtype", DTYPES)
def test_elementwise_restatement_matches_numpy(dtype):
    rng = np.random.default_rng(10)
    a, b = rnd(rng, (3, 9, 7), dtype), rnd(rng, (3, 9, 7), dtype) + dtype(2)
    for op, f in zip(LA.OPS, (np.add, np.subtract, np.multiply, np.divide)):
        exact, mag = LA.elementwise_exact(op, a, b)
        ok, worst = LA.elementwise_within(f(a, b), exact, mag, dtype)
        assert ok, (op, worst)
    exact, mag = LA.axpby_exact(dtype(1.5), a, dtype(-0.25), b)
    ok, worst = LA.elementwise_within(dtype(1.5) * a + dtype(-0.25) * b, exact, mag, dtype)
    assert ok, worst
