"""NumPy front end (batchlas_b200.api): the contract BatchLAS's Python tests pin for gemm
(python/tests/test_batchlas.py:33-44, 65-80, 209-221), computed on the GPU."""
import numpy as np
import pytest

from batchlas_b200 import api as bl


def test_argument_contract_needs_no_gpu():
    a = np.eye(2)
    with pytest.raises(ValueError):
        bl.gemm(a, a, beta=1.0)                      # beta requires an out operand
    with pytest.raises(RuntimeError):
        bl.gemm(a, a, backend="netlib")              # only the CUDA arm exists
    with pytest.raises(RuntimeError):
        bl.gemm(a, a, compute_precision="tf32")      # no reduced-precision shortcut
    with pytest.raises(ValueError):
        bl.gemm(np.ones((2, 3)), np.ones((2, 3)))    # inner dimensions disagree
    with pytest.raises(ValueError):
        bl.gemm(a, a, trans_a="x")
    assert bl.available_backends() == ["cuda"]


@pytest.mark.gpu
def test_gemm_and_out_contract():
    a = np.array([[1.0, 2.0], [3.0, 4.0]])
    b = np.array([[5.0, 6.0], [7.0, 8.0]])
    out = np.empty((2, 2))
    result = bl.gemm(a, b, out=out)
    assert result is out
    np.testing.assert_allclose(out, a @ b)
    np.testing.assert_allclose(a, [[1.0, 2.0], [3.0, 4.0]])
    np.testing.assert_allclose(b, [[5.0, 6.0], [7.0, 8.0]])


@pytest.mark.gpu
def test_gemm_applies_beta_to_the_out_operand():
    rng = np.random.default_rng(0)
    a, b, c = (rng.standard_normal((2, 3, 3)) for _ in range(3))
    got = bl.gemm(a, b, alpha=2.0, beta=0.5, out=c.copy())
    np.testing.assert_allclose(got, 2.0 * (a @ b) + 0.5 * c, rtol=1e-10, atol=1e-10)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64, np.complex128])
def test_transposes_and_batches_match_numpy(dtype):
    rng = np.random.default_rng(1)

    def rnd(*shape):
        x = rng.standard_normal(shape)
        if np.issubdtype(dtype, np.complexfloating):
            x = x + 1j * rng.standard_normal(shape)
        return x.astype(dtype)

    tol = 2e-4 if dtype in (np.float32, np.complex64) else 1e-10
    ops = {"n": lambda x: x, "t": lambda x: np.swapaxes(x, -1, -2), "c": lambda x: np.conj(np.swapaxes(x, -1, -2))}
    for ta in "ntc":
        for tb in "ntc":
            m, n, k, batch = 37, 29, 41, 5
            a = rnd(batch, m, k) if ta == "n" else rnd(batch, k, m)
            b = rnd(batch, k, n) if tb == "n" else rnd(batch, n, k)
            got = bl.gemm(a, b, alpha=1.5, trans_a=ta, trans_b=tb)
            np.testing.assert_allclose(got, 1.5 * (ops[ta](a) @ ops[tb](b)), rtol=tol, atol=tol * 10)
    a, b = rnd(64, 64), rnd(64, 64)
    np.testing.assert_allclose(bl.gemm(a, b), a @ b, rtol=tol, atol=tol * 20)


@pytest.mark.gpu
def test_gemm_heterogeneous_returns_python_list():
    a = [np.array([[1.0, 2.0], [3.0, 4.0]]), np.array([[2.0, 0.0, 1.0]])]
    b = [np.array([[1.0], [2.0]]), np.array([[1.0], [0.0], [1.0]])]
    result = bl.gemm_heterogeneous(a, b)
    assert isinstance(result, list) and len(result) == 2
    np.testing.assert_allclose(result[0], a[0] @ b[0])
    np.testing.assert_allclose(result[1], a[1] @ b[1])
    rng = np.random.default_rng(2)
    shapes = [(5, 7, 3), (33, 2, 40), (1, 1, 1), (17, 45, 9)]
    a = [rng.standard_normal((k, m)) for m, n, k in shapes]      # trans_a = "t"
    b = [rng.standard_normal((k, n)) for m, n, k in shapes]
    for got, x, y in zip(bl.gemm_heterogeneous(a, b, alpha=2.0, trans_a="t"), a, b):
        np.testing.assert_allclose(got, 2.0 * (x.T @ y), rtol=1e-10, atol=1e-10)
