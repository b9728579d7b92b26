"""Parity of gemv and the elementwise helpers against the CPU oracle, through the library's own
kernels.  Acceptance rules (entrywise):

    gemv:         |y_gpu - exact| <= 4 * K * eps_T * (|alpha| * |op(A)| * |x| + |beta| * |y0|),  K = length of x
    elementwise:  |c_gpu - exact| <= 8 * eps_T * mag,   mag = |a|+|b| (add, subtract), |a|*|b|, |a|/|b|,
                  |alpha|*|a| + |beta|*|b| (axpby)

`exact` accumulated in long double.  Shapes follow the reference's tests (BatchLAS tests/gemv_tests.cc:
square fixtures, single and batched, N and T, alpha/beta; tests/linalg_layer_tests.cc for the
elementwise layer) and add ragged sizes, padded leading dimensions, vector increments and batch gaps;
memory that must not be written carries canaries."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import linalg as LA  # noqa: E402

pytestmark = pytest.mark.gpu

NP_DT = {"s": np.float32, "d": np.float64, "c": np.complex64, "z": np.complex128}


@pytest.fixture(scope="module")
def bl(lib):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    import batchlas_b200
    return batchlas_b200


def rnd(rng, shape, dtype):
    x = rng.uniform(-1, 1, shape)
    if np.issubdtype(dtype, np.complexfloating):
        x = x + 1j * rng.uniform(-1, 1, shape)
    return x.astype(dtype)


def mat_to_dev(x, pad=0, gap=0):
    """(batch, rows, cols) -> column-major view (batch, cols, rows), ld = rows + pad, `gap` unused
    elements between items; returns (view, backing)."""
    b, r, c = x.shape
    back = torch.full((b, c * (r + pad) + gap), 7.0, dtype=torch.from_numpy(x[:0]).dtype, device="cuda")
    view = back[:, :c * (r + pad)].view(b, c, r + pad)[:, :, :r]
    view.copy_(torch.from_numpy(np.ascontiguousarray(np.swapaxes(x, 1, 2))).cuda())
    return view, back


def vec_to_dev(v, inc=1, gap=0):
    b, n = v.shape
    back = torch.full((b, max(n, 1) * inc + gap), 7.0, dtype=torch.from_numpy(v[:0]).dtype, device="cuda")
    view = back[:, :n * inc:inc] if n else back[:, :0]
    view.copy_(torch.from_numpy(v).cuda())
    return view, back


GEMV_SHAPES = [(32, 32, 5), (64, 64, 3), (37, 23, 4), (1, 50, 2), (50, 1, 2), (130, 70, 3), (257, 300, 2),
               (1024, 1024, 1), (8, 2048, 1), (2048, 8, 1), (33, 1000, 40)]


@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("shape", GEMV_SHAPES, ids=str)
def test_gemv(bl, dt, shape):
    dtype = NP_DT[dt]
    m, n, batch = shape
    rng = np.random.default_rng(500 + m + n)
    a = rnd(rng, (batch, m, n), dtype)
    dA, _ = mat_to_dev(a, pad=3, gap=5)
    for op in (0, 1, 2):
        xl, yl = (n, m) if op == 0 else (m, n)
        x, y0 = rnd(rng, (batch, xl), dtype), rnd(rng, (batch, yl), dtype)
        for alpha, beta, incx, incy in [(1.0, 0.0, 1, 1), (1.5, 0.8, 2, 3)]:
            if dt in "cz":
                alpha, beta = alpha + 0.5j, beta * (1 - 0.25j)
            y_in = y0.copy()
            if beta == 0:
                y_in[:] = np.nan  # never read then
            dX, _ = vec_to_dev(x, incx, gap=2)
            dY, backY = vec_to_dev(y_in, incy, gap=4)
            bl.linalg.gemv(dA, dX, dY, alpha, beta, op)
            exact, bound = LA.gemv_exact(a, x, y_in, alpha, beta, op)
            ok, worst = LA.gemv_within(dY.cpu().numpy(), exact, bound, xl, dtype)
            assert ok, f"op={op} alpha={alpha} beta={beta} worst {worst:.3g}"
            mask = torch.ones_like(backY, dtype=torch.bool)
            mask[:, :yl * incy:incy] = False
            assert bool((backY[mask] == 7.0).all()), "gemv wrote between or behind the elements of y"


def test_gemv_large_batch_of_small_matrices(bl):
    """The shape the headline gemm workload has: 32 x 32 float, many items."""
    rng = np.random.default_rng(77)
    batch = 20011
    a, x, y0 = rnd(rng, (batch, 32, 32), np.float32), rnd(rng, (batch, 32), np.float32), rnd(rng, (batch, 32), np.float32)
    dA, _ = mat_to_dev(a)
    for op in (0, 1):
        dX, _ = vec_to_dev(x)
        dY, _ = vec_to_dev(y0)
        bl.linalg.gemv(dA, dX, dY, 1.5, -0.5, op)
        exact, bound = LA.gemv_exact(a, x, y0, 1.5, -0.5, op)
        ok, worst = LA.gemv_within(dY.cpu().numpy(), exact, bound, 32, np.float32)
        assert ok, worst


@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("shape", [(32, 32), (64, 64), (24, 40), (128, 8), (8, 128), (20, 20), (100, 12)], ids=str)
def test_gemv_ring_kernel(bl, dt, shape):
    """Large batches of small packed matrices go through the TMA ring; every dtype, both operand
    transforms, ragged shapes whose item size is still a multiple of 16 bytes."""
    dtype = NP_DT[dt]
    m, n = shape
    if m * n * np.dtype(dtype).itemsize > 16384:
        pytest.skip("item larger than a ring slot")
    batch = 1500 if m * n >= 1024 else 2500
    rng = np.random.default_rng(700 + m * n)
    a = rnd(rng, (batch, m, n), dtype)
    dA, _ = mat_to_dev(a)
    for op in (0, 1, 2):
        xl, yl = (n, m) if op == 0 else (m, n)
        x, y0 = rnd(rng, (batch, xl), dtype), rnd(rng, (batch, yl), dtype)
        for alpha, beta in [(1.5, -0.5), (2.0, 0.0)]:
            if dt in "cz":
                alpha = alpha + 0.5j
            y_in = y0.copy()
            if beta == 0:
                y_in[:] = np.nan
            dX, _ = vec_to_dev(x)
            dY, backY = vec_to_dev(y_in, gap=4)  # items stay 16-byte aligned
            bl.linalg.gemv(dA, dX, dY, alpha, beta, op)
            assert bl.last_kernel_name() == "gemv_ring"
            exact, bound = LA.gemv_exact(a, x, y_in, alpha, beta, op)
            ok, worst = LA.gemv_within(dY.cpu().numpy(), exact, bound, xl, dtype)
            assert ok, f"op={op} beta={beta} worst {worst:.3g}"
            assert bool((backY[:, yl:] == 7.0).all())
    assert bl.device_status() == 0


def test_gemv_empty_and_errors(bl, lib):
    y = torch.full((2, 5), 3.0, device="cuda", dtype=torch.float64)
    a = torch.zeros((2, 0, 5), device="cuda", dtype=torch.float64)  # 5 x 0: empty x scales y by beta
    x = torch.zeros((2, 0), device="cuda", dtype=torch.float64)
    bl.linalg.gemv(a, x, y, 1.0, 0.5, 0)
    assert bool((y == 1.5).all())
    bl.linalg.gemv(a, x, y, 1.0, 0.0, 0)
    assert bool((y == 0.0).all())
    with pytest.raises(RuntimeError, match="GEMV: incompatible dimensions"):
        bl.linalg.gemv(torch.zeros((2, 4, 5), device="cuda"), torch.zeros((2, 5), device="cuda"),
                       torch.zeros((2, 5), device="cuda"))
    d = bl._lib.GemvDesc()
    d.m, d.n, d.batch, d.lda, d.incx, d.incy, d.dtype = 4, 4, 1, 2, 1, 1, 0
    assert lib.blb200_gemv_strided_batched(d, None) == bl._lib.E_SHAPE  # lda < m
    d.lda, d.incx = 4, 0
    assert lib.blb200_gemv_strided_batched(d, None) == bl._lib.E_SHAPE
    d.incx = 1
    assert lib.blb200_gemv_strided_batched(d, None) == bl._lib.E_NULL
    assert lib.blb200_gemv_strided_batched(None, None) == bl._lib.E_NULL


EW_SHAPES = [(10, 10, 3), (33, 7, 5), (1, 1, 1), (256, 256, 4), (1000, 3, 2), (5, 700, 3)]


@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("packed", [True, False], ids=["packed", "strided"])
@pytest.mark.parametrize("shape", EW_SHAPES, ids=str)
def test_elementwise_and_axpby(bl, dt, packed, shape):
    dtype = NP_DT[dt]
    rows, cols, batch = shape
    rng = np.random.default_rng(600 + rows)
    a = rnd(rng, (batch, rows, cols), dtype)
    b = rnd(rng, (batch, rows, cols), dtype) + dtype(2)  # away from zero for the division
    pad, gap = (0, 0) if packed else (3, 5)
    dA, _ = mat_to_dev(a, pad, gap)
    dB, _ = mat_to_dev(b, pad + (0 if packed else 1), gap)
    fns = {"add": bl.linalg.add_into, "subtract": bl.linalg.subtract_into, "multiply": bl.linalg.multiply_into,
           "divide": bl.linalg.divide_into}
    for op, fn in fns.items():
        dC, backC = mat_to_dev(np.zeros_like(a), pad, gap)
        fn(dA, dB, dC)
        exact, mag = LA.elementwise_exact(op, a, b)
        ok, worst = LA.elementwise_within(np.swapaxes(dC.cpu().numpy(), 1, 2), exact, mag, dtype)
        assert ok, f"{op} worst {worst:.3g}"
        if not packed:
            assert bool((backC[:, cols * (rows + pad):] == 7.0).all()) and bool(
                (backC[:, :cols * (rows + pad)].view(batch, cols, rows + pad)[:, :, rows:] == 7.0).all())
    alpha, beta = (1.5, -0.25) if dt in "sd" else (1.5 - 0.5j, -0.25 + 2j)
    dC, _ = mat_to_dev(np.zeros_like(a), pad, gap)
    bl.linalg.axpby_into(alpha, dA, beta, dB, dC)
    exact, mag = LA.axpby_exact(alpha, a, beta, b)
    ok, worst = LA.elementwise_within(np.swapaxes(dC.cpu().numpy(), 1, 2), exact, mag, dtype)
    assert ok, worst
    # aliasing: C = A, and scaling in place
    bl.linalg.add_into(dA, dB, dA)
    exact, mag = LA.elementwise_exact("add", a, b)
    ok, worst = LA.elementwise_within(np.swapaxes(dA.cpu().numpy(), 1, 2), exact, mag, dtype)
    assert ok, worst
    bl.linalg.scale(dB, alpha)
    exact, mag = LA.axpby_exact(alpha, b, 0.0, b)
    ok, worst = LA.elementwise_within(np.swapaxes(dB.cpu().numpy(), 1, 2), exact, mag, dtype)
    assert ok, worst


def test_elementwise_shape_errors(bl, lib):
    a = torch.zeros((2, 3, 4), device="cuda")
    with pytest.raises(ValueError, match="linalg::elementwise_into: operands must have the same shape"):
        bl.linalg.add_into(a, torch.zeros((2, 4, 3), device="cuda"), a)
    with pytest.raises(ValueError, match="linalg::axpby_into: operands must have the same shape"):
        bl.linalg.axpby_into(1.0, a, 1.0, a, torch.zeros((1, 3, 4), device="cuda"))
    d = bl._lib.EwiseDesc()
    d.rows, d.cols, d.batch, d.lda, d.ldb, d.ldc = 4, 3, 2, 4, 4, 3
    assert lib.blb200_elementwise(d, 0, None) == bl._lib.E_SHAPE
    d.ldc = 4
    assert lib.blb200_elementwise(d, 4, None) == bl._lib.E_DTYPE
    assert lib.blb200_elementwise(d, 0, None) == bl._lib.E_NULL


def test_matmul_matches_gemm(bl):
    rng = np.random.default_rng(12)
    a, b = rnd(rng, (3, 40, 24), np.float64), rnd(rng, (3, 24, 56), np.float64)
    dA, _ = mat_to_dev(a)
    dB, _ = mat_to_dev(b)
    c = bl.linalg.matmul(dA, dB, alpha=2.0)
    ref = 2.0 * np.matmul(a.astype(np.longdouble), b.astype(np.longdouble))
    assert np.allclose(np.swapaxes(c.cpu().numpy(), 1, 2), np.asarray(ref, float), rtol=0, atol=1e-12)
    ct = bl.linalg.matmul(dB, dA, transA=1, transB=1)
    assert np.allclose(np.swapaxes(ct.cpu().numpy(), 1, 2), np.swapaxes(np.asarray(ref / 2, float), 1, 2), rtol=0, atol=1e-12)
