"""Parity of the level-3 calls that run on the gemm kernels (symm, hemm, trmm, syrk, herk) against the
CPU oracle, on the shapes and option sweeps of the reference's own tests (BatchLAS tests/symm_tests.cc,
hemm_tests.cc, trmm_tests.cc, syrk_tests.cc, herk_tests.cc).  Acceptance rule, entrywise:

    |C_gpu - exact| <= 4 * k * eps_T * (|alpha| * |A| * |B| + |beta| * |C0|)

with `exact` and the magnitude sum accumulated in long double, A the expanded (full / triangular)
operand.  Storage the operation must not reference is poisoned with NaN on the way in (the other
triangle of A, the diagonal under Diag::Unit) and storage it must not write has to come back
bit-identical (the other triangle of C, padding rows)."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import level3 as L  # noqa: E402

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


def to_dev(x, pad=0, pad_value=7.0):
    """(batch, rows, cols) array -> column-major device tensor (batch, cols, rows) with ld = rows + pad;
    returns (view, backing) so the padding rows can be checked afterwards."""
    b, r, c = x.shape
    back = torch.full((b, c, r + pad), pad_value, dtype=torch.from_numpy(x[:0]).dtype, device="cuda")
    back[:, :, :r] = torch.from_numpy(np.ascontiguousarray(np.swapaxes(x, 1, 2))).cuda()
    return back[:, :, :r], back


def from_dev(view):
    return np.swapaxes(view.cpu().numpy(), 1, 2)


def poison_other_triangle(a, uplo, diag_too=False):
    """NaN where the operation must not look."""
    p = a.copy()
    n = a.shape[-1]
    other = np.triu(np.ones((n, n), bool), 1) if uplo == 1 else np.tril(np.ones((n, n), bool), -1)
    if diag_too:
        other |= np.eye(n, dtype=bool)
    p[:, other] = np.nan
    return p


@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("side", [0, 1])
@pytest.mark.parametrize("uplo", [0, 1])
@pytest.mark.parametrize("shape", [(96, 64, 3), (33, 7, 5), (128, 128, 8)], ids=str)
def test_symm_hemm(bl, dt, side, uplo, shape):
    dtype = NP_DT[dt]
    n, m, batch = shape
    rng = np.random.default_rng(100 + n)
    rows, cols = (n, m) if side == 0 else (m, n)
    a, b, c0 = rnd(rng, (batch, n, n), dtype), rnd(rng, (batch, rows, cols), dtype), rnd(rng, (batch, rows, cols), dtype)
    alpha, beta = (1.25, -0.5) if dt in "sd" else (1.25 + 0.5j, -0.5 + 0.25j)
    for herm in ([False, True] if dt in "cz" else [False]):
        a_in = poison_other_triangle(a, uplo)
        if herm:  # the imaginary part of a Hermitian diagonal is not referenced either
            idx = np.arange(n)
            diag = a[:, idx, idx].copy()
            diag.imag = np.nan
            a_in[:, idx, idx] = diag
        dA, _ = to_dev(a_in, pad=3)
        dB, _ = to_dev(b, pad=1)
        dC, backC = to_dev(c0, pad=5)
        bl.symm(dA, dB, dC, alpha, beta, side, uplo, hermitian=herm)
        torch.cuda.synchronize()
        exact, bound = L.symm_exact(a, b, c0, alpha, beta, side, uplo, herm)
        ok, worst = L.within(from_dev(dC), exact, bound, n, dtype)
        assert ok, f"herm={herm} worst ratio {worst:.3g}"
        assert bool((backC[:, :, rows:] == 7.0).all()), "padding rows of C were written"


def test_symm_beta_zero_ignores_nan_in_c(bl):
    rng = np.random.default_rng(3)
    a, b = rnd(rng, (2, 40, 40), np.float64), rnd(rng, (2, 40, 24), np.float64)
    c0 = np.full((2, 40, 24), np.nan)
    dA, _ = to_dev(a)
    dB, _ = to_dev(b)
    dC, _ = to_dev(c0)
    bl.symm(dA, dB, dC, 2.0, 0.0, 0, 1)
    exact, bound = L.symm_exact(a, b, c0, 2.0, 0.0, 0, 1)
    ok, worst = L.within(from_dev(dC), exact, bound, 40, np.float64)
    assert ok, worst


def apad(rows, aligned, odd):
    """Padding rows: `odd` as given, or what makes the leading dimension a multiple of 4 elements
    (16-byte aligned columns for every dtype) when the tile kernels are to be reached."""
    return (-rows) % 4 + 4 if aligned else odd


@pytest.mark.parametrize("aligned", [False, True], ids=["oddld", "alignedld"])
@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("shape", [(48, 32, 2), (17, 33, 3), (128, 128, 4), (200, 136, 2)], ids=str)
def test_trmm_all_combinations(bl, dt, shape, aligned):
    dtype = NP_DT[dt]
    m, n, batch = shape
    rng = np.random.default_rng(200 + m)
    alpha = 0.9 if dt in "sd" else 0.9 - 0.3j
    for side in (0, 1):
        k = m if side == 0 else n
        a, b = rnd(rng, (batch, k, k), dtype), rnd(rng, (batch, m, n), dtype)
        dB, _ = to_dev(b, pad=apad(m, aligned, 2))
        for uplo in (0, 1):
            for unit in (False, True):
                dA, _ = to_dev(poison_other_triangle(a, uplo, diag_too=unit), pad=1)
                for op in (0, 1, 2):
                    dC, backC = to_dev(np.full((batch, m, n), np.nan, dtype), pad=apad(m, aligned, 5))
                    bl.trmm(dA, dB, dC, alpha, side, uplo, op, int(unit))
                    exact, bound = L.trmm_exact(a, b, alpha, side, uplo, op, unit)
                    ok, worst = L.within(from_dev(dC), exact, bound, k, dtype)
                    assert ok, f"side={side} uplo={uplo} unit={unit} op={op} worst {worst:.3g}"
                    assert bool((backC[:, :, m:] == 7.0).all())


@pytest.mark.parametrize("aligned", [False, True], ids=["oddld", "alignedld"])
@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("shape", [(65, 40, 4), (32, 24, 3), (128, 200, 3), (7, 1, 2), (300, 72, 2)], ids=str)
def test_syrk_herk(bl, dt, shape, aligned):
    dtype = NP_DT[dt]
    n, k, batch = shape
    rng = np.random.default_rng(300 + n)
    idx = np.arange(n)
    for herm in ([False, True] if dt in "cz" else [False]):
        for op in ((0, 2) if herm else (0, 1)):
            a = rnd(rng, (batch, n, k) if op == 0 else (batch, k, n), dtype)
            c0 = rnd(rng, (batch, n, n), dtype)
            dA, _ = to_dev(a, pad=apad(a.shape[1], aligned, 2))
            for uplo in (0, 1):
                for alpha, beta in [(0.9, -0.35), (1.5, 0.0)]:
                    if not herm and dt in "cz":
                        alpha, beta = alpha + 0.25j, beta * (1 + 0.5j)
                    c_in = c0.copy()
                    if beta == 0:  # C is not an input at all then
                        mask_ref = np.tril(np.ones((n, n), bool)) if uplo == 1 else np.triu(np.ones((n, n), bool))
                        c_in[:, mask_ref] = np.nan
                    if herm:  # the imaginary part of a Hermitian diagonal is not an input either
                        diag = c_in[:, idx, idx].copy()
                        diag.imag = np.nan
                        c_in[:, idx, idx] = diag
                    dC, backC = to_dev(c_in, pad=apad(n, aligned, 3))
                    bl.syrk(dA, dC, alpha, beta, uplo, op, hermitian=herm)
                    got = from_dev(dC)
                    exact, bound, mask = L.syrk_exact(a, c_in, alpha, beta, uplo, op, herm)
                    ok, worst = L.within(got, exact, bound, k, dtype, mask)
                    assert ok, f"herm={herm} op={op} uplo={uplo} beta={beta} worst {worst:.3g}"
                    # the other triangle and the padding come back bit-identical
                    assert np.ascontiguousarray(got[:, ~mask]).tobytes() == np.ascontiguousarray(c_in[:, ~mask]).tobytes()
                    assert bool((backC[:, :, n:] == 7.0).all())
                    if herm:
                        assert np.all(got[:, idx, idx].imag == 0), "herk left an imaginary part on the diagonal"


@pytest.mark.parametrize("aligned", [False, True], ids=["oddld", "alignedld"])
@pytest.mark.parametrize("dt", "sdcz")
@pytest.mark.parametrize("shape", [(48, 20, 3), (65, 40, 2), (130, 70, 2), (5, 3, 4)], ids=str)
def test_syr2k_her2k(bl, dt, shape, aligned):
    dtype = NP_DT[dt]
    n, k, batch = shape
    rng = np.random.default_rng(400 + n)
    idx = np.arange(n)
    for herm in ([False, True] if dt in "cz" else [False]):
        for op in ((0, 2) if herm else (0, 1)):
            shp = (batch, n, k) if op == 0 else (batch, k, n)
            a, b, c0 = rnd(rng, shp, dtype), rnd(rng, shp, dtype), rnd(rng, (batch, n, n), dtype)
            dA, _ = to_dev(a, pad=apad(shp[1], aligned, 1))
            dB, _ = to_dev(b, pad=apad(shp[1], aligned, 2))
            for uplo in (0, 1):
                for alpha, beta in [(0.9, -0.35), (1.5, 0.0)]:
                    if dt in "cz":
                        alpha = alpha - 0.4j
                        if not herm:
                            beta = beta * (1 + 0.5j)
                    c_in = c0.copy()
                    if beta == 0:
                        mask_ref = np.tril(np.ones((n, n), bool)) if uplo == 1 else np.triu(np.ones((n, n), bool))
                        c_in[:, mask_ref] = np.nan
                    if herm:
                        diag = c_in[:, idx, idx].copy()
                        diag.imag = np.nan
                        c_in[:, idx, idx] = diag
                    dC, backC = to_dev(c_in, pad=apad(n, aligned, 3))
                    bl.syr2k(dA, dB, dC, alpha, beta, uplo, op, hermitian=herm)
                    got = from_dev(dC)
                    exact, bound, mask = L.syr2k_exact(a, b, c_in, alpha, beta, uplo, op, herm)
                    ok, worst = L.within(got, exact, bound, 2 * k, dtype, mask)
                    assert ok, f"herm={herm} op={op} uplo={uplo} beta={beta} worst {worst:.3g}"
                    assert np.ascontiguousarray(got[:, ~mask]).tobytes() == np.ascontiguousarray(c_in[:, ~mask]).tobytes()
                    assert bool((backC[:, :, n:] == 7.0).all())
                    if herm:
                        assert np.all(got[:, idx, idx].imag == 0)


def test_herk_triangles_agree_across_uplo(bl):
    """A*A^H is Hermitian: what Lower writes below the diagonal is the conjugate of what Upper writes
    above it (tests/herk_tests.cc:238-280)."""
    rng = np.random.default_rng(11)
    n, k, batch = 65, 40, 4
    a = rnd(rng, (batch, n, k), np.complex128)
    dA, _ = to_dev(a)
    lo, _ = to_dev(np.zeros((batch, n, n), np.complex128))
    up, _ = to_dev(np.zeros((batch, n, n), np.complex128))
    bl.herk(dA, lo, 1.0, 0.0, 1, 0)
    bl.herk(dA, up, 1.0, 0.0, 0, 0)
    l, u = from_dev(lo), from_dev(up)
    assert np.allclose(np.tril(l), np.conj(np.swapaxes(np.triu(u), 1, 2)), rtol=0, atol=1e-12)
    assert np.all(np.triu(l, 1) == 0) and np.all(np.tril(u, -1) == 0)


def test_syrk_needs_no_scratch_on_aligned_operands(bl, lib):
    """16-byte aligned operands go straight to a tile kernel that writes the triangle itself, so the
    scratch may be absent; anything else needs it and says so."""
    rng = np.random.default_rng(23)
    n, k, batch = 160, 96, 3
    a, c0 = rnd(rng, (batch, n, k), np.float64), rnd(rng, (batch, n, n), np.float64)
    dA, _ = to_dev(a)
    dC, _ = to_dev(c0)
    d = bl.make_desc(dA.data_ptr(), 0, dC.data_ptr(), 1, 0, 0, n, n, k, batch, n, 1, n, n * k, 0, n * n, 0.9, -0.35)
    assert lib.blb200_syrk(d, 1, 0, None, 0, torch.cuda.current_stream().cuda_stream) == 0
    exact, bound, mask = L.syrk_exact(a, c0, 0.9, -0.35, 1, 0)
    ok, worst = L.within(from_dev(dC), exact, bound, k, np.float64, mask)
    assert ok, worst
    dA2, _ = to_dev(a, pad=1)  # ld 161: columns no longer 16-byte aligned
    d2 = bl.make_desc(dA2.data_ptr(), 0, dC.data_ptr(), 1, 0, 0, n, n, k, batch, n + 1, 1, n, (n + 1) * k, 0, n * n)
    assert lib.blb200_syrk(d2, 1, 0, None, 0, None) == bl._lib.E_NULL


def test_level3_error_paths(bl, lib):
    a = torch.zeros(2, 8, 8, device="cuda")
    b = torch.zeros(2, 4, 8, device="cuda")
    c = torch.zeros(2, 4, 8, device="cuda")
    need = bl.level3.workspace_bytes(torch.float32, 8, 2)
    assert need == 8 * 8 * 2 * 4
    small = torch.empty(need - 1, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        bl.symm(a, b, c, workspace=small)
    d = bl.make_desc(a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, 0, 0, 8, 4, 8, 2, 8, 8, 8, 64, 32, 32)
    assert lib.blb200_symm(d, 0, 1, 0, small.data_ptr(), need - 1, None) == bl._lib.E_TOO_LARGE
    assert lib.blb200_symm(d, 0, 1, 0, None, need, None) == bl._lib.E_NULL
    assert lib.blb200_symm(d, 0, 1, 1, small.data_ptr(), need, None) == bl._lib.E_DTYPE  # real hemm
    assert lib.blb200_symm(d, 2, 1, 0, small.data_ptr(), need, None) == bl._lib.E_DTYPE
    assert lib.blb200_trmm(d, 0, 1, 0, small.data_ptr(), need - 1, None) == bl._lib.E_TOO_LARGE
    assert lib.blb200_syrk(d, 1, 0, small.data_ptr(), 0, None) == bl._lib.E_TOO_LARGE
    with pytest.raises(RuntimeError, match="SYMM: incompatible matrix dimensions"):
        bl.symm(a, b, c, side=1)
    with pytest.raises(RuntimeError, match="TRMM: A must be square"):
        bl.trmm(b, b, c)
    with pytest.raises(RuntimeError, match="SYRK: C must be square"):
        bl.syrk(a, c)
    with pytest.raises(TypeError):
        bl.herk(a, a)
    torch.cuda.synchronize()


def test_symm_large_batch_runs_on_a_tuned_kernel(bl):
    """n = 128, batch 64, float (tests/symm_tests.cc:120-140): after the expansion the product is an
    ordinary aligned batched gemm, so it must land on a tile kernel, not the generic one."""
    rng = np.random.default_rng(17)
    n, batch = 128, 64
    a, b, c0 = (rnd(rng, (batch, n, n), np.float32) for _ in range(3))
    dA, _ = to_dev(a)
    dB, _ = to_dev(b)
    for side in (0, 1):
        dC, _ = to_dev(c0)
        bl.symm(dA, dB, dC, 1.1, -0.3, side, 1)
        assert bl.last_kernel_name() != "generic"
        exact, bound = L.symm_exact(a, b, c0, 1.1, -0.3, side, 1)
        ok, worst = L.within(from_dev(dC), exact, bound, n, np.float32)
        assert ok, worst
