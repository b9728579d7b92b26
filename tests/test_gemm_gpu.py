"""Parity tests proper: the CUDA path, called through the C ABI, against the CPU oracle on the
same seeded inputs.  Acceptance rule (written here because it is the contract):

    |C_gpu - (alpha*S + beta*C0)| <= 4 * K * eps_T * (|alpha| * (|A|*|B|) + |beta| * |C0|)   entrywise

with S and the bound accumulated in long double by the oracle, eps_T = 2^-23 (float, complex<float>)
or 2^-52 (double, complex<double>).  Everything outside the m x n windows of C must come back
bit-identical (padding rows within ldc, stride gaps)."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tests._cases import DTYPE_NAMES, EDGE_SHAPES, REFERENCE_SHAPES, make_inputs, scalar_for  # noqa: E402

pytestmark = pytest.mark.gpu

TORCH_DT = {0: torch.float32, 1: torch.float64, 2: torch.complex64, 3: torch.complex128}


@pytest.fixture(scope="module")
def bl(lib):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    import batchlas_b200
    return batchlas_b200


def run_device(bl, p, A, B, C0, kernel="auto", offset_elems=0):
    """Upload, launch through the C ABI, download.  offset_elems shifts every base pointer to
    exercise unaligned views (slices)."""
    def up(x):
        buf = torch.empty(x.size + offset_elems, dtype=TORCH_DT[p.dtype], device="cuda")
        buf[offset_elems:] = torch.from_numpy(x).cuda()
        return buf
    dA, dB, dC = up(A), up(B), up(C0)
    es = dA.element_size()
    desc = bl.make_desc(dA.data_ptr() + offset_elems * es, dB.data_ptr() + offset_elems * es,
                        dC.data_ptr() + offset_elems * es, p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, p.batch,
                        p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta, kernel)
    bl.gemm_strided_batched(desc)
    torch.cuda.synchronize()
    return dC[offset_elems:].cpu().numpy(), bl.last_kernel_name()


def assert_parity(p, A, B, C0, C, items=None, what=""):
    bad, worst = oracle.check(p, A, B, C0, C, items)
    assert bad == 0, f"{what}: {bad} entries beyond the bound, worst ratio {worst:.3g}"
    assert oracle.untouched_outside_window(p, C0, C), f"{what}: wrote outside the m x n windows"


@pytest.mark.parametrize("dt", DTYPE_NAMES)
@pytest.mark.parametrize("case", REFERENCE_SHAPES + EDGE_SHAPES, ids=lambda c: "x".join(map(str, c[:4])) + c[4] + c[5])
def test_reference_test_shapes_padded(bl, dt, case):
    m, n, k, batch, oa, ob, alpha, beta = case
    code = oracle.DTYPES[dt]
    ar = m if oa == "N" else k
    br = k if ob == "N" else n
    p = oracle.make_problem(dt, oa, ob, m, n, k, batch, lda=ar + 3, ldb=br + 1, ldc=m + 5,
                            alpha=scalar_for(code, alpha), beta=scalar_for(code, beta))
    p.stride_c += 11
    A, B, C0 = make_inputs(p)
    C, kern = run_device(bl, p, A, B, C0)
    assert_parity(p, A, B, C0, C, what=f"{dt} {case} via {kern}")


@pytest.mark.parametrize("dt", DTYPE_NAMES)
@pytest.mark.parametrize("oa", ["N", "T", "C"])
@pytest.mark.parametrize("ob", ["N", "T", "C"])
def test_all_nine_op_pairs_packed_and_generic_agree(bl, dt, oa, ob):
    code = oracle.DTYPES[dt]
    for (m, n, k, batch) in [(32, 32, 32, 5), (64, 64, 64, 3), (48, 40, 24, 2), (128, 64, 96, 2)]:
        p = oracle.make_problem(dt, oa, ob, m, n, k, batch, alpha=scalar_for(code, 1.5), beta=scalar_for(code, -0.5))
        A, B, C0 = make_inputs(p)
        C, kern = run_device(bl, p, A, B, C0)
        assert_parity(p, A, B, C0, C, what=f"{dt} {oa}{ob} {m}x{n}x{k} via {kern}")
        Cg, kg = run_device(bl, p, A, B, C0, kernel="generic")
        assert kg == "generic"
        assert_parity(p, A, B, C0, Cg, what=f"{dt} {oa}{ob} {m}x{n}x{k} via generic")


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_beta_zero_never_reads_c(bl, dt):
    # linalg::matmul hands in uninitialised C on that promise (BatchLAS include/blas/linalg-ops.hh:168-184).
    for (m, n, k, batch) in [(32, 32, 32, 9), (64, 64, 64, 3), (50, 30, 20, 2), (256, 128, 64, 1)]:
        p = oracle.make_problem(dt, "N", "T", m, n, k, batch, alpha=2.0, beta=0.0)
        A, B, C0 = make_inputs(p)
        Cnan = C0.copy()
        Cnan[:] = np.nan
        C, kern = run_device(bl, p, A, B, Cnan)
        assert not np.isnan(C[: p.alloc_len("c")]).any(), kern
        bad, worst = oracle.check(p, A, B, C0, C)
        assert bad == 0, (kern, worst)


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_identity_product_is_exact(bl, dt):
    # BatchLAS tests/gemm_tests.cc:355-396
    for batch in (1, 3):
        p = oracle.make_problem(dt, "N", "N", 10, 10, 10, batch)
        A, B, C0 = make_inputs(p, tail=0)
        B[:] = np.tile(np.eye(10, dtype=A.dtype).ravel(), batch)
        C, _ = run_device(bl, p, A, B, C0)
        assert np.array_equal(C, A)


@pytest.mark.parametrize("dt", ["s", "z"])
def test_unaligned_views_take_a_safe_path(bl, dt):
    # Views can be slices (BatchLAS include/blas/matrix.hh:855-869): base pointers need not be 16-byte
    # aligned and ld need not be a multiple of the vector width; fast paths must decline them.
    for (m, n, k, batch, ld_extra) in [(32, 32, 32, 4, 0), (64, 64, 64, 2, 1), (130, 66, 40, 2, 1)]:
        ar = m
        p = oracle.make_problem(dt, "N", "N", m, n, k, batch, lda=ar + ld_extra, ldb=k + ld_extra,
                                ldc=m + ld_extra, alpha=1.0, beta=1.0)
        A, B, C0 = make_inputs(p)
        C, kern = run_device(bl, p, A, B, C0, offset_elems=1)
        assert_parity(p, A, B, C0, C, what=f"offset view via {kern}")


@pytest.mark.parametrize("dt", ["s", "d", "c"])
def test_unaligned_operands_stay_on_a_tile_kernel(bl, dt):
    """Operands that are only element-aligned (a slice starting one element in, ld = 258: the
    reference's own unaligned case, BatchLAS tests/gemm_tests.cc:320-332) keep a tile kernel and
    only switch its load policy (as src/sycl/gemm/load_policies.hh:18-34 does) — every op pair,
    ragged edges, beta != 0, canaries in the padding."""
    code = oracle.DTYPES[dt]
    ops = ["N", "T"] if dt in "sd" else ["N", "T", "C"]
    for oa in ops:
        for ob in ops:
            for (m, n, k, batch, ld_extra, off) in [(256, 256, 256, 1, 2, 0), (130, 66, 40, 2, 1, 1), (64, 96, 17, 3, 0, 1)]:
                ar = m if oa == "N" else k
                br = k if ob == "N" else n
                p = oracle.make_problem(dt, oa, ob, m, n, k, batch, lda=ar + ld_extra, ldb=br + ld_extra,
                                        ldc=m + ld_extra, alpha=scalar_for(code, 1.5), beta=scalar_for(code, -0.5))
                p.stride_a += 1
                p.stride_c += 3
                A, B, C0 = make_inputs(p)
                C, kern = run_device(bl, p, A, B, C0, offset_elems=off)
                assert kern in ("tiled", "dmma", "sgemm128"), (dt, oa, ob, m, n, k, kern)
                assert_parity(p, A, B, C0, C, what=f"element-aligned {dt} {oa}{ob} {m}x{n}x{k} via {kern}")


@pytest.mark.parametrize("kernel", ["tiled", "dmma"])
@pytest.mark.parametrize("dt", ["d", "z"])
def test_both_fp64_tile_kernels_on_ragged_and_aligned_shapes(bl, kernel, dt):
    """The register-blocked DFMA tiles and the tensor-core DMMA tiles are interchangeable: both must
    meet the bound on every op pair, including ragged edges in m, n and k (the reference's ragged
    case is 200 x 130 x 70, alpha = 2, beta = -1: tests/gemm_tests.cc:1995-2033)."""
    code = oracle.DTYPES[dt]
    ops = ["N", "T"] if dt == "d" else ["N", "T", "C"]
    for oa in ops:
        for ob in ops:
            for (m, n, k, batch, alpha, beta) in [(200, 130, 70, 3, 2.0, -1.0), (128, 64, 96, 2, 1.0, 0.0),
                                                 (66, 34, 6, 2, 1.0, 1.0), (256, 256, 40, 1, 0.5, 0.0)]:
                p = oracle.make_problem(dt, oa, ob, m, n, k, batch, alpha=scalar_for(code, alpha),
                                        beta=scalar_for(code, beta))
                A, B, C0 = make_inputs(p)
                C, kern = run_device(bl, p, A, B, C0, kernel=kernel)
                assert kern == kernel
                assert_parity(p, A, B, C0, C, what=f"{kernel} {dt} {oa}{ob} {m}x{n}x{k}")


@pytest.mark.parametrize("oa", ["N", "T"])
@pytest.mark.parametrize("ob", ["N", "T"])
def test_tma_fed_dmma_tiles(bl, oa, ob):
    """The tensor-map fed DMMA kernel (128-byte swizzled stages, permuted row ownership) on full,
    ragged and tiny shapes, padded even leading dimensions with canaries, stride gaps, many items,
    beta == 0 over NaN and beta != 0; and it must agree with the cp.async DMMA kernel bit for bit
    (same products summed in the same order)."""
    shapes = [(256, 256, 256, 3, 2.0, 0.5, 8), (200, 130, 70, 3, 2.0, -1.0, 2), (64, 64, 16, 5, 1.0, 0.0, 0),
              (66, 34, 6, 2, 1.0, 1.0, 4), (40, 190, 33, 2, -1.5, 0.0, 2), (128, 64, 1, 2, 1.0, 0.5, 0),
              (1024, 96, 48, 1, 1.0, 1.0, 0), (33, 33, 100, 7, 1.0, 0.0, 6)]
    for (m, n, k, batch, alpha, beta, pad) in shapes:
        ar = m if oa == "N" else k
        br = k if ob == "N" else n
        ev = lambda x: x + (x & 1)  # tensor-map strides are multiples of 16 bytes: even ld
        p = oracle.make_problem("d", oa, ob, m, n, k, batch, lda=ev(ar) + pad, ldb=ev(br) + pad, ldc=m + pad + 1,
                                alpha=alpha, beta=beta)
        p.stride_a += 2
        p.stride_b += 4
        p.stride_c += 5
        A, B, C0 = make_inputs(p)
        if beta == 0.0:
            idx = (np.arange(p.batch)[:, None, None] * p.stride_c + np.arange(n)[None, :, None] * p.ldc
                   + np.arange(m)[None, None, :]).ravel()
            C0[idx] = np.nan
        C, kern = run_device(bl, p, A, B, C0, kernel="dmma_tma")
        assert kern == "dmma_tma"
        C0chk = np.where(np.isnan(C0), 0.0, C0) if beta == 0.0 else C0
        bad, worst = oracle.check(p, A, B, C0chk, C)
        assert bad == 0, f"dmma_tma {oa}{ob} {m}x{n}x{k}: worst ratio {worst:.3g}"
        assert oracle.untouched_outside_window(p, C0, C)
        C2, kern2 = run_device(bl, p, A, B, C0, kernel="dmma")
        assert kern2 == "dmma" and np.array_equal(C, C2, equal_nan=True)
    # the dispatcher takes it for plain aligned double problems, and leaves odd ld to the cp.async kernel
    p = oracle.make_problem("d", oa, ob, 128, 128, 64, 2, alpha=1.0, beta=0.0)
    A, B, C0 = make_inputs(p)
    assert run_device(bl, p, A, B, C0)[1] == "dmma_tma"
    p = oracle.make_problem("d", oa, ob, 129, 127, 65, 2, alpha=1.0, beta=0.0)
    A, B, C0 = make_inputs(p)
    C, kern = run_device(bl, p, A, B, C0)
    assert kern in ("dmma", "dmma_tma")
    assert_parity(p, A, B, C0, C, what=f"odd dims via {kern}")
    assert bl.device_status() == 0


@pytest.mark.parametrize("ob", ["N", "T"])
def test_tma_fed_sgemm_tiles(bl, ob):
    """The tensor-map fed float tile kernel (128 x 128 x 32 stages, 16 x 8 blocks, the last warp out of a
    stage refills it) on full, ragged and tiny shapes, k that is and is not a multiple of the stage depth and
    shorter than the ring, padded leading dimensions (multiples of 4 floats) with canaries, stride gaps,
    several items, beta == 0 over NaN and beta != 0; and it must agree with the cp.async kernel of the
    same tile bit for bit (same products in the same order)."""
    shapes = [(256, 256, 256, 3, 2.0, 0.5, 8), (200, 136, 70, 3, 2.0, -1.0, 4), (128, 128, 32, 5, 1.0, 0.0, 0),
              (64, 64, 1, 2, 1.0, 1.0, 4), (68, 196, 33, 2, -1.5, 0.0, 0), (132, 64, 97, 2, 1.0, 0.5, 0),
              (1024, 96, 200, 1, 1.0, 1.0, 0), (260, 300, 129, 2, 1.0, 0.0, 12), (128, 128, 1024, 1, 1.0, 0.0, 0)]
    r4 = lambda x: (x + 3) // 4 * 4  # tensor-map strides are multiples of 16 bytes
    for (m, n, k, batch, alpha, beta, pad) in shapes:
        br = k if ob == "N" else n
        p = oracle.make_problem("s", "N", ob, m, n, k, batch, lda=r4(m) + pad, ldb=r4(br) + pad, ldc=r4(m) + pad,
                                alpha=alpha, beta=beta)
        p.stride_a += 4
        p.stride_b += 8
        p.stride_c += 12
        A, B, C0 = make_inputs(p)
        if beta == 0.0:
            idx = (np.arange(p.batch)[:, None, None] * p.stride_c + np.arange(n)[None, :, None] * p.ldc
                   + np.arange(m)[None, None, :]).ravel()
            C0[idx] = np.nan
        C, kern = run_device(bl, p, A, B, C0, kernel="sgemm_tma")
        assert kern == "sgemm_tma"
        C0chk = np.where(np.isnan(C0), 0.0, C0) if beta == 0.0 else C0
        bad, worst = oracle.check(p, A, B, C0chk, C)
        assert bad == 0, f"sgemm_tma N{ob} {m}x{n}x{k}: worst ratio {worst:.3g}"
        assert oracle.untouched_outside_window(p, C0, C)
        C2, kern2 = run_device(bl, p, A, B, C0, kernel="sgemm128")
        assert kern2 == "sgemm128" and np.array_equal(C, C2, equal_nan=True)
    if ob == "T":
        # A^T B^T runs as the transposed product with a transposing epilogue: ragged in both dimensions,
        # k shorter than the ring and not a multiple of the stage depth, beta on and off, several items
        for (m, n, k, batch, alpha, beta, pad) in [(256, 256, 256, 2, 2.0, 0.5, 8), (200, 136, 70, 3, 2.0, -1.0, 4),
                                                   (64, 68, 1, 2, 1.0, 1.0, 0), (132, 260, 97, 2, -1.5, 0.0, 4),
                                                   (1024, 96, 200, 1, 1.0, 1.0, 0), (68, 516, 129, 2, 1.0, 0.0, 0)]:
            p = oracle.make_problem("s", "T", "T", m, n, k, batch, lda=r4(k) + pad, ldb=r4(n) + pad, ldc=r4(m) + pad,
                                    alpha=alpha, beta=beta)
            p.stride_a += 4
            p.stride_b += 8
            p.stride_c += 12
            A, B, C0 = make_inputs(p)
            if beta == 0.0:
                idx = (np.arange(p.batch)[:, None, None] * p.stride_c + np.arange(n)[None, :, None] * p.ldc
                       + np.arange(m)[None, None, :]).ravel()
                C0[idx] = np.nan
            C, kern = run_device(bl, p, A, B, C0, kernel="sgemm_tma")
            assert kern == "sgemm_tma"
            C0chk = np.where(np.isnan(C0), 0.0, C0) if beta == 0.0 else C0
            bad, worst = oracle.check(p, A, B, C0chk, C)
            assert bad == 0, f"sgemm_tma TT {m}x{n}x{k}: worst ratio {worst:.3g}"
            assert oracle.untouched_outside_window(p, C0, C)
        p = oracle.make_problem("s", "T", "T", 256, 128, 512, 2, alpha=1.0, beta=0.0)
        A, B, C0 = make_inputs(p)
        C, kern = run_device(bl, p, A, B, C0)
        assert kern == "sgemm_tma", kern
        assert_parity(p, A, B, C0, C, what="dispatched TT 256x128x512")
    if ob == "N":
        # A^T B: (even-k, odd-k) partial sums from k-pairs of both operands, four stages, eight warps; odd k,
        # k shorter than the ring, ragged in both dimensions, beta on and off, several items
        for (m, n, k, batch, alpha, beta, pad) in [(256, 256, 256, 2, 2.0, 0.5, 8), (200, 136, 70, 3, 2.0, -1.0, 4),
                                                   (64, 68, 1, 2, 1.0, 1.0, 0), (132, 260, 97, 2, -1.5, 0.0, 4),
                                                   (1024, 96, 203, 1, 1.0, 1.0, 0), (68, 516, 129, 2, 1.0, 0.0, 0),
                                                   (128, 128, 1024, 1, 1.0, 0.0, 0)]:
            p = oracle.make_problem("s", "T", "N", m, n, k, batch, lda=r4(k) + pad, ldb=r4(k) + pad, ldc=r4(m) + pad,
                                    alpha=alpha, beta=beta)
            p.stride_a += 4
            p.stride_b += 8
            p.stride_c += 12
            A, B, C0 = make_inputs(p)
            if beta == 0.0:
                idx = (np.arange(p.batch)[:, None, None] * p.stride_c + np.arange(n)[None, :, None] * p.ldc
                       + np.arange(m)[None, None, :]).ravel()
                C0[idx] = np.nan
            C, kern = run_device(bl, p, A, B, C0, kernel="sgemm_tma")
            assert kern == "sgemm_tma"
            C0chk = np.where(np.isnan(C0), 0.0, C0) if beta == 0.0 else C0
            bad, worst = oracle.check(p, A, B, C0chk, C)
            assert bad == 0, f"sgemm_tma TN {m}x{n}x{k}: worst ratio {worst:.3g}"
            assert oracle.untouched_outside_window(p, C0, C)
        p = oracle.make_problem("s", "T", "N", 256, 128, 512, 2, alpha=1.0, beta=0.0)
        A, B, C0 = make_inputs(p)
        C, kern = run_device(bl, p, A, B, C0)
        assert kern == "sgemm_tma", kern
        assert_parity(p, A, B, C0, C, what="dispatched TN 256x128x512")
    # operands that are only float-aligned are not its business
    p = oracle.make_problem("s", "N", ob, 128, 128, 64, 2, lda=129, alpha=1.0, beta=0.0)
    A, B, C0 = make_inputs(p)
    with pytest.raises(Exception):
        run_device(bl, p, A, B, C0, kernel="sgemm_tma")
    assert bl.device_status() == 0


@pytest.mark.parametrize("oa", ["N", "T", "C"])
@pytest.mark.parametrize("ob", ["N", "T", "C"])
def test_tma_fed_dmma_tiles_complex(bl, oa, ob):
    """The complex<double> form of the tensor-map fed DMMA kernel: all nine op pairs on full, ragged
    and tiny shapes (row counts that are and are not multiples of 8: one grouped copy or eight small
    ones per M-major operand), padded leading dimensions with canaries, stride gaps, beta == 0 over
    NaN; bit-for-bit agreement with the cp.async DMMA kernel."""
    shapes = [(128, 64, 256, 3, 1.0 + 0.5j, 0.0, 0), (70, 50, 37, 3, 2.0 - 1.0j, -1.0 + 0.25j, 3), (64, 64, 8, 4, 1.0, 0.0, 0),
              (36, 20, 5, 2, 1.0, 1.0, 1), (200, 24, 64, 2, -1.5j, 0.5, 2), (33, 129, 19, 2, 1.0, 0.0, 5)]
    for (m, n, k, batch, alpha, beta, pad) in shapes:
        ar = m if oa == "N" else k
        br = k if ob == "N" else n
        p = oracle.make_problem("z", oa, ob, m, n, k, batch, lda=ar + pad, ldb=br + pad, ldc=m + pad + 1,
                                alpha=alpha, beta=beta)
        p.stride_a += 1
        p.stride_b += 2
        p.stride_c += 3
        A, B, C0 = make_inputs(p)
        if beta == 0.0:
            idx = (np.arange(p.batch)[:, None, None] * p.stride_c + np.arange(n)[None, :, None] * p.ldc
                   + np.arange(m)[None, None, :]).ravel()
            C0[idx] = np.nan
        C, kern = run_device(bl, p, A, B, C0, kernel="dmma_tma")
        assert kern == "dmma_tma"
        C0chk = np.where(np.isnan(C0), 0.0, C0) if beta == 0.0 else C0
        bad, worst = oracle.check(p, A, B, C0chk, C)
        assert bad == 0, f"dmma_tma z {oa}{ob} {m}x{n}x{k}: worst ratio {worst:.3g}"
        assert oracle.untouched_outside_window(p, C0, C)
        C2, kern2 = run_device(bl, p, A, B, C0, kernel="dmma")
        assert kern2 == "dmma" and np.array_equal(C, C2, equal_nan=True)
    assert bl.device_status() == 0


@pytest.mark.parametrize("dt", ["s", "d", "c"])
def test_64x64_tiles_of_the_tiled_kernel(bl, dt):
    """The 64 x 64 tile configuration (float below 1024^2, double and complex<float> up to one tile):
    every op pair on full, ragged and tiny-k shapes; float also on shapes of several tiles."""
    code = oracle.DTYPES[dt]
    ops = ["N", "T"] if dt in "sd" else ["N", "T", "C"]
    shapes = [(64, 64, 32, 3, 1.0, 0.0), (48, 48, 48, 2, 1.5, -0.5), (40, 36, 72, 2, 2.0, 1.0), (64, 20, 5, 2, 1.0, 0.5)]
    if dt == "s":
        shapes += [(200, 132, 70, 2, 2.0, -1.0), (320, 100, 64, 1, 1.0, 0.0), (96, 96, 96, 2, 1.0, 1.0)]
    for oa in ops:
        for ob in ops:
            for (m, n, k, batch, alpha, beta) in shapes:
                al = 4 if dt == "s" else 2  # elements per 16 bytes: the tile kernels want aligned columns
                up = lambda rows: (rows + al - 1) // al * al
                p = oracle.make_problem(dt, oa, ob, m, n, k, batch, lda=up(m if oa == "N" else k),
                                        ldb=up(k if ob == "N" else n), ldc=up(m), alpha=scalar_for(code, alpha),
                                        beta=scalar_for(code, beta))
                A, B, C0 = make_inputs(p)
                C, kern = run_device(bl, p, A, B, C0, kernel="tiled")
                assert kern == "tiled"
                assert_parity(p, A, B, C0, C, what=f"tiled {dt} {oa}{ob} {m}x{n}x{k}")


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_small_packed_matrices_of_every_type_through_the_ring(bl, dt):
    """Large batches of packed matrices up to 32 x 32 (complex<double>: 8 x 8), any k up to 64: the
    general whole-matrix-per-warp ring kernel, every op pair, beta on and off, ragged shapes whose
    operands are still multiples of 16 bytes."""
    code = oracle.DTYPES[dt]
    ops = ["N", "T"] if dt in "sd" else ["N", "T", "C"]
    shapes = [(8, 8, 8), (8, 4, 64), (5, 8, 16)]
    if dt != "z":
        shapes += [(16, 16, 16), (12, 20, 28), (16, 4, 64), (32, 32, 16), (24, 24, 24), (32, 20, 36)]
    if dt in "dc":
        shapes += [(32, 32, 32)]
    for oa in ops:
        for ob in ops:
            for (m, n, k) in shapes:
                for alpha, beta in [(1.5, -0.5), (2.0, 0.0)]:
                    batch = 1300
                    p = oracle.make_problem(dt, oa, ob, m, n, k, batch, alpha=scalar_for(code, alpha),
                                            beta=scalar_for(code, beta))
                    A, B, C0 = make_inputs(p)
                    if beta == 0.0:
                        C0[:] = np.nan
                    C, kern = run_device(bl, p, A, B, C0)
                    assert kern == "small_ring", (kern, dt, oa, ob, m, n, k)
                    Cz = np.zeros_like(C0) if beta == 0.0 else C0  # beta == 0: the NaNs must not be read
                    bad, worst = oracle.check(p, A, B, Cz, C, [0, 1, 2, 147, 148, 149, 700, 1297, 1298, 1299])
                    assert bad == 0, f"small_ring {dt} {oa}{ob} {m}x{n}x{k} beta={beta}: worst ratio {worst:.3g}"
                    assert not np.isnan(C[: p.alloc_len("c")].view(np.float32 if dt in "sc" else np.float64)).any()
                    assert oracle.untouched_outside_window(p, C0, C)
    assert bl.device_status() == 0


def test_large_float_tiles_with_packed_fma(bl):
    """sgemm128 (A not transposed, B either way): aligned and ragged shapes, beta on and off; the
    float shapes the reference tunes by hand (256^3 aligned, 200 x 130 x 70 ragged with alpha = 2,
    beta = -1: tests/gemm_tests.cc:1964-2033)."""
    for ob in ["N", "T"]:
        for (m, n, k, batch, alpha, beta) in [(256, 256, 256, 2, 1.0, 0.0), (200, 130, 70, 3, 2.0, -1.0),
                                             (128, 128, 128, 2, 1.0, 1.0), (64, 68, 33, 2, 1.5, 0.0),
                                             (512, 256, 96, 1, 1.0, 0.5), (132, 260, 257, 1, -1.0, 1.0), (196, 132, 76, 2, 2.0, -1.0),
                                             (100, 260, 44, 1, 1.0, 0.0)]:
            p = oracle.make_problem("s", "N", ob, m, n, k, batch, alpha=alpha, beta=beta)
            A, B, C0 = make_inputs(p)
            C, kern = run_device(bl, p, A, B, C0)
            # every shape goes to whichever tile wastes less; an ld that is not a multiple of 4 floats
            # (33, 257, 70 here) only switches the tile kernel's load policy
            # (and from k = 256 on, 16-byte aligned operands take the TMA-fed form of the 128 x 128 tile)
            assert kern in ("sgemm128", "sgemm_tma", "tiled"), kern
            if (m, n, k) == (256, 256, 256):
                assert kern == "sgemm_tma", kern
            if k < 256:
                assert kern != "sgemm_tma", (kern, m, n, k)
            assert_parity(p, A, B, C0, C, what=f"{kern} N{ob} {m}x{n}x{k}")
            C, kern = run_device(bl, p, A, B, C0, kernel="sgemm128")
            assert kern == "sgemm128"
            assert_parity(p, A, B, C0, C, what=f"forced sgemm128 N{ob} {m}x{n}x{k}")
            Cn = C0.copy()
            Cn[:] = np.nan if beta == 0.0 else Cn
            if beta == 0.0:
                C2, _ = run_device(bl, p, A, B, Cn)
                assert not np.isnan(C2[: p.alloc_len("c")]).any()


@pytest.mark.parametrize("size", [32, 64])
@pytest.mark.parametrize("oa", ["N", "T"])
@pytest.mark.parametrize("ob", ["N", "T"])
def test_small_kernel_rings_over_many_items(bl, size, oa, ob):
    """Batch sizes around the SM count and far beyond it walk every ring slot through many rounds;
    a sample of items is checked against the oracle and every item against the generic kernel."""
    rng = np.random.default_rng(size)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    # 6 + r items per SM for r = 1..5: the 64^3 kernel's six warp pairs with a partly filled last round
    tails = [(sms * (6 + r) - (r & 1), 0.0 if r & 1 else -0.5) for r in range(1, 6)] if size == 64 else []
    for batch, beta in [(1, 0.0), (7, -0.5), (147, 0.0), (149, 1.0), (1000, -0.5), (1250, 1.0), (5003, 0.0)] + tails:
        p = oracle.make_problem("s", oa, ob, size, size, size, batch, alpha=1.5, beta=beta)
        A, B, C0 = make_inputs(p)
        C, kern = run_device(bl, p, A, B, C0)
        assert kern == f"small{size}"
        items = sorted(set([0, batch - 1] + [int(x) for x in rng.integers(0, batch, 12)]))
        assert_parity(p, A, B, C0, C, items, what=f"{kern} {oa}{ob} b{batch}")
        Cg, _ = run_device(bl, p, A, B, C0, kernel="generic")
        assert np.allclose(C, Cg, rtol=2e-5, atol=2e-5), f"{kern} {oa}{ob} b{batch} vs generic"


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_heterogeneous_batch_in_one_launch(bl, dt):
    """Per-item active dims inside a common capacity (BatchLAS tests/gemm_tests.cc:398-586: includes an
    item with m == 0 and one with k == 0, which scales C by beta).  Every item is checked against the
    oracle as a batch-1 problem; everything outside the active windows must be untouched."""
    code = oracle.DTYPES[dt]
    cap_m, cap_n, cap_k = 70, 45, 50
    ms = [70, 2, 0, 33, 17, 64]
    ns = [45, 2, 4, 45, 0, 31]
    ks = [50, 3, 3, 0, 9, 50]
    batch = len(ms)
    for oa, ob in [("N", "N"), ("T", "N"), ("N", "C"), ("C", "T")]:
        p = oracle.make_problem(dt, oa, ob, cap_m, cap_n, cap_k, batch, alpha=scalar_for(code, 1.5),
                                beta=scalar_for(code, -0.5))
        A, B, C0 = make_inputs(p)
        dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
        dm, dn, dk = (torch.tensor(v, dtype=torch.int32, device="cuda") for v in (ms, ns, ks))
        desc = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, p.op_a, p.op_b, cap_m, cap_n, cap_k,
                            batch, p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)
        bl._lib.check(bl._lib.load().blb200_gemm_heterogeneous(desc, dm.data_ptr(), dn.data_ptr(), dk.data_ptr(),
                                                               torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        # 16-byte aligned capacities (double, complex here) are taken by a tile kernel, the rest by the generic one
        assert bl.last_kernel_name() in ("generic_hetero", "dmma", "tiled"), bl.last_kernel_name()
        C = dC.cpu().numpy()
        expect_untouched = np.ones(C.size, bool)
        es = A.itemsize
        for b in range(batch):
            pi = oracle.make_problem(dt, oa, ob, ms[b], ns[b], ks[b], 1, lda=p.lda, ldb=p.ldb, ldc=p.ldc,
                                     alpha=p.alpha, beta=p.beta)
            sl = lambda x, st: x[b * st:]
            bad, worst = oracle.check(pi, sl(A, p.stride_a), sl(B, p.stride_b), sl(C0, p.stride_c), sl(C, p.stride_c))
            assert bad == 0, (dt, oa, ob, b, worst)
            for j in range(ns[b]):
                expect_untouched[b * p.stride_c + j * p.ldc: b * p.stride_c + j * p.ldc + ms[b]] = False
        assert np.array_equal(C.view(np.uint8).reshape(C.size, -1)[expect_untouched],
                              C0.view(np.uint8).reshape(C0.size, -1)[expect_untouched])
    # null arrays fall back to the homogeneous dispatcher
    bl._lib.check(bl._lib.load().blb200_gemm_heterogeneous(desc, None, None, None, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert bl.last_kernel_name() != "generic_hetero"


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_heterogeneous_batch_on_the_tile_kernels(bl, dt):
    """Capacities of a tile and more with 16-byte aligned operands: the per-item dims are read by the
    tile kernels themselves (one launch, tiles outside an item's dims return at once).  Includes the
    reference benchmark's pattern of full / half / empty items (benchmarks/gemm_heterogeneous_benchmark.cc:47-97)."""
    code = oracle.DTYPES[dt]
    cap_m, cap_n, cap_k = 160, 136, 72
    ms = [160, 80, 0, 129, 1, 160, 33]
    ns = [136, 68, 0, 136, 136, 0, 7]
    ks = [72, 72, 72, 0, 5, 72, 72]
    batch = len(ms)
    for oa, ob in [("N", "N"), ("T", "N"), ("N", "C"), ("C", "T")]:
        p = oracle.make_problem(dt, oa, ob, cap_m, cap_n, cap_k, batch, alpha=scalar_for(code, 1.5),
                                beta=scalar_for(code, -0.5))
        A, B, C0 = make_inputs(p)
        dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
        dm, dn, dk = (torch.tensor(v, dtype=torch.int32, device="cuda") for v in (ms, ns, ks))
        desc = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, p.op_a, p.op_b, cap_m, cap_n, cap_k,
                            batch, p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)
        bl._lib.check(bl._lib.load().blb200_gemm_heterogeneous(desc, dm.data_ptr(), dn.data_ptr(), dk.data_ptr(),
                                                               torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert bl.last_kernel_name() in ("dmma", "sgemm128", "tiled"), bl.last_kernel_name()
        C = dC.cpu().numpy()
        expect_untouched = np.ones(C.size, bool)
        for b in range(batch):
            pi = oracle.make_problem(dt, oa, ob, ms[b], ns[b], ks[b], 1, lda=p.lda, ldb=p.ldb, ldc=p.ldc,
                                     alpha=p.alpha, beta=p.beta)
            sl = lambda x, st: x[b * st:]
            bad, worst = oracle.check(pi, sl(A, p.stride_a), sl(B, p.stride_b), sl(C0, p.stride_c), sl(C, p.stride_c))
            assert bad == 0, (dt, oa, ob, b, worst)
            for j in range(ns[b]):
                expect_untouched[b * p.stride_c + j * p.ldc: b * p.stride_c + j * p.ldc + ms[b]] = False
        assert np.array_equal(C.view(np.uint8).reshape(C.size, -1)[expect_untouched],
                              C0.view(np.uint8).reshape(C0.size, -1)[expect_untouched])


def run_splitk(bl, p, A, B, C0, splits):
    L = bl._lib.load()
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
    desc = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, p.batch,
                        p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)
    need = ctypes.c_size_t(0)
    used = L.blb200_gemm_splitk_plan(desc, splits, ctypes.byref(need))
    ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
    bl._lib.check(L.blb200_gemm_splitk(desc, splits, ws.data_ptr(), need.value, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return dC.cpu().numpy(), used, need.value, bl.last_kernel_name()


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_split_k_matches_the_oracle(bl, dt):
    """Long-k, few-tile problems computed as side-by-side k chunks into scratch partials plus a
    reduce pass (the reference's experimental split-K, src/sycl/gemm/split_k.hh:52-162)."""
    code = oracle.DTYPES[dt]
    ops = ["N", "T"] if dt in "sd" else ["N", "C"]
    for oa in ops:
        for ob in ops:
            for (m, n, k, batch, splits, beta) in [(64, 48, 1000, 2, 4, 0.5), (33, 17, 515, 1, 7, 0.0),
                                                   (128, 64, 2048, 1, 0, 1.0), (20, 10, 300, 3, 3, -1.0)]:
                p = oracle.make_problem(dt, oa, ob, m, n, k, batch, ldc=m + 3, alpha=scalar_for(code, 1.25),
                                        beta=scalar_for(code, beta))
                A, B, C0 = make_inputs(p)
                C, used, need, kern = run_splitk(bl, p, A, B, C0, splits)
                assert used >= 2 and need > 0 and kern == "splitk", (m, n, k, used, kern)
                assert_parity(p, A, B, C0, C, what=f"splitk {dt} {oa}{ob} {m}x{n}x{k} s={used}")


def test_split_k_plan_declines_when_the_gpu_is_already_full(bl):
    L = bl._lib.load()
    need = ctypes.c_size_t(7)
    d = bl.make_desc(16, 16, 16, 1, 0, 0, 256, 256, 256, 2048, 256, 256, 256, 65536, 65536, 65536)
    assert L.blb200_gemm_splitk_plan(d, 0, ctypes.byref(need)) == 1 and need.value == 0
    d = bl.make_desc(16, 16, 16, 1, 0, 0, 64, 64, 100000, 1, 64, 100000, 64, 0, 0, 0)
    s = L.blb200_gemm_splitk_plan(d, 0, ctypes.byref(need))
    assert 2 <= s <= 64 and need.value == s * 64 * 64 * 8
    # too little scratch is refused, not overrun
    p = oracle.make_problem("d", "N", "N", 64, 64, 4096, 1)
    A, B, C0 = make_inputs(p)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
    desc = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 1, 0, 0, 64, 64, 4096, 1, 64, 4096, 64, 0, 0, 0)
    ws = torch.empty(1024, dtype=torch.uint8, device="cuda")
    assert L.blb200_gemm_splitk(desc, 8, ws.data_ptr(), 1024, None) == bl._lib.E_TOO_LARGE


def test_back_to_back_dependent_launches_keep_stream_order(bl):
    """The 64^3 kernel is launched with programmatic dependent launch: its CTAs may be placed while
    the previous kernel of the stream is still draining.  A chain in which every call consumes the
    previous call's output (and torch kernels write operands in between) must still see finished
    data: X1 = A*B, X2 = X1*B + X1 (in place through beta), X3 = (2*X2)^T-free product X2*X1."""
    batch = 700
    p = oracle.make_problem("s", "N", "N", 64, 64, 64, batch)
    A, B, _ = make_inputs(p, scale=0.125, tail=0)
    A *= np.float32(0.125)
    B *= np.float32(0.125)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    X1 = torch.full_like(dA, float("nan"))
    X2 = torch.empty_like(dA)
    X3 = torch.full_like(dA, float("nan"))

    def call(a, b, c, alpha, beta):
        d = bl.make_desc(a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, 0, 0, 64, 64, 64, batch, 64, 64, 64, 4096, 4096,
                         4096, alpha, beta)
        bl.gemm_strided_batched(d)
        assert bl.last_kernel_name() == "small64"

    for _ in range(3):  # repeated so that launches really queue up behind each other
        call(dA, dB, X1, 1.0, 0.0)
        X2.copy_(X1)                 # torch kernel between two of ours
        call(X1, dB, X2, 1.0, 1.0)   # reads X1 written by the first call, accumulates into the copy
        X2.mul_(2.0)                 # torch kernel writes an operand of the next call
        call(X2, X1, X3, 1.0, 0.0)
    torch.cuda.synchronize()

    a = A.reshape(batch, 64, 64).transpose(0, 2, 1).astype(np.float64)  # math layout [b, row, col]
    b = B.reshape(batch, 64, 64).transpose(0, 2, 1).astype(np.float64)
    x1 = a @ b
    x2 = 2.0 * (x1 @ b + x1)
    x3 = x2 @ x1
    got = X3.cpu().numpy().reshape(batch, 64, 64).transpose(0, 2, 1)
    assert np.allclose(got, x3, rtol=2e-4, atol=1e-6), float(np.max(np.abs(got - x3)))


def test_forced_kernel_that_cannot_run_reports_unsupported(bl):
    p = oracle.make_problem("d", "N", "N", 20, 20, 20, 1)
    A, B, C0 = make_inputs(p)
    with pytest.raises(bl.BlasError) as e:
        run_device(bl, p, A, B, C0, kernel="small32")
    assert e.value.status == bl._lib.E_UNSUPPORTED


def test_tensor_front_end_and_shape_errors(bl):
    # Argument meaning of batchlas::gemm(ctx, A, B, C, {.alpha,.beta,.transA,.transB}).
    from batchlas_b200.gemm import col_major_view
    p = oracle.make_problem("d", "T", "N", 24, 20, 16, 3, alpha=2.0, beta=0.5)
    A, B, C0 = make_inputs(p, tail=0)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
    vA = col_major_view(dA, 16, 24, batch=3)
    vB = col_major_view(dB, 16, 20, batch=3)
    vC = col_major_view(dC, 24, 20, batch=3)
    bl.gemm(vA, vB, vC, alpha=2.0, beta=0.5, transA=bl.Transpose.Trans)
    torch.cuda.synchronize()
    assert_parity(p, A, B, C0, dC.cpu().numpy(), what="tensor front end")
    with pytest.raises(bl.BlasError, match="GEMM: incompatible matrix dimensions"):
        bl.gemm(vA, vB, vC)  # without transA the inner dimensions disagree
    with pytest.raises(RuntimeError):
        bl.gemm(vA.cpu(), vB.cpu(), vC.cpu())  # no CPU path


def test_config_shapes_sampled(bl):
    """The five benchmark configurations at reduced batch, every item checked."""
    cfgs = [
        ("s", "N", "N", 64, 64, 64, 37, 1.0, 0.0, {}, "uniform", "uniform", 1.0),
        ("s", "N", "T", 32, 32, 32, 1000, 1.5, -0.5, {}, "uniform", "uniform", 1.0),
        ("s", "T", "N", 32, 32, 32, 1000, 1.5, -0.5, {}, "uniform", "uniform", 1.0),
        ("d", "N", "N", 256, 256, 256, 3, 2.0, 0.5, dict(lda=264, ldb=264, ldc=264), "normal", "uniform", 1.0),
        ("d", "N", "T", 256, 256, 256, 2, 2.0, 0.5, dict(lda=264, ldb=264, ldc=264), "normal", "uniform", 1.0),
        ("d", "T", "N", 256, 256, 256, 2, 2.0, 0.5, dict(lda=264, ldb=264, ldc=264), "normal", "uniform", 1.0),
        ("d", "T", "T", 256, 256, 256, 2, 2.0, 0.5, dict(lda=264, ldb=264, ldc=264), "normal", "uniform", 1.0),
        ("z", "C", "N", 128, 64, 256, 4, 1.0 + 0.5j, 0.0, {}, "normal", "uniform", 1.0),
        ("d", "N", "N", 1024, 1024, 1024, 1, 1.0, 1.0, {}, "normal", "uniform", 1.0 / 32.0),
    ]
    for dt, oa, ob, m, n, k, batch, alpha, beta, lds, dab, dc, scale in cfgs:
        p = oracle.make_problem(dt, oa, ob, m, n, k, batch, alpha=alpha, beta=beta, **lds)
        A, B, C0 = make_inputs(p, dist_ab=dab, dist_c=dc, scale=scale)
        C, kern = run_device(bl, p, A, B, C0)
        items = None if m < 1024 else [0]
        if m >= 1024:  # the long-double arbiter is O(mnk): check a 96-column slab of the big item
            p_chk = oracle.make_problem(dt, oa, ob, m, 96, k, 1, lda=p.lda, ldb=p.ldb, ldc=p.ldc, alpha=alpha, beta=beta)
            bad, worst = oracle.check(p_chk, A, B, C0, C)
            assert bad == 0, (kern, worst)
            ref = C0.copy()
            assert oracle.gemm_netlib(p, A, B, ref, provider=1 if oracle.load_cblas() else 0) == 0
            assert np.max(np.abs(ref - C)) < 1e-11
        else:
            assert_parity(p, A, B, C0, C, items, what=f"{dt} {oa}{ob} {m}x{n}x{k} via {kern}")


def test_host_buffer_entry_matches_device_entry(bl):
    for (dt, m, n, k, batch, beta, ldc_extra) in [("s", 32, 32, 32, 3000, -0.5, 0), ("d", 48, 40, 24, 50, 0.0, 3),
                                                  ("z", 20, 10, 30, 7, 0.0, 0), ("s", 64, 64, 64, 100, 0.0, 0)]:
        p = oracle.make_problem(dt, "N", "T", m, n, k, batch, ldc=m + ldc_extra, alpha=1.5, beta=beta)
        A, B, C0 = make_inputs(p)
        hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
        hC = torch.from_numpy(C0.copy()).pin_memory()
        desc = bl.make_desc(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), p.dtype, p.op_a, p.op_b, m, n, k, batch,
                            p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)
        for chunk in (0, 7):
            hC.copy_(torch.from_numpy(C0))
            bl._lib.check(bl._lib.load().blb200_gemm_strided_batched_host(desc, 0, chunk))
            assert_parity(p, A, B, C0, hC.numpy(), what=f"host entry {dt} chunk={chunk}")


def test_multi_gpu_host_entry_matches_one_gpu_bit_for_bit(bl):
    """One call over every visible GPU (contiguous batch ranges, no exchange) gives exactly the bytes
    the one-GPU host entry gives, padding and stride gaps included; with one GPU visible the device
    list is [0] and the same comparison still exercises the entry.  Called twice: the second call
    reuses the per-device streams and the library's own staging pool."""
    import ctypes
    ndev = torch.cuda.device_count()
    devices = list(range(ndev))
    L = bl._lib.load()
    for (dt, oa, ob, m, n, k, batch, beta, ldc_extra) in [("s", "N", "T", 32, 32, 32, 4001, -0.5, 0),
                                                         ("d", "T", "N", 72, 40, 56, 37, 0.5, 3),
                                                         ("z", "C", "N", 24, 16, 40, 3, 0.0, 0)]:
        p = oracle.make_problem(dt, oa, ob, m, n, k, batch, ldc=m + ldc_extra, alpha=1.5, beta=beta)
        A, B, C0 = make_inputs(p)
        hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
        hC1 = torch.from_numpy(C0.copy()).pin_memory()
        hCn = torch.from_numpy(C0.copy()).pin_memory()

        def desc(hc):
            return bl.make_desc(hA.data_ptr(), hB.data_ptr(), hc.data_ptr(), p.dtype, p.op_a, p.op_b, m, n, k, batch,
                                p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)
        bl._lib.check(L.blb200_gemm_strided_batched_host(desc(hC1), 0, 0))
        arr = (ctypes.c_int32 * ndev)(*devices)
        for _ in range(2):
            hCn.copy_(torch.from_numpy(C0))
            bl._lib.check(L.blb200_gemm_strided_batched_host_multi(desc(hCn), arr, ndev, 0))
            assert np.array_equal(hCn.numpy().view(np.uint8), hC1.numpy().view(np.uint8)), (dt, ndev)
        assert_parity(p, A, B, C0, hCn.numpy(), what=f"multi-GPU host entry {dt} on {ndev} GPU(s)")
    # more shards than items: the empty shards do nothing
    if ndev > 1:
        p = oracle.make_problem("d", "N", "N", 8, 8, 8, 1, alpha=1.0, beta=0.0)
        A, B, C0 = make_inputs(p, tail=0)
        hA, hB, hC = (torch.from_numpy(x.copy()).pin_memory() for x in (A, B, C0))
        d = bl.make_desc(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), p.dtype, 0, 0, 8, 8, 8, 1, 8, 8, 8, 64, 64, 64)
        bl._lib.check(L.blb200_gemm_strided_batched_host_multi(d, (ctypes.c_int32 * ndev)(*devices), ndev, 0))
        assert_parity(p, A, B, C0, hC.numpy(), what="one item over several GPUs")
    for dev in devices:
        assert L.blb200_host_staging_trim(dev) == 0
    torch.cuda.set_device(0)


def test_device_fill_matches_numpy_statement(bl):
    t = torch.empty(5000, dtype=torch.float32, device="cuda")
    bl.fill(t, 42, 1, "uniform", first_index=123)
    assert np.array_equal(t.cpu().numpy(), oracle.fill(0, 5000, 42, 1, "uniform", first=123))
    z = torch.empty(3000, dtype=torch.complex128, device="cuda")
    bl.fill(z, 7, 4, "normal", scale=0.5)
    ref = oracle.fill(3, 3000, 7, 4, "normal", scale=0.5)
    assert np.allclose(z.cpu().numpy(), ref, rtol=1e-12, atol=1e-14)


def test_device_arena_lifecycle(bl):
    L = bl._lib.load()
    h = ctypes.c_void_p()
    s = torch.cuda.Stream()
    assert L.blb200_arena_create(0, s.cuda_stream, ctypes.byref(h)) == 0
    a, b = bl._lib.Lease(), bl._lib.Lease()
    assert L.blb200_arena_acquire(h, 1 << 20, ctypes.byref(a)) == 0
    assert L.blb200_arena_acquire(h, 1 << 10, ctypes.byref(b)) == 0
    assert a.ptr % 256 == 0 and b.ptr >= a.ptr + (1 << 20)
    cap = L.blb200_arena_capacity(h)
    assert L.blb200_arena_trim(h) == 0
    L.blb200_arena_release(h, ctypes.byref(b))
    L.blb200_arena_release(h, ctypes.byref(a))
    c = bl._lib.Lease()
    assert L.blb200_arena_acquire(h, 1 << 20, ctypes.byref(c)) == 0
    assert c.ptr == a.ptr and L.blb200_arena_capacity(h) == cap  # repeated calls do not grow the arena
    L.blb200_arena_release(h, ctypes.byref(c))
    assert L.blb200_arena_trim(h) == 1 and L.blb200_arena_capacity(h) == 0
    assert L.blb200_arena_destroy(h) == 0


def test_no_wait_was_abandoned(bl):
    assert bl.device_status() == 0
