"""Pins the CPU oracle (test infrastructure) before anything is compared against it.

Sources of truth, in order: the committed golden vectors (numpy extended precision, see
tests/golden/make_golden.py); the reference's own known-answer tests re-stated here (identity
products, k == 0 scaling, matmul vs a naive triple loop, the configure-time dgemm health check);
agreement between the oracle's two BLAS providers; and the oracle's own long-double arbiter.
"""
import os

import numpy as np
import pytest

from oracle import oracle
from tests._cases import DTYPE_NAMES, EDGE_SHAPES, REFERENCE_SHAPES, make_inputs, scalar_for

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemm_golden.npz")


def golden_cases():
    z = np.load(GOLDEN)
    names = sorted(k[:-5] for k in z.files if k.endswith("_meta"))
    return z, names


def eps_of(code):
    return np.finfo(np.float32).eps if code in (0, 2) else np.finfo(np.float64).eps


@pytest.mark.parametrize("provider", [0, 1])
def test_oracle_matches_golden_vectors(provider):
    if provider == 1 and not oracle.load_cblas():
        pytest.skip("no CBLAS could be bound in this environment")
    z, names = golden_cases()
    assert len(names) >= 8
    for name in names:
        code, oa, ob, m, n, k, batch = (int(v) for v in z[name + "_meta"])
        alpha, beta = z[name + "_scal"]
        p = oracle.make_problem(code, oa, ob, m, n, k, batch, alpha=alpha, beta=beta)
        A, B, C0 = (np.ascontiguousarray(z[name + s]).ravel() for s in ("_A", "_B", "_C0"))
        C = C0.copy()
        assert oracle.gemm_netlib(p, A, B, C, provider=provider) == 0
        got = C.reshape(batch, n, m)
        err = np.abs(got - z[name + "_expect"])
        lim = 4 * max(k, 1) * eps_of(code) * z[name + "_bound"] + 1e-300
        assert np.all(err <= lim), f"{name}: worst ratio {np.max(err / lim):.3g}"
        # the oracle's own arbiter must agree with the golden expectation as well
        bad, worst = oracle.check(p, A, B, C0, C)
        assert bad == 0 and worst <= 1.0, name


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_identity_product_is_exact(dt):
    # A * I == A bit for bit (BatchLAS tests/gemm_tests.cc:355-396: GemmWithIdentityMatrix, BatchedGemm).
    for batch in (1, 3):
        p = oracle.make_problem(dt, "N", "N", 10, 10, 10, batch)
        A, B, C = make_inputs(p, tail=0)
        eye = np.eye(10, dtype=A.dtype).ravel()
        B[:] = np.tile(eye, batch)
        C[:] = np.nan
        assert oracle.gemm_netlib(p, A, B, C) == 0
        assert np.array_equal(C, A)


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_k_zero_scales_c_and_empty_output_is_noop(dt):
    # netlib_lapack.cc:148-158 and gemm_tests.cc:398-586: m*n == 0 -> skip, k == 0 -> C *= beta.
    p = oracle.make_problem(dt, "N", "N", 5, 4, 0, 2, beta=0.5)
    A, B, C = make_inputs(p)
    C0 = C.copy()
    assert oracle.gemm_netlib(p, A, B, C) == 0
    win = np.zeros(C.size, bool)
    for b in range(2):
        for j in range(4):
            win[b * p.stride_c + j * p.ldc: b * p.stride_c + j * p.ldc + 5] = True
    assert np.array_equal(C[win], (C0[win] * C0.dtype.type(0.5)).astype(C0.dtype))
    assert np.array_equal(C[~win], C0[~win])
    p0 = oracle.make_problem(dt, "N", "N", 0, 4, 3, 2)
    A, B, C = make_inputs(p0)
    C0 = C.copy()
    assert oracle.gemm_netlib(p0, A, B, C) == 0
    assert np.array_equal(C, C0)


def test_incompatible_dimensions_are_rejected():
    # gemm_variant.hh:19-44; the reference throws "GEMM: incompatible matrix dimensions".
    L = oracle.lib()
    assert L.oracle_gemm_validate(4, 4, 4, 1, 0, 0, 4, 4, 4) == 1
    assert L.oracle_gemm_validate(-1, 4, 4, 1, 0, 0, 4, 4, 4) == 0
    assert L.oracle_gemm_validate(4, 4, 4, 1, 0, 0, 3, 4, 4) == 0   # lda < rows of A
    assert L.oracle_gemm_validate(4, 4, 8, 1, 1, 0, 4, 8, 4) == 0   # op T: A stored k x m needs lda >= k
    assert L.oracle_gemm_validate(4, 4, 4, 1, 0, 0, 4, 4, 3) == 0   # ldc < m


def test_matmul_against_naive_triple_loop():
    # BatchLAS tests/linalg_layer_tests.cc:120-142 compares matmul with a naive loop at 1e-4.
    p = oracle.make_problem("s", "N", "N", 7, 5, 6, 2)
    A, B, C = make_inputs(p, tail=0)
    assert oracle.gemm_netlib(p, A, B, C) == 0
    for b in range(2):
        for i in range(7):
            for j in range(5):
                ref = sum(float(A[b * 42 + l * 7 + i]) * float(B[b * 30 + j * 6 + l]) for l in range(6))
                assert abs(float(C[b * 35 + j * 7 + i]) - ref) < 1e-4


@pytest.mark.parametrize("provider", [0, 1])
def test_dgemm_health_check(provider):
    # cmake/BatchLASBlasHealthCheck.cmake:33-88: dgemm on sin/cos inputs vs a naive loop,
    # n in {64,128,200,256,512}, max abs error <= 1e-6.  Guards against a broken host BLAS.
    if provider == 1 and not oracle.load_cblas():
        pytest.skip("no CBLAS could be bound in this environment")
    for n in (64, 128, 200, 256):
        i = np.arange(n * n, dtype=np.float64)
        A = np.sin(0.001 * i)
        B = np.cos(0.002 * i)
        C = np.zeros(n * n)
        p = oracle.make_problem("d", "N", "N", n, n, n)
        assert oracle.gemm_netlib(p, A, B, C, provider=provider) == 0
        ref = (A.reshape(n, n).T @ B.reshape(n, n).T).T.ravel()  # column-major product
        assert np.max(np.abs(C - ref)) <= 1e-6


@pytest.mark.parametrize("dt", DTYPE_NAMES)
def test_providers_agree_and_pass_the_acceptance_rule(dt):
    have_cblas = bool(oracle.load_cblas())
    code = oracle.DTYPES[dt]
    for (m, n, k, batch, oa, ob, alpha, beta) in REFERENCE_SHAPES[:7] + EDGE_SHAPES:
        p = oracle.make_problem(dt, oa, ob, m, n, k, batch, lda=0, ldc=m + 3 if m else 0,
                                alpha=scalar_for(code, alpha), beta=scalar_for(code, beta))
        A, B, C0 = make_inputs(p)
        for provider in ([0, 1] if have_cblas else [0]):
            C = C0.copy()
            assert oracle.gemm_netlib(p, A, B, C, provider=provider) == 0
            bad, worst = oracle.check(p, A, B, C0, C)
            assert bad == 0, (dt, m, n, k, oa, ob, provider, worst)
            assert oracle.untouched_outside_window(p, C0, C)


def test_threaded_batch_split_matches_serial_loop():
    p = oracle.make_problem("d", "T", "N", 13, 11, 9, 17, alpha=2.0, beta=0.5)
    A, B, C0 = make_inputs(p)
    C1, C2 = C0.copy(), C0.copy()
    assert oracle.gemm_netlib(p, A, B, C1, threads=1) == 0
    assert oracle.gemm_netlib(p, A, B, C2, threads=4) == 0
    assert np.array_equal(C1, C2)


def test_checker_rejects_a_wrong_answer():
    p = oracle.make_problem("s", "N", "N", 8, 8, 8, 1)
    A, B, C0 = make_inputs(p, tail=0)
    C = C0.copy()
    oracle.gemm_netlib(p, A, B, C)
    assert oracle.check(p, A, B, C0, C)[0] == 0
    C[5] += np.float32(1e-3)
    assert oracle.check(p, A, B, C0, C)[0] == 1
    C[5] = np.nan
    assert oracle.check(p, A, B, C0, C)[0] == 1


def test_seeded_generator_is_shard_invariant():
    full = oracle.fill(0, 1000, 42, 1)
    part = oracle.fill(0, 300, 42, 1, first=500)
    assert np.array_equal(full[500:800], part)
    assert full.min() >= -1.0 and full.max() <= 1.0 and abs(float(full.mean())) < 0.1
    nrm = oracle.fill(1, 20000, 42, 2, "normal")
    assert abs(float(nrm.mean())) < 0.05 and abs(float(nrm.std()) - 1.0) < 0.05
