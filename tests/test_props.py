"""The full-size checksum property (tests/_props.py) pinned on CPU against the oracle: it accepts the
oracle's own result for every dtype and op pair, and it notices one wrong entry, a dropped k-slice
and two swapped items."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tests import _props  # noqa: E402
from tests._cases import DTYPE_NAMES, make_inputs, scalar_for  # noqa: E402


def _views(p, A, B, C):
    ar, ac = p.a_shape
    br, bc = p.b_shape
    tA = _props.strided_view(torch, torch.from_numpy(A), ar, ac, p.lda, p.stride_a, p.batch)
    tB = _props.strided_view(torch, torch.from_numpy(B), br, bc, p.ldb, p.stride_b, p.batch)
    tC = _props.strided_view(torch, torch.from_numpy(C), p.m, p.n, p.ldc, p.stride_c, p.batch)
    return tA, tB, tC


@pytest.mark.parametrize("dt", DTYPE_NAMES)
@pytest.mark.parametrize("ops", ["NN", "NT", "TN", "TT", "CN", "NC", "CC"])
def test_checksum_accepts_the_oracle_and_rejects_corruption(dt, ops):
    code = oracle.DTYPES[dt]
    m, n, k, batch = 24, 20, 36, 5
    ar = m if ops[0] == "N" else k
    br = k if ops[1] == "N" else n
    p = oracle.make_problem(dt, ops[0], ops[1], m, n, k, batch, lda=ar + 2, ldb=br + 4, ldc=m + 2,
                            alpha=scalar_for(code, 1.5), beta=scalar_for(code, -0.5))
    A, B, C0 = make_inputs(p)
    C = C0.copy()
    oracle.gemm_netlib(p, A, B, C, provider=0)
    tA, tB, tC0 = _views(p, A, B, C0)
    before = _props.sums_before(torch, tC0)
    letter = dt
    _, _, tC = _views(p, A, B, C)
    bad, worst = _props.checksum_check(torch, tA, tB, tC, ops[0], ops[1], p.alpha, p.beta, k, letter, before)
    assert bad == 0 and worst < 1.0, worst

    wrong = C.copy()
    wrong[2 * p.stride_c + 3 * p.ldc + 1] += 1.0          # one entry of item 2
    _, _, tW = _views(p, A, B, wrong)
    bad, _ = _props.checksum_check(torch, tA, tB, tW, ops[0], ops[1], p.alpha, p.beta, k, letter, before)
    assert bad == 1

    swapped = C.copy()                                      # items 0 and 1 exchanged
    swapped[:p.stride_c], swapped[p.stride_c:2 * p.stride_c] = C[p.stride_c:2 * p.stride_c], C[:p.stride_c]
    _, _, tS = _views(p, A, B, swapped)
    bad, _ = _props.checksum_check(torch, tA, tB, tS, ops[0], ops[1], p.alpha, p.beta, k, letter, before)
    assert bad == 2


def test_checksum_with_beta_zero_ignores_nan_in_old_c():
    p = oracle.make_problem("d", "N", "N", 16, 16, 16, 3, alpha=1.0, beta=0.0)
    A, B, C0 = make_inputs(p, tail=0)
    C0[:] = np.nan
    C = C0.copy()
    oracle.gemm_netlib(p, A, B, C, provider=0)
    tA, tB, tC0 = _views(p, A, B, C0)
    _, _, tC = _views(p, A, B, C)
    bad, worst = _props.checksum_check(torch, tA, tB, tC, "N", "N", 1.0, 0.0, 16, "d", _props.sums_before(torch, tC0))
    assert bad == 0 and worst < 1.0
