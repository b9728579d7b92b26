"""Size-independent parity property for the full-size configurations, where the long-double arbiter
(O(mnk) per item on one core) can only sample: the checksum identity

    sum_ij C_new(i,j) = alpha * sum_l (sum_i op(A)(i,l)) * (sum_j op(B)(l,j)) + beta * sum_ij C_old(i,j)

evaluated for EVERY batch item with float64 reductions (torch, on the device that holds the data —
none of the library's own kernels take part).  The tolerance is the entrywise acceptance rule of
the parity tests summed over the item,

    |lhs - rhs| <= 4*K*eps_T * (|alpha| * sum_l (sum_i |op(A)|)(sum_j |op(B)|) + |beta| * sum_ij |C_old|),

so a single wrong tile, a dropped k-chunk or a misplaced item shows up in the item's sum.
TEST INFRASTRUCTURE: used by tests/ and by bench.py's post-timing verification only.
"""
from __future__ import annotations

EPS = {"s": 2.0 ** -23, "c": 2.0 ** -23, "d": 2.0 ** -52, "z": 2.0 ** -52}


def _acc_dtype(torch, t):
    return torch.complex128 if t.is_complex() else torch.float64


def strided_view(torch, flat, rows, cols, ld, stride, batch):
    """(batch, cols, rows) view of a flat column-major buffer: [b, j, i] = element (i, j) of item b."""
    return torch.as_strided(flat, (batch, cols, rows), (stride, ld, 1))


def sums_before(torch, tC):
    """Per-item sum and absolute sum of C before the product overwrites it."""
    acc = _acc_dtype(torch, tC)
    return tC.sum(dim=(1, 2), dtype=acc), tC.abs().sum(dim=(1, 2), dtype=torch.float64)


def checksum_check(torch, tA, tB, tC_new, op_a, op_b, alpha, beta, k, dtype_letter, before):
    """Returns (items beyond the bound, worst |error| / bound) over all batch items.
    tA, tB, tC_new are (batch, cols, rows) views; op_a / op_b in "NTC"; `before` = sums_before(C_old)."""
    acc = _acc_dtype(torch, tA)

    def col_or_row_sums(t, reduce_rows, conj):
        s = t.sum(dim=2 if reduce_rows else 1, dtype=acc)
        s_abs = t.abs().sum(dim=2 if reduce_rows else 1, dtype=torch.float64)
        return (s.conj() if conj and s.is_complex() else s), s_abs

    u, u_abs = col_or_row_sums(tA, op_a == "N", op_a == "C")      # sum over m of op(A): (batch, k)
    v, v_abs = col_or_row_sums(tB, op_b != "N", op_b == "C")      # sum over n of op(B): (batch, k)
    sum_c0, abs_c0 = before
    al, be = complex(alpha), complex(beta)
    if not tA.is_complex():
        al, be = al.real, be.real
    want = al * (u * v).sum(dim=1) + (be * sum_c0 if be != 0 else 0)
    got = tC_new.sum(dim=(1, 2), dtype=acc)
    bound = 4.0 * max(k, 1) * EPS[dtype_letter] * (abs(al) * (u_abs * v_abs).sum(dim=1) + (abs(be) * abs_c0 if be != 0 else 0.0))
    err = (got - want).abs().to(torch.float64)
    # the check's own float64 summation error is far below the bound for every shape used here
    tiny = torch.finfo(torch.float64).tiny
    ratio = err / bound.clamp_min(tiny)
    bad = int((err > bound).sum().item())
    return bad, float(ratio.max().item()) if ratio.numel() else 0.0
