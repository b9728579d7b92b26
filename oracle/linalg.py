"""CPU oracle for gemv and the elementwise helpers.  TEST INFRASTRUCTURE ONLY: nothing in the product
imports this module.

``gemv_blas`` is the BLAS routine itself (``?gemv`` of the OpenBLAS SciPy ships) called once per batch
item, which is what the reference's host backend does (BatchLAS src/backends/netlib_lapack.cc:174-215);
``gemv_exact`` is the definition in extended precision with the magnitude sum that scales the
tolerance.  The elementwise functions restate src/extra/elementwise.cc:24-29,84-112 (one operation
per element; ``axpby`` always forms both products).

Arrays: matrices (batch, rows, cols), vectors (batch, size), mathematical orientation.
op: 0 = N, 1 = T, 2 = H.
"""
from __future__ import annotations

import numpy as np

from .level3 import _PREFIX, _wide, apply_op, eps_of


def gemv_exact(a, x, y, alpha, beta, op):
    oa = _wide(apply_op(a, op))
    xv = _wide(x)[..., None]
    prod = np.matmul(oa, xv)[..., 0]
    mag = np.matmul(np.abs(oa).real, np.abs(xv).real)[..., 0]
    exact = alpha * prod + (beta * _wide(y) if beta != 0 else 0)
    bound = abs(alpha) * mag + (abs(beta) * np.abs(_wide(y)).real if beta != 0 else 0)
    return exact, bound


def gemv_blas(a, x, y, alpha, beta, op):
    import scipy.linalg.blas as sb
    f = getattr(sb, _PREFIX[np.dtype(y.dtype)] + "gemv")
    out = np.empty_like(y)
    for i in range(y.shape[0]):
        out[i] = f(alpha, np.asfortranarray(a[i]), x[i], beta=beta, y=y[i].copy(), trans=op)
    return out


def gemv_within(got, exact, bound, k, dtype):
    """Entrywise |got - exact| <= 4*max(k,1)*eps*bound."""
    tol = 4.0 * max(k, 1) * eps_of(dtype) * np.asarray(bound, dtype=np.longdouble) + np.finfo(np.dtype(dtype)).tiny
    err = np.abs(_wide(got) - exact)
    worst = float(np.max(err / tol)) if err.size else 0.0
    return bool(np.all(err <= tol)), worst


OPS = ("add", "subtract", "multiply", "divide")


def elementwise_exact(op: str, a, b):
    """(exact result, magnitude that one rounding error is relative to)."""
    wa, wb = _wide(a), _wide(b)
    if op == "add":
        return wa + wb, np.abs(wa) + np.abs(wb)
    if op == "subtract":
        return wa - wb, np.abs(wa) + np.abs(wb)
    if op == "multiply":
        return wa * wb, np.abs(wa) * np.abs(wb)
    if op == "divide":
        return wa / wb, np.abs(wa) / np.abs(wb)
    raise ValueError(op)


def axpby_exact(alpha, a, beta, b):
    wa, wb = _wide(a), _wide(b)
    return alpha * wa + beta * wb, abs(alpha) * np.abs(wa) + abs(beta) * np.abs(wb)


def elementwise_within(got, exact, mag, dtype, ulps=8.0):
    """|got - exact| <= ulps*eps*mag: real add/sub/mul/div are correctly rounded (0.5 ulp); complex
    products and quotients and the two roundings of axpby stay within a few."""
    tol = ulps * eps_of(dtype) * np.asarray(mag, dtype=np.longdouble).real + np.finfo(np.dtype(dtype)).tiny
    err = np.abs(_wide(got) - exact)
    worst = float(np.max(err / tol)) if err.size else 0.0
    return bool(np.all(err <= tol)), worst
