"""CPU oracle for the level-3 operations BatchLAS implements through gemm.  TEST INFRASTRUCTURE ONLY:
nothing in the product imports this module.

Two independent statements of each operation:

* ``*_blas``  — the BLAS routine itself (``?symm``, ``?hemm``, ``?trmm``, ``?syrk``, ``?herk``, ``?syr2k``, ``?her2k`` from the
  OpenBLAS that SciPy ships), called once per batch item.  This is what the reference's host
  backend does: a serial loop of ``cblas_?symm`` / ``?hemm`` / ``?herk`` / ``?syrk`` / ``?trmm`` over the
  batch (BatchLAS src/backends/netlib_lapack.cc:333-760).
* ``*_exact`` — the definition written out in extended precision (x87 long double), returning the
  exact result and the magnitude sum ``|alpha|*|A|*|B| + |beta|*|C|`` that scales the tolerance.

All arrays are (batch, rows, cols) NumPy arrays in the mathematical orientation; column-major
storage is the caller's business.  side: 0 = Left, 1 = Right; uplo: 0 = Upper, 1 = Lower;
op: 0 = N, 1 = T, 2 = H (the reference's Side / Uplo / Transpose enumerators).
"""
from __future__ import annotations

import numpy as np

_PREFIX = {np.dtype(np.float32): "s", np.dtype(np.float64): "d", np.dtype(np.complex64): "c",
           np.dtype(np.complex128): "z"}


def _wide(x: np.ndarray) -> np.ndarray:
    return x.astype(np.clongdouble if np.iscomplexobj(x) else np.longdouble)


def apply_op(x: np.ndarray, op: int) -> np.ndarray:
    if op == 0:
        return x
    xt = np.swapaxes(x, -1, -2)
    return np.conj(xt) if op == 2 else xt


def expand_full(a: np.ndarray, uplo: int, hermitian: bool = False) -> np.ndarray:
    """Full matrix whose `uplo` triangle is a's; the other triangle is its (conjugate) transpose.
    For the Hermitian case the stored diagonal's imaginary part is dropped, as BLAS does not
    reference it (the reference: expand_mirrored, src/backends/triangular_expand.hh)."""
    tri = np.tril(a) if uplo == 1 else np.triu(a)
    strict = np.tril(a, -1) if uplo == 1 else np.triu(a, 1)
    other = np.swapaxes(strict, -1, -2)
    if hermitian:
        other = np.conj(other)
        full = tri + other
        idx = np.arange(a.shape[-1])
        full[..., idx, idx] = full[..., idx, idx].real
        return full
    return tri + other


def expand_triangular(a: np.ndarray, uplo: int, unit_diag: bool) -> np.ndarray:
    """The `uplo` triangle of a with zeros elsewhere and, on request, a unit diagonal
    (the reference: expand_triangular, src/backends/triangular_expand.hh)."""
    t = (np.tril(a) if uplo == 1 else np.triu(a)).copy()
    if unit_diag:
        idx = np.arange(a.shape[-1])
        t[..., idx, idx] = 1
    return t


def _mm_exact(x, y):
    return np.matmul(_wide(x), _wide(y)), np.matmul(np.abs(_wide(x)).real, np.abs(_wide(y)).real)


def symm_exact(a, b, c, alpha, beta, side, uplo, hermitian=False):
    """C <- alpha*A*B + beta*C (Left) or alpha*B*A + beta*C (Right)."""
    full = expand_full(a, uplo, hermitian)
    prod, mag = _mm_exact(full, b) if side == 0 else _mm_exact(b, full)
    exact = alpha * prod + (beta * _wide(c) if beta != 0 else 0)
    bound = abs(alpha) * mag + (abs(beta) * np.abs(_wide(c)).real if beta != 0 else 0)
    return exact, bound


def trmm_exact(a, b, alpha, side, uplo, op, unit_diag):
    """C <- alpha*op(tri(A))*B (Left) or alpha*B*op(tri(A)) (Right), out of place."""
    t = apply_op(expand_triangular(a, uplo, unit_diag), op)
    prod, mag = _mm_exact(t, b) if side == 0 else _mm_exact(b, t)
    return alpha * prod, abs(alpha) * mag


def syrk_exact(a, c, alpha, beta, uplo, op, hermitian=False):
    """The `uplo` triangle of C <- alpha*op(A)*op(A)^T|H + beta*C; the other triangle is c's,
    untouched.  Hermitian: alpha, beta real, the diagonal of C is read and written as real."""
    left = apply_op(a, op)
    right = apply_op(left, 2 if hermitian else 1)
    prod, mag = _mm_exact(left, right)
    cw = _wide(c).copy()
    n = c.shape[-1]
    idx = np.arange(n)
    if hermitian:
        cw[..., idx, idx] = cw[..., idx, idx].real
    full = alpha * prod + (beta * cw if beta != 0 else 0)
    if hermitian:
        full[..., idx, idx] = full[..., idx, idx].real
    bound = abs(alpha) * mag + (abs(beta) * np.abs(cw).real if beta != 0 else 0)
    mask = np.tril(np.ones((n, n), bool)) if uplo == 1 else np.triu(np.ones((n, n), bool))
    exact = np.where(mask, full, _wide(c))
    return exact, bound, mask


def syr2k_exact(a, b, c, alpha, beta, uplo, op, hermitian=False):
    """The `uplo` triangle of C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C (syr2k) or
    alpha*op(A)*op(B)^H + conj(alpha)*op(B)*op(A)^H + beta*C (her2k: beta real, diagonal real)."""
    la, lb = apply_op(a, op), apply_op(b, op)
    t = 2 if hermitian else 1
    p1, m1 = _mm_exact(la, apply_op(lb, t))
    p2, m2 = _mm_exact(lb, apply_op(la, t))
    alpha2 = np.conj(alpha) if hermitian else alpha
    cw = _wide(c).copy()
    n = c.shape[-1]
    idx = np.arange(n)
    if hermitian:
        cw[..., idx, idx] = cw[..., idx, idx].real
    full = alpha * p1 + alpha2 * p2 + (beta * cw if beta != 0 else 0)
    if hermitian:
        full[..., idx, idx] = full[..., idx, idx].real
    bound = abs(alpha) * (m1 + m2) + (abs(beta) * np.abs(cw).real if beta != 0 else 0)
    mask = np.tril(np.ones((n, n), bool)) if uplo == 1 else np.triu(np.ones((n, n), bool))
    return np.where(mask, full, _wide(c)), bound, mask


# ---- the BLAS routines themselves -----------------------------------------------------------------
def _blas(name: str, dtype):
    import scipy.linalg.blas as sb
    return getattr(sb, _PREFIX[np.dtype(dtype)] + name)


def symm_blas(a, b, c, alpha, beta, side, uplo, hermitian=False):
    f = _blas("hemm" if hermitian else "symm", c.dtype)
    out = np.empty_like(c)
    for i in range(c.shape[0]):
        out[i] = f(alpha, np.asfortranarray(a[i]), np.asfortranarray(b[i]), beta=beta, c=np.asfortranarray(c[i]),
                   side=side, lower=uplo)
    return out


def trmm_blas(a, b, alpha, side, uplo, op, unit_diag):
    f = _blas("trmm", b.dtype)
    out = np.empty_like(b)
    for i in range(b.shape[0]):
        out[i] = f(alpha, np.asfortranarray(a[i]), np.asfortranarray(b[i]), side=side, lower=uplo, trans_a=op,
                   diag=int(bool(unit_diag)))
    return out


def syrk_blas(a, c, alpha, beta, uplo, op, hermitian=False):
    f = _blas("herk" if hermitian else "syrk", c.dtype)
    out = np.empty_like(c)
    for i in range(c.shape[0]):
        out[i] = f(alpha, np.asfortranarray(a[i]), beta=beta, c=np.asfortranarray(c[i]), trans=op, lower=uplo)
    return out


def syr2k_blas(a, b, c, alpha, beta, uplo, op, hermitian=False):
    f = _blas("her2k" if hermitian else "syr2k", c.dtype)
    out = np.empty_like(c)
    for i in range(c.shape[0]):
        out[i] = f(alpha, np.asfortranarray(a[i]), np.asfortranarray(b[i]), beta=beta, c=np.asfortranarray(c[i]),
                   trans=op, lower=uplo)
    return out


def eps_of(dtype) -> float:
    return float(np.finfo(np.dtype(dtype)).eps)


def within(got, exact, bound, k: int, dtype, mask=None):
    """Entrywise |got - exact| <= 4*k*eps*bound (+ one ulp of slack for the final rounding)."""
    tol = 4.0 * max(k, 1) * eps_of(dtype) * np.asarray(bound, dtype=np.longdouble) + np.finfo(np.dtype(dtype)).tiny
    err = np.abs(_wide(got) - exact)
    ok = err <= tol
    if mask is not None:
        ok = ok | ~mask
    worst = float(np.max(np.where(tol > 0, err / np.maximum(tol, np.finfo(np.longdouble).tiny), 0)))
    return bool(np.all(ok)), worst
