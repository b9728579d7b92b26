"""Host-side mirror of the calls either side of gemm in a BatchLAS pipeline — ``gemv``, the elementwise
``*_into`` helpers, ``axpby_into``, ``scale`` and ``matmul`` — over torch tensors (device memory and
streams only; the arithmetic runs in the library's own kernels).

Matrices use the convention of :mod:`batchlas_b200.gemm`: a column-major ``rows x cols`` matrix is a
tensor of shape ``(batch, cols, rows)`` (or ``(cols, rows)``) with unit stride along ``rows``.  A batch
of vectors is a tensor of shape ``(batch, size)`` (or ``(size,)``); its strides are the batch stride
and the increment of ``VectorView`` (BatchLAS include/blas/matrix.hh:1320-1380).  Argument meaning
follows ``gemv(ctx, A, X, Y, alpha, beta, transA)`` (include/blas/functions/gemv.hh:22-29) and
``linalg::add_into / subtract_into / multiply_into / divide_into / axpby_into / scale / matmul``
(include/blas/linalg-ops.hh:59-184); shape errors raise the reference's messages
(src/extra/elementwise.cc:31-38).
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import EwiseDesc, GemvDesc, check, load
from .gemm import DTYPE_CODES, Transpose, _as3, gemm


def _ld(t):
    return t.stride(1) if t.shape[1] > 1 else max(t.shape[2], 1, t.stride(1))


def _st(t):
    return t.stride(0) if t.shape[0] > 1 else 0


def _vec(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 1:
        t = t.unsqueeze(0)
    if t.dim() != 2:
        raise ValueError("expected a (batch, size) or (size,) tensor")
    return t


def _stream(stream):
    return torch.cuda.current_stream().cuda_stream if stream is None else stream


def gemv(A, X, Y, alpha=1.0, beta=0.0, transA: Transpose = Transpose.NoTrans, stream=None):
    """Y <- alpha * op(A) * X + beta * Y for every batch item; returns Y.  Asynchronous."""
    A, X, Y = _as3(A), _vec(X), _vec(Y)
    if not (A.is_cuda and X.is_cuda and Y.is_cuda):
        raise RuntimeError("batchlas_b200.gemv needs CUDA tensors; there is no CPU path")
    if not (A.dtype == X.dtype == Y.dtype) or A.dtype not in DTYPE_CODES:
        raise TypeError("A, X, Y must share one of float32/float64/complex64/complex128")
    ta = Transpose(transA)
    m, n = A.shape[2], A.shape[1]
    x_len, y_len = (n, m) if ta == Transpose.NoTrans else (m, n)
    if not (A.shape[0] == X.shape[0] == Y.shape[0]) or X.shape[1] != x_len or Y.shape[1] != y_len:
        raise RuntimeError("GEMV: incompatible dimensions")

    def inc(v):
        return v.stride(1) if v.shape[1] > 1 else 1

    d = GemvDesc()
    d.a, d.x, d.y = A.data_ptr(), X.data_ptr(), Y.data_ptr()
    d.m, d.n, d.batch = m, n, A.shape[0]
    d.lda, d.stride_a = _ld(A), _st(A)
    d.incx, d.stride_x = inc(X), (X.stride(0) if X.shape[0] > 1 else 0)
    d.incy, d.stride_y = inc(Y), (Y.stride(0) if Y.shape[0] > 1 else 0)
    al, be = complex(alpha), complex(beta)
    d.alpha[0], d.alpha[1], d.beta[0], d.beta[1] = al.real, al.imag, be.real, be.imag
    d.dtype, d.op_a = DTYPE_CODES[A.dtype], int(ta)
    with torch.cuda.device(Y.device):
        check(load().blb200_gemv_strided_batched(d, _stream(stream)))
    return Y


def _ewise_desc(where, A, B, C):
    A, B, C = _as3(A), _as3(B), _as3(C)
    if not (A.is_cuda and B.is_cuda and C.is_cuda):
        raise RuntimeError(f"{where} needs CUDA tensors; there is no CPU path")
    if not (A.dtype == B.dtype == C.dtype) or A.dtype not in DTYPE_CODES:
        raise TypeError("operands must share one of float32/float64/complex64/complex128")
    if A.shape != B.shape or A.shape != C.shape:
        raise ValueError(f"{where}: operands must have the same shape")
    d = EwiseDesc()
    d.a, d.b, d.c = A.data_ptr(), B.data_ptr(), C.data_ptr()
    d.rows, d.cols, d.batch = A.shape[2], A.shape[1], A.shape[0]
    d.lda, d.ldb, d.ldc = _ld(A), _ld(B), _ld(C)
    d.stride_a, d.stride_b, d.stride_c = _st(A), _st(B), _st(C)
    d.dtype = DTYPE_CODES[A.dtype]
    return d, C


def _elementwise(op: int, A, B, C, stream):
    d, C3 = _ewise_desc("linalg::elementwise_into", A, B, C)
    with torch.cuda.device(C3.device):
        check(load().blb200_elementwise(d, op, _stream(stream)))
    return C


def add_into(A, B, C, stream=None):
    """C <- A + B."""
    return _elementwise(0, A, B, C, stream)


def subtract_into(A, B, C, stream=None):
    """C <- A - B."""
    return _elementwise(1, A, B, C, stream)


def multiply_into(A, B, C, stream=None):
    """C <- A .* B (Hadamard)."""
    return _elementwise(2, A, B, C, stream)


def divide_into(A, B, C, stream=None):
    """C <- A ./ B."""
    return _elementwise(3, A, B, C, stream)


def axpby_into(alpha, A, beta, B, C, stream=None):
    """C <- alpha*A + beta*B."""
    d, C3 = _ewise_desc("linalg::axpby_into", A, B, C)
    al, be = complex(alpha), complex(beta)
    a2 = (ctypes.c_double * 2)(al.real, al.imag)
    b2 = (ctypes.c_double * 2)(be.real, be.imag)
    with torch.cuda.device(C3.device):
        check(load().blb200_axpby(d, a2, b2, _stream(stream)))
    return C


def scale(A, alpha, stream=None):
    """A <- alpha * A, in place."""
    return axpby_into(alpha, A, 0.0, A, A, stream)


def matmul(A, B, alpha=1.0, transA: Transpose = Transpose.NoTrans, transB: Transpose = Transpose.NoTrans):
    """alpha * op(A) * op(B) as a new column-major tensor (batch, n, m); beta is zero by construction,
    so the fresh storage is never read (linalg::matmul, include/blas/linalg-ops.hh:168-184)."""
    A3, B3 = _as3(A), _as3(B)
    m = A3.shape[2] if Transpose(transA) == Transpose.NoTrans else A3.shape[1]
    n = B3.shape[1] if Transpose(transB) == Transpose.NoTrans else B3.shape[2]
    C = torch.empty((A3.shape[0], n, m), dtype=A3.dtype, device=A3.device)
    gemm(A3, B3, C, alpha, 0.0, transA, transB)
    return C
