"""NumPy front end with the call shape of BatchLAS's Python package for this path:

    bl.gemm(a, b, *, alpha=1, beta=0, trans_a="n", trans_b="n", out=None)
    bl.gemm_heterogeneous([a0, a1, ...], [b0, b1, ...])

(BatchLAS python/batchlas/_api.py:287-314, bindings python/batchlas/bindings/ops_blas.cc:339-376;
contract pinned by python/tests/test_batchlas.py:33-44, 65-80, 209-221: `out` is returned when given,
inputs are not modified, `beta != 0` needs `out`.)

Arrays are mathematical row-major (..., rows, cols), 2-D or batched 3-D.  A C-contiguous row-major
matrix X is, read column-major, the matrix X^T with ld = cols, so no repacking is needed:
C = op(A) op(B)  <=>  C^T = op(B)^T op(A)^T, i.e. one column-major GEMM with the operands swapped
and the same transpose flags.  Host arrays go through the library's host-buffer entry point
(chunked upload / kernel / download on the GPU); there is no CPU arithmetic here.
"""
from __future__ import annotations

import ctypes
from typing import Any, Sequence

import numpy as np

from . import _lib
from ._lib import check, load

_NP_CODES = {np.dtype(np.float32): _lib.S, np.dtype(np.float64): _lib.D, np.dtype(np.complex64): _lib.C,
             np.dtype(np.complex128): _lib.Z}
_OPS = {"n": _lib.OP_N, "t": _lib.OP_T, "c": _lib.OP_H, "h": _lib.OP_H}


def available_backends() -> list[str]:
    return ["cuda"]


def _coerce(x: Any, dtype=None) -> np.ndarray:
    arr = np.asarray(x)
    if arr.dtype not in _NP_CODES:
        arr = arr.astype(np.float64 if not np.iscomplexobj(arr) else np.complex128)
    if dtype is not None and arr.dtype != dtype:
        arr = arr.astype(dtype)
    if arr.ndim not in (2, 3):
        raise ValueError("expected a matrix (rows, cols) or a batch (batch, rows, cols)")
    return np.ascontiguousarray(arr)


def _op(flag: str) -> int:
    try:
        return _OPS[flag.lower()]
    except (KeyError, AttributeError):
        raise ValueError(f"transpose flag must be one of n/t/c, got {flag!r}") from None


def _check_backend(backend: str, compute_precision: str) -> None:
    if backend.lower() not in ("auto", "cuda"):
        raise RuntimeError(f"backend {backend!r} is not compiled into this build (only 'cuda')")
    if compute_precision.lower() not in ("default", "f32", "f64"):
        raise RuntimeError("reduced compute precision is not available on this path")


def gemm(a: Any, b: Any, *, alpha: Any = 1, beta: Any = 0, trans_a: str = "n", trans_b: str = "n",
         compute_precision: str = "default", backend: str = "auto", device: int | str | None = None,
         out: Any = None):
    """alpha * op(a) @ op(b) + beta * out, computed on the GPU.  Returns `out` when given."""
    _check_backend(backend, compute_precision)
    A = _coerce(a)
    B = _coerce(b, A.dtype)
    oa, ob = _op(trans_a), _op(trans_b)
    if complex(beta) != 0 and out is None:
        raise ValueError("beta != 0 needs an `out` operand to scale")
    batched = A.ndim == 3 or B.ndim == 3
    A3 = A if A.ndim == 3 else A[None]
    B3 = B if B.ndim == 3 else B[None]
    if A3.shape[0] != B3.shape[0]:
        raise ValueError("GEMM: incompatible matrix dimensions")
    batch = A3.shape[0]
    m, k = (A3.shape[1], A3.shape[2]) if oa == _lib.OP_N else (A3.shape[2], A3.shape[1])
    kb, n = (B3.shape[1], B3.shape[2]) if ob == _lib.OP_N else (B3.shape[2], B3.shape[1])
    if k != kb:
        raise ValueError("GEMM: incompatible matrix dimensions")
    if out is None:
        C3 = np.empty((batch, m, n), dtype=A.dtype)
        result = C3 if batched else C3[0]
    else:
        if not isinstance(out, np.ndarray) or out.dtype != A.dtype or not out.flags.c_contiguous:
            raise ValueError("`out` must be a C-contiguous ndarray of the operands' dtype")
        C3 = out if out.ndim == 3 else out[None]
        if C3.shape != (batch, m, n):
            raise ValueError("GEMM: incompatible matrix dimensions")
        result = out
    if isinstance(device, str):
        device = 0
    # column-major call: C^T (n x m) = op_b(B^T-as-stored) * op_a(A^T-as-stored)
    d = _lib.GemmDesc()
    d.a, d.b, d.c = B3.ctypes.data, A3.ctypes.data, C3.ctypes.data
    d.m, d.n, d.k, d.batch = n, m, k, batch
    d.lda, d.ldb, d.ldc = max(B3.shape[2], 1), max(A3.shape[2], 1), max(n, 1)
    d.stride_a, d.stride_b, d.stride_c = B3.shape[1] * B3.shape[2], A3.shape[1] * A3.shape[2], m * n
    al, be = complex(alpha), complex(beta)
    d.alpha[0], d.alpha[1], d.beta[0], d.beta[1] = al.real, al.imag, be.real, be.imag
    d.dtype, d.op_a, d.op_b, d.kernel_hint = _NP_CODES[A.dtype], ob, oa, 0
    check(load().blb200_gemm_strided_batched_host(d, int(device or 0), 0))
    return result


def gemm_heterogeneous(a: Sequence[Any], b: Sequence[Any], *, alpha: Any = 1, trans_a: str = "n",
                       trans_b: str = "n", backend: str = "auto", device: int | None = None) -> list[np.ndarray]:
    """Products of differently shaped pairs in one launch; returns a Python list of results
    (BatchLAS python/tests/test_batchlas.py:65-80)."""
    import torch

    _check_backend(backend, "default")
    if len(a) != len(b) or len(a) == 0:
        raise ValueError("need equally many, at least one, operands")
    oa, ob = _op(trans_a), _op(trans_b)
    As = [_coerce(x) for x in a]
    dt = np.result_type(*[x.dtype for x in As])
    As = [_coerce(x, dt) for x in As]
    Bs = [_coerce(x, dt) for x in b]
    if any(x.ndim != 2 for x in As + Bs):
        raise ValueError("heterogeneous operands are single matrices")
    dims = []
    for X, Y in zip(As, Bs):
        mi, ki = X.shape if oa == _lib.OP_N else X.shape[::-1]
        kj, ni = Y.shape if ob == _lib.OP_N else Y.shape[::-1]
        if ki != kj:
            raise ValueError("GEMM: incompatible matrix dimensions")
        dims.append((mi, ni, ki))
    batch = len(As)
    ar, ac = max(x.shape[0] for x in As), max(x.shape[1] for x in As)
    br, bc = max(x.shape[0] for x in Bs), max(x.shape[1] for x in Bs)
    cm, cn, ck = max(d[0] for d in dims), max(d[1] for d in dims), max(d[2] for d in dims)
    Ap = np.zeros((batch, ar, ac), dt)
    Bp = np.zeros((batch, br, bc), dt)
    for i, (X, Y) in enumerate(zip(As, Bs)):
        Ap[i, :X.shape[0], :X.shape[1]] = X
        Bp[i, :Y.shape[0], :Y.shape[1]] = Y
    dev = torch.device("cuda", int(device or 0))
    with torch.cuda.device(dev):
        dA, dB = torch.from_numpy(Ap).to(dev), torch.from_numpy(Bp).to(dev)
        dC = torch.zeros((batch, cm, cn), dtype=dA.dtype, device=dev)
        # swapped column-major call (see module docstring): per-item dims are (n_i, m_i, k_i)
        dm = torch.tensor([d[1] for d in dims], dtype=torch.int32, device=dev)
        dn = torch.tensor([d[0] for d in dims], dtype=torch.int32, device=dev)
        dk = torch.tensor([d[2] for d in dims], dtype=torch.int32, device=dev)
        desc = _lib.GemmDesc()
        desc.a, desc.b, desc.c = dB.data_ptr(), dA.data_ptr(), dC.data_ptr()
        desc.m, desc.n, desc.k, desc.batch = cn, cm, ck, batch
        desc.lda, desc.ldb, desc.ldc = max(bc, 1), max(ac, 1), max(cn, 1)
        desc.stride_a, desc.stride_b, desc.stride_c = br * bc, ar * ac, cm * cn
        al = complex(alpha)
        desc.alpha[0], desc.alpha[1] = al.real, al.imag
        desc.dtype, desc.op_a, desc.op_b = _NP_CODES[np.dtype(dt)], ob, oa
        check(load().blb200_gemm_heterogeneous(desc, dm.data_ptr(), dn.data_ptr(), dk.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream))
        C = dC.cpu().numpy()
    return [np.array(C[i, :d[0], :d[1]]) for i, d in enumerate(dims)]
