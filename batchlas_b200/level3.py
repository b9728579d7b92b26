"""Host-side mirror of the level-3 calls BatchLAS implements through gemm — ``symm``, ``hemm``,
``trmm``, ``syrk``, ``herk``, ``syr2k``, ``her2k`` — over torch tensors (device memory and streams only).

Tensors use the convention of :mod:`batchlas_b200.gemm`: a column-major ``rows x cols`` matrix is a
tensor of shape ``(batch, cols, rows)`` with unit stride along ``rows``.  Argument meaning follows
the reference's positional overloads (BatchLAS include/blas/functions/symm.hh, hemm.hh, trmm.hh,
syrk.hh, herk.hh); shape errors raise with the reference's messages (src/backends/cublas.cc:190-213,
:513-530, :707-721, :913-935).  The scratch for the expanded triangle / the full product comes from
torch's caching allocator on the current stream unless the caller passes ``workspace=`` (a CUDA
uint8 tensor of at least :func:`workspace_bytes` bytes).
"""
from __future__ import annotations

import enum

import torch

from . import _lib
from ._lib import check, load
from .gemm import DTYPE_CODES, Transpose, _as3, make_desc


class Side(enum.IntEnum):
    """Same ordinals as batchlas::Side (BatchLAS include/blas/enums.hh)."""
    Left = 0
    Right = 1


class Uplo(enum.IntEnum):
    """Same ordinals as batchlas::Uplo."""
    Upper = 0
    Lower = 1


class Diag(enum.IntEnum):
    """Same ordinals as batchlas::Diag."""
    NonUnit = 0
    Unit = 1


def workspace_bytes(dtype: torch.dtype, order: int, batch: int) -> int:
    return int(load().blb200_level3_workspace_bytes(DTYPE_CODES[dtype], order, batch))


def _ld(t):
    return t.stride(1) if t.shape[1] > 1 else max(t.shape[2], 1, t.stride(1))


def _st(t):
    return t.stride(0) if t.shape[0] > 1 else 0


def _prep(*ts):
    ts = [_as3(t) for t in ts]
    if any(not t.is_cuda for t in ts):
        raise RuntimeError("batchlas_b200 level-3 calls need CUDA tensors; there is no CPU path")
    if len({t.dtype for t in ts}) != 1 or ts[0].dtype not in DTYPE_CODES:
        raise TypeError("operands must share one of float32/float64/complex64/complex128")
    return ts


def _scratch(workspace, need: int, device):
    if workspace is None:
        return torch.empty(max(need, 16), dtype=torch.uint8, device=device)
    if not workspace.is_cuda or workspace.dtype != torch.uint8 or workspace.numel() < need:
        raise ValueError(f"workspace must be a CUDA uint8 tensor of at least {need} bytes")
    return workspace


def _stream(stream):
    return torch.cuda.current_stream().cuda_stream if stream is None else stream


def symm(A, B, C, alpha=1.0, beta=0.0, side: Side = Side.Left, uplo: Uplo = Uplo.Lower, *, hermitian=False,
         workspace=None, stream=None):
    """C <- alpha*A*B + beta*C (Left) or alpha*B*A + beta*C (Right); A symmetric (or Hermitian), only
    its `uplo` triangle is read."""
    name = "HEMM" if hermitian else "SYMM"
    A, B, C = _prep(A, B, C)
    if A.shape[1] != A.shape[2]:
        raise RuntimeError(f"{name}: A must be square")
    if not (A.shape[0] == B.shape[0] == C.shape[0]):
        raise RuntimeError(f"{name}: batch size mismatch")
    m, n = C.shape[2], C.shape[1]
    k = m if Side(side) == Side.Left else n
    if A.shape[1] != k or B.shape[2] != m or B.shape[1] != n:
        raise RuntimeError(f"{name}: incompatible matrix dimensions")
    if hermitian and not A.is_complex():
        raise TypeError("HEMM needs a complex dtype")
    d = make_desc(A.data_ptr(), B.data_ptr(), C.data_ptr(), DTYPE_CODES[A.dtype], 0, 0, m, n, k, A.shape[0],
                  _ld(A), _ld(B), _ld(C), _st(A), _st(B), _st(C), alpha, beta)
    with torch.cuda.device(C.device):
        need = workspace_bytes(A.dtype, k, A.shape[0])
        ws = _scratch(workspace, need, C.device)
        check(load().blb200_symm(d, int(side), int(uplo), int(bool(hermitian)), ws.data_ptr(), ws.numel(),
                                 _stream(stream)))
        ws.record_stream(torch.cuda.current_stream())
    return C


def hemm(A, B, C, alpha=1.0, beta=0.0, side: Side = Side.Left, uplo: Uplo = Uplo.Lower, **kw):
    return symm(A, B, C, alpha, beta, side, uplo, hermitian=True, **kw)


def trmm(A, B, C, alpha=1.0, side: Side = Side.Left, uplo: Uplo = Uplo.Lower,
         transA: Transpose = Transpose.NoTrans, diag: Diag = Diag.NonUnit, *, workspace=None, stream=None):
    """C <- alpha*op(tri(A))*B (Left) or alpha*B*op(tri(A)) (Right), out of place."""
    A, B, C = _prep(A, B, C)
    if A.shape[1] != A.shape[2]:
        raise RuntimeError("TRMM: A must be square")
    if not (A.shape[0] == B.shape[0] == C.shape[0]):
        raise RuntimeError("TRMM: batch size mismatch")
    m, n = B.shape[2], B.shape[1]
    k = m if Side(side) == Side.Left else n
    if A.shape[1] != k or C.shape[2] != m or C.shape[1] != n:
        raise RuntimeError("TRMM: incompatible matrix dimensions")
    d = make_desc(A.data_ptr(), B.data_ptr(), C.data_ptr(), DTYPE_CODES[A.dtype], Transpose(transA), 0, m, n, k,
                  A.shape[0], _ld(A), _ld(B), _ld(C), _st(A), _st(B), _st(C), alpha, 0.0)
    with torch.cuda.device(C.device):
        need = workspace_bytes(A.dtype, k, A.shape[0])
        ws = _scratch(workspace, need, C.device)
        check(load().blb200_trmm(d, int(side), int(uplo), int(Diag(diag) == Diag.Unit), ws.data_ptr(), ws.numel(),
                                 _stream(stream)))
        ws.record_stream(torch.cuda.current_stream())
    return C


def syrk(A, C, alpha=1.0, beta=0.0, uplo: Uplo = Uplo.Lower, transA: Transpose = Transpose.NoTrans, *,
         hermitian=False, workspace=None, stream=None):
    """The `uplo` triangle of C <- alpha*op(A)*op(A)^T + beta*C (syrk) or alpha*op(A)*op(A)^H + beta*C
    (herk: alpha, beta real; the diagonal comes out real)."""
    name = "HERK" if hermitian else "SYRK"
    A, C = _prep(A, C)
    if C.shape[1] != C.shape[2]:
        raise RuntimeError(f"{name}: C must be square")
    if A.shape[0] != C.shape[0]:
        raise RuntimeError(f"{name}: batch size mismatch")
    ta = Transpose(transA)
    n = C.shape[2]
    a_rows, a_cols = A.shape[2], A.shape[1]
    expected_n, k = (a_rows, a_cols) if ta == Transpose.NoTrans else (a_cols, a_rows)
    if expected_n != n or k <= 0:
        raise RuntimeError(f"{name}: incompatible matrix dimensions")
    if hermitian:
        if not A.is_complex():
            raise TypeError("HERK needs a complex dtype")
        if ta == Transpose.Trans:
            raise RuntimeError("HERK: transA must be NoTrans or ConjTrans")
        alpha, beta = float(alpha), float(beta)
    elif ta == Transpose.ConjTrans:
        if A.is_complex():
            raise RuntimeError("SYRK: transA must be NoTrans or Trans for complex types")
        ta = Transpose.Trans
    d = make_desc(A.data_ptr(), 0, C.data_ptr(), DTYPE_CODES[A.dtype], ta, 0, n, n, k, A.shape[0],
                  _ld(A), 1, _ld(C), _st(A), 0, _st(C), alpha, beta)
    with torch.cuda.device(C.device):
        need = workspace_bytes(A.dtype, n, A.shape[0])
        ws = _scratch(workspace, need, C.device)
        check(load().blb200_syrk(d, int(uplo), int(bool(hermitian)), ws.data_ptr(), ws.numel(), _stream(stream)))
        ws.record_stream(torch.cuda.current_stream())
    return C


def syr2k(A, B, C, alpha=1.0, beta=0.0, uplo: Uplo = Uplo.Lower, transA: Transpose = Transpose.NoTrans, *,
          hermitian=False, workspace=None, stream=None):
    """The `uplo` triangle of C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C (syr2k) or
    alpha*op(A)*op(B)^H + conj(alpha)*op(B)*op(A)^H + beta*C (her2k: beta real, real diagonal)."""
    name = "HER2K" if hermitian else "SYR2K"
    A, B, C = _prep(A, B, C)
    if C.shape[1] != C.shape[2]:
        raise RuntimeError(f"{name}: C must be square")
    if not (A.shape[0] == B.shape[0] == C.shape[0]):
        raise RuntimeError(f"{name}: batch size mismatch")
    ta = Transpose(transA)
    if hermitian:
        if not A.is_complex():
            raise TypeError("HER2K needs a complex dtype")
        if ta == Transpose.Trans:
            raise RuntimeError("HER2K: transA must be NoTrans or ConjTrans")
        beta = float(beta)
    elif ta == Transpose.ConjTrans:
        if A.is_complex():
            raise RuntimeError("SYR2K: transA must be NoTrans or Trans for complex types")
        ta = Transpose.Trans
    n = C.shape[2]
    no_trans = ta == Transpose.NoTrans
    expected_n, k = (A.shape[2], A.shape[1]) if no_trans else (A.shape[1], A.shape[2])
    b_n, b_k = (B.shape[2], B.shape[1]) if no_trans else (B.shape[1], B.shape[2])
    if expected_n != n or b_n != n or b_k != k or k <= 0:
        raise RuntimeError(f"{name}: incompatible matrix dimensions")
    d = make_desc(A.data_ptr(), B.data_ptr(), C.data_ptr(), DTYPE_CODES[A.dtype], ta, 0, n, n, k, A.shape[0],
                  _ld(A), _ld(B), _ld(C), _st(A), _st(B), _st(C), alpha, beta)
    with torch.cuda.device(C.device):
        need = workspace_bytes(A.dtype, n, A.shape[0])
        ws = _scratch(workspace, need, C.device)
        check(load().blb200_syr2k(d, int(uplo), int(bool(hermitian)), ws.data_ptr(), ws.numel(), _stream(stream)))
        ws.record_stream(torch.cuda.current_stream())
    return C


def her2k(A, B, C, alpha=1.0, beta=0.0, uplo: Uplo = Uplo.Lower, transA: Transpose = Transpose.NoTrans, **kw):
    return syr2k(A, B, C, alpha, beta, uplo, transA, hermitian=True, **kw)


def herk(A, C, alpha=1.0, beta=0.0, uplo: Uplo = Uplo.Lower, transA: Transpose = Transpose.NoTrans, **kw):
    return syrk(A, C, alpha, beta, uplo, transA, hermitian=True, **kw)
