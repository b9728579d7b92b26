"""Host-side mirror of BatchLAS's gemm call over torch tensors (device memory and streams only;
torch does no arithmetic here).

A column-major ``rows x cols`` matrix with leading dimension ``ld`` and batch stride ``stride`` is
passed as a tensor ``t`` of shape ``(batch, cols, rows)`` (or ``(cols, rows)``) with
``t.stride() == (stride, ld, 1)``: ``t[b, j, i]`` is element (i, j) of item b — the addressing rule
of ``MatrixView`` (BatchLAS include/blas/matrix.hh:765-800).  `col_major_view` builds such a tensor
from a flat buffer.

``gemm(A, B, C, alpha, beta, transA, transB)`` has the argument meaning of
``batchlas::gemm(ctx, A, B, C, {.alpha, .beta, .transA, .transB})`` (BatchLAS
include/blas/options.hh:39-46,210-222): C <- alpha*op(A)*op(B) + beta*C, asynchronous on the current
stream, shape errors raise with the reference's message.
"""
from __future__ import annotations

import enum

import torch

from . import _lib
from ._lib import GemmDesc, KERNEL_IDS, check, load


class Transpose(enum.IntEnum):
    """Same ordinals as batchlas::Transpose (BatchLAS include/blas/enums.hh:78-82)."""
    NoTrans = 0
    Trans = 1
    ConjTrans = 2


DTYPE_CODES = {torch.float32: _lib.S, torch.float64: _lib.D, torch.complex64: _lib.C, torch.complex128: _lib.Z}


def col_major_view(buf: torch.Tensor, rows: int, cols: int, ld: int = 0, stride: int = 0, batch: int = 1,
                   offset: int = 0) -> torch.Tensor:
    """View of flat `buf` as `batch` column-major rows x cols matrices; ld/stride default the way
    MatrixView's constructor does (ld = rows, stride = ld*cols; BatchLAS src/matrix.cc:1554-1560)."""
    ld = ld or max(rows, 1)
    stride = stride or ld * cols
    return torch.as_strided(buf, (batch, cols, rows), (stride, ld, 1), storage_offset=buf.storage_offset() + offset)


def _as3(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if t.dim() != 3:
        raise ValueError("expected a (batch, cols, rows) or (cols, rows) tensor")
    if t.shape[2] > 1 and t.stride(2) != 1:
        raise ValueError("rows must be contiguous (column-major storage)")
    return t


def make_desc(a_ptr: int, b_ptr: int, c_ptr: int, dtype: int, op_a: int, op_b: int, m: int, n: int, k: int,
              batch: int, lda: int, ldb: int, ldc: int, stride_a: int, stride_b: int, stride_c: int,
              alpha=1.0, beta=0.0, kernel: str | int = "auto") -> GemmDesc:
    d = GemmDesc()
    d.a, d.b, d.c = a_ptr, b_ptr, c_ptr
    d.m, d.n, d.k, d.batch = m, n, k, batch
    d.lda, d.ldb, d.ldc = lda, ldb, ldc
    d.stride_a, d.stride_b, d.stride_c = stride_a, stride_b, stride_c
    al, be = complex(alpha), complex(beta)
    d.alpha[0], d.alpha[1] = al.real, al.imag
    d.beta[0], d.beta[1] = be.real, be.imag
    d.dtype, d.op_a, d.op_b = dtype, int(op_a), int(op_b)
    d.kernel_hint = KERNEL_IDS[kernel] if isinstance(kernel, str) else int(kernel)
    return d


def _desc_from_tensors(A, B, C, alpha, beta, transA, transB, kernel) -> GemmDesc:
    A, B, C = _as3(A), _as3(B), _as3(C)
    if not (A.dtype == B.dtype == C.dtype) or A.dtype not in DTYPE_CODES:
        raise TypeError("A, B, C must share one of float32/float64/complex64/complex128")
    ta, tb = Transpose(transA), Transpose(transB)
    a_rows, a_cols = A.shape[2], A.shape[1]
    b_rows, b_cols = B.shape[2], B.shape[1]
    m, k = (a_rows, a_cols) if ta == Transpose.NoTrans else (a_cols, a_rows)
    kb, n = (b_rows, b_cols) if tb == Transpose.NoTrans else (b_cols, b_rows)
    # Same checks as gemm_batch_dimensions_compatible (BatchLAS src/backends/gemm_variant.hh:19-44).
    if not (A.shape[0] == B.shape[0] == C.shape[0]) or k != kb or C.shape[2] != m or C.shape[1] != n:
        raise _lib.BlasError(_lib.E_SHAPE)

    def ld_of(t):
        return t.stride(1) if t.shape[1] > 1 else max(t.shape[2], 1, t.stride(1))

    def st_of(t):
        return t.stride(0) if t.shape[0] > 1 else 0

    return make_desc(A.data_ptr(), B.data_ptr(), C.data_ptr(), DTYPE_CODES[A.dtype], ta, tb, m, n, k,
                     A.shape[0], ld_of(A), ld_of(B), ld_of(C), st_of(A), st_of(B), st_of(C), alpha, beta, kernel)


def gemm_strided_batched(desc: GemmDesc, stream: int | None = None) -> None:
    """Raw C-ABI launch (device pointers) on `stream` (a cudaStream_t as int; default: torch's
    current stream)."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    check(load().blb200_gemm_strided_batched(desc, stream))


def gemm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, alpha=1.0, beta=0.0,
         transA: Transpose = Transpose.NoTrans, transB: Transpose = Transpose.NoTrans,
         kernel: str | int = "auto", stream: int | None = None) -> torch.Tensor:
    """C <- alpha*op(A)*op(B) + beta*C on the GPU holding the tensors; returns C.  Asynchronous."""
    if not (A.is_cuda and B.is_cuda and C.is_cuda):
        raise RuntimeError("batchlas_b200.gemm needs CUDA tensors; there is no CPU path (use gemm_host for "
                           "host-resident operands, which still computes on the GPU)")
    desc = _desc_from_tensors(A, B, C, alpha, beta, transA, transB, kernel)
    with torch.cuda.device(C.device):
        gemm_strided_batched(desc, stream)
    return C


def gemm_host(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, alpha=1.0, beta=0.0,
              transA: Transpose = Transpose.NoTrans, transB: Transpose = Transpose.NoTrans,
              device: int = 0, chunk_items: int = 0, kernel: str | int = "auto") -> torch.Tensor:
    """Same operation with HOST tensors (pinned for full speed): chunked H2D -> kernel -> D2H
    pipeline on `device`.  Synchronous; returns C."""
    if A.is_cuda or B.is_cuda or C.is_cuda:
        raise RuntimeError("gemm_host takes host tensors")
    desc = _desc_from_tensors(A, B, C, alpha, beta, transA, transB, kernel)
    check(load().blb200_gemm_strided_batched_host(desc, device, chunk_items))
    return C


def gemm_host_multi(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, alpha=1.0, beta=0.0,
                    transA: Transpose = Transpose.NoTrans, transB: Transpose = Transpose.NoTrans,
                    devices=None, chunk_items: int = 0) -> torch.Tensor:
    """gemm_host over several GPUs of the box in one call: contiguous batch ranges, one host thread
    and one copy/compute pipeline per GPU, each writing its own slice of C.  `devices` defaults to
    every visible GPU.  Synchronous; returns C."""
    import ctypes
    if A.is_cuda or B.is_cuda or C.is_cuda:
        raise RuntimeError("gemm_host_multi takes host tensors")
    if devices is None:
        devices = list(range(torch.cuda.device_count()))
    desc = _desc_from_tensors(A, B, C, alpha, beta, transA, transB, "auto")
    arr = (ctypes.c_int32 * len(devices))(*devices)
    check(load().blb200_gemm_strided_batched_host_multi(desc, arr, len(devices), chunk_items))
    return C


def fill(t: torch.Tensor, seed: int, tensor_id: int, dist: str = "uniform", scale: float = 1.0,
         first_index: int = 0) -> torch.Tensor:
    """Fill contiguous CUDA tensor `t` from the library's counter-based generator."""
    if not t.is_cuda or not t.is_contiguous():
        raise RuntimeError("fill needs a contiguous CUDA tensor")
    with torch.cuda.device(t.device):
        check(load().blb200_fill(t.data_ptr(), DTYPE_CODES[t.dtype], t.numel(), first_index, seed, tensor_id,
                                 {"uniform": 0, "normal": 1}[dist], scale,
                                 torch.cuda.current_stream().cuda_stream))
    return t


def last_kernel_name() -> str:
    return load().blb200_last_kernel_name().decode()


def launch_count() -> int:
    return int(load().blb200_launch_count())


def device_status() -> int:
    import ctypes
    out = ctypes.c_int(0)
    check(load().blb200_device_status(ctypes.byref(out)))
    return out.value


def measure_pipe_peak(dtype: str = "s") -> float:
    """Measured FFMA ("s") or DFMA ("d") issue rate of the current device, TFLOP/s; "dmma" gives the
    FP64 tensor-core (mma.sync m8n8k4) rate."""
    import ctypes
    out = ctypes.c_double(0.0)
    check(load().blb200_measure_pipe_peak({"s": _lib.S, "d": _lib.D, "dmma": _lib.Z, "ffma2": _lib.C, "ffma2_outer": 100 + _lib.C}[dtype], ctypes.byref(out)))
    return out.value
