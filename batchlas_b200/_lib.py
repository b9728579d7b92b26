"""ctypes binding of libbatchlas_b200.so (the C ABI declared in include/blb200.h).

There is no CPU fallback: importing this module when the library has not been built raises, and
every compute entry point needs an sm_100 GPU.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbatchlas_b200.so")

S, D, C, Z = 0, 1, 2, 3
OP_N, OP_T, OP_H = 0, 1, 2
K_AUTO, K_GENERIC, K_SMALL32, K_SMALL64, K_TILED, K_DMMA, K_SGEMM128, K_SMALL_RING, K_DMMA_TMA, K_SGEMM_TMA = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9
KERNEL_IDS = {"auto": K_AUTO, "generic": K_GENERIC, "small32": K_SMALL32, "small64": K_SMALL64,
              "tiled": K_TILED, "dmma": K_DMMA, "sgemm128": K_SGEMM128, "small_ring": K_SMALL_RING, "dmma_tma": K_DMMA_TMA, "sgemm_tma": K_SGEMM_TMA}

E_NULL, E_SHAPE, E_DTYPE, E_UNSUPPORTED, E_NO_DEVICE, E_TOO_LARGE, E_INTERNAL = -1, -2, -3, -4, -5, -6, -7


class GemmDesc(ctypes.Structure):
    """Mirror of `blb200_gemm_desc`."""
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p),
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("batch", ctypes.c_int32),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64),
        ("alpha", ctypes.c_double * 2), ("beta", ctypes.c_double * 2),
        ("dtype", ctypes.c_int32), ("op_a", ctypes.c_int32), ("op_b", ctypes.c_int32),
        ("kernel_hint", ctypes.c_int32),
    ]


class Lease(ctypes.Structure):
    """Mirror of `blb200_lease`."""
    _fields_ = [("ptr", ctypes.c_void_p), ("bytes", ctypes.c_size_t), ("block", ctypes.c_size_t),
                ("offset", ctypes.c_size_t), ("seq", ctypes.c_uint64)]


# Every symbol include/blb200.h declares, with its signature.
class GemvDesc(ctypes.Structure):
    """Mirror of blb200_gemv_desc."""
    _fields_ = [("a", ctypes.c_void_p), ("x", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("batch", ctypes.c_int32),
                ("lda", ctypes.c_int64), ("stride_a", ctypes.c_int64),
                ("incx", ctypes.c_int64), ("stride_x", ctypes.c_int64),
                ("incy", ctypes.c_int64), ("stride_y", ctypes.c_int64),
                ("alpha", ctypes.c_double * 2), ("beta", ctypes.c_double * 2),
                ("dtype", ctypes.c_int32), ("op_a", ctypes.c_int32)]


class EwiseDesc(ctypes.Structure):
    """Mirror of blb200_ewise_desc."""
    _fields_ = [("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p),
                ("rows", ctypes.c_int32), ("cols", ctypes.c_int32), ("batch", ctypes.c_int32),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
                ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64),
                ("dtype", ctypes.c_int32)]


SIGNATURES = {
    "blb200_gemm_validate": (ctypes.c_int, [ctypes.POINTER(GemmDesc)]),
    "blb200_gemm_strided_batched": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_void_p]),
    "blb200_gemm_heterogeneous": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p,
                                                 ctypes.c_void_p, ctypes.c_void_p]),
    "blb200_gemm_splitk_plan": (ctypes.c_int32, [ctypes.POINTER(GemmDesc), ctypes.c_int32,
                                                 ctypes.POINTER(ctypes.c_size_t)]),
    "blb200_gemm_splitk": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t,
                                          ctypes.c_void_p]),
    "blb200_gemm_splitk_static_capacity": (ctypes.c_size_t, []),
    "blb200_gemm_splitk_static": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_void_p]),
    "blb200_level3_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
    "blb200_symm": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                   ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "blb200_trmm": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                   ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "blb200_syrk": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                   ctypes.c_size_t, ctypes.c_void_p]),
    "blb200_syr2k": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                    ctypes.c_size_t, ctypes.c_void_p]),
    "blb200_gemv_strided_batched": (ctypes.c_int, [ctypes.POINTER(GemvDesc), ctypes.c_void_p]),
    "blb200_elementwise": (ctypes.c_int, [ctypes.POINTER(EwiseDesc), ctypes.c_int32, ctypes.c_void_p]),
    "blb200_axpby": (ctypes.c_int, [ctypes.POINTER(EwiseDesc), ctypes.POINTER(ctypes.c_double),
                                    ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]),
    "blb200_gemm_strided_batched_host": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.c_int, ctypes.c_int32]),
    "blb200_gemm_strided_batched_host_multi": (ctypes.c_int, [ctypes.POINTER(GemmDesc), ctypes.POINTER(ctypes.c_int32),
                                                              ctypes.c_int32, ctypes.c_int32]),
    "blb200_shard_range": (None, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_int64),
                                  ctypes.POINTER(ctypes.c_int64)]),
    "blb200_host_staging_trim": (ctypes.c_int, [ctypes.c_int]),
    "blb200_last_kernel_name": (ctypes.c_char_p, []),
    "blb200_launch_count": (ctypes.c_uint64, []),
    "blb200_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "blb200_version": (ctypes.c_char_p, []),
    "blb200_trace_flush": (ctypes.c_int, []),
    "blb200_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "blb200_device_status_reset": (ctypes.c_int, []),
    "blb200_selftest_wait_expiry": (ctypes.c_int, [ctypes.c_uint32, ctypes.c_void_p]),
    "blb200_arena_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]),
    "blb200_arena_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "blb200_arena_acquire": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(Lease)]),
    "blb200_arena_release": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Lease)]),
    "blb200_arena_trim": (ctypes.c_int, [ctypes.c_void_p]),
    "blb200_arena_capacity": (ctypes.c_size_t, [ctypes.c_void_p]),
    "blb200_arena_block_count": (ctypes.c_size_t, [ctypes.c_void_p]),
    "blb200_arena_alignment": (ctypes.c_size_t, [ctypes.c_void_p]),
    "blb200_measure_pipe_peak": (ctypes.c_int, [ctypes.c_int32, ctypes.POINTER(ctypes.c_double)]),
    "blb200_fill": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64,
                                   ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_double,
                                   ctypes.c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library (once).  Raises if it has not been built — there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m batchlas_b200.build` "
                "(needs nvcc with sm_100a support). batchlas_b200 has no CPU or eager fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class BlasError(RuntimeError):
    """Raised for a non-zero status; the text matches the reference's for shape errors
    ("GEMM: incompatible matrix dimensions", BatchLAS src/backends/cublas.cc:119-121)."""

    def __init__(self, status: int):
        self.status = status
        super().__init__(load().blb200_status_string(status).decode())


def check(status: int) -> None:
    if status != 0:
        raise BlasError(status)
