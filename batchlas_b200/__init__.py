"""batchlas_b200 — B200 (sm_100a) batched GEMM behind BatchLAS's gemm call.

The product is `libbatchlas_b200.so` (hand-written CUDA kernels + a C ABI, see include/blb200.h);
this package is its Python host side: a ctypes binding (`_lib`), a torch-tensor convenience layer
over device memory (`gemm`, and `level3` for the symm/hemm/trmm/syrk/herk calls that run on the
same kernels, `linalg` for gemv and the elementwise helpers), and the batch-sharding helper used for multi-GPU runs (`sharding`).
"""
from . import _lib
from . import linalg
from ._lib import BlasError, GemmDesc, KERNEL_IDS
from .gemm import (DTYPE_CODES, Transpose, device_status, fill, gemm, gemm_host, gemm_host_multi, gemm_strided_batched,
                   last_kernel_name, launch_count, make_desc, measure_pipe_peak)
from .level3 import Diag, Side, Uplo, hemm, her2k, herk, symm, syr2k, syrk, trmm
from .sharding import shard_range

__all__ = ["_lib", "BlasError", "GemmDesc", "KERNEL_IDS", "DTYPE_CODES", "Transpose", "device_status",
           "fill", "gemm", "gemm_host", "gemm_host_multi", "gemm_strided_batched", "last_kernel_name", "launch_count",
           "make_desc", "measure_pipe_peak", "shard_range", "Side", "Uplo", "Diag", "symm", "hemm", "trmm", "syrk",
           "herk", "syr2k", "her2k", "linalg"]
