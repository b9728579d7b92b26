"""ctypes front end of the CPU oracle (liboracle_gemm.so).  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / ``--impl reference`` legs may
import this module.  It restates BatchLAS's host GEMM path
(src/backends/netlib_lapack.cc:108-171) — see oracle_gemm.c for the line-by-line mapping — and
adds the long-double arbiter and the entrywise acceptance rule

    |C_got - (alpha*S + beta*C0)| <= 4*K*eps_T*(|alpha|*(|A|*|B|) + |beta|*|C0|).
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_gemm.so")

DTYPES = {"s": 0, "d": 1, "c": 2, "z": 3}
NP_DTYPES = {0: np.float32, 1: np.float64, 2: np.complex64, 3: np.complex128}
OPS = {"N": 0, "T": 1, "C": 2, "H": 2}

_lib = None
_cblas_state = None  # None = not tried, "" = unavailable, else description


def build(force: bool = False) -> str:
    """Compile oracle_gemm.c with gcc (a few hundred ms).  Returns the library path."""
    src = os.path.join(_HERE, "oracle_gemm.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle_gemm.so"])
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i, i64, vp, dp = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER(ctypes.c_double)
        L.oracle_gemm_validate.argtypes = [i, i, i, i, i, i, i64, i64, i64]
        L.oracle_gemm_validate.restype = i
        L.oracle_load_cblas.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
        L.oracle_load_cblas.restype = i
        L.oracle_cblas_loaded.restype = i
        L.oracle_cblas_set_threads.argtypes = [i]
        L.oracle_cblas_config.restype = ctypes.c_char_p
        L.oracle_gemm_netlib.argtypes = [i, i, i, i, i, i, i, i, dp, vp, i64, i64, vp, i64, i64, dp, vp,
                                         i64, i64, i]
        L.oracle_gemm_netlib.restype = i
        L.oracle_gemm_exact_item.argtypes = [i, i, i, i, i, i, dp, vp, i64, vp, i64, dp, vp, i64, dp, dp, dp]
        L.oracle_gemm_exact_item.restype = None
        L.oracle_check_item.argtypes = [i, i, i, i, vp, i64, dp, dp, dp, dp]
        L.oracle_check_item.restype = i64
        _lib = L
    return _lib


def load_cblas() -> str:
    """Bind the CBLAS that ships inside SciPy (OpenBLAS, LP64, scipy_cblas_?gemm).  Returns a
    description string, or "" when none could be bound (callers then use provider 0)."""
    global _cblas_state
    if _cblas_state is not None:
        return _cblas_state
    _cblas_state = ""
    try:
        import scipy  # noqa: F401

        root = os.path.join(os.path.dirname(scipy.__file__), os.pardir, "scipy.libs")
        for path in sorted(glob.glob(os.path.join(root, "libscipy_openblas-*.so"))):
            if lib().oracle_load_cblas(os.path.abspath(path).encode(), b"scipy_"):
                cfg = lib().oracle_cblas_config() or b""
                _cblas_state = "scipy-openblas: " + cfg.decode(errors="replace").strip()
                break
    except Exception:  # pragma: no cover - scipy absent
        _cblas_state = ""
    return _cblas_state


def _scalar2(x) -> ctypes.Array:
    z = complex(x)
    return (ctypes.c_double * 2)(z.real, z.imag)


@dataclass
class Problem:
    """One strided-batched GEMM in the C-ABI's terms (elements, column-major)."""
    dtype: int
    op_a: int
    op_b: int
    m: int
    n: int
    k: int
    batch: int
    lda: int
    ldb: int
    ldc: int
    stride_a: int
    stride_b: int
    stride_c: int
    alpha: complex
    beta: complex

    @property
    def a_shape(self):  # stored rows, cols
        return (self.m, self.k) if self.op_a == 0 else (self.k, self.m)

    @property
    def b_shape(self):
        return (self.k, self.n) if self.op_b == 0 else (self.n, self.k)

    def alloc_len(self, which: str) -> int:
        """Elements a flat buffer needs for operand `which` ('a','b','c')."""
        ld, st = {"a": (self.lda, self.stride_a), "b": (self.ldb, self.stride_b),
                  "c": (self.ldc, self.stride_c)}[which]
        rows, cols = {"a": self.a_shape, "b": self.b_shape, "c": (self.m, self.n)}[which]
        if self.batch == 0:
            return 0
        last = (cols - 1) * ld + rows if cols > 0 and rows > 0 else 0
        return (self.batch - 1) * st + max(last, 0)


def make_problem(dtype, op_a, op_b, m, n, k, batch=1, lda=0, ldb=0, ldc=0, stride_a=0, stride_b=0,
                 stride_c=0, alpha=1.0, beta=0.0) -> Problem:
    """Defaults follow MatrixView's: ld = stored rows, stride = ld * stored cols
    (BatchLAS src/matrix.cc:1554-1560)."""
    dt = DTYPES[dtype] if isinstance(dtype, str) else int(dtype)
    oa = OPS[op_a] if isinstance(op_a, str) else int(op_a)
    ob = OPS[op_b] if isinstance(op_b, str) else int(op_b)
    ar, ac = (m, k) if oa == 0 else (k, m)
    br, bc = (k, n) if ob == 0 else (n, k)
    lda = lda or max(ar, 1)
    ldb = ldb or max(br, 1)
    ldc = ldc or max(m, 1)
    return Problem(dt, oa, ob, m, n, k, batch, lda, ldb, ldc, stride_a or lda * ac, stride_b or ldb * bc,
                   stride_c or ldc * n, complex(alpha), complex(beta))


def gemm_netlib(p: Problem, A: np.ndarray, B: np.ndarray, C: np.ndarray, provider: int = 0,
                threads: int = 1) -> int:
    """In-place on C (flat arrays of the problem's dtype).  Returns the oracle's status."""
    npdt = NP_DTYPES[p.dtype]
    assert A.dtype == npdt and B.dtype == npdt and C.dtype == npdt
    assert A.size >= p.alloc_len("a") and B.size >= p.alloc_len("b") and C.size >= p.alloc_len("c")
    if provider == 1 and not load_cblas():
        raise RuntimeError("no CBLAS could be bound")
    return lib().oracle_gemm_netlib(provider, p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, p.batch,
                                    _scalar2(p.alpha), A.ctypes.data, p.lda, p.stride_a, B.ctypes.data,
                                    p.ldb, p.stride_b, _scalar2(p.beta), C.ctypes.data, p.ldc,
                                    p.stride_c, threads)


def check(p: Problem, A: np.ndarray, B: np.ndarray, C0: np.ndarray, C_got: np.ndarray, items=None):
    """Apply the acceptance rule to the batch items in `items` (default: all).
    Returns (violations, worst_ratio)."""
    L = lib()
    es = np.dtype(NP_DTYPES[p.dtype]).itemsize
    mn = max(p.m * p.n, 1)
    er = np.empty(mn, np.float64)
    ei = np.empty(mn, np.float64)
    bd = np.empty(mn, np.float64)
    dp = ctypes.POINTER(ctypes.c_double)
    worst = ctypes.c_double(0.0)
    total_bad, worst_all = 0, 0.0
    al, be = _scalar2(p.alpha), _scalar2(p.beta)
    rng = range(p.batch) if items is None else items
    if p.m == 0 or p.n == 0:
        return 0, 0.0
    for b in rng:
        L.oracle_gemm_exact_item(p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, al,
                                 A.ctypes.data + b * p.stride_a * es, p.lda,
                                 B.ctypes.data + b * p.stride_b * es, p.ldb, be,
                                 C0.ctypes.data + b * p.stride_c * es, p.ldc,
                                 er.ctypes.data_as(dp), ei.ctypes.data_as(dp), bd.ctypes.data_as(dp))
        bad = L.oracle_check_item(p.dtype, p.m, p.n, p.k, C_got.ctypes.data + b * p.stride_c * es, p.ldc,
                                  er.ctypes.data_as(dp), ei.ctypes.data_as(dp), bd.ctypes.data_as(dp),
                                  ctypes.byref(worst))
        total_bad += int(bad)
        worst_all = max(worst_all, worst.value)
    return total_bad, worst_all


def untouched_outside_window(p: Problem, C0: np.ndarray, C_got: np.ndarray) -> bool:
    """True when every element of C outside the m x n windows (padding rows within ldc, gaps between
    ldc*n and stride_c, tail) is bit-identical to C0."""
    mask = np.ones(C0.size, dtype=bool)
    if p.m > 0 and p.n > 0:
        col = (np.arange(p.n, dtype=np.int64) * p.ldc)[:, None] + np.arange(p.m, dtype=np.int64)[None, :]
        for b in range(p.batch):
            mask[(b * p.stride_c + col).ravel()] = False
    a = C0.view(np.uint8).reshape(C0.size, -1)[mask]
    g = C_got.view(np.uint8).reshape(C_got.size, -1)[mask]
    return bool(np.array_equal(a, g))


# ---- seeded inputs -------------------------------------------------------------------------
def _mix64(x: np.ndarray) -> np.ndarray:
    """SplitMix64 finaliser on uint64 arrays (wrap-around arithmetic)."""
    x = x.copy()
    with np.errstate(over="ignore"):
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def counter_bits(seed: int, tensor_id: int, first: int, count: int, lane: int = 0) -> np.ndarray:
    """64 random bits per element index; the same function the library's device fill uses."""
    with np.errstate(over="ignore"):
        key = _mix64(np.array([seed], np.uint64) ^ (np.uint64(tensor_id) << np.uint64(32))
                     ^ (np.uint64(lane) << np.uint64(56)))
        idx = np.arange(first, first + count, dtype=np.uint64)
        return _mix64(idx * np.uint64(0x9E3779B97F4A7C15) + key[0])


def _unit(bits: np.ndarray) -> np.ndarray:
    return (bits >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def fill(dtype: int, count: int, seed: int, tensor_id: int, dist: str = "uniform", scale: float = 1.0,
         first: int = 0) -> np.ndarray:
    """uniform: U[-1,1]; normal: N(0,1)*scale (Box-Muller).  Complex: re and im independent."""
    def real_part(lane0):
        if dist == "uniform":
            return 2.0 * _unit(counter_bits(seed, tensor_id, first, count, lane0)) - 1.0
        u1 = _unit(counter_bits(seed, tensor_id, first, count, lane0))
        u2 = _unit(counter_bits(seed, tensor_id, first, count, lane0 + 1))
        return np.sqrt(-2.0 * np.log(1.0 - u1)) * np.cos(2.0 * np.pi * u2) * scale

    npdt = NP_DTYPES[dtype]
    if dtype < 2:
        return real_part(0).astype(npdt)
    out = np.empty(count, npdt)
    out.real = real_part(0)
    out.imag = real_part(2)
    return out
