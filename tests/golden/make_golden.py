"""Regenerates tests/golden/gemm_golden.npz.

The reference ships no golden-vector files for gemm and cannot be built or imported in this image
(its sources need a SYCL compiler and CBLAS headers), so these vectors come from an independent
statement of the same operation: numpy's einsum over extended-precision operands
(longdouble / clongdouble), C = alpha*op(A)@op(B) + beta*C.  They pin the C oracle (and through it
the CUDA kernels) against a second implementation that shares no code with it.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402  (only its seeded generator is used here)

CASES = [  # name, dtype, opA, opB, m, n, k, batch, alpha, beta
    ("s_nn_10", "s", "N", "N", 10, 10, 10, 3, 1.0, 0.0),
    ("s_nt_32", "s", "N", "T", 32, 32, 32, 4, 1.5, -0.5),
    ("s_tn_32", "s", "T", "N", 32, 32, 32, 4, 1.5, -0.5),
    ("d_tt_24", "d", "T", "T", 24, 20, 16, 3, 1.0, 0.0),
    ("d_nn_ragged", "d", "N", "N", 50, 34, 19, 2, 2.0, -1.0),
    ("c_cn_18", "c", "C", "N", 18, 14, 12, 2, 1.0 + 0.5j, 0.0),
    ("z_cn_18", "z", "C", "N", 18, 14, 12, 2, 1.0 + 0.5j, 0.25 - 1.0j),
    ("z_nc_9", "z", "N", "C", 9, 11, 7, 2, -0.5 + 2.0j, 1.0),
]


def op(x, o):
    if o == "N":
        return x
    x = np.swapaxes(x, -1, -2)
    return np.conj(x) if o == "C" else x


def main():
    out = {}
    for name, dt, oa, ob, m, n, k, batch, alpha, beta in CASES:
        code = oracle.DTYPES[dt]
        ar, ac = (m, k) if oa == "N" else (k, m)
        br, bc = (k, n) if ob == "N" else (n, k)
        # stored column-major, packed: array[b, col, row]
        A = oracle.fill(code, batch * ar * ac, 42, 1).reshape(batch, ac, ar)
        B = oracle.fill(code, batch * br * bc, 42, 2).reshape(batch, bc, br)
        C = oracle.fill(code, batch * m * n, 42, 3).reshape(batch, n, m)
        wide = np.clongdouble if code >= 2 else np.longdouble
        Am = op(np.swapaxes(A, 1, 2).astype(wide), oa)  # math layout [b, row, col]
        Bm = op(np.swapaxes(B, 1, 2).astype(wide), ob)
        Cm = np.swapaxes(C, 1, 2).astype(wide)
        al = wide(np.asarray(alpha).astype(oracle.NP_DTYPES[code]))
        be = wide(np.asarray(beta).astype(oracle.NP_DTYPES[code]))
        R = al * np.einsum("bik,bkj->bij", Am, Bm) + (be * Cm if beta != 0 else 0)
        P = abs(al) * np.einsum("bik,bkj->bij", np.abs(Am), np.abs(Bm)) + abs(be) * np.abs(Cm)
        out[name + "_A"], out[name + "_B"], out[name + "_C0"] = A, B, C
        out[name + "_expect"] = np.swapaxes(R, 1, 2).astype(np.complex128 if code >= 2 else np.float64)
        out[name + "_bound"] = np.swapaxes(P, 1, 2).astype(np.float64)
        out[name + "_meta"] = np.array([code, oracle.OPS[oa], oracle.OPS[ob], m, n, k, batch], np.int64)
        out[name + "_scal"] = np.array([alpha, beta], np.complex128)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
