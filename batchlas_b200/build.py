"""Builds libbatchlas_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch headers).

    python -m batchlas_b200.build            # incremental
    python -m batchlas_b200.build --force
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libbatchlas_b200.so")
SOURCES = ["dispatch.cu", "gemm_generic.cu", "gemm_small.cu", "gemm_small_ring.cu", "gemm_tiled.cu", "gemm_tiled_s.cu", "gemm_tiled_d.cu", "gemm_tiled_c.cu", "gemm_tiled_z.cu", "gemm_dmma.cu", "gemm_dmma_tma.cu", "gemm_sgemm128.cu", "gemm_sgemm_tma.cu", "gemm_splitk.cu", "level3.cu", "gemv.cu", "gemv_ring.cu", "elementwise.cu", "arena.cu", "fill.cu",
           "host_pipeline.cu", "status.cu", "peak.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libbatchlas_b200.so cannot be built")


def _newest_header() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(HERE, os.pardir, "include", "blb200.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src: str, force: bool, log_dir: str) -> str:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    srcp = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(srcp), _newest_header()):
        return obj
    res = subprocess.run([_nvcc(), *NVCC_FLAGS, "-c", srcp, "-o", obj], capture_output=True, text=True)
    with open(os.path.join(log_dir, src + ".ptxas.log"), "w") as f:
        f.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    return obj


def _source_hash() -> str:
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    files = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h")))
    files.append(os.path.join(HERE, os.pardir, "include", "blb200.h"))
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build(force: bool = False) -> str:
    # A library whose recorded source hash matches is current, whatever the file times say
    # (a copied tree does not keep them).
    stamp = LIB + ".srchash"
    digest = _source_hash()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return LIB
    _build_objects_and_link(force)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


def _build_objects_and_link(force: bool) -> None:
    os.makedirs(OBJ, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, OBJ), SOURCES))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        subprocess.check_call([_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static", "-lpthread", "-ldl"])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
