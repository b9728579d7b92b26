"""Environment knobs, exercised in a child process because they are read once per process:
BATCHLAS_GEMM_B200_KERNEL (forced kernel, the role BATCHLAS_GEMM_SYCL_KERNEL plays in the reference),
BATCHLAS_KERNEL_TRACE / BATCHLAS_KERNEL_TRACE_PATH (Chrome trace of every launch, as the
reference's kernel tracer writes, src/util/kernel-trace.hh:46-215) and BATCHLAS_NVTX (an NVTX range
around every call; without a profiler attached it must simply change nothing)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
import batchlas_b200 as bl
from oracle import oracle
from tests._cases import make_inputs
names = []
for (dt, m) in [("s", 64), ("d", 128), ("s", 32)]:
    p = oracle.make_problem(dt, "N", "N", m, m, m, 5, alpha=1.0, beta=0.0)
    A, B, C0 = make_inputs(p, tail=0)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
    d = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, 0, 0, m, m, m, 5, m, m, m, m*m, m*m, m*m)
    bl.gemm_strided_batched(d)
    torch.cuda.synchronize()
    bad, worst = oracle.check(p, A, B, C0, dC.cpu().numpy())
    assert bad == 0
    names.append(bl.last_kernel_name())
bl._lib.load().blb200_trace_flush()
print("KERNELS", ",".join(names))
"""


@pytest.mark.gpu
def test_forced_kernel_and_trace_file(lib, tmp_path):
    trace = str(tmp_path / "trace.json")
    env = dict(os.environ, BATCHLAS_GEMM_B200_KERNEL="tiled", BATCHLAS_KERNEL_TRACE="1", BATCHLAS_KERNEL_TRACE_PATH=trace,
               BATCHLAS_NVTX="1")
    out = subprocess.run([sys.executable, "-c", CHILD % ROOT], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("KERNELS")][0]
    # 64^3 float and 128^3 double can run on the forced tile kernel; 32^3 cannot and is dispatched normally
    assert line.split()[1].split(",") == ["tiled", "tiled", "small32"]
    events = json.load(open(trace))["traceEvents"]
    assert [e["name"] for e in events] == ["gemm.tiled", "gemm.tiled", "gemm.small32"]
    assert all(e["ph"] == "X" and e["dur"] > 0 and e["args"]["batch"] == 5 for e in events)
    assert events[0]["ts"] <= events[1]["ts"] <= events[2]["ts"]
