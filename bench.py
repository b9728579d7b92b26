#!/usr/bin/env python
"""Benchmark of the batched-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|cublas] [--no-extra]

Headline workload (``config.workload`` = "C2"): tiny-matrix SGEMM, float32, M=N=K=32, packed
column-major (ld 32, batch stride 1024), alpha=1.5, beta=-0.5, A/B/C ~ U[-1,1], batch 1,000,000,
ops NT and TN.  One *step* = one NT call plus one TN call over the whole batch (2 kernel launches
per GPU).  Inputs are 12.3 GB, far larger than the 126 MB L2, so no explicit L2 flush is needed
between iterations.  Multi-GPU: the 1,000,000 items are sharded contiguously over the ranks, one
process per GPU, no collective on the data path ("strong": the total batch is fixed, 125,000 items
per GPU at 8 GPUs).

Reported on one JSON line: ``value`` (GFLOP/s, inputs resident in HBM, CUDA-event timed, max over
ranks), ``e2e`` (same metric through the host-buffer C-ABI entry with H2D/D2H inside the timed
region), ``roofline`` (algorithmic bytes / measured launch time against the measured HBM copy
bandwidth), ``cpu_baseline`` (the CPU oracle — a port of the reference's serial CBLAS loop — on a
bounded sample), ``clocks``, ``gpu_launches``, ``sustained`` (the same steps repeated for 2 s or
more, with the SM clock the power cap allows) and, unless --no-extra, ``strong`` and ``configs``:
device-timed figures for the other four benchmark configurations (C1, C3, C4, C5), batch-sharded
over the ranks, each with a burst figure, a sustained figure, the cuBLAS figure on the same
buffers and, with more than one GPU, the speed-up over rank 0 running the whole batch alone.

Timing patterns.  The headline times exactly K steps inside one event pair (C drifts under
beta = -0.5 but stays bounded; timing does not depend on the values).  The per-configuration
figures follow the reference's harness (BatchLAS include/util/bench_structured.hh:118-150): when
beta != 0, C is restored from the generator before every launch, outside the timed interval; every
launch then has its own event pair and only those intervals are summed.  With beta == 0 the
launches run back to back inside one event pair.

cuBLAS leg: ``cublas{S,D,C,Z}gemmStridedBatched`` through ctypes on the libcublas that ships with
torch, default math mode (FP32 / FP64 arithmetic, no TF32) — what the reference's CUDA backend
executes on this GPU (BatchLAS src/backends/cublas.cc:125-147).  It is a yardstick inside this file
only; the library never links or calls cuBLAS.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "batched GEMM GFLOP/s (device-timed)"
NOMINAL_HBM_GBS = 8000.0          # the roofline definition of the task statement uses 8 TB/s
FALLBACK_HBM_GBS = 6650.0         # earlier measurement on this pool, used when no peaks file exists
# dram__bytes_read.sum + dram__bytes_write.sum per item of the dominant kernel, from the committed
# ncu summary of a 100 000-item capture (mean of NT and TN); traffic grows in proportion to the
# batch, so it is scaled to the full launch by the item count.
NCU_TRAFFIC_BYTES_PER_ITEM = 16040.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ---- the five configurations ---------------------------------------------------------------------
def configs():
    """name -> dict(dtype, ops, m, n, k, batch, alpha, beta, ld pad, dists)."""
    return {
        "C1": dict(dtype="s", ops=[("N", "N")], m=64, n=64, k=64, batch=10_000, alpha=1.0, beta=0.0, pad=0,
                   dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0), zero_c=True),
        "C2": dict(dtype="s", ops=[("N", "T"), ("T", "N")], m=32, n=32, k=32, batch=1_000_000, alpha=1.5,
                   beta=-0.5, pad=0, dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0)),
        "C3": dict(dtype="d", ops=[("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")], m=256, n=256, k=256,
                   batch=2048, alpha=2.0, beta=0.5, pad=8, dist_ab=("normal", 1.0), dist_c=("uniform", 1.0)),
        "C4": dict(dtype="z", ops=[("C", "N")], m=128, n=64, k=256, batch=8192, alpha=1.0 + 0.5j, beta=0.0,
                   pad=0, dist_ab=("normal", 1.0), dist_c=("uniform", 1.0)),
        "C5": dict(dtype="d", ops=[("N", "N")], m=1024, n=1024, k=1024, batch=512, alpha=1.0, beta=1.0, pad=0,
                   dist_ab=("normal", 1.0 / 32.0), dist_c=("uniform", 1.0)),
        # the reference's own published SGEMM shapes (RTX 4090 numbers in experiments/sycl_vs_cuda/FINDINGS.md:
        # 512^3 b512, 1024^3 b64, 256^3 b1024, beta = 1), reachable through --case S512 / S1024 / S256
        "S512": dict(dtype="s", ops=[("N", "N")], m=512, n=512, k=512, batch=512, alpha=1.0, beta=1.0, pad=0,
                     dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0)),
        "S1024": dict(dtype="s", ops=[("N", "N")], m=1024, n=1024, k=1024, batch=64, alpha=1.0, beta=1.0, pad=0,
                      dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0)),
        "S256": dict(dtype="s", ops=[("N", "N")], m=256, n=256, k=256, batch=1024, alpha=1.0, beta=1.0, pad=0,
                     dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0)),
        "S128": dict(dtype="s", ops=[("N", "N")], m=128, n=128, k=128, batch=4096, alpha=1.0, beta=1.0, pad=0,
                     dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0)),
        # not a BASELINE configuration: a Gram-matrix shaped product (few output tiles, long k) for
        # the split-K path, only reachable through --case SK [--splitk]
        "SK": dict(dtype="d", ops=[("T", "N")], m=64, n=64, k=262144, batch=2, alpha=1.0, beta=0.0, pad=0,
                   dist_ab=("normal", 1.0 / 512.0), dist_c=("uniform", 1.0)),
    }


ELEM_BYTES = {"s": 4, "d": 8, "c": 8, "z": 16}
PIPE_PEAK_TFLOPS = {"s": 148 * 128 * 2 * 1.965e9 / 1e12, "d": 148 * 64 * 2 * 1.965e9 / 1e12}
PIPE_PEAK_TFLOPS["c"] = PIPE_PEAK_TFLOPS["s"]
PIPE_PEAK_TFLOPS["z"] = PIPE_PEAK_TFLOPS["d"]


def flops_per_item(c):
    real = 2.0 * c["m"] * c["n"] * c["k"]
    return real * (4.0 if c["dtype"] in "cz" else 1.0)  # real flops: a complex FMA is 4 real FMAs


def algorithmic_bytes_per_item(c):
    es = ELEM_BYTES[c["dtype"]]
    a = c["m"] * c["k"] * es
    b = c["k"] * c["n"] * es
    cc = c["m"] * c["n"] * es
    return a + b + cc + (cc if c["beta"] != 0 else 0)


# ---- clocks sampler ------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        sm, smax, reasons = [], [], set()
        for ts, line in self.lines:
            if ts < t0 or ts > t1 + 0.2:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU baseline (oracle: test infrastructure, timed here as the reference arm) -----------------------
def cpu_baseline(cfg_name: str, budget_s: float = 20.0):
    """Times the CPU oracle — a port of the reference's host path (serial loop over batch items
    calling CBLAS ?gemm, BatchLAS src/backends/netlib_lapack.cc:108-171) — on a bounded contiguous
    sub-batch of the configuration, (1) exactly as the reference runs it and (2) batch-parallel over
    all host cores with the BLAS pinned to one thread.  Returns the dict for the JSON line."""
    import numpy as np
    from oracle import oracle

    c = configs()[cfg_name]
    cores = len(os.sched_getaffinity(0))
    provider = 1 if oracle.load_cblas() else 0
    code = oracle.DTYPES[c["dtype"]]
    per_item = flops_per_item(c)
    # size the sample for roughly budget_s at a guessed 2 GFLOP/s/core serial rate, capped by memory
    sample = int(max(1, min(c["batch"], budget_s * 0.25 * 2e9 / per_item)))
    oa, ob = c["ops"][0]
    ar = c["m"] if oa == "N" else c["k"]
    br = c["k"] if ob == "N" else c["n"]
    p = oracle.make_problem(code, oa, ob, c["m"], c["n"], c["k"], sample, lda=ar + c["pad"], ldb=br + c["pad"],
                            ldc=c["m"] + c["pad"], alpha=c["alpha"], beta=c["beta"])
    A = oracle.fill(code, p.alloc_len("a"), 42, 1, c["dist_ab"][0], c["dist_ab"][1])
    B = oracle.fill(code, p.alloc_len("b"), 42, 2, c["dist_ab"][0], c["dist_ab"][1])
    C = oracle.fill(code, p.alloc_len("c"), 42, 3, c["dist_c"][0], c["dist_c"][1])
    out = {}
    for label, threads in (("serial", 1), ("batch_parallel", cores)):
        if provider == 1:
            oracle.lib().oracle_cblas_set_threads(1 if threads > 1 else max(1, cores))
        times = []
        for oa_, ob_ in c["ops"]:
            p.op_a, p.op_b = oracle.OPS[oa_], oracle.OPS[ob_]
            oracle.gemm_netlib(p, A, B, C.copy(), provider=provider, threads=threads)  # warm
            Cw = C.copy()
            t0 = time.perf_counter()
            oracle.gemm_netlib(p, A, B, Cw, provider=provider, threads=threads)
            times.append(time.perf_counter() - t0)
        out[label] = per_item * sample * len(c["ops"]) / sum(times) / 1e9
    # The headline CPU figure is the path exactly as the reference runs it (one thread walks the
    # batch; the BLAS may thread inside a call but does not for matrices this small).  The
    # batch-parallel figure is reported beside it as the fairer all-cores number.
    return {"value": out["serial"], "unit": "GFLOP/s", "cores": 1, "kind": "port",
            "sample": f"{cfg_name}: {sample} of {c['batch']} items per op, ops " +
            "+".join(a + b for a, b in c["ops"]) + f"; provider={'scipy-openblas cblas' if provider else 'built-in loops'}"
            + f"; serial batch loop as in netlib_lapack.cc, BLAS allowed {cores} threads",
            "as_reference_runs_it_gflops": out["serial"], "batch_parallel_gflops": out["batch_parallel"],
            "batch_parallel_cores": cores, "host_cores": cores}


# ---- device helpers ----------------------------------------------------------------------------------
def alloc_config(bl, torch, c, batch, first_item, device):
    """Device operands for `batch` items of configuration c starting at global item `first_item`."""
    dt = {"s": torch.float32, "d": torch.float64, "c": torch.complex64, "z": torch.complex128}[c["dtype"]]
    pad = c["pad"]
    tensors, meta = {}, {}
    for tid, which in ((1, "a"), (2, "b"), (3, "c")):
        if which == "c":
            rows, cols = c["m"], c["n"]
        else:
            # stored shape depends on the op; allocate for the largest stored shape over the op list
            rows = max(((c["m"] if oa == "N" else c["k"]) if which == "a" else (c["k"] if ob == "N" else c["n"]))
                       for oa, ob in c["ops"])
            cols = max(((c["k"] if oa == "N" else c["m"]) if which == "a" else (c["n"] if ob == "N" else c["k"]))
                       for oa, ob in c["ops"])
        ld = rows + pad
        stride = ld * cols
        t = torch.empty(batch * stride, dtype=dt, device=device)
        dist, scale = c["dist_c"] if which == "c" else c["dist_ab"]
        bl.fill(t, 42, tid, dist, scale, first_index=first_item * stride)
        if which == "c" and c.get("zero_c"):
            t.zero_()
        tensors[which] = t
        meta[which] = (ld, stride)
    return tensors, meta


def desc_for(bl, c, op, tensors, meta, batch, kernel="auto"):
    from batchlas_b200 import _lib
    oa, ob = op
    code = {"s": 0, "d": 1, "c": 2, "z": 3}[c["dtype"]]
    opc = {"N": 0, "T": 1, "C": 2}
    return bl.make_desc(tensors["a"].data_ptr(), tensors["b"].data_ptr(), tensors["c"].data_ptr(), code, opc[oa],
                        opc[ob], c["m"], c["n"], c["k"], batch, meta["a"][0], meta["b"][0], meta["c"][0],
                        meta["a"][1], meta["b"][1], meta["c"][1], c["alpha"], c["beta"], kernel)


def verify_sample(bl, torch, c, op, tensors, meta, batch, first_item, n_check=4, kernel="auto"):
    """Restore C from the generator, run one launch, check a few items against the oracle."""
    import numpy as np
    from oracle import oracle
    ldc, sc = meta["c"]
    dist, scale = c["dist_c"]
    bl.fill(tensors["c"], 42, 3, dist, scale, first_index=first_item * sc)
    if c.get("zero_c"):
        tensors["c"].zero_()
    items = sorted(set([0, batch - 1] + [int(i) for i in np.linspace(0, batch - 1, n_check)]))
    c0 = {i: tensors["c"][i * sc:(i + 1) * sc].cpu().numpy() for i in items}
    bl.gemm_strided_batched(desc_for(bl, c, op, tensors, meta, batch, kernel=kernel))
    torch.cuda.synchronize()
    code = oracle.DTYPES[c["dtype"]]
    worst_all = 0.0
    for i in items:
        lda, sa = meta["a"]
        ldb, sb = meta["b"]
        A = tensors["a"][i * sa:(i + 1) * sa].cpu().numpy()
        B = tensors["b"][i * sb:(i + 1) * sb].cpu().numpy()
        got = tensors["c"][i * sc:(i + 1) * sc].cpu().numpy()
        n_chk = min(c["n"], 64)  # the long-double arbiter is O(mnk): a column slab of big items
        p = oracle.make_problem(code, op[0], op[1], c["m"], n_chk, c["k"], 1, lda=lda, ldb=ldb, ldc=ldc,
                                alpha=c["alpha"], beta=c["beta"])
        bad, worst = oracle.check(p, A, B, c0[i], got)
        if bad:
            raise SystemExit(f"PARITY FAILURE {op} item {i}: {bad} entries beyond the bound (worst {worst:.3g})")
        worst_all = max(worst_all, worst)
    return worst_all


def time_launches(torch, launch, reps):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        launch()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / reps  # ms per rep


def time_restored(torch, launch, restore, reps):
    """ms per launch with C restored before every launch, outside the timed intervals: one event
    pair per launch, only those intervals are summed."""
    pairs = []
    for _ in range(reps):
        restore()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        launch()
        e.record()
        pairs.append((s, e))
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in pairs) / reps


def time_op(torch, launch, restore, reps):
    return time_restored(torch, launch, restore, reps) if restore else time_launches(torch, launch, reps)


def sustained_run(torch, launch, restore, one_ms, local_rank, seconds=2.0):
    """The same launch repeated for `seconds` or more of device time; returns ms per launch and the
    clocks sampled meanwhile (median SM MHz under load, throttle reasons)."""
    reps = int(max(3, min(150000, seconds * 1e3 / max(one_ms, 1e-3))))
    smp = ClockSampler(local_rank)
    smp.start()
    time.sleep(0.15)
    t0 = time.time()
    ms = time_op(torch, launch, restore, reps)
    t1 = time.time()
    smp.stop()
    clk = smp.summary(t0 + 0.3, t1)  # skip the ramp: the clock under a held load is what is wanted
    return ms, reps, clk


# ---- cuBLAS yardstick (bench only) --------------------------------------------------------------------
class Cublas:
    """cublas{S,D,C,Z}gemmStridedBatched on the caller's device buffers and stream: the call the
    reference's CUDA backend ends in (BatchLAS src/backends/cublas.cc:125-147).  Default math mode:
    FP32 / FP64 arithmetic, no TF32."""

    def __init__(self, torch):
        import ctypes
        import glob
        self.ct = ctypes
        self.torch = torch
        cands = []
        try:
            import nvidia.cublas.lib as nl
            cands += glob.glob(os.path.join(os.path.dirname(nl.__file__), "libcublas.so*"))
        except Exception:
            pass
        cands += ["libcublas.so.12", "libcublas.so"]
        self.lib = None
        for c in cands:
            try:
                self.lib = ctypes.CDLL(c)
                break
            except OSError:
                continue
        if self.lib is None:
            raise RuntimeError("libcublas not found")
        self.handle = ctypes.c_void_p()
        self.lib.cublasCreate_v2.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        if self.lib.cublasCreate_v2(ctypes.byref(self.handle)) != 0:
            raise RuntimeError("cublasCreate failed")
        self.lib.cublasSetStream_v2.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        self.fns = {}
        for letter, name in (("s", "cublasSgemmStridedBatched"), ("d", "cublasDgemmStridedBatched"),
                             ("c", "cublasCgemmStridedBatched"), ("z", "cublasZgemmStridedBatched")):
            fn = getattr(self.lib, name)
            fn.argtypes = [vp, i, i, i, i, i, vp, vp, i, ll, vp, i, ll, vp, vp, i, ll, i]
            fn.restype = i
            self.fns[letter] = fn
        ver = ctypes.c_int(0)
        self.lib.cublasGetVersion_v2.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        self.lib.cublasGetVersion_v2(self.handle, ctypes.byref(ver))
        self.version = ver.value

    def launcher(self, c, op, tensors, meta, batch):
        ct = self.ct
        letter = c["dtype"]
        real = {"s": ct.c_float, "d": ct.c_double, "c": ct.c_float, "z": ct.c_double}[letter]
        al, be = complex(c["alpha"]), complex(c["beta"])
        alpha = (real * 2)(al.real, al.imag)
        beta = (real * 2)(be.real, be.imag)
        opc = {"N": 0, "T": 1, "C": 2}
        fn = self.fns[letter]
        args = (opc[op[0]], opc[op[1]], c["m"], c["n"], c["k"], ct.cast(alpha, ct.c_void_p),
                tensors["a"].data_ptr(), meta["a"][0], meta["a"][1], tensors["b"].data_ptr(), meta["b"][0], meta["b"][1],
                ct.cast(beta, ct.c_void_p), tensors["c"].data_ptr(), meta["c"][0], meta["c"][1], batch)
        handle, lib, torch = self.handle, self.lib, self.torch

        def launch(_keep=(alpha, beta)):
            lib.cublasSetStream_v2(handle, torch.cuda.current_stream().cuda_stream)
            rc = fn(handle, *args)
            if rc != 0:
                raise RuntimeError(f"cuBLAS status {rc}")
        return launch


def checksum_all_items(torch, c, op, tensors, meta, batch, launch, restore):
    """Full-size parity property: restore C, run `launch` once, and hold EVERY item to the summed
    entrywise bound through the checksum identity (tests/_props.py).  Returns the worst ratio."""
    from tests import _props
    restore()
    torch.cuda.synchronize()
    oa, ob = op
    ar, ac = (c["m"], c["k"]) if oa == "N" else (c["k"], c["m"])
    br, bc = (c["k"], c["n"]) if ob == "N" else (c["n"], c["k"])
    tA = _props.strided_view(torch, tensors["a"], ar, ac, meta["a"][0], meta["a"][1], batch)
    tB = _props.strided_view(torch, tensors["b"], br, bc, meta["b"][0], meta["b"][1], batch)
    tC = _props.strided_view(torch, tensors["c"], c["m"], c["n"], meta["c"][0], meta["c"][1], batch)
    before = _props.sums_before(torch, tC)
    launch()
    torch.cuda.synchronize()
    bad, worst = _props.checksum_check(torch, tA, tB, tC, oa, ob, c["alpha"], c["beta"], c["k"], c["dtype"], before)
    if bad:
        raise SystemExit(f"PARITY FAILURE (checksum) {op}: {bad} of {batch} items beyond the bound (worst {worst:.3g})")
    return worst


# ---- the two arms ------------------------------------------------------------------------------------
def run_reference_arm(args, rank):
    if rank != 0:
        return
    t0 = time.perf_counter()
    base = cpu_baseline("C2", budget_s=8.0)
    # K timed "steps", each a bounded sample; the sample rate is what is reported.
    vals = [base["value"]]
    for _ in range(max(0, min(args.steps, 3) - 1)):
        vals.append(cpu_baseline("C2", budget_s=8.0)["value"])
    value = sorted(vals)[len(vals) // 2]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C2", "note": "reference CPU path (port of the serial CBLAS batch "
                       "loop of netlib_lapack.cc:108-171, BLAS threading at its default) on a bounded sub-batch "
                       "per step; cpu_baseline.batch_parallel_gflops is the same loop split over all host cores"},
            "cpu_baseline": dict(base, value=value),
            "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


def restore_fn(bl, torch, c, tensors, meta, first_item):
    """Device-side restore of C from the generator (None when beta == 0: C is never read)."""
    if c["beta"] == 0:
        return None
    dist, scale = c["dist_c"]
    sc = meta["c"][1]

    def restore():
        bl.fill(tensors["c"], 42, 3, dist, scale, first_index=first_item * sc)
    return restore


def measure_config_op(bl, torch, c, op, tens, mt, nb, b0, local_rank, barrier, max_over_ranks, world, cublas,
                      do_sustained=True, kernel="auto"):
    """Burst, sustained and cuBLAS figures for one op pair of one configuration on this rank's shard."""
    d = desc_for(bl, c, op, tens, mt, nb, kernel=kernel)
    launch = (lambda d=d: bl.gemm_strided_batched(d))
    restore = restore_fn(bl, torch, c, tens, mt, b0)
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    one = time_launches(torch, launch, 1)
    # about 60 ms of launches after a short idle: a kernel timed alone.  Held for 150 ms or more, the
    # FP32 64^3 case reaches the 1000 W cap and the SM clock falls from 1965 to about 1710 MHz.
    reps = int(max(3, min(1000, 60.0 / max(one, 1e-3))))
    barrier()
    smp = ClockSampler(local_rank)
    smp.start()
    time.sleep(0.4)
    tw0 = time.time()
    ms = max_over_ranks(time_op(torch, launch, restore, reps))
    tw1 = time.time()
    smp.stop()
    clk = smp.summary(tw0, tw1)
    kern = bl.last_kernel_name()
    w = verify_sample(bl, torch, c, op, tens, mt, nb, b0, n_check=2)
    full_restore = restore or (lambda: None)
    wsum = checksum_all_items(torch, c, op, tens, mt, nb, launch, full_restore)
    total_flops = flops_per_item(c) * c["batch"]
    tfl = total_flops / (ms * 1e-3) / 1e12
    ai = flops_per_item(c) / algorithmic_bytes_per_item(c)
    roof = min(PIPE_PEAK_TFLOPS[c["dtype"]] * world, ai * NOMINAL_HBM_GBS * 1e9 / 1e12 * world)
    out = {"gflops": tfl * 1e3, "ms": ms, "kernel": kern, "frac_of_roofline": tfl / roof,
           "worst_error_ratio": w, "checksum_all_items_worst_ratio": wsum, "reps": reps,
           "timing": "C restored before each launch, per-launch events" if restore else "back-to-back, one event pair",
           "sm_mhz": clk["sm_mhz"], "clock_reasons": clk["reasons"],
           "hbm_gbs": algorithmic_bytes_per_item(c) * c["batch"] / (ms * 1e-3) / 1e9}
    if do_sustained:
        time.sleep(0.3)
        barrier()
        sms, sreps, sclk = sustained_run(torch, launch, restore, ms, local_rank)
        sms = max_over_ranks(sms)
        stfl = total_flops / (sms * 1e-3) / 1e12
        out["sustained"] = {"gflops": stfl * 1e3, "ms": sms, "launches": sreps, "seconds": sms * sreps * 1e-3,
                            "frac_of_roofline": stfl / roof, "sm_mhz": sclk["sm_mhz"], "clock_reasons": sclk["reasons"],
                            "gflops_per_mhz": (stfl * 1e3 / sclk["sm_mhz"]) if sclk["sm_mhz"] else None}
    if cublas is not None:
        try:
            cl = cublas.launcher(c, op, tens, mt, nb)
            for _ in range(3):
                cl()
            torch.cuda.synchronize()
            cw = checksum_all_items(torch, c, op, tens, mt, nb, cl, full_restore)  # the yardstick computes the same thing
            time.sleep(0.3)
            barrier()
            cms = max_over_ranks(time_op(torch, cl, restore, reps))
            out["cublas_gflops"] = total_flops / (cms * 1e-3) / 1e9
            out["cublas_ms"] = cms
            out["vs_cublas"] = cms / ms
            out["cublas_checksum_worst_ratio"] = cw
        except Exception as exc:  # the yardstick must never take the benchmark down
            out["cublas_error"] = str(exc)[:200]
    return out


def bind_to_gpu_numa_node(torch, local_rank):
    """Best effort: run this process on the cores of the NUMA node its GPU hangs off, so that host
    staging buffers allocated afterwards land in that node's memory.  Returns what was done."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read().strip())
        if node < 0:
            return {"pci": bdf, "numa_node": node, "bound": False}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"pci": bdf, "numa_node": node, "bound": False, "why": "no allowed core on that node"}
        os.sched_setaffinity(0, allowed)
        return {"pci": bdf, "numa_node": node, "bound": True, "cores": len(allowed)}
    except Exception as exc:
        return {"bound": False, "why": str(exc)[:120]}


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    import batchlas_b200 as bl
    from batchlas_b200 import _lib
    from batchlas_b200.sharding import shard_range

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: batchlas_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL announces its version on stdout when the first communicator comes up; stdout must
        # carry exactly one JSON line, so that chatter is sent to stderr.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cublas = None
    if not args.no_cublas:
        try:
            cublas = Cublas(torch)
        except Exception:
            cublas = None

    cfgs = configs()
    c2 = cfgs["C2"]
    first_item, batch = shard_range(c2["batch"], rank, world)   # strong scaling: the 10^6 items are shared out
    tensors, meta = alloc_config(bl, torch, c2, batch, first_item, device)
    descs = [desc_for(bl, c2, op, tensors, meta, batch) for op in c2["ops"]]

    def step():
        for d in descs:
            bl.gemm_strided_batched(d)

    # Clocks are sampled (nvidia-smi, 50 ms period) from the first warm-up step to the last timed
    # step: K timed steps alone can be shorter than one sampling period.
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    t_load0 = time.time()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    kernel_name = bl.last_kernel_name()
    launches0 = bl.launch_count()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_wall1 = time.time()
    launches = bl.launch_count() - launches0
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    time.sleep(0.2)
    sampler.stop()
    clocks = sampler.summary(t_load0, t_wall1)
    clocks["window"] = "warm-up + timed steps"
    ms_per_step = ms_total / args.steps
    flops_step = flops_per_item(c2) * c2["batch"] * len(c2["ops"])
    value = flops_step / (ms_per_step * 1e-3) / 1e9

    per_op_ms = {}
    for (oa, ob), d in zip(c2["ops"], descs):
        per_op_ms[oa + ob] = max_over_ranks(time_launches(torch, lambda d=d: bl.gemm_strided_batched(d), max(3, args.steps)))

    # the same steps held for two seconds or more: what the 1000 W cap allows
    time.sleep(0.3)
    barrier()
    s_ms, s_reps, s_clk = sustained_run(torch, step, None, ms_per_step, local_rank)
    s_ms = max_over_ranks(s_ms)
    sustained = {"value": flops_step / (s_ms * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": s_ms, "steps": s_reps,
                 "seconds": s_ms * s_reps * 1e-3, "sm_mhz": s_clk["sm_mhz"], "clock_reasons": s_clk["reasons"],
                 "hbm_gbs": algorithmic_bytes_per_item(c2) * batch * len(c2["ops"]) / (s_ms * 1e-3) / 1e9,
                 "gflops_per_mhz": (flops_step / (s_ms * 1e-3) / 1e9 / s_clk["sm_mhz"]) if s_clk["sm_mhz"] else None}

    # parity on the exact buffers that were timed (restores C first): sampled items against the
    # long-double arbiter, and every item through the checksum identity
    worst = max(verify_sample(bl, torch, c2, op, tensors, meta, batch, first_item) for op in c2["ops"])
    c2_restore = restore_fn(bl, torch, c2, tensors, meta, first_item)
    worst_sum = max(checksum_all_items(torch, c2, op, tensors, meta, batch,
                                       (lambda d=d: bl.gemm_strided_batched(d)), c2_restore)
                    for op, d in zip(c2["ops"], descs))

    cublas_c2 = None
    if cublas is not None:
        try:
            cms = {}
            for op in c2["ops"]:
                cl = cublas.launcher(c2, op, tensors, meta, batch)
                for _ in range(2):
                    cl()
                torch.cuda.synchronize()
                cms[op[0] + op[1]] = max_over_ranks(time_launches(torch, cl, max(3, min(args.steps, 5))))
            cublas_c2 = {"ms_by_op": cms, "gflops": flops_step / (sum(cms.values()) * 1e-3) / 1e9,
                         "vs_cublas": sum(cms.values()) / ms_per_step, "version": cublas.version,
                         "call": "cublasSgemmStridedBatched, default math (no TF32), same device buffers"}
        except Exception as exc:
            cublas_c2 = {"error": str(exc)[:200]}

    # roofline of the dominant kernel: one launch = one op over this GPU's share of the batch
    peak, peak_kind = measured_peaks()
    bytes_launch = algorithmic_bytes_per_item(c2) * batch
    launch_ms = ms_per_step / len(c2["ops"])
    achieved = bytes_launch / (launch_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"{peak_kind} STREAM-style copy (burst; kernel timed alone)",
                "traffic": (NCU_TRAFFIC_BYTES_PER_ITEM * batch if NCU_TRAFFIC_BYTES_PER_ITEM else None),
                "algorithmic_bytes_per_launch": bytes_launch, "kernel": kernel_name, "launch_ms": launch_ms,
                "launch_ms_by_op": per_op_ms,
                "frac_of_8TBs_definition": achieved / NOMINAL_HBM_GBS}

    # ---- end to end: host buffers through the C ABI, copies inside the timed region ----------------
    e2e = None
    if not args.no_e2e:
        import psutil
        numa = bind_to_gpu_numa_node(torch, local_rank) if args.numa_bind else {"bound": False, "why": "not requested"}
        es = 4
        need = 3 * batch * 1024 * es
        avail = psutil.virtual_memory().available / max(world, 1)
        e2e_batch = batch if avail > 2.5 * need else max(1000, int(batch * avail / (2.5 * need)))
        hA = torch.empty(e2e_batch * 1024, dtype=torch.float32).pin_memory()
        hB = torch.empty(e2e_batch * 1024, dtype=torch.float32).pin_memory()
        hC = torch.empty(e2e_batch * 1024, dtype=torch.float32).pin_memory()
        hA.copy_(tensors["a"][: e2e_batch * 1024])
        hB.copy_(tensors["b"][: e2e_batch * 1024])
        hC.copy_(tensors["c"][: e2e_batch * 1024])
        hdescs = []
        for (oa, ob) in c2["ops"]:
            opc = {"N": 0, "T": 1, "C": 2}
            hdescs.append(bl.make_desc(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), 0, opc[oa], opc[ob], 32, 32, 32,
                                       e2e_batch, 32, 32, 32, 1024, 1024, 1024, c2["alpha"], c2["beta"]))
        L = _lib.load()

        def e2e_step():
            for d in hdescs:
                _lib.check(L.blb200_gemm_strided_batched_host(d, local_rank, 0))

        e2e_step()  # warm-up (pool growth, stream creation)
        e2e_steps = max(1, min(args.steps, 3))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt_e2e = max_over_ranks(time.perf_counter() - t0)
        all_items = e2e_batch
        if world > 1:
            t = torch.tensor([float(e2e_batch)], dtype=torch.float64, device=device)
            dist.all_reduce(t)
            all_items = int(t.item())
        e2e_flops = flops_per_item(c2) * all_items * len(c2["ops"]) * e2e_steps
        # the ceiling of this box for the same bytes: plain pinned copies, all ranks at once
        barrier()
        t0 = time.perf_counter()
        for src in (hA, hB, hC):
            tensors["a"][: e2e_batch * 1024].copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        dt_copy = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": e2e_flops / dt_e2e / 1e9, "unit": "GFLOP/s",
               "h2d_bytes_per_step": 3 * all_items * 4096 * len(c2["ops"]),
               "d2h_bytes_per_step": all_items * 4096 * len(c2["ops"]), "steps": e2e_steps,
               "batch_per_gpu": e2e_batch, "api": "blb200_gemm_strided_batched_host (pinned host A,B,C; chunked "
               "H2D -> kernel -> D2H on 3 streams)", "ms_per_step": dt_e2e / e2e_steps * 1e3,
               "h2d_gbs_in_step": 3 * all_items * 4096 * len(c2["ops"]) * e2e_steps / dt_e2e / 1e9,
               "h2d_gbs_plain_copies_all_ranks": 3 * all_items * 4096 / dt_copy / 1e9, "numa": numa}
        del hA, hB, hC

    del tensors
    torch.cuda.empty_cache()

    # ---- the other configurations, device-timed, batch sharded over the ranks (strong) ------------
    extra, strong = {}, {}
    pipe_peaks = None
    if not args.no_extra:
        pipe_peaks = {"fp32_tflops_measured": bl.measure_pipe_peak("s"), "fp64_tflops_measured": bl.measure_pipe_peak("d"),
                      "fp32_tflops_nominal": PIPE_PEAK_TFLOPS["s"], "fp64_tflops_nominal": PIPE_PEAK_TFLOPS["d"]}
        for name in ("C1", "C3", "C4", "C5"):
            c = cfgs[name]
            b0, nb = shard_range(c["batch"], rank, world)
            if nb == 0:
                continue
            tens, mt = alloc_config(bl, torch, c, nb, b0, device)
            per_op = {}
            for op in c["ops"]:
                per_op[op[0] + op[1]] = measure_config_op(bl, torch, c, op, tens, mt, nb, b0, local_rank, barrier,
                                                         max_over_ranks, world, cublas, do_sustained=not args.no_sustained)
            extra[name] = per_op
            del tens
            torch.cuda.empty_cache()
            if world > 1:
                # strong scaling inside this run: rank 0 alone runs the whole batch on its GPU while the
                # others wait; speed-up = that time / the sharded time measured above
                alone = {}
                if rank == 0:
                    tens, mt = alloc_config(bl, torch, c, c["batch"], 0, device)
                    for op in c["ops"]:
                        d = desc_for(bl, c, op, tens, mt, c["batch"])
                        launch = (lambda d=d: bl.gemm_strided_batched(d))
                        restore = restore_fn(bl, torch, c, tens, mt, 0)
                        for _ in range(3):
                            launch()
                        torch.cuda.synchronize()
                        one = time_launches(torch, launch, 1)
                        time.sleep(0.4)
                        alone[op[0] + op[1]] = time_op(torch, launch, restore, int(max(3, min(1000, 60.0 / max(one, 1e-3)))))
                    del tens
                    torch.cuda.empty_cache()
                barrier()
                for opn, r in per_op.items():
                    a_ms = alone.get(opn)
                    strong[f"{name}:{opn}"] = {"ms_1gpu_whole_batch": a_ms, "ms_sharded": r["ms"],
                                               "speedup": (a_ms / r["ms"]) if a_ms else None, "gflops": r["gflops"]}
            else:
                for opn, r in per_op.items():
                    strong[f"{name}:{opn}"] = {"ms_sharded": r["ms"], "gflops": r["gflops"],
                                               "frac_of_roofline": r["frac_of_roofline"],
                                               "sustained_frac": r.get("sustained", {}).get("frac_of_roofline"),
                                               "vs_cublas": r.get("vs_cublas")}

    status = bl.device_status()
    if status != 0:
        raise SystemExit(f"a kernel abandoned a bounded wait (code {status})")

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "C2", "shape": "SGEMM 32x32x32, ops NT+TN per step, alpha=1.5 beta=-0.5, "
                           "packed column-major (ld 32, stride 1024)", "global_batch": c2["batch"],
                           "batch_per_gpu": batch, "sharding": f"contiguous batch ranges x{world}, no collective",
                           "l2": f"inputs ({3 * batch * 4096 / 1e9:.1f} GB per GPU) exceed the 126 MB L2; no flush needed",
                           "seed": 42},
                "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches) * world, "clocks": clocks,
                "sustained": sustained, "parity_worst_error_ratio": worst,
                "parity_checksum_all_items_worst_ratio": worst_sum, "cublas": cublas_c2}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline("C2")
        if extra:
            line["strong"] = strong     # compact, ahead of the long per-configuration block
            line["pipe_peaks"] = pipe_peaks
            line["configs_note"] = ("device-timed, whole BASELINE batch sharded contiguously over the ranks; "
                                    "frac_of_roofline = achieved / min(nominal pipe peak, AI x 8 TB/s); beta != 0: C "
                                    "restored before each launch outside the timed intervals")
            line["configs"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_case(args):
    """One configuration, one op, a chosen batch: the small case that ncu captures.
    Prints one JSON line with the CUDA-event time per launch."""
    import torch

    import batchlas_b200 as bl
    name, _, op = args.case.partition(":")
    import re
    shape = re.fullmatch(r"([sdcz])(\d+)x(\d+)x(\d+)", name)
    if shape:  # an arbitrary packed shape, e.g. d32x32x32:TN: uniform inputs, alpha 1.5, beta from --beta
        c = dict(dtype=shape.group(1), ops=[("N", "N")], m=int(shape.group(2)), n=int(shape.group(3)),
                 k=int(shape.group(4)), batch=100_000, alpha=1.5, beta=args.beta, pad=0,
                 dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0))
    else:
        c = configs()[name]
    ops = [tuple(op)] if op else c["ops"]
    batch = args.batch or c["batch"]
    if args.ld_extra:  # e.g. 1: leading dimensions that are not multiples of 16 bytes (element-granular copies)
        c = dict(c, pad=c["pad"] + args.ld_extra)
    torch.cuda.set_device(0)
    tens, mt = alloc_config(bl, torch, c, batch, 0, torch.device("cuda", 0))
    out = {"case": name, "batch": batch, "ld_extra": args.ld_extra, "ops": {}}
    for o in ops:
        d = desc_for(bl, c, o, tens, mt, batch, kernel=args.kernel)
        launch = lambda: bl.gemm_strided_batched(d)
        if args.impl == "cublas":  # the yardstick on the same buffers
            launch = Cublas(torch).launcher(c, o, tens, mt, batch)
        if args.splitk:
            import ctypes
            from batchlas_b200 import _lib
            need = ctypes.c_size_t(0)
            splits = _lib.load().blb200_gemm_splitk_plan(d, 0, ctypes.byref(need))
            ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
            stream = torch.cuda.current_stream().cuda_stream
            launch = lambda: _lib.check(_lib.load().blb200_gemm_splitk(d, splits, ws.data_ptr(), need.value, stream))
            out["splits"] = splits
        for _ in range(args.warmup):
            launch()
        torch.cuda.synchronize()
        ms = time_op(torch, launch, restore_fn(bl, torch, c, tens, mt, 0), args.steps)
        kern = "cublas" if args.impl == "cublas" else bl.last_kernel_name()
        w = verify_sample(bl, torch, c, o, tens, mt, batch, 0, n_check=2, kernel=args.kernel)
        if args.impl == "cublas":
            out["impl"] = "cublas"
        out["ops"][o[0] + o[1]] = {"ms": ms, "kernel": kern, "worst_error_ratio": w,
                                   "gflops": flops_per_item(c) * batch / (ms * 1e-3) / 1e9,
                                   "hbm_gbs": algorithmic_bytes_per_item(c) * batch / (ms * 1e-3) / 1e9}
    print(json.dumps(out), flush=True)


# BatchLAS's own batched-gemm benchmark sizes: cubes with these batches (include/util/minibench.hh:869-887,
# `CubeBatchSizes`), run by BM_GEMM with alpha = beta = 1, NN (benchmarks/gemm_benchmark.cc:8-33).
CUBE_BATCH_SIZES = ((16, (4096, 8192, 16384)), (32, (2048, 4096, 8192)), (64, (1024, 2048, 4096)),
                    (128, (512, 1024, 2048)), (256, (128, 256, 512, 1024)), (512, (32, 64, 128, 256)),
                    (1024, (8, 16, 32, 64)), (2048, (2, 4, 8, 16)), (4096, (1, 2, 4, 8)))


def run_sweep(args):
    """The reference's cube sizes (largest batch of each), float and double, alpha = beta = 1, NN: our
    launch and cuBLAS on the same buffers, one JSON line per point.  Where the three operands of the
    listed batch would fit in L2, the batch is doubled until they exceed 256 MiB (`batch` against
    `listed_batch`), so that every figure is measured from HBM."""
    import torch

    import batchlas_b200 as bl
    torch.cuda.set_device(0)
    cublas = Cublas(torch)
    dtypes = args.sweep.split(",") if args.sweep != "all" else ["s", "d"]
    for dt in dtypes:
        es = {"s": 4, "d": 8, "c": 8, "z": 16}[dt]
        for size, batches in CUBE_BATCH_SIZES:
            listed = batches[-1]
            batch = listed
            while 3 * size * size * es * batch < (256 << 20):
                batch *= 2
            c = dict(dtype=dt, ops=[("N", "N")], m=size, n=size, k=size, batch=batch, alpha=1.0, beta=1.0, pad=0,
                     dist_ab=("uniform", 1.0), dist_c=("uniform", 1.0))
            tens, mt = alloc_config(bl, torch, c, batch, 0, torch.device("cuda", 0))
            d = desc_for(bl, c, ("N", "N"), tens, mt, batch)
            restore = restore_fn(bl, torch, c, tens, mt, 0)
            ours = lambda: bl.gemm_strided_batched(d)
            theirs = cublas.launcher(c, ("N", "N"), tens, mt, batch)
            res = {}
            for label, launch in (("ours", ours), ("cublas", theirs)):
                for _ in range(args.warmup):
                    launch()
                torch.cuda.synchronize()
                res[label] = time_op(torch, launch, restore, args.steps)
            ours()
            kern = bl.last_kernel_name()
            worst = verify_sample(bl, torch, c, ("N", "N"), tens, mt, batch, 0, n_check=2)
            fl = flops_per_item(c) * batch / 1e6
            print(json.dumps({"sweep": f"{dt}{size}", "listed_batch": listed, "batch": batch, "kernel": kern,
                              "ms": res["ours"], "gflops": fl / res["ours"], "cublas_ms": res["cublas"],
                              "cublas_gflops": fl / res["cublas"], "vs_cublas": res["cublas"] / res["ours"],
                              "hbm_gbs": algorithmic_bytes_per_item(c) * batch / res["ours"] / 1e6,
                              "worst_error_ratio": worst}), flush=True)
            del tens, d
            torch.cuda.empty_cache()


def run_level3(args):
    """symm / hemm / trmm / syrk / herk / syr2k / her2k (the calls BatchLAS builds on gemm) on square operands, each
    beside the plain gemm of the same shape: the difference is the cost of expanding the triangle
    (or of accumulating one).  One JSON line; times are CUDA events per call, after warm-up."""
    import torch

    import batchlas_b200 as bl
    torch.cuda.set_device(0)
    tdt = {"s": torch.float32, "d": torch.float64, "c": torch.complex64, "z": torch.complex128}
    out = {"level3": []}
    shapes = [("s", 128, 4096), ("d", 256, 512), ("z", 128, 1024), ("d", 1024, 32)]
    for dt, n, batch in shapes:
        if args.batch:
            batch = args.batch
        t = tdt[dt]
        A, B, C = (bl.fill(torch.empty(batch, n, n, dtype=t, device="cuda"), 42, i) for i in range(3))
        ws = torch.empty(bl.level3.workspace_bytes(t, n, batch), dtype=torch.uint8, device="cuda")
        cplx = dt in "cz"
        mul = 4 if cplx else 1  # real flops per complex fma pair, BLAS convention 8 per complex multiply-add
        calls = {
            "gemm": (lambda: bl.gemm(A, B, C, 1.0, 0.5), 2.0 * n * n * n),
            "symm": (lambda: bl.symm(A, B, C, 1.0, 0.5, 0, 1, workspace=ws), 2.0 * n * n * n),
            "trmm": (lambda: bl.trmm(A, B, C, 1.0, 0, 1, 0, 0, workspace=ws), 1.0 * n * n * n),
            "syrk": (lambda: bl.syrk(A, C, 1.0, 0.5, 1, 0, workspace=ws), 1.0 * n * n * (n + 1)),
            "syr2k": (lambda: bl.syr2k(A, B, C, 1.0, 0.5, 1, 0, workspace=ws), 2.0 * n * n * (n + 1)),
        }
        if cplx:
            calls["hemm"] = (lambda: bl.hemm(A, B, C, 1.0, 0.5, 0, 1, workspace=ws), 2.0 * n * n * n)
            calls["herk"] = (lambda: bl.herk(A, C, 1.0, 0.5, 1, 0, workspace=ws), 1.0 * n * n * (n + 1))
            calls["her2k"] = (lambda: bl.her2k(A, B, C, 1.0, 0.5, 1, 0, workspace=ws), 2.0 * n * n * (n + 1))
        row = {"dtype": dt, "n": n, "batch": batch, "ops": {}}
        for name, (fn, fl) in calls.items():
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            ms = time_launches(torch, fn, args.steps)
            row["ops"][name] = {"ms": round(ms, 4), "blas_gflops": round(fl * mul * batch / (ms * 1e-3) / 1e9, 1),
                                "kernel": bl.last_kernel_name()}
        g = row["ops"]["gemm"]["ms"]
        for name in row["ops"]:
            row["ops"][name]["time_vs_gemm"] = round(row["ops"][name]["ms"] / g, 3)
        out["level3"].append(row)
    print(json.dumps(out), flush=True)


def run_hetero(args):
    """Heterogeneous batches (per-item m, n inside a common capacity) on the reference's benchmark
    pattern (benchmarks/gemm_heterogeneous_benchmark.cc:47-110): items cycle full size / half size /
    empty, float, k = 32; plus a double case with a long k.  GFLOP/s counts the active sizes only."""
    import ctypes

    import numpy as np
    import torch

    import batchlas_b200 as bl
    from batchlas_b200 import _lib
    torch.cuda.set_device(0)
    tdt = {"s": torch.float32, "d": torch.float64}
    out = {"hetero": []}
    for dt, mx, nx, k, batch in [("s", 64, 64, 32, 4096), ("s", 128, 128, 32, 1024), ("s", 256, 256, 32, 256),
                                 ("s", 256, 256, 256, 2048), ("d", 256, 256, 256, 2048)]:
        t = tdt[dt]
        A = bl.fill(torch.empty(batch, k, mx, dtype=t, device="cuda"), 42, 0)
        B = bl.fill(torch.empty(batch, nx, k, dtype=t, device="cuda"), 42, 1)
        C = bl.fill(torch.empty(batch, nx, mx, dtype=t, device="cuda"), 42, 2)
        idx = np.arange(batch) % 3
        m_items = np.where(idx == 0, mx, np.where(idx == 1, mx // 2, 0)).astype(np.int32)
        n_items = np.where(idx == 0, nx, np.where(idx == 1, nx // 2, 0)).astype(np.int32)
        flops = float(np.sum(2.0 * m_items.astype(np.float64) * n_items * k))
        dm, dn = torch.from_numpy(m_items).cuda(), torch.from_numpy(n_items).cuda()
        d = bl.make_desc(A.data_ptr(), B.data_ptr(), C.data_ptr(), bl.DTYPE_CODES[t], 0, 0, mx, nx, k, batch, mx, k, mx,
                         mx * k, k * nx, mx * nx, 1.0, 0.0)
        stream = torch.cuda.current_stream().cuda_stream
        fn = lambda: _lib.check(_lib.load().blb200_gemm_heterogeneous(d, dm.data_ptr(), dn.data_ptr(), None, stream))
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        ms = time_launches(torch, fn, args.steps)
        kernel = bl.last_kernel_name()
        full = lambda: bl.gemm_strided_batched(d)
        for _ in range(3):
            full()
        torch.cuda.synchronize()
        ms_full = time_launches(torch, full, args.steps)
        out["hetero"].append({"dtype": dt, "max_m": mx, "max_n": nx, "k": k, "batch": batch, "ms": round(ms, 4),
                              "gflops_active": round(flops / (ms * 1e-3) / 1e9, 1), "kernel": kernel,
                              "ms_full_size_homogeneous": round(ms_full, 4)})
    print(json.dumps(out), flush=True)


def run_aux(args):
    """gemv and the elementwise helpers (the steps either side of gemm): achieved HBM GB/s against the
    measured copy bandwidth.  Algorithmic bytes: gemv reads A once (m*n*sizeof(T); x and y are noise and
    not counted); elementwise / axpby read two operands and write one (3*rows*cols*sizeof(T))."""
    import torch

    import batchlas_b200 as bl
    torch.cuda.set_device(0)
    peak, src = measured_peaks()
    tdt = {"s": torch.float32, "d": torch.float64, "c": torch.complex64, "z": torch.complex128}
    out = {"hbm_peak_gbs": peak, "peak_source": src, "gemv": [], "elementwise": []}
    gemv_cases = [("s", 32, 32, 1_000_000), ("s", 64, 64, 200_000), ("d", 256, 256, 8192), ("d", 1024, 1024, 512),
                  ("s", 8192, 8192, 8), ("d", 16384, 16384, 1), ("z", 128, 128, 8192)]
    ew_cases = [("s", 32, 32, 1_000_000, True), ("d", 1024, 1024, 128, True), ("d", 1000, 1000, 128, False),
                ("s", 32, 32, 500_000, False)]
    if args.aux_gemv:  # one small gemv case only: what a profiler captures
        dt, m, n, batch = args.aux_gemv.split(",")
        gemv_cases, ew_cases = [(dt, int(m), int(n), int(batch))], []
    for dt, m, n, batch in gemv_cases:
        t = tdt[dt]
        A = bl.fill(torch.empty(batch, n, m, dtype=t, device="cuda"), 42, 0)
        row = {"dtype": dt, "m": m, "n": n, "batch": batch, "ops": {}}
        nbytes = A.numel() * A.element_size()
        for op, name in ((0, "N"), (1, "T")):
            X = bl.fill(torch.empty(batch, n if op == 0 else m, dtype=t, device="cuda"), 42, 1)
            Y = bl.fill(torch.empty(batch, m if op == 0 else n, dtype=t, device="cuda"), 42, 2)
            fn = lambda: bl.linalg.gemv(A, X, Y, 1.5, -0.5, op)
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            ms = time_launches(torch, fn, args.steps)
            gbs = nbytes / (ms * 1e-3) / 1e9
            row["ops"][name] = {"ms": round(ms, 4), "hbm_gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 3)}
        out["gemv"].append(row)
        del A
    for dt, rows, cols, batch, packed in ew_cases:
        t = tdt[dt]
        ld = rows if packed else rows + 8
        def mk(i):
            back = bl.fill(torch.empty(batch, cols, ld, dtype=t, device="cuda"), 42, i)
            return back[:, :, :rows]
        A, B, C = mk(0), mk(1), mk(2)
        nbytes = 3 * batch * rows * cols * A.element_size()
        row = {"dtype": dt, "rows": rows, "cols": cols, "batch": batch, "packed": packed, "ops": {}}
        for name, fn in (("add", lambda: bl.linalg.add_into(A, B, C)),
                         ("axpby", lambda: bl.linalg.axpby_into(1.5, A, -0.5, B, C))):
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            ms = time_launches(torch, fn, args.steps)
            gbs = nbytes / (ms * 1e-3) / 1e9
            row["ops"][name] = {"ms": round(ms, 4), "hbm_gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 3)}
        out["elementwise"].append(row)
        del A, B, C
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "cublas"])
    ap.add_argument("--no-extra", action="store_true", help="skip the C1/C3/C4/C5 figures")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-cublas", action="store_true", help="skip the cuBLAS yardstick legs")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 2 s sustained figures of the configurations")
    ap.add_argument("--numa-bind", action="store_true", help="bind each rank to its GPU's NUMA node before pinning host buffers")
    ap.add_argument("--case", default="", help="profiling mode: CONFIG[:OP], e.g. C2:NT or C3:TN, or a packed shape such as d32x32x32:NN (1 GPU)")
    ap.add_argument("--batch", type=int, default=0, help="batch override for --case")
    ap.add_argument("--beta", type=float, default=-0.5, help="beta of a --case given as a shape (DTYPE MxNxK, e.g. d32x32x32:TN)")
    ap.add_argument("--kernel", default="auto", help="forced kernel for --case")
    ap.add_argument("--ld-extra", type=int, default=0, help="extra elements on every leading dimension of a --case")
    ap.add_argument("--sweep", default="", help="the reference's cube benchmark sizes against cuBLAS: all, s or d (1 GPU)")
    ap.add_argument("--hetero", action="store_true", help="time heterogeneous batches on the reference's pattern (1 GPU)")
    ap.add_argument("--aux", action="store_true", help="time gemv and the elementwise helpers against HBM bandwidth (1 GPU)")
    ap.add_argument("--aux-gemv", default="", help="with --aux: only this gemv case, DTYPE,M,N,BATCH (e.g. s,32,32,100000)")
    ap.add_argument("--level3", action="store_true", help="time symm/hemm/trmm/syrk/herk beside gemm (1 GPU)")
    ap.add_argument("--splitk", action="store_true", help="--case through blb200_gemm_splitk with planned scratch")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.impl == "cublas" and not args.case:
        raise SystemExit("--impl cublas times one configuration: give --case CONFIG[:OP] (the full run reports "
                         "cublas_gflops beside every figure already)")
    if args.case:
        run_case(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    if args.level3:
        run_level3(args)
        return
    if args.aux:
        run_aux(args)
        return
    if args.hetero:
        run_hetero(args)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
