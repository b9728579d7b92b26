"""Failure detection without a GPU fault: every wait inside the ring kernels is bounded, and a wait
that runs out records a code in a device status word that the host reads (the counterpart of
BatchLAS surfacing asynchronous errors at Queue::wait_and_throw, src/util/queue-impl.cc).

The expiry branch is made to run by the library's own self-test: one warp waits, with the same
bounded-wait routine the kernels use and a limit of a few hundred polls, on a barrier that nothing
ever completes.  The kernel returns normally; nothing traps, faults or hangs; the device is used for
an ordinary product straight afterwards.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tests._cases import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu

WAIT_SELFTEST = 901  # BLB200_WAIT_SELFTEST in include/blb200.h


def test_bounded_wait_runs_out_and_is_reported_then_cleared(lib):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    import batchlas_b200 as bl
    L = bl._lib.load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    assert bl.device_status() == 0
    # limits outside 1..65536 polls are refused before anything is launched
    assert L.blb200_selftest_wait_expiry(0, stream) == bl._lib.E_TOO_LARGE
    assert L.blb200_selftest_wait_expiry(1 << 20, stream) == bl._lib.E_TOO_LARGE
    try:
        bl._lib.check(L.blb200_selftest_wait_expiry(300, stream))
        assert bl.device_status() == WAIT_SELFTEST      # the wait gave up and said so
        assert bl.device_status() == WAIT_SELFTEST      # sticky until cleared
    finally:
        bl._lib.check(L.blb200_device_status_reset())
    assert bl.device_status() == 0

    # the context is intact: a ring kernel (forced by id) runs and meets the parity bound
    p = oracle.make_problem("d", "T", "N", 16, 16, 16, 8 * 160, alpha=1.5, beta=-0.5)
    A, B, C0 = make_inputs(p, tail=0)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C0))
    desc = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, p.batch,
                        p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta, "small_ring")
    bl.gemm_strided_batched(desc)
    torch.cuda.synchronize()
    assert bl.last_kernel_name() == "small_ring"
    got = dC.cpu().numpy()
    bad, worst = oracle.check(p, A, B, C0, got, items=list(range(0, p.batch, 97)))
    assert bad == 0, worst
    assert bl.device_status() == 0
