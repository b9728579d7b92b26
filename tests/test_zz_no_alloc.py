"""The allocation-free split-K entry point (blb200_gemm_splitk_static) against the ordinary one.

Some callers may not allocate device memory at all — the whole of HBM belongs to their own pool, or
an allocator call is not allowed where they run — so they can neither lease scratch for
blb200_gemm_splitk nor let the library call cudaMalloc.  For them the partials live in a fixed
8 MiB array inside the library.  This file is collected last on purpose (its name sorts after the
others): a run that stops at the first failure has then already exercised everything else.

Checked here, through the C ABI: two calls in a row (the second on a smaller problem, so stale
partials of the first are still lying in the array) give the same C as blb200_gemm_splitk with
caller scratch and meet the entrywise bound of the parity tests
    |C - (alpha*S + beta*C0)| <= 4*K*eps*(|alpha|*|A|*|B| + |beta|*|C0|);
a plan beyond the capacity is refused with the library's "too large" status.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tests._cases import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def _desc(bl, p, dA, dB, dC):
    return bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), p.dtype, p.op_a, p.op_b, p.m, p.n, p.k, p.batch,
                        p.lda, p.ldb, p.ldc, p.stride_a, p.stride_b, p.stride_c, p.alpha, p.beta)


def test_static_scratch_split_k_matches_caller_scratch_split_k(lib):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    import batchlas_b200 as bl
    L = bl._lib.load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    cap = L.blb200_gemm_splitk_static_capacity()
    assert cap == 8 << 20

    cases = [("d", "T", "N", 96, 80, 5000, 2, 2.0, -0.5, 8),     # first call: 8 splits, ~1 MB of partials
             ("z", "C", "N", 24, 20, 900, 1, 1.0 + 0.5j, 0.0, 3),  # second call: smaller, stale partials around it
             ("s", "N", "T", 64, 64, 4096, 1, 1.5, 1.0, 0)]        # third: library-chosen split count
    for dt, oa, ob, m, n, k, batch, alpha, beta, splits in cases:
        p = oracle.make_problem(dt, oa, ob, m, n, k, batch, ldc=m + 2, alpha=alpha, beta=beta)
        A, B, C0 = make_inputs(p)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        dC_static, dC_ref = torch.from_numpy(C0).cuda(), torch.from_numpy(C0).cuda()

        need = ctypes.c_size_t(0)
        used = L.blb200_gemm_splitk_plan(_desc(bl, p, dA, dB, dC_ref), splits, ctypes.byref(need))
        assert used >= 2 and 0 < need.value <= cap
        ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        bl._lib.check(L.blb200_gemm_splitk(_desc(bl, p, dA, dB, dC_ref), splits, ws.data_ptr(), need.value, stream))

        bl._lib.check(L.blb200_gemm_splitk_static(_desc(bl, p, dA, dB, dC_static), splits, stream))
        torch.cuda.synchronize()
        assert bl.last_kernel_name() == "splitk"

        got, ref = dC_static.cpu().numpy(), dC_ref.cpu().numpy()
        assert np.array_equal(got, ref), f"{dt} {oa}{ob}: static-scratch result differs from caller-scratch result"
        bad, worst = oracle.check(p, A, B, C0, got)
        assert bad == 0, (dt, oa, ob, worst)
        assert oracle.untouched_outside_window(p, C0, got)

    # "allocates nothing": with every kernel already loaded by the calls above, one more call leaves
    # the device's free memory exactly where it was
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    bl._lib.check(L.blb200_gemm_splitk_static(_desc(bl, p, dA, dB, dC_static), splits, stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before

    # a plan that does not fit the fixed array is refused, nothing is launched
    big = bl.make_desc(dA.data_ptr(), dB.data_ptr(), dC_ref.data_ptr(), 1, 0, 0, 512, 512, 1 << 20, 1, 512, 1 << 20, 512,
                       0, 0, 0)
    need = ctypes.c_size_t(0)
    assert L.blb200_gemm_splitk_plan(big, 16, ctypes.byref(need)) == 16 and need.value > cap
    assert L.blb200_gemm_splitk_static(big, 16, stream) == bl._lib.E_TOO_LARGE
    assert "exceeds the fixed capacity" in L.blb200_status_string(bl._lib.E_TOO_LARGE).decode()
    assert bl.device_status() == 0
