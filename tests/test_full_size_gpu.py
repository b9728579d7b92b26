"""The five benchmark configurations at their FULL sizes (SGEMM 64^3 x 10 000; SGEMM 32^3 x 1 000 000
NT and TN; DGEMM 256^3 x 2 048, ld 264, all four op pairs; ZGEMM 128 x 64 x 256 x 8 192 A^H B; DGEMM
1024^3 x 512), on the seeded synthetic inputs the benchmark uses.  The long-double arbiter is O(mnk)
per item on one core, so at these sizes it checks sampled items; EVERY item is held to the checksum
identity of tests/_props.py (float64 device reductions, none of the library's kernels) against the
entrywise acceptance bound summed over the item.  beta == 0 configurations run over a NaN-filled C.
"""
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["C1", "C2", "C3", "C4", "C5"])
def test_full_size_configuration_every_item(lib, name):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    import bench
    import batchlas_b200 as bl
    torch.cuda.set_device(0)
    c = bench.configs()[name]
    need = 3.2 * c["batch"] * max(c["m"] * c["k"], c["k"] * c["n"], c["m"] * c["n"]) * bench.ELEM_BYTES[c["dtype"]]
    if torch.cuda.mem_get_info()[0] < need:
        pytest.skip("not enough free device memory for the full-size configuration")
    tens, mt = bench.alloc_config(bl, torch, c, c["batch"], 0, torch.device("cuda", 0))
    restore = bench.restore_fn(bl, torch, c, tens, mt, 0)
    for op in c["ops"]:
        d = bench.desc_for(bl, c, op, tens, mt, c["batch"])
        if c["beta"] == 0:
            tens["c"].fill_(float("nan"))   # beta == 0 must not read C
        worst_sampled = bench.verify_sample(bl, torch, c, op, tens, mt, c["batch"], 0, n_check=3) if c["beta"] != 0 else 0.0
        if c["beta"] == 0:
            # verify_sample restores C from the generator; here C must stay NaN before the launch
            worst_all = bench.checksum_all_items(torch, c, op, tens, mt, c["batch"], lambda: bl.gemm_strided_batched(d),
                                                 lambda: tens["c"].fill_(float("nan")))
        else:
            worst_all = bench.checksum_all_items(torch, c, op, tens, mt, c["batch"], lambda: bl.gemm_strided_batched(d), restore)
        assert worst_all < 1.0 and worst_sampled < 1.0, (name, op, worst_all, worst_sampled)
        assert not torch.isnan(tens["c"]).any()
    assert bl.device_status() == 0
    del tens
    torch.cuda.empty_cache()
