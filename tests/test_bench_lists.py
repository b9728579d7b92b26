"""bench.py's `--sweep` walks the cube sizes of BatchLAS's own batched-gemm benchmark.  Where the
reference tree is at hand (this container; not the GPU box) the list is checked against its source,
include/util/minibench.hh `CubeBatchSizes`."""
import os
import re

import pytest

import bench

# the reference checkout, when there is one: BATCHLAS_SOURCE_DIR, else a `reference` folder beside this repository
_ROOT = os.environ.get("BATCHLAS_SOURCE_DIR") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
REF = os.path.join(_ROOT, "include", "util", "minibench.hh")


def test_cube_list_is_well_formed():
    sizes = [s for s, _ in bench.CUBE_BATCH_SIZES]
    assert sizes == sorted(sizes) and len(set(sizes)) == len(sizes)
    for size, batches in bench.CUBE_BATCH_SIZES:
        assert size > 0 and list(batches) == sorted(batches) and batches[0] > 0


@pytest.mark.skipif(not os.path.exists(REF), reason="reference tree not present")
def test_cube_list_matches_the_reference():
    text = open(REF).read()
    body = text[text.index("inline void CubeBatchSizes("):]
    body = body[:body.index("\n}\n")]
    found = tuple((int(s), tuple(int(b) for b in bs.split(",")))
                  for s, bs in re.findall(r"add_batches\((\d+),\s*\{([^}]*)\}\)", body))
    assert found == bench.CUBE_BATCH_SIZES
