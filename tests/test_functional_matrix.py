"""Runs the C++ functional matrix (tests/functional/functional_test.cpp) as plain processes: every
collective x 12 datatypes x reductions x element counts x buffers in flight x in / out of place x start
and completion orders x wait / test x cached x synchronous, sampled by a deterministic hash, under several
runtime configurations.  The binary prints the failing configuration, so a failure here names it."""
import tempfile
from pathlib import Path

import pytest

from test_cpp_examples import ROOT, _build, _run_ranks


@pytest.fixture(scope="module")
def exe():
    out = Path(tempfile.mkdtemp(prefix="cclx_ft_")) / "functional_test"
    _build(ROOT / "tests" / "functional" / "functional_test.cpp", out)
    return out


CASES = [
    (2, "97", {}),
    (4, "53", {}),  # alltoallv blocks on both sides of the algorithm threshold within one call
    (3, "97", {"CCL_WORKER_COUNT": "2", "CCL_FUSION": "1", "CCL_PRIORITY": "lifo"}),
    (3, "97", {"CCL_CACHE_KEY": "full"}),  # cache hits differ between ranks (keys hold buffer addresses)
    (2, "97", {"FUNCTIONAL_TEST_DYNAMIC_POINTER": "1", "CCL_SCHED_CACHE_MAX_ENTRIES": "16"}),
    (3, "97", {"CCL_UNORDERED_COLL": "1", "CCL_ATL_SHM": "0", "CCL_MAX_FLOW_CREDITS": "2"}),
    (4, "97", {"CCL_ALLREDUCE": "ring_rma", "CCL_ATL_RMA": "1", "CCL_ALLTOALL": "scatter", "CCL_ALLTOALLV": "scatter",
               "CCL_REDUCE": "rabenseifner", "CCL_ALLGATHERV": "ring", "CCL_REDUCE_SCATTER": "ring",
               "CCL_RS_CHUNK_COUNT": "3", "CCL_RS_MIN_CHUNK_SIZE": "64", "CCL_CHUNK_COUNT": "2",
               "CCL_MIN_CHUNK_SIZE": "256"}),
    (4, "97", {"CCL_ALLREDUCE": "2d", "CCL_ALLREDUCE_2D_CHUNK_COUNT": "3", "CCL_ALLREDUCE_2D_MIN_CHUNK_SIZE": "64",
               "CCL_BCAST": "double_tree", "CCL_BROADCAST": "ring", "CCL_REDUCE": "double_tree",
               "CCL_ALLGATHERV": "multi_bcast", "CCL_ALLGATHER": "ring", "CCL_WORKER_OFFLOAD": "0"}),
]


@pytest.mark.parametrize("world,keep,env", CASES,
                         ids=["w2", "w4-dense", "w3-workers-fusion", "w3-full-cache-key", "w2-dynamic-pointers",
                              "w3-unordered-sockets",
                              "w4-ring-algorithms", "w4-tree-algorithms"])
def test_functional_matrix(exe, world, keep, env):
    outs = _run_ranks(exe, world, extra_args=(keep,), env=env, timeout=300)
    for rank, (rc, out, err) in enumerate(outs):
        failed = [l for l in out.splitlines() if l.startswith("FAILED")]
        assert rc == 0 and not failed, f"rank {rank} rc={rc}\n" + "\n".join(failed[:5]) + "\n" + err[-1500:]
    summary = [l for l in outs[0][1].splitlines() if l.startswith("functional:")]
    assert summary and "PASSED" in summary[0]
    assert int(summary[0].split()[1]) >= 2000
