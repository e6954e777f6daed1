"""The host path over libfabric (CCL_ATL_TRANSPORT=ofi): the library is opened at run time, a
reliable-datagram provider carries tagged messages, the closed-form checks of the socket transport's
suite must hold unchanged.  Needs a libfabric.so: CCL_OFI_LIBRARY_PATH, else the one that the
reference installation under baseline/_ref ships; skipped when neither exists."""
import os
from pathlib import Path

import numpy as np
import pytest

from mp_util import run_ranks
from test_cpu_collectives import _allreduce_matrix, _cfg1, _double_tree_ops, _others, _split_ops


def _libfabric():
    p = os.environ.get("CCL_OFI_LIBRARY_PATH")
    if p and Path(p).exists():
        return p
    q = Path(__file__).resolve().parent.parent / "baseline" / "_ref" / "opt" / "mpi" / "libfabric" / "lib" / "libfabric.so"
    return str(q) if q.exists() else None


LIB = _libfabric()
pytestmark = pytest.mark.skipif(LIB is None, reason="no libfabric.so available")


def _env(**extra):
    env = {"CCL_ATL_TRANSPORT": "ofi", "CCL_OFI_LIBRARY_PATH": LIB or ""}
    env.update(extra)
    return env


def _name_and_cfg1(comm):
    return comm.transport_name, _cfg1(comm)


def test_baseline_config1_over_libfabric():
    for name, errs in run_ranks(_name_and_cfg1, 2, env=_env()):
        assert name.startswith("ofi:"), name
        assert max(errs) < 1e-5


@pytest.mark.parametrize("provider", ["shm", "tcp"])
def test_every_collective_over_two_providers(provider):
    assert all(run_ranks(_others, 3, env=_env(FI_PROVIDER=provider)))


@pytest.mark.parametrize("algo", ["ring", "recursive_doubling", "rabenseifner", "nreduce", "double_tree", "2d", "ring_rma"])
def test_allreduce_algorithms_over_libfabric(algo):
    # ring_rma: the transport has no one-sided writes, the two-sided ring runs instead
    assert all(run_ranks(_allreduce_matrix, 3, algo, env=_env(CCL_ALLREDUCE=algo, CCL_ATL_RMA="1")))


def test_workers_partitions_and_trees_over_libfabric():
    env = _env(CCL_WORKER_COUNT="2", CCL_ALLGATHER="ring", CCL_ALLGATHERV="ring", CCL_ALLTOALL="naive",
               CCL_ATL_LARGE_MSG_SIZE="8192")
    assert all(run_ranks(_split_ops, 3, env=env))
    env = _env(CCL_BCAST="double_tree", CCL_BROADCAST="double_tree", CCL_REDUCE="double_tree", CCL_ALLREDUCE="double_tree")
    assert all(run_ranks(_double_tree_ops, 4, env=env))


def _long(comm):
    """Messages above any eager limit of the provider."""
    W, r = comm.size, comm.rank
    n = 3_000_000
    x = np.full(n, float(r + 1), np.float32)
    comm.allreduce(x).wait()
    assert np.all(x == W * (W + 1) / 2)
    nxt, prv = (r + 1) % W, (r - 1) % W
    got = np.zeros(500_000, np.int32)
    e1 = comm.recv(got, prv)
    e2 = comm.send(np.arange(500_000, dtype=np.int32) + r, nxt)
    e2.wait()
    e1.wait()
    assert np.array_equal(got, np.arange(500_000, dtype=np.int32) + prv)
    return True


@pytest.mark.parametrize("provider", ["shm", "tcp"])
def test_long_messages(provider):
    assert all(run_ranks(_long, 3, env=_env(FI_PROVIDER=provider)))


def test_missing_library_falls_back_to_the_socket_transport():
    res = run_ranks(_name_and_cfg1, 2, env={"CCL_ATL_TRANSPORT": "ofi", "CCL_OFI_LIBRARY_PATH": "/nonexistent/libfabric.so"})
    for name, errs in res:
        assert name.endswith("tcp") and not name.startswith("ofi") and max(errs) < 1e-5
