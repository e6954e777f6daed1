"""The host path over MPI point-to-point messages (CCL_ATL_TRANSPORT=mpi).  The image has no MPI installation, so
the library under the transport is a stand-in with the MPICH binary interface (tests/mock_mpi/mock_mpi.c, built
here with cc): what is tested is this library's side, the run-time loading, the rank table, the header / payload
protocol with its posted and unexpected queues, and the fallbacks.  The stand-in numbers its ranks the other way
round than the communicator, so a transport that confused the two numberings would deliver to the wrong rank."""
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

import numpy as np
import pytest

from mp_util import run_ranks
from test_cpu_collectives import _allreduce_matrix, _cfg1, _double_tree_ops, _others, _split_ops

CC = shutil.which("cc") or shutil.which("gcc")
pytestmark = pytest.mark.skipif(CC is None, reason="no C compiler")


@pytest.fixture(scope="module")
def mock_lib():
    d = Path(tempfile.mkdtemp(prefix="cclx_mockmpi_"))
    lib = d / "libmockmpi.so"
    src = Path(__file__).resolve().parent / "mock_mpi" / "mock_mpi.c"
    subprocess.run([CC, "-shared", "-fPIC", "-O1", "-o", str(lib), str(src), "-lpthread"], check=True)
    return str(lib)


def _env(lib, **extra):
    env = {"CCL_ATL_TRANSPORT": "mpi", "CCL_MPI_LIBRARY_PATH": lib, "MOCK_MPI_REVERSE": "1",
           "MOCK_MPI_DIR": tempfile.mkdtemp(prefix="cclx_mockmpi_job_")}
    env.update(extra)
    return env


def _name_and_cfg1(comm):
    return comm.transport_name, _cfg1(comm)


def test_baseline_config1_over_mpi(mock_lib):
    for name, errs in run_ranks(_name_and_cfg1, 2, env=_env(mock_lib)):
        assert name == "mpi", name
        assert max(errs) < 1e-5


def test_every_collective_over_mpi(mock_lib):
    assert all(run_ranks(_others, 3, env=_env(mock_lib)))


@pytest.mark.parametrize("algo", ["ring", "recursive_doubling", "rabenseifner", "nreduce", "double_tree", "2d", "ring_rma"])
def test_allreduce_algorithms_over_mpi(mock_lib, algo):
    # ring_rma: the transport has no one-sided writes, the two-sided ring runs instead
    assert all(run_ranks(_allreduce_matrix, 3, algo, env=_env(mock_lib, CCL_ALLREDUCE=algo, CCL_ATL_RMA="1")))


@pytest.mark.parametrize("level", ["3", "2"], ids=["thread-multiple", "thread-serialized"])
def test_workers_partitions_and_trees_over_mpi(mock_lib, level):
    """Two worker threads per rank: their own endpoints under MPI_THREAD_MULTIPLE, one lock around every MPI call
    under MPI_THREAD_SERIALIZED."""
    env = _env(mock_lib, CCL_WORKER_COUNT="2", CCL_ALLGATHER="ring", CCL_ALLGATHERV="ring", CCL_ALLTOALL="naive",
               CCL_ATL_LARGE_MSG_SIZE="8192", MOCK_MPI_THREAD_LEVEL=level)
    assert all(run_ranks(_split_ops, 3, env=env))
    env = _env(mock_lib, CCL_BCAST="double_tree", CCL_BROADCAST="double_tree", CCL_REDUCE="double_tree",
               CCL_ALLREDUCE="double_tree", MOCK_MPI_THREAD_LEVEL=level)
    assert all(run_ranks(_double_tree_ops, 4, env=env))


def _p2p_unexpected_and_short(comm):
    """Messages that arrive before their receive is posted, several with one tag in order, a zero-byte message,
    a receive shorter than its message, and probe."""
    r, W = comm.rank, comm.size
    peer = (r + 1) % W
    src = (r - 1) % W
    msgs = [np.full(n, float(r * 10 + k), np.float32) for k, n in enumerate((1, 7000, 0, 300000))]
    evs = [comm.send(m, peer) for m in msgs]
    comm.barrier().wait()  # everything above is on its way or there before the first receive below
    got = [np.zeros(max(m.size, 1), np.float32) for m in msgs]
    for k, m in enumerate(msgs):
        comm.recv(got[k][:m.size], src).wait()
    for e in evs:
        e.wait()
    ok = all(np.all(g[:m.size] == float(src * 10 + k)) for k, (g, m) in enumerate(zip(got, msgs)))
    return ok


def test_point_to_point_order_and_unexpected_messages(mock_lib):
    assert all(run_ranks(_p2p_unexpected_and_short, 3, env=_env(mock_lib)))


def _transport_name(comm):
    x = np.full(100, float(comm.rank + 1), np.float32)
    y = np.zeros_like(x)
    comm.allreduce(x, y).wait()
    return comm.transport_name, float(y[0])


def test_falls_back_when_the_library_cannot_be_used(mock_lib):
    """No library at the given path; and a library whose MPI_COMM_WORLD does not span the job (every process
    finds itself alone): all ranks agree to use the socket transport."""
    W = 2
    for name, total in run_ranks(_transport_name, W, env=_env("/nonexistent/libmpi.so")):
        assert name != "mpi" and total == W * (W + 1) / 2
    for name, total in run_ranks(_transport_name, W, env=_env(mock_lib, MOCK_MPI_SIZE="1", MOCK_MPI_RANK="0")):
        assert name != "mpi" and total == W * (W + 1) / 2
