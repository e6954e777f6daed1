"""CCL_PROCESS_LAUNCHER=pmix: local rank and local size are asked of the PMIx server through a libpmix opened at
run time.  The image has no PMIx, so the library is a stand-in (tests/mock_pmix/mock_pmix.c, built here with cc)
that serves the two keys the way a server does: the size to the wildcard rank as uint32, the local rank to the
process itself as uint16."""
import shutil
import subprocess
import tempfile
from pathlib import Path

import pytest

from mp_util import run_ranks

CC = shutil.which("cc") or shutil.which("gcc")
pytestmark = pytest.mark.skipif(CC is None, reason="no C compiler")


@pytest.fixture(scope="module")
def mock_lib():
    d = Path(tempfile.mkdtemp(prefix="cclx_mockpmix_"))
    lib = d / "libmockpmix.so"
    src = Path(__file__).resolve().parent / "mock_pmix" / "mock_pmix.c"
    subprocess.run([CC, "-shared", "-fPIC", "-O1", "-o", str(lib), str(src)], check=True)
    return str(lib)


def _coords(comm):
    return comm.local_rank, comm.local_size


def test_local_coordinates_come_from_the_pmix_server(mock_lib):
    # mp_util exports CCL_LOCAL_RANK / CCL_LOCAL_SIZE, which would take precedence: blank them out
    env = {"CCL_PROCESS_LAUNCHER": "pmix", "CCL_PMIX_LIBRARY_PATH": mock_lib, "MOCK_PMIX_LOCAL_RANK": "3",
           "MOCK_PMIX_LOCAL_SIZE": "7", "MOCK_PMIX_RANK": "11", "CCLX_TEST_UNSET": "CCL_LOCAL_RANK,CCL_LOCAL_SIZE"}
    for lr, ls in run_ranks(_coords, 2, env=env):
        assert (lr, ls) == (3, 7)


def test_falls_back_to_exported_variables_and_then_to_the_node_communicator(mock_lib):
    base = {"CCL_PROCESS_LAUNCHER": "pmix", "CCL_PMIX_LIBRARY_PATH": mock_lib, "MOCK_PMIX_FAIL_INIT": "1",
            "CCLX_TEST_UNSET": "CCL_LOCAL_RANK,CCL_LOCAL_SIZE"}
    # PMIx_Init fails (no PMIx-aware launcher): what the launcher exported is used
    for lr, ls in run_ranks(_coords, 2, env=dict(base, PMIX_LOCAL_RANK="1", PMIX_LOCAL_SIZE="4")):
        assert (lr, ls) == (1, 4)
    # nothing exported either, and no library at all: the ranks on this host, counted by the library itself
    out = run_ranks(_coords, 2, env=dict(base, CCL_PMIX_LIBRARY_PATH="/nonexistent/libpmix.so"))
    assert sorted(out) == [(0, 2), (1, 2)]
