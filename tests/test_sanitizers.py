"""Host runtime under AddressSanitizer / ThreadSanitizer: an instrumented copy of the library is built
into build/lib-<sanitizer>/ and the all-operations C++ example runs against it as three ranks, in several
runtime modes.  Two extra full builds: opt-in with CCLX_RUN_SANITIZERS=1."""
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

pytestmark = pytest.mark.skipif(os.environ.get("CCLX_RUN_SANITIZERS") != "1",
                                reason="set CCLX_RUN_SANITIZERS=1 (builds two instrumented copies of the library)")

MODES = [{}, {"CCL_FUSION": "1"}, {"CCL_WORKER_COUNT": "2"}, {"CCL_WORKER_OFFLOAD": "0"},
         {"CCL_ATL_SHM": "0", "CCL_PRIORITY": "lifo"}]


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_all_operations_under_sanitizer(sanitizer):
    from oneccl_b200._build import build_native

    lib = build_native(sanitize=sanitizer)
    exe = Path(tempfile.mkdtemp(prefix="cclx_san_")) / f"all_ops_{sanitizer}"
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer",
           str(ROOT / "examples" / "cpu" / "cpu_all_ops_test.cpp"), "-o", str(exe), f"-I{ROOT / 'csrc' / 'include'}",
           f"-I{ROOT / 'examples' / 'include'}", f"-L{lib.parent}", "-lccl_b200", f"-Wl,-rpath,{lib.parent}", "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    marker = "ERROR: AddressSanitizer" if sanitizer == "address" else "WARNING: ThreadSanitizer"
    for mode in MODES:
        addr = os.path.join(tempfile.mkdtemp(prefix="cclx_san_addr_"), "addr")
        env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0", **mode)
        procs = [subprocess.Popen([str(exe), str(rk), "3", addr], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                  text=True, env=env) for rk in range(3)]
        outs = [p.communicate(timeout=300)[0] for p in procs]
        for o in outs:
            assert marker not in o and "LeakSanitizer" not in o, (mode, o[-4000:])
        assert outs[0].count("PASSED") == 71, (mode, outs[0][-2000:])
    # the MPI transport with two worker threads per rank (their own endpoints; then one lock around every MPI call),
    # against the stand-in MPI library of tests/mock_mpi
    cc = shutil.which("cc") or shutil.which("gcc")
    if cc:
        mock = exe.parent / "libmockmpi.so"
        subprocess.run([cc, "-shared", "-fPIC", "-O1", "-o", str(mock), str(ROOT / "tests" / "mock_mpi" / "mock_mpi.c"),
                        "-lpthread"], check=True)
        for level in ("3", "2"):
            job = tempfile.mkdtemp(prefix="cclx_san_mpi_")
            addr = os.path.join(job, "addr")
            procs = []
            for rk in range(3):
                env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0",
                           CCL_ATL_TRANSPORT="mpi", CCL_MPI_LIBRARY_PATH=str(mock), CCL_WORKER_COUNT="2", MOCK_MPI_DIR=job,
                           MOCK_MPI_RANK=str(rk), MOCK_MPI_SIZE="3", MOCK_MPI_THREAD_LEVEL=level)
                procs.append(subprocess.Popen([str(exe), str(rk), "3", addr], stdout=subprocess.PIPE,
                                              stderr=subprocess.STDOUT, text=True, env=env))
            outs = [p.communicate(timeout=300)[0] for p in procs]
            for o in outs:
                assert marker not in o and "LeakSanitizer" not in o, ("mpi", level, o[-4000:])
            assert outs[0].count("PASSED") == 71, ("mpi", level, outs[0][-2000:])
    # the functional matrix, thinly sampled, over the paths the example does not reach: one-sided writes
    # (as messages: the sanitizers cannot see a cross-memory copy), rendezvous for every message, bounded cache
    ft = exe.parent / f"functional_{sanitizer}"
    cmd[cmd.index(str(ROOT / "examples" / "cpu" / "cpu_all_ops_test.cpp"))] = str(ROOT / "tests" / "functional" /
                                                                              "functional_test.cpp")
    cmd[cmd.index(str(exe))] = str(ft)
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    for mode in ({"CCL_ALLREDUCE": "ring_rma", "CCL_ATL_RMA": "1", "CCL_ATL_CMA": "0"},
                 {"CCL_ATL_CMA_THRESHOLD": "1", "CCL_SCHED_CACHE_MAX_ENTRIES": "4", "CCL_WORKER_COUNT": "2"},
                 {"CCL_RS_CHUNK_COUNT": "3", "CCL_RS_MIN_CHUNK_SIZE": "64", "CCL_CHUNK_COUNT": "2", "CCL_MIN_CHUNK_SIZE": "64",
                  "CCL_ALLREDUCE": "ring", "CCL_REDUCE_SCATTER": "ring", "CCL_ALLTOALLV": "scatter"}):
        addr = os.path.join(tempfile.mkdtemp(prefix="cclx_san_addr_"), "addr")
        env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0", **mode)
        procs = [subprocess.Popen([str(ft), str(rk), "3", addr, "797"], stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True, env=env) for rk in range(3)]
        outs = [p.communicate(timeout=900)[0] for p in procs]
        for o in outs:
            assert marker not in o and "LeakSanitizer" not in o, (mode, o[-4000:])
        assert "PASSED" in outs[0].splitlines()[-1], (mode, outs[0][-2000:])
