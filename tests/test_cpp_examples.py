"""Builds the C++ examples against the public header and runs them as plain processes
(no mpirun), like the reference's examples double as smoke tests; also the stub backend."""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIBDIR = ROOT / "oneccl_b200" / "lib"


def _build(src: Path, out: Path, extra=()):
    from oneccl_b200 import _lib

    _lib.load()  # makes sure the library exists
    cmd = ["g++", "-std=c++17", "-O1", str(src), "-o", str(out), f"-I{ROOT / 'csrc' / 'include'}",
           f"-I{ROOT / 'examples' / 'include'}", f"-L{LIBDIR}", "-lccl_b200", f"-Wl,-rpath,{LIBDIR}", "-pthread",
           *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


def _run_ranks(exe, world, extra_args=(), env=None, timeout=120):
    d = tempfile.mkdtemp(prefix="cclx_ex_")
    addr = os.path.join(d, "addr")
    e = dict(os.environ, **(env or {}))
    procs = [subprocess.Popen([str(exe), str(r), str(world), addr, *extra_args], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True, env=e) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, err = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, err = p.communicate()
        outs.append((p.returncode, o, err))
    return outs


@pytest.fixture(scope="module")
def bindir():
    return Path(tempfile.mkdtemp(prefix="cclx_bin_"))


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_allreduce_example(bindir, world):
    exe = bindir / "cpu_allreduce_test"
    if not exe.exists():
        _build(ROOT / "examples" / "cpu" / "cpu_allreduce_test.cpp", exe)
    outs = _run_ranks(exe, world)
    for rc, o, err in outs:
        assert rc == 0, err[-2000:]
    assert "PASSED" in outs[0][1]


def test_stub_backend_completes_without_transport(bindir):
    exe = bindir / "cpu_allreduce_test"
    if not exe.exists():
        _build(ROOT / "examples" / "cpu" / "cpu_allreduce_test.cpp", exe)
    # with the stub backend nothing is communicated: the example runs (and reports FAILED values)
    outs = _run_ranks(exe, 1, env={"CCL_BACKEND": "stub"})
    assert outs[0][0] in (0, 1)
    assert "PASSED" in outs[0][1] or "FAILED" in outs[0][1]


def test_benchmark_tool(bindir):
    exe = bindir / "benchmark"
    _build(ROOT / "examples" / "benchmark" / "benchmark.cpp", exe)
    outs = _run_ranks(exe, 2, extra_args=("allreduce", "1", "4096", "4", "2"))
    for rc, o, err in outs:
        assert rc == 0, err[-2000:]
    lines = [l for l in outs[0][1].splitlines() if l.startswith("allreduce,")]
    assert len(lines) == 13 and lines[-1].split(",")[1] == "4096"


def test_external_launcher_reforms_the_communicator(bindir):
    """No process manager: rank / size / address file on the command line, five incarnations."""
    exe = bindir / "external_launcher"
    _build(ROOT / "examples" / "external_launcher" / "external_launcher.cpp", exe)
    d = tempfile.mkdtemp(prefix="cclx_el_")
    world = 3
    procs = []
    for r in range(world):
        env = dict(os.environ, CCL_PROCESS_LAUNCHER="none", CCL_LOCAL_RANK=str(r), CCL_LOCAL_SIZE=str(world))
        procs.append(subprocess.Popen([str(exe), str(world), str(r), os.path.join(d, "addr"), "5"],
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env))
    outs = [p.communicate(timeout=180) + (p.returncode,) for p in procs]
    for o, err, rc in outs:
        assert rc == 0, err[-2000:]
    assert "PASSED after 5" in outs[0][0]


def test_point_to_point_latency_and_bandwidth_tools(bindir):
    lat, bw = bindir / "ccl_latency", bindir / "ccl_bw"
    _build(ROOT / "examples" / "pt2pt" / "ccl_latency.cpp", lat)
    _build(ROOT / "examples" / "pt2pt" / "ccl_bw.cpp", bw)
    outs = _run_ranks(lat, 2, extra_args=("1", "4096", "20"))
    for rc, o, err in outs:
        assert rc == 0, err[-2000:]
    rows = [l for l in outs[0][1].splitlines() if l and l[0].isdigit()]
    assert len(rows) == 13 and all(float(r.split(",")[1]) > 0 for r in rows) and "PASSED" in outs[0][1]
    outs = _run_ranks(bw, 2, extra_args=("1024", "262144", "4", "4"))
    for rc, o, err in outs:
        assert rc == 0, err[-2000:]
    rows = [l for l in outs[0][1].splitlines() if l and l[0].isdigit()]
    assert len(rows) == 9 and all(float(r.split(",")[1]) > 0 for r in rows) and "PASSED" in outs[0][1]


@pytest.mark.parametrize("world", [2, 4])
def test_all_operations_through_the_typed_api(bindir, world):
    exe = bindir / "cpu_all_ops_test"
    if not exe.exists():
        _build(ROOT / "examples" / "cpu" / "cpu_all_ops_test.cpp", exe)
    outs = _run_ranks(exe, world, timeout=240)
    for rc, o, err in outs:
        assert rc == 0, (o[-3000:], err[-2000:])
    text = outs[0][1]
    assert "FAILED" not in text
    # 5 datatypes x 2 iterations x 7 operation groups + the final line
    assert text.count("PASSED") == 5 * 2 * 7 + 1


CUDA_FLAGS = ("-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64", "-lcudart")


@pytest.mark.parametrize("name", ["cuda_allreduce", "cuda_all_ops"])
def test_cuda_examples_build_against_the_public_header(bindir, name):
    """The device-buffer examples compile and link with g++ and the CUDA runtime alone; without a GPU they say so
    and exit cleanly (their run on GPUs is tests/test_zzz_cuda_examples.py)."""
    import torch

    exe = bindir / name
    _build(ROOT / "examples" / "cuda" / f"{name}.cpp", exe, extra=CUDA_FLAGS)
    if not torch.cuda.is_available():
        outs = _run_ranks(exe, 1)
        assert outs[0][0] == 0 and "no CUDA device" in outs[0][1]
    # the benchmark tool with device buffers compiled in
    _build(ROOT / "examples" / "benchmark" / "benchmark.cpp", bindir / "benchmark_cuda", extra=("-DCCL_BENCH_CUDA",) + CUDA_FLAGS)


def test_benchmark_tool_options_and_result_check(bindir, tmp_path):
    """The option set of the reference's benchmark: lists of collectives / datatypes / reductions, explicit
    element counts, several operations in flight, in-place buffers, persistent operations, result check on
    every iteration, CSV file."""
    exe = bindir / "benchmark"
    if not exe.exists():
        _build(ROOT / "examples" / "benchmark" / "benchmark.cpp", exe)
    csv = tmp_path / "out.csv"
    outs = _run_ranks(exe, 3, extra_args=("-l", "all", "-d", "int8,bfloat16,float32", "-r", "sum,max", "-y", "1,17,1027",
                                          "-c", "all", "-i", "3", "-w", "1", "-n", "2", "-x", "on", "-o", str(csv)))
    for rc, o, err in outs:
        assert rc == 0 and "CHECK FAILED" not in o, o[-2000:] + err[-2000:]
    rows = [l for l in outs[0][1].splitlines() if l and not l.startswith("#") and "," in l]
    # 3 reducing collectives x 2 reductions + 5 others, x 3 datatypes x 3 counts
    assert len(rows) == (3 * 2 + 5) * 3 * 3
    assert all(len(r.split(",")) == 11 for r in rows)  # with wait_t_avg
    assert outs[0][1].strip().endswith("PASSED")
    assert len(csv.read_text().splitlines()) == len(rows) + 1
    # in place, not persistent, automatic iteration count
    outs = _run_ranks(exe, 2, extra_args=("-l", "allreduce,allgatherv,reduce-scatter,alltoall", "-q", "1", "-p", "0",
                                          "-f", "1024", "-t", "262144", "-i", "8", "-c", "last"))
    for rc, o, err in outs:
        assert rc == 0 and "CHECK FAILED" not in o, o[-2000:] + err[-2000:]
    reps = [int(l.split(",")[5]) for l in outs[0][1].splitlines() if l.startswith("allreduce,")]
    assert reps[0] == 8 and reps[-1] < 8  # 1 MiB of float32 runs fewer repetitions


def _free_port_pair():
    """A port p such that p + 1 is free as well (the store of a torchrun-style job listens next to the
    rendezvous port)."""
    import socket

    for _ in range(50):
        a = socket.socket()
        a.bind(("127.0.0.1", 0))
        p = a.getsockname()[1]
        b = socket.socket()
        try:
            b.bind(("127.0.0.1", p + 1))
        except OSError:
            a.close()
            b.close()
            continue
        a.close()
        b.close()
        return p
    raise RuntimeError("no free port pair")
