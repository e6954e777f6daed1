"""The C++ device-buffer examples on real GPUs: one rank on one GPU, and one rank per GPU (up to four) when the
machine has several.  Ranks never share a GPU: their kernels wait on one another."""
import tempfile
from pathlib import Path

import pytest
import torch

from test_cpp_examples import CUDA_FLAGS, ROOT, _build, _run_ranks

pytestmark = pytest.mark.gpu


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [1] + ([min(n, 4)] if n >= 2 else [])


@pytest.mark.parametrize("name,expected", [("cuda_allreduce", 1), ("cuda_all_ops", 12)])
def test_cuda_example(name, expected):
    exe = Path(tempfile.mkdtemp(prefix="cclx_cuda_ex_")) / name
    _build(ROOT / "examples" / "cuda" / f"{name}.cpp", exe, extra=CUDA_FLAGS)
    for world in _worlds():
        outs = _run_ranks(exe, world, env={"CCL_CUDA_SYMM_HEAP_SIZE": "256M", "CCL_CUDA_TMP_BUF_SIZE": "32M"}, timeout=240)
        for rank, (rc, out, err) in enumerate(outs):
            assert rc == 0 and "FAILED" not in out, f"world {world} rank {rank} rc={rc}\n{out[-2000:]}\n{err[-2000:]}"
        passed = outs[0][1].count("PASSED")
        # one line per operation and datatype; send/recv only with more than one rank
        want = expected if (world == 1 or name == "cuda_allreduce") else expected + 2
        assert passed == want, outs[0][1]


def test_benchmark_tool_on_device_buffers():
    """`benchmark -b cuda`: every collective with its result check on device buffers (one rank per GPU)."""
    exe = Path(tempfile.mkdtemp(prefix="cclx_cuda_ex_")) / "benchmark_cuda"
    _build(ROOT / "examples" / "benchmark" / "benchmark.cpp", exe, extra=("-DCCL_BENCH_CUDA",) + CUDA_FLAGS)
    for world in _worlds():
        outs = _run_ranks(exe, world, extra_args=("-b", "cuda", "-l", "all", "-d", "float32,bfloat16", "-y", "17,4099,65536",
                                                  "-c", "all", "-i", "3", "-w", "2", "-p", "0"),
                          env={"CCL_CUDA_SYMM_HEAP_SIZE": "256M", "CCL_CUDA_TMP_BUF_SIZE": "32M"}, timeout=300)
        for rank, (rc, out, err) in enumerate(outs):
            assert rc == 0 and "CHECK FAILED" not in out, f"world {world} rank {rank} rc={rc}\n{out[-2000:]}\n{err[-2000:]}"
        assert outs[0][1].strip().endswith("PASSED"), outs[0][1][-1000:]
