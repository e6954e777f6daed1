"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on one GPU.

    python -m oneccl_b200.benchmarks.gemm_bench [--shapes MxNxK,...] [--iters 20]

Timing: CUDA events around `iters` back-to-back launches after 5 warm-up
launches; operands are rotated through a pool larger than the L2 so that every
launch streams from HBM."""
from __future__ import annotations

import argparse
import json

import torch

from ..ops.gemm import gemm_bf16


def time_fn(fn, pool, iters, warmup=5):
    for i in range(warmup):
        fn(*pool[i % len(pool)])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(*pool[i % len(pool)])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x1792x4096,8192x4096x1792,8192x8192x8192,4096x4096x4096")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ctas", type=int, default=0)
    args = ap.parse_args()
    rows = []
    for spec in args.shapes.split(","):
        M, N, K = (int(v) for v in spec.split("x"))
        per = (M * K + N * K + M * N) * 2
        n_pool = max(2, min(8, (256 << 20) // per + 1))
        pool = [(torch.randn(M, K, device="cuda").to(torch.bfloat16),
                 (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16),
                 torch.empty(M, N, device="cuda", dtype=torch.bfloat16)) for _ in range(n_pool)]
        ours = time_fn(lambda a, w, o: gemm_bf16(a, w, out=o, ctas=args.ctas), pool, args.iters)
        ref = time_fn(lambda a, w, o: torch.matmul(a, w.t(), out=o), pool, args.iters)
        a, w, o = pool[0]
        gemm_bf16(a, w, out=o, check=True)
        err = (o.float() - a.float() @ w.float().t()).abs().max().item()
        fl = 2.0 * M * N * K
        rows.append({"shape": spec, "ours_ms": ours, "cublas_ms": ref, "ours_tflops": fl / ours / 1e9,
                     "cublas_tflops": fl / ref / 1e9, "ratio": ref / ours, "max_abs_err": err})
        print(json.dumps(rows[-1]))
    return rows


if __name__ == "__main__":
    main()
