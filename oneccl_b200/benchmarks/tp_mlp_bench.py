"""Tensor-parallel MLP block: fused (all-gather+GEMM, GEMM+reduce-scatter) against
NCCL collectives + cuBLAS on the same GPUs.

    python -m torch.distributed.run --nproc-per-node 8 ... -m oneccl_b200.benchmarks.tp_mlp_bench

Shapes: X [8192 x 4096] normal(0,1) sharded over tokens, W_up [4096 x 14336] and
W_down [14336 x 4096] normal(0, 0.02) sharded over the 14336 dimension, bf16.
Timing: CUDA events around `iters` block evaluations after `warmup`, max over
ranks.  Roofline of the fused block = max(compute at the measured GEMM peak,
bytes over NVLink at the measured 770 GB/s per direction) summed over its two
kernels; the fraction achieved is printed with both denominators.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--n-comm", type=int, default=0)
    ap.add_argument("--peak-tflops", type=float, default=1400.3)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("CCL_CUDA_SYMM_HEAP_SIZE", "2G")
    from oneccl_b200.comm import init_from_env
    from oneccl_b200.parallel.tp import TensorParallelMLP

    comm = init_from_env()
    grp = comm.device_group
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mlp = TensorParallelMLP(grp, args.tokens, args.d_model, args.d_ff, n_comm=args.n_comm)
    per = args.tokens // world
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    x_local = torch.randn(per, args.d_model, generator=gen, device="cuda").to(torch.bfloat16)
    mlp.x_shard.copy_(x_local)

    def fused():
        return mlp.forward()

    def unfused_ours():
        return mlp.forward_unfused(x_local)

    xf = torch.empty((args.tokens, args.d_model), dtype=torch.bfloat16, device="cuda")
    yb = torch.empty((per, args.d_model), dtype=torch.bfloat16, device="cuda")

    def nccl_cublas():
        dist.all_gather_into_tensor(xf, x_local)
        h = torch.nn.functional.silu(xf @ mlp.w_up.t())
        part = h @ mlp.w_down.t()
        dist.reduce_scatter_tensor(yb, part)
        return yb

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        grp.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
        grp.allreduce(t, t, op="max")
        torch.cuda.synchronize()
        return float(t.item())

    # correctness of the fused path against the unfused one
    y_f = fused().float().clone()
    y_u = nccl_cublas().float()
    torch.cuda.synchronize()
    err = (y_f - y_u).abs().max().item()
    scale = y_u.abs().max().item()
    res = {"config": {"tokens": args.tokens, "d_model": args.d_model, "d_ff": args.d_ff, "tp": world, "dtype": "bf16"},
           "max_abs_diff_vs_nccl_cublas": err, "ref_abs_max": scale}
    res["fused_ms"] = timeit(fused)
    # the two fused stages on their own, and the bare GEMMs they contain (no communication)
    res["fused_up_ms"] = timeit(lambda: mlp.up.run(None, mlp.w_up, out=mlp.h))
    res["fused_down_ms"] = timeit(lambda: mlp.down.run(mlp.h, mlp.w_down, out=mlp.y))
    from oneccl_b200.ops.gemm import gemm_bf16
    tmp = torch.empty((args.tokens, args.d_model), dtype=torch.bfloat16, device="cuda")
    res["gemm_up_only_ms"] = timeit(lambda: gemm_bf16(xf, mlp.w_up, out=mlp.h, epilogue="silu"))
    res["gemm_down_only_ms"] = timeit(lambda: gemm_bf16(mlp.h, mlp.w_down, out=tmp))
    res["unfused_ours_ms"] = timeit(unfused_ours)
    res["nccl_cublas_ms"] = timeit(nccl_cublas)
    flops = 2.0 * args.tokens * args.d_model * (args.d_ff // world) * 2
    t_compute = flops / (args.peak_tflops * 1e12) * 1e3
    bytes_ag = (world - 1) / world * args.tokens * args.d_model * 2
    bytes_rs = (world - 1) / world * args.tokens * args.d_model * 2
    t_up = max(flops / 2 / (args.peak_tflops * 1e12), bytes_ag / (args.link_gbs * 1e9)) * 1e3
    t_down = max(flops / 2 / (args.peak_tflops * 1e12), bytes_rs / (args.link_gbs * 1e9)) * 1e3
    res["roofline_ms"] = t_up + t_down
    res["compute_only_ms"] = t_compute
    res["fraction_of_roofline"] = (t_up + t_down) / res["fused_ms"]
    res["speedup_vs_nccl_cublas"] = res["nccl_cublas_ms"] / res["fused_ms"]
    res["peaks_used"] = {"bf16_tflops_sustained_measured": args.peak_tflops, "nvlink_gbs_measured": args.link_gbs}
    if rank == 0:
        print(json.dumps(res), flush=True)
    mlp.close()
    dist.barrier()
    dist.destroy_process_group()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
