"""Collective bandwidth sweep against NCCL on the same GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m oneccl_b200.benchmarks.coll_bench [--colls allreduce,reduce_scatter,allgather,alltoall] \
        [--dtypes bf16,fp32] [--min-bytes 8] [--max-bytes 1G] [--warmup 20] [--iters 100] [--out file.jsonl]

Method (the reference's benchmark tool measures start+wait on the host,
examples/benchmark/src/benchmark.cpp:47-222; here timing is on the device):
buffers filled with seeded normal(0,1) values, `warmup` untimed and `iters`
timed launches between two CUDA events on the launching stream, time = max
over ranks / iters.  Bus bandwidth uses the NCCL-tests convention: allreduce
2(n-1)/n * S/t, reduce_scatter / allgather / alltoall (n-1)/n * S/t with S the
full message size.  Every size is reported for three arms: "ours" (ordinary
device tensors: staged through the symmetric heap below 256 KiB, shared with the
peers automatically and reduced zero-copy from there on), "ours_symm" (tensors
allocated from the symmetric heap: zero-copy, NVLS when available) and "nccl",
with the ratios NCCL time / our time per arm ("ordinary_vs_nccl",
"symmetric_vs_nccl"; above 1 = faster than NCCL).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mul = 1
    for suf, m in (("K", 1 << 10), ("M", 1 << 20), ("G", 1 << 30)):
        if s.endswith(suf):
            mul = m
            s = s[:-1]
    return int(float(s) * mul)


def time_op(fn, warmup, iters, sync):
    for _ in range(warmup):
        fn()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3  # seconds


def time_graph(fn, iters, sync):
    """Device time of one launch with the host out of the loop: `iters` launches are
    captured into a CUDA graph and replayed (one untimed replay, one timed)."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(iters):
            fn()
    sync()
    g.replay()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--graph", action="store_true",
                    help="time graph replays (device time without per-launch host overhead)")
    ap.add_argument("--colls", default="allreduce,reduce_scatter,allgather,alltoall")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", default="8")
    ap.add_argument("--max-bytes", default="1G")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--out", default="")
    ap.add_argument("--arms", default="ours,ours_symm,nccl")
    ap.add_argument("--heap", default="6G")
    ap.add_argument("--shrink-large", action="store_true",
                    help="a fifth of the iterations above 64 MiB (the counts used are recorded in every row)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("CCL_CUDA_SYMM_HEAP_SIZE", args.heap)
    os.environ.setdefault("CCL_CUDA_TMP_BUF_SIZE", "256M")
    from oneccl_b200.comm import init_from_env

    comm = init_from_env()
    grp = comm.device_group
    arms = args.arms.split(",")
    if "nccl" in arms:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    sizes = []
    s = lo
    while s <= hi:
        sizes.append(s)
        s *= 2
    dts = {"bf16": torch.bfloat16, "fp32": torch.float32}
    rows = []
    fout = open(args.out, "w") if (args.out and rank == 0) else None

    def sync():
        grp.barrier()
        torch.cuda.synchronize()

    def maxr(t):
        x = torch.tensor([t], dtype=torch.float32, device="cuda")
        grp.allreduce(x, x, op="max")
        torch.cuda.synchronize()
        return float(x.item())

    for coll in args.colls.split(","):
        for dname in args.dtypes.split(","):
            dt = dts[dname]
            esz = torch.empty((), dtype=dt).element_size()
            for S in sizes:
                if S < esz:
                    continue
                # S = full message: allreduce buffer, or the gathered / scattered total
                if coll == "allreduce":
                    n_in = n_out = S // esz
                else:
                    per = max(1, S // esz // world)
                    n_in, n_out = (per * world, per) if coll == "reduce_scatter" else (
                        (per, per * world) if coll == "allgather" else (per * world, per * world))
                if n_in == 0 or n_out == 0:
                    continue
                Sb = max(n_in, n_out) * esz
                shrink = args.shrink_large and Sb > (64 << 20)
                iters = max(10, args.iters // 5) if shrink else args.iters
                warm = max(3, args.warmup // 5) if shrink else args.warmup
                gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
                factor = {"allreduce": 2.0 * (world - 1) / world}.get(coll, (world - 1) / world)
                row = {"coll": coll, "dtype": dname, "bytes": Sb, "n_gpus": world, "iters": iters, "warmup": warm,
                       "timing": "graph" if args.graph else "stream"}
                for arm in arms:
                    symm = arm == "ours_symm"
                    if arm == "nccl":
                        a = torch.randn(n_in, generator=gen, device="cuda").to(dt)
                        b = torch.empty(n_out, device="cuda", dtype=dt)
                        if coll == "allreduce":
                            fn = lambda: dist.all_reduce(a)  # noqa: E731
                        elif coll == "reduce_scatter":
                            fn = lambda: dist.reduce_scatter_tensor(b, a)  # noqa: E731
                        elif coll == "allgather":
                            fn = lambda: dist.all_gather_into_tensor(b, a)  # noqa: E731
                        else:
                            fn = lambda: dist.all_to_all_single(b, a)  # noqa: E731
                    else:
                        if symm:
                            a = grp.symm_empty((n_in,), dtype=dt)
                            b = grp.symm_empty((n_out,), dtype=dt) if coll != "allreduce" else a
                            a.copy_(torch.randn(n_in, generator=gen, device="cuda").to(dt))
                        else:
                            a = torch.randn(n_in, generator=gen, device="cuda").to(dt)
                            b = torch.empty(n_out, device="cuda", dtype=dt) if coll != "allreduce" else a
                        if coll == "allreduce":
                            fn = lambda: grp.allreduce(a, a)  # noqa: E731
                        elif coll == "reduce_scatter":
                            fn = lambda: grp.reduce_scatter(a, b)  # noqa: E731
                        elif coll == "allgather":
                            fn = lambda: grp.allgatherv(a, b)  # noqa: E731
                        else:
                            fn = lambda: grp.alltoallv(a, b)  # noqa: E731
                    t = maxr(time_graph(fn, iters, sync) if args.graph else time_op(fn, warm, iters, sync))
                    row[arm + "_us"] = t * 1e6
                    row[arm + "_busbw_gbs"] = factor * Sb / t / 1e9
                    if symm:
                        grp.symm_free(a)
                        if b is not a:
                            grp.symm_free(b)
                    del a, b
                if "nccl" in arms:
                    if "ours" in arms:
                        row["ordinary_vs_nccl"] = row["nccl_us"] / row["ours_us"]
                    if "ours_symm" in arms:
                        row["symmetric_vs_nccl"] = row["nccl_us"] / row["ours_symm_us"]
                rows.append(row)
                if rank == 0:
                    line = json.dumps(row)
                    print(line, flush=True)
                    if fout:
                        fout.write(line + "\n")
                        fout.flush()
    torch.cuda.synchronize()
    grp.check()
    if "nccl" in arms:
        dist.barrier()
        dist.destroy_process_group()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
