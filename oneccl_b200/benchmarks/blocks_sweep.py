"""Grid width of the zero-copy collective kernels: time per (collective, size, thread blocks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m oneccl_b200.benchmarks.blocks_sweep [--out file.jsonl] [--colls allreduce,...] [--ordinary]

Buffers come from the symmetric heap (``--ordinary``: plain torch tensors, shared automatically), bf16,
in place where the collective allows it.  Device-timed with CUDA events, max over ranks.  The table that
comes out is what the launchers' automatic width (``blocks=0``) is derived from; ``blocks=0`` itself is
the last column, so a later run shows whether the automatic choice matches the best fixed width.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--colls", default="allreduce,reduce_scatter,allgather,alltoall")
    ap.add_argument("--sizes", default="65536,262144,1048576,4194304,16777216,67108864,268435456,1073741824")
    ap.add_argument("--blocks", default="1,2,4,8,16,32,64,148,0")
    ap.add_argument("--ordinary", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("CCL_CUDA_SYMM_HEAP_SIZE", "5G")
    from oneccl_b200.comm import init_from_env

    comm = init_from_env()
    grp = comm.device_group
    fout = open(args.out, "w") if (args.out and rank == 0) else None

    def maxr(t):
        x = torch.tensor([t], dtype=torch.float32, device="cuda")
        grp.allreduce(x, x, op="max")
        torch.cuda.synchronize()
        return float(x.item())

    dt = torch.bfloat16
    for coll in args.colls.split(","):
        for S in [int(x) for x in args.sizes.split(",")]:
            per = S // 2 // world
            if coll == "allreduce":
                n_in = n_out = S // 2
            elif coll == "reduce_scatter":
                n_in, n_out = per * world, per
            elif coll == "allgather":
                n_in, n_out = per, per * world
            else:
                n_in = n_out = per * world

            def alloc(n):
                if args.ordinary:
                    return torch.empty(n, device="cuda", dtype=dt)
                return grp.symm_empty((n,), dtype=dt)

            a = alloc(n_in)
            a.normal_()
            b = a if coll == "allreduce" else alloc(n_out)
            iters = 20 if S <= (64 << 20) else 6
            row = {"coll": coll, "bytes": S, "n_gpus": world, "ordinary": args.ordinary, "us": {}}
            for w in [int(x) for x in args.blocks.split(",")]:
                if coll == "allreduce":
                    fn = lambda: grp.allreduce(a, a, blocks=w)  # noqa: E731
                elif coll == "reduce_scatter":
                    fn = lambda: grp.reduce_scatter(a, b, blocks=w)  # noqa: E731
                elif coll == "allgather":
                    fn = lambda: grp.allgatherv(a, b, blocks=w)  # noqa: E731
                else:
                    fn = lambda: grp.alltoall(a, b, blocks=w)  # noqa: E731
                for _ in range(3):
                    fn()
                grp.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                row["us"][str(w)] = round(maxr(e0.elapsed_time(e1) / iters * 1e3), 2)
            best = min((v, k) for k, v in row["us"].items() if k != "0")
            row["best_blocks"], row["best_us"], row["auto_us"] = int(best[1]), best[0], row["us"].get("0")
            if rank == 0:
                line = json.dumps(row)
                print(line, flush=True)
                if fout:
                    fout.write(line + "\n")
                    fout.flush()
            if not args.ordinary:
                grp.symm_free(a)
                if b is not a:
                    grp.symm_free(b)
            del a, b
    grp.check()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
