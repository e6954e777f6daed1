"""Point-to-point on device buffers between two GPUs: this library's send / recv against NCCL's.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P \
        -m oneccl_b200.benchmarks.p2p_bench [--out file.jsonl] [--min-bytes 8] [--max-bytes 256M]

The counterpart of the reference's ccl_latency / ccl_bw examples (examples/pt2pt/src/ccl_latency.cpp,
ccl_bw.cpp: half round-trip time of a ping-pong, and a window of back-to-back sends answered by one
acknowledgement) with the timing moved onto the device: CUDA events on the launching stream, max over the two
ranks.  Per size: ``lat_us`` = half the time of one ping-pong, ``uni_gbs`` = bytes / time of a window of 16
messages 0 -> 1, ``bidi_gbs`` = both directions at once (send and recv posted in one group), each for "ours"
and "nccl".
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .coll_bench import parse_size


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--min-bytes", default="8")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == 2, "two ranks"
    torch.cuda.set_device(local)
    from oneccl_b200.comm import group_end, group_start, init_from_env

    comm = init_from_env()
    grp = comm.device_group
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peer = 1 - rank
    fout = open(args.out, "w") if (args.out and rank == 0) else None

    def maxr(t):
        x = torch.tensor([t], dtype=torch.float32, device="cuda")
        grp.allreduce(x, x, op="max")
        torch.cuda.synchronize()
        return float(x.item())

    def timed(fn, iters):
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
        return maxr(e0.elapsed_time(e1) / iters * 1e-3)

    S = parse_size(args.min_bytes)
    hi = parse_size(args.max_bytes)
    WINDOW = 16
    while S <= hi:
        a = torch.empty(S, dtype=torch.uint8, device="cuda").random_(0, 255)
        b = torch.empty(S, dtype=torch.uint8, device="cuda")
        iters = args.iters if S <= (16 << 20) else max(5, args.iters // 5)
        row = {"bytes": S, "iters": iters}

        # ---- ours
        def ours_pingpong():
            if rank == 0:
                comm.send(a, peer)
                comm.recv(b, peer)
            else:
                comm.recv(b, peer)
                comm.send(a, peer)

        def ours_window():
            for _ in range(WINDOW):
                if rank == 0:
                    comm.send(a, peer)
                else:
                    comm.recv(b, peer)

        def ours_bidi():
            group_start()
            comm.send(a, peer)
            comm.recv(b, peer)
            group_end()

        # ---- nccl
        def nccl_pingpong():
            if rank == 0:
                dist.send(a, peer)
                dist.recv(b, peer)
            else:
                dist.recv(b, peer)
                dist.send(a, peer)

        def nccl_window():
            for _ in range(WINDOW):
                if rank == 0:
                    dist.send(a, peer)
                else:
                    dist.recv(b, peer)

        def nccl_bidi():
            ops = [dist.P2POp(dist.isend, a, peer), dist.P2POp(dist.irecv, b, peer)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()

        for name, pp, win, bidi in (("ours", ours_pingpong, ours_window, ours_bidi),
                                    ("nccl", nccl_pingpong, nccl_window, nccl_bidi)):
            row[name + "_lat_us"] = timed(pp, iters) / 2 * 1e6
            row[name + "_uni_gbs"] = S * WINDOW / timed(win, max(3, iters // 4)) / 1e9
            row[name + "_bidi_gbs"] = S / timed(bidi, iters) / 1e9  # per direction
        if rank == 0:
            line = json.dumps(row)
            print(line, flush=True)
            if fout:
                fout.write(line + "\n")
                fout.flush()
        del a, b
        S *= 4
    grp.check()
    dist.barrier()
    dist.destroy_process_group()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
