"""How wide should a gradient allreduce be while backward is still running?

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m oneccl_b200.benchmarks.ddp_overlap_bench [--out file.jsonl] [--timeline prefix]

Three measurements in one process group, all device-timed (CUDA events, max over ranks):

1. ``allreduce_alone``: the symmetric in-place bf16 allreduce of one 25 MB bucket (and of 100 MB) with nothing
   else on the GPU, for a range of grid widths: bus bandwidth per width.
2. ``step``: the data-parallel GPT-2-medium step (batch 8 x 1024 per GPU) for a range of widths of the overlapped
   bucket allreduces, with the side stream at high and at normal priority, launched eagerly and as one CUDA
   graph.  The width whose step is shortest is what ``oneccl_b200.parallel.ddp.OVERLAP_BLOCKS`` records.
3. ``timeline`` (``--timeline``): for one eager step per-bucket ready / start / end times against the end of
   backward, written per rank.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--timeline", default="")
    ap.add_argument("--widths", default="4,8,12,16,24,32,48,64,0")
    ap.add_argument("--step-widths", default="8,16,24,32,64,0")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--skip-graph", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("CCL_CUDA_SYMM_HEAP_SIZE", "3G")
    os.environ.setdefault("CCL_CUDA_WAIT_TIMEOUT_MS", "20000")
    from oneccl_b200.comm import init_from_env
    from oneccl_b200.models.gpt2 import GPT2, GPT2Config
    from oneccl_b200.parallel.ddp import DataParallel, GraphedTrainStep, train_step

    comm = init_from_env()
    grp = comm.device_group
    fout = open(args.out, "w") if (args.out and rank == 0) else None

    def emit(row):
        if rank == 0:
            line = json.dumps(row)
            print(line, flush=True)
            if fout:
                fout.write(line + "\n")
                fout.flush()

    def sync():
        grp.barrier()
        torch.cuda.synchronize()

    def maxr(t):
        x = torch.tensor([t], dtype=torch.float32, device="cuda")
        grp.allreduce(x, x, op="max")
        torch.cuda.synchronize()
        return float(x.item())

    # ---- 1. the allreduce alone, per grid width
    for mb in (25, 100):
        n = mb * (1 << 20) // 2
        buf = grp.symm_empty((n,), dtype=torch.bfloat16)
        buf.normal_()
        for w in [int(x) for x in args.widths.split(",")]:
            for _ in range(5):
                grp.allreduce(buf, buf, blocks=w, scale=1.0 / world)
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            iters = 30
            e0.record()
            for _ in range(iters):
                grp.allreduce(buf, buf, blocks=w, scale=1.0 / world)
            e1.record()
            torch.cuda.synchronize()
            t = maxr(e0.elapsed_time(e1) / iters * 1e-3)
            emit({"what": "allreduce_alone", "mbytes": mb, "blocks": w, "n_gpus": world, "us": t * 1e6,
                  "busbw_gbs": 2.0 * (world - 1) / world * n * 2 / t / 1e9})
        grp.symm_free(buf)

    # ---- 2. the training step per width / priority / launch mode
    cfg = GPT2Config.named(args.model)
    B, S = 8, cfg.seq_len
    gen = torch.Generator().manual_seed(1000 + rank)
    idx = [torch.randint(0, cfg.vocab, (B, S), generator=gen).cuda() for _ in range(args.steps)]
    tgt = [torch.randint(0, cfg.vocab, (B, S), generator=gen).cuda() for _ in range(args.steps)]

    def run(width, high, graph, timeline=""):
        torch.manual_seed(1234)
        model = GPT2(cfg, fused_ops=True).cuda().to(torch.bfloat16)
        ddp = DataParallel(model, grp, comm_blocks=width, high_priority=high)
        opt = ddp.make_optimizer(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, max_norm=1.0, device_step=graph)
        if graph:
            step = GraphedTrainStep(ddp, opt, idx[0], tgt[0])
        else:
            def step(i, t):
                return train_step(ddp, opt, i, t)
        for w in range(args.warmup):
            step(idx[w], tgt[w])
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(args.steps):
            step(idx[k], tgt[k])
        e1.record()
        sync()
        ms = maxr(e0.elapsed_time(e1)) / args.steps
        emit({"what": "step", "blocks": width, "high_priority": high, "graph": graph, "n_gpus": world,
              "ms_per_step": ms, "tokens_per_s": world * B * S / (ms * 1e-3)})
        if timeline and not graph:
            ddp.record_timeline = True
            for k in range(2):
                train_step(ddp, opt, idx[k], tgt[k])
            torch.cuda.synchronize()
            tl = ddp.timeline()
            tl.update({"rank": rank, "blocks": width, "n_gpus": world})
            with open(f"{timeline}.rank{rank}.json", "w") as f:
                json.dump(tl, f)
            ddp.record_timeline = False
        del step
        ddp.close()
        del ddp, opt, model
        gc.collect()
        torch.cuda.empty_cache()
        return ms

    widths = [int(x) for x in args.step_widths.split(",")]
    best = None
    for w in widths:
        ms = run(w, True, False)
        if best is None or ms < best[0]:
            best = (ms, w)
    run(best[1], False, False)  # the side stream without priority, at the best width
    if args.timeline:
        run(best[1], True, False, args.timeline)
    if not args.skip_graph:
        for w in sorted({best[1], 16, 0}):
            run(w, True, True)
    grp.check()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
