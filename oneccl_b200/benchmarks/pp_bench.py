"""Pipeline-parallel training step (GPipe fill / drain) over device send / recv, against the same schedule on
NCCL's point-to-point.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port P \
        -m oneccl_b200.benchmarks.pp_bench [--layers 24] [--micro 8] [--micro-batch 4] [--seq 1024] [--steps 5]

The model is the stack of transformer blocks of GPT-2 medium (hidden 1024, 16 heads, bf16, random weights) cut into one
stage per GPU; the activation that crosses a stage boundary is [micro_batch, seq, 1024] in bf16 (8 MiB at the
defaults).  A step is all forwards, all backwards (gradients accumulate), timed with CUDA events on every rank,
max over ranks.  Both arms run the same modules and the same schedule (``run_gpipe``); only the transport of the
stage differs: this library's send / recv kernels on a side stream, or ``torch.distributed.send`` / ``recv`` on
NCCL.  Also printed: the time of the stage's compute alone (same micro-batches, no transfers), which gives the ideal
step time compute * (micro + stages - 1) / micro of a fill / drain schedule.
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
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    from oneccl_b200.comm import init_from_env
    from oneccl_b200.models.gpt2 import Block, GPT2Config
    from oneccl_b200.parallel.pp import PipelineStage, run_gpipe

    comm = init_from_env()
    grp = comm.device_group
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    cfg = GPT2Config(args.layers, 16, 1024, args.seq)
    per = args.layers // world
    torch.manual_seed(1 + rank)
    stage_mod = torch.nn.Sequential(*[Block(cfg) for _ in range(per)]).cuda().to(torch.bfloat16)
    act = torch.empty(args.micro_batch, args.seq, cfg.d_model, device="cuda", dtype=torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(3)
    micro = [torch.randn(act.shape, generator=gen, device="cuda").to(torch.bfloat16) for _ in range(args.micro)]

    class NcclStage(PipelineStage):
        def _send(self, t, peer):
            dist.send(t, peer)

        def _recv(self, buf, peer):
            dist.recv(buf, peer)

    def maxr(t):
        x = torch.tensor([t], dtype=torch.float32, device="cuda")
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return maxr(e0.elapsed_time(e1) / args.steps)

    def step_with(stage):
        def f():
            for p in stage_mod.parameters():
                p.grad = None
            run_gpipe(stage, stage_mod, micro, act)
        return f

    def compute_only():
        for p in stage_mod.parameters():
            p.grad = None
        for m in range(args.micro):
            x = micro[m].clone().requires_grad_(True)
            y = stage_mod(x)
            y.float().mean().backward() if rank == world - 1 else y.backward(micro[m])

    out = {"stages": world, "layers_per_stage": per, "micro_batches": args.micro,
           "activation_bytes": act.numel() * 2, "steps": args.steps, "warmup": args.warmup}
    out["compute_only_ms"] = timed(compute_only)
    out["ideal_ms"] = out["compute_only_ms"] * (args.micro + world - 1) / args.micro
    out["ours_ms"] = timed(step_with(PipelineStage(comm)))
    grp.check()
    out["nccl_ms"] = timed(step_with(NcclStage(comm)))
    out["nccl_over_ours"] = out["nccl_ms"] / out["ours_ms"]
    out["ours_over_ideal"] = out["ours_ms"] / out["ideal_ms"]
    out["tokens_per_s_ours"] = args.micro * args.micro_batch * args.seq / (out["ours_ms"] * 1e-3)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
