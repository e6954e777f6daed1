#!/usr/bin/env python
"""Headline benchmark: data-parallel GPT-2-medium training throughput (tokens/s).

Config (the data-parallel row of the baseline): 24 layers, d_model 1024,
16 heads, seq 1024, vocab 50257, bf16 weights with fp32 master copies, AdamW,
per-GPU batch 8 of uniform-random token ids, gradients reduced in 25 MB buckets
by the library's own allreduce kernels overlapped with backward.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line.  ``value`` is the device-timed whole-job tokens/s
(max over ranks), ``e2e`` the same metric through the public API including the
per-step host->device copy of the batch from pinned memory and the
device->host read of the loss.

Arms (``--impl``):

* ``ours`` (default): the library's layer kernels, flat symmetric gradients, its own bucket allreduce
  on a high-priority side stream, fused loss and flat AdamW, the step replayed from one CUDA graph
  (``--no-graph``: launched eagerly).  Unless ``--no-arms`` is given the same process then measures the
  comparison arms below with the same K and W and reports them under ``arms``; ``vs_baseline`` is
  the headline value divided by the ``nccl`` arm (stock PyTorch over NCCL), the baseline that can be
  measured on this hardware.
* ``nccl``: the same network on stock PyTorch modules, ``torch.nn.parallel.DistributedDataParallel``
  over NCCL, ``F.cross_entropy``, torch's fused AdamW.
* ``nccl-flat``: the ``ours`` step launched eagerly with one change: the bucket allreduce is NCCL's.  Against
  ``ours --no-graph`` it isolates what the collective kernels themselves contribute.
* ``ccl-ddp``: stock ``DistributedDataParallel`` over this library's ``torch.distributed`` backend
  ``"ccl"``, with a communication hook that has the allreduce average in place (scale fused).
* ``reference``: the unmodified reference library (``baseline/_ref``, built from its CMake project:
  CPU path over libfabric; it has no CUDA path).  A stock Hugging Face GPT-2 and torch AdamW run on the
  GPU; gradients travel to pinned host memory, through the reference's ``ccl::allreduce`` and back.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODEL = "gpt2-medium"
PER_GPU_BATCH = 8


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl", "nccl-flat", "ccl-ddp"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--batch", type=int, default=PER_GPU_BATCH)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--comm-blocks", type=int, default=-1,
                    help="thread blocks of a gradient allreduce that overlaps backward (-1 = the measured default, "
                         "0 = the kernel's own full-width choice)")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-arms", action="store_true", help="measure only the requested arm")
    ap.add_argument("--timeline", default="", help="write the per-bucket timeline of one eager step to this file")
    return ap.parse_args()


def env_world():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


class Harness:
    """What every arm shares: the synthetic batches, barriers, max over ranks, the timed regions."""

    def __init__(self, args, cfg, world, rank, local_rank):
        import torch

        self.torch = torch
        self.args, self.cfg, self.world, self.rank, self.local_rank = args, cfg, world, rank, local_rank
        self.B, self.S = args.batch, cfg.seq_len
        n_batches = args.steps + args.warmup
        gen = torch.Generator().manual_seed(1000 + rank)
        # synthetic data: uniform-random token ids, a fresh pinned batch per step
        self.host_idx = [torch.randint(0, cfg.vocab, (self.B, self.S), generator=gen).pin_memory() for _ in range(n_batches)]
        self.host_tgt = [torch.randint(0, cfg.vocab, (self.B, self.S), generator=gen).pin_memory() for _ in range(n_batches)]
        self.dev_idx = [t.cuda() for t in self.host_idx[: args.steps]]
        self.dev_tgt = [t.cuda() for t in self.host_tgt[: args.steps]]
        self.h2d = sum(t.numel() * t.element_size() for t in (self.host_idx[0], self.host_tgt[0]))
        self.group = None  # the library's device group ("ours"); None: torch.distributed is initialised
        self.tokens_per_step = world * self.B * self.S

    def barrier(self):
        if self.world > 1:
            if self.group is not None:
                self.group.barrier()
            else:
                self.torch.distributed.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        torch = self.torch
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float32, device="cuda")
        if self.group is not None:
            self.group.allreduce(t, t, op="max")
        else:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.cuda.synchronize()
        return float(t.item())

    def measure(self, step, clocks=None, e2e=True):
        """W warm-up steps, K device-timed steps on device-resident batches, then (e2e) K steps whose batch comes
        from pinned host memory and whose loss is read back every step."""
        torch, args = self.torch, self.args
        for w in range(args.warmup):
            loss = step(self.dev_idx[w % len(self.dev_idx)], self.dev_tgt[w % len(self.dev_tgt)])
        self.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        if clocks:
            clocks.begin()
        ev0.record()
        for k in range(args.steps):
            loss = step(self.dev_idx[k], self.dev_tgt[k])
        ev1.record()
        self.barrier()
        if clocks:
            clocks.end()
        ms_dev = self.max_over_ranks(ev0.elapsed_time(ev1))
        out = {"ms_dev": ms_dev, "value": self.tokens_per_step * args.steps / (ms_dev / 1e3),
               "ms_per_step": ms_dev / args.steps, "final_loss": float(loss.item())}
        if not e2e:
            return out
        self.barrier()
        if clocks:
            clocks.begin()
        t0 = time.perf_counter()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record()
        for k in range(args.steps):
            idx = self.host_idx[args.warmup + k].cuda(non_blocking=True)
            tgt = self.host_tgt[args.warmup + k].cuda(non_blocking=True)
            loss = step(idx, tgt)
            _ = float(loss.item())  # 4-byte device->host read of the step's result
        ev3.record()
        self.barrier()
        if clocks:
            clocks.end()
        ms_e2e = self.max_over_ranks(ev2.elapsed_time(ev3))
        out.update({"ms_e2e": ms_e2e, "e2e_value": self.tokens_per_step * args.steps / (ms_e2e / 1e3),
                    "e2e_ms_per_step": ms_e2e / args.steps, "wall_e2e": time.perf_counter() - t0})
        return out


def init_torch_dist(h: Harness):
    import torch
    import torch.distributed as dist

    if h.world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", h.local_rank))


# ---- arms ---------------------------------------------------------------------------------------------

def arm_ours(h: Harness, graph: bool, clocks=None, e2e=True, reducer=None, timeline_path=""):
    """The library's own step.  `reducer` replaces the bucket allreduce (the nccl-flat arm)."""
    import torch

    from oneccl_b200.models.gpt2 import GPT2
    from oneccl_b200.ops import train as train_ops
    from oneccl_b200.parallel.ddp import DataParallel, GraphedTrainStep, train_step

    args = h.args
    torch.manual_seed(1234)
    model = GPT2(h.cfg, fused_ops=True).cuda().to(torch.bfloat16)
    ddp = DataParallel(model, h.ours_group, bucket_mb=args.bucket_mb, comm_blocks=args.comm_blocks, reducer=reducer)
    opt = ddp.make_optimizer(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, max_norm=1.0, device_step=graph)
    if graph:
        step = GraphedTrainStep(ddp, opt, h.dev_idx[0], h.dev_tgt[0])
        per_step = step.launches_per_step
    else:
        def step(idx, tgt):
            return train_step(ddp, opt, idx, tgt)

        c0 = train_ops.launch_count + ddp.launches
        step(h.dev_idx[0], h.dev_tgt[0])  # also the first warm-up step
        per_step = train_ops.launch_count + ddp.launches - c0
    out = h.measure(step, clocks, e2e)
    out["launches_per_step"] = per_step
    out["buckets"] = len(ddp.buckets)
    if timeline_path and not graph:
        ddp.record_timeline = True
        for k in range(2):
            train_step(ddp, opt, h.dev_idx[k], h.dev_tgt[k])
        torch.cuda.synchronize()
        tl = ddp.timeline()
        tl["rank"] = h.rank
        ddp.record_timeline = False
        with open(f"{timeline_path}.rank{h.rank}.json", "w") as f:
            json.dump(tl, f)
    del step
    ddp.close()
    del ddp, opt, model
    gc.collect()
    torch.cuda.empty_cache()
    return out


def arm_torch_ddp(h: Harness, backend: str, e2e=False):
    """Stock PyTorch: nn modules, DistributedDataParallel over `backend` ("nccl" or this library's "ccl"),
    F.cross_entropy on fp32 logits, clip_grad_norm_, torch's fused AdamW."""
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as TorchDDP

    from oneccl_b200.models.gpt2 import GPT2

    torch.manual_seed(1234)
    model = GPT2(h.cfg, fused_ops=False).cuda().to(torch.bfloat16)
    net = model
    if h.world > 1:
        pg = None
        if backend == "ccl":
            import oneccl_b200.torch_backend  # noqa: F401  (registers the backend)

            pg = dist.new_group(backend="ccl")
        net = TorchDDP(model, device_ids=[h.local_rank], bucket_cap_mb=h.args.bucket_mb, gradient_as_bucket_view=True,
                       process_group=pg)
        if backend == "ccl":
            def avg_hook(state, bucket):
                # one allreduce per bucket that also divides by the world size (scale fused into the kernel)
                work = dist.all_reduce(bucket.buffer(), op=dist.ReduceOp.AVG, group=state, async_op=True)
                return work.get_future().then(lambda f: f.value()[0])

            net.register_comm_hook(pg, avg_hook)
    decay, no_decay = model.decay_split()
    topt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                             lr=3e-4, betas=(0.9, 0.95), fused=True)

    def step(idx, tgt):
        topt.zero_grad(set_to_none=True)
        lg = net(idx)
        loss = torch.nn.functional.cross_entropy(lg.float(), tgt.reshape(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        topt.step()
        return loss

    return h.measure(step, None, e2e)


def arm_reference(h: Harness):
    """The unmodified reference as the gradient allreduce of a stock PyTorch training step."""
    import torch
    from transformers import GPT2Config as HFConfig, GPT2LMHeadModel

    from baseline.reference_arm import ReferenceComm

    c = h.cfg
    torch.manual_seed(1234)
    hf = HFConfig(n_layer=c.n_layer, n_embd=c.d_model, n_head=c.n_head, n_positions=c.seq_len, vocab_size=c.vocab,
                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, attn_implementation="sdpa", use_cache=False)
    model = GPT2LMHeadModel(hf).cuda().to(torch.bfloat16)
    params = [p for p in model.parameters() if p.requires_grad]
    decay = [p for p in params if p.dim() >= 2]
    no_decay = [p for p in params if p.dim() < 2]
    topt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                             lr=3e-4, betas=(0.9, 0.95), fused=True)
    ref = None
    if h.world > 1:
        store = torch.distributed.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"),
                                           int(os.environ.get("MASTER_PORT", "29500")) + 17, h.world, h.rank == 0)
        ref = ReferenceComm(h.rank, h.world, h.local_rank, h.world, store)
        total = sum(p.numel() for p in params)
        flat_dev = torch.empty(total, dtype=torch.bfloat16, device="cuda")
        flat_host = torch.empty(total, dtype=torch.bfloat16).pin_memory()
        h.ref = ref

    def step(idx, tgt):
        topt.zero_grad(set_to_none=True)
        lg = model(idx).logits
        loss = torch.nn.functional.cross_entropy(lg.float().view(-1, lg.shape[-1]), tgt.reshape(-1))
        loss.backward()
        if ref is not None:
            grads = [p.grad for p in params]
            torch.cat([g.reshape(-1) for g in grads], out=flat_dev)
            flat_host.copy_(flat_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            ref.allreduce_(flat_host)
            flat_dev.copy_(flat_host, non_blocking=True)
            flat_dev.mul_(1.0 / h.world)
            o = 0
            for g in grads:
                g.copy_(flat_dev[o:o + g.numel()].view_as(g))
                o += g.numel()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        topt.step()
        return loss

    return h.measure(step, None, True)


# ---- main ---------------------------------------------------------------------------------------------

def base_record(h: Harness, impl: str, res: dict, clocks_summary, launches):
    args = h.args
    return {
        "metric": "dp_training_tokens_per_sec",
        "value": res["value"],
        "unit": "tokens/s",
        "n_gpus": h.world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": res["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform-random token ids, random-init weights",
        "impl": impl,
        "config": {"model": args.model, "global_batch": h.world * h.B, "seq_len": h.S, "parallelism": f"dp{h.world}",
                   "per_gpu_batch": h.B, "optimizer": "AdamW fp32 master", "bucket_mb": args.bucket_mb,
                   "l2": "working set (0.7 GB weights + activations) far larger than the 126 MB L2"},
        "clocks": clocks_summary,
        "e2e": {"value": res.get("e2e_value"), "unit": "tokens/s", "h2d_bytes_per_step": h.h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": res.get("e2e_ms_per_step"), "wall_s": res.get("wall_e2e")},
        "gpu_launches": launches,
        "final_loss": res["final_loss"],
    }


def main():
    args = parse()
    world, rank, local_rank = env_world()
    if args.impl == "reference":
        from baseline import reference_arm

        why = reference_arm.available()
        if why:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            return 0
    os.environ.setdefault("CCL_CUDA_WAIT_TIMEOUT_MS", "20000")
    os.environ.setdefault("CCL_CUDA_SYMM_HEAP_SIZE", "2G")
    import torch

    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # launched directly: re-exec under torchrun so that one process drives one GPU
            import subprocess

            port = 29000 + os.getpid() % 2000
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), __file__] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    torch.backends.cuda.matmul.allow_tf32 = True

    from oneccl_b200.models.gpt2 import GPT2Config
    from oneccl_b200.utils.clocks import ClockSampler

    cfg = GPT2Config.named(args.model)
    h = Harness(args, cfg, world, rank, local_rank)

    # the clock sampler starts before the warm-up (nvidia-smi needs a moment to come up); only the samples
    # that arrive inside the timed regions are summarised.  Rank 0 watches every GPU of the job.
    clocks = ClockSampler(list(range(world)) if rank == 0 else [])
    clocks.__enter__()
    comm = None
    try:
        if args.impl in ("ours", "nccl-flat"):
            from oneccl_b200.ops.device_group import DeviceGroup

            if world == 1:
                h.ours_group = DeviceGroup.emulated(1, heap_bytes=(2 << 30), staging_bytes=16 << 20)
            else:
                from oneccl_b200.comm import init_from_env

                comm = init_from_env()
                h.ours_group = comm.device_group
        if args.impl == "ours":
            h.group = h.ours_group
            graph = not args.no_graph
            res = arm_ours(h, graph, clocks, e2e=True)
            clocks.__exit__(None, None, None)
            out = base_record(h, "ours", res, clocks.summary(), res["launches_per_step"] * args.steps)
            out["config"]["step_launch"] = "one CUDA graph per step" if graph else "eager"
            out["config"]["buckets"] = res["buckets"]
            arms = {}

            def aux(name, fn):
                """A comparison arm must not take the headline down with it: an error that every rank raises is
                recorded under the arm's name and the run goes on."""
                try:
                    return fn()
                except Exception as e:  # noqa: BLE001 - reported, not hidden
                    arms[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                    return None

            if not args.no_arms:
                # the same step launched eagerly (also what the per-bucket timeline is taken from)
                r = aux("ours_eager", lambda: arm_ours(h, False, None, e2e=False, timeline_path=args.timeline))
                if r:
                    arms["ours_eager"] = {"value": r["value"], "ms_per_step": r["ms_per_step"]}
                h.group = None
                init_torch_dist(h)
                if world > 1:
                    r = aux("nccl_flat_eager", lambda: arm_ours(h, False, None, e2e=False, reducer="nccl"))
                    if r:
                        arms["nccl_flat_eager"] = {"value": r["value"], "ms_per_step": r["ms_per_step"],
                                                   "what": "this library's step with NCCL as the bucket allreduce"}
                r = aux("nccl", lambda: arm_torch_ddp(h, "nccl", e2e=True))
                if r:
                    arms["nccl"] = {"value": r["value"], "ms_per_step": r["ms_per_step"], "e2e_value": r["e2e_value"],
                                    "what": "stock PyTorch modules, DistributedDataParallel over NCCL, torch fused AdamW"}
                    out["vs_baseline"] = out["value"] / r["value"]
                    out["e2e"]["vs_baseline"] = out["e2e"]["value"] / r["e2e_value"]
                if world > 1:
                    r = aux("ccl_ddp", lambda: arm_torch_ddp(h, "ccl", e2e=False))
                    if r:
                        arms["ccl_ddp"] = {"value": r["value"], "ms_per_step": r["ms_per_step"],
                                           "what": "stock DistributedDataParallel over this library's torch backend"}
                out["arms"] = arms
                out["baseline_note"] = ("the reference publishes no number; vs_baseline is value / arms.nccl.value "
                                        "measured in this run")
        else:
            if args.impl == "nccl-flat":
                h.group = None
                init_torch_dist(h)
                res = arm_ours(h, False, clocks, e2e=True, reducer="nccl")
                launches = res["launches_per_step"] * args.steps
            elif args.impl == "reference":
                res = arm_reference(h) if world == 1 else None
                if world > 1:
                    init_torch_dist(h)
                    res = arm_reference(h)
                launches = 0
            else:
                init_torch_dist(h)
                res = arm_torch_ddp(h, "nccl" if args.impl == "nccl" else "ccl", e2e=True)
                launches = 0
            clocks.__exit__(None, None, None)
            out = base_record(h, args.impl, res, clocks.summary(), launches)
            if args.impl == "reference":
                out["config"]["optimizer"] = "torch AdamW (fused) on bf16 parameters"
                out["config"]["reference"] = ("oneCCL 2021.14 built from its CMake project (CPU path, libfabric); stock "
                                              "Hugging Face GPT-2 + torch AdamW on the GPU, gradients through pinned "
                                              "host memory and ccl::allreduce (the reference has no CUDA path)")
        if rank == 0:
            print(json.dumps(out))
    finally:
        clocks.__exit__(None, None, None)
    if getattr(h, "ref", None) is not None:
        h.ref.close()
    if comm is not None:
        comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
