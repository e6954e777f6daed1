"""One kernel family, a few launches, on one GPU: the small cases that profiler captures are taken on.

    python -m oneccl_b200.benchmarks.kernel_cases <case> [--launches 3] [--world 8]

Multi-rank kernels run with all ranks emulated on the one GPU (one cooperative launch, blockIdx.y = rank),
so what a capture shows is the kernel's HBM traffic, occupancy and stall reasons; NVLink bytes are not
in it (those are reported as bytes moved / device time from the multi-GPU sweeps).  Working sets are larger
than the 126 MB L2 and at most a few GB.  Each case prints the algorithmic bytes (or FLOPs) of one launch
and its device time from CUDA events, so a summary can state achieved / measured peak next to the
counters.

Cases: ar_oneshot ar_twoshot ar_pipelined ar_symm rs_symm ag_symm a2a_symm bcast pack_fused sendrecv
       moe_dispatch_combine moe_route gemm_rows ln_fwd_bwd colsum xent adamw gemm_2sm ag_gemm gemm_rs
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def _time(fn, launches):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--world", type=int, default=8)
    args = ap.parse_args()
    from oneccl_b200.ops.device_group import DeviceGroup

    W = args.world
    case = args.case
    out = {"case": case, "world": W}
    dt = torch.bfloat16

    def emu(heap_mb, staging_mb=32):
        return DeviceGroup.emulated(W, heap_bytes=heap_mb << 20, staging_bytes=staging_mb << 20)

    if case in ("ar_oneshot", "ar_twoshot", "ar_pipelined"):
        n = {"ar_oneshot": 128 << 10, "ar_twoshot": 8 << 20, "ar_pipelined": 64 << 20}[case]  # elements per rank
        g = emu(64)
        xs = [torch.randn(n, device="cuda").to(dt) for _ in range(W)]
        algo = case[3:]
        t = _time(lambda: g.allreduce(xs, xs, algo=algo), args.launches)
        out.update(bytes_per_rank=n * 2, algorithmic_hbm_bytes=W * n * 2 * 2, seconds=t)
    elif case in ("ar_symm", "rs_symm", "ag_symm", "a2a_symm"):
        n = 32 << 20  # elements per rank: 64 MB each, 512 MB for 8 ranks
        g = emu(160)
        a = g.symm_empty((n,), dtype=dt)
        for x in a:
            x.normal_()
        if case == "ar_symm":
            t = _time(lambda: g.allreduce(a, a, algo="symm"), args.launches)
            alg = W * n * 2 * 2  # every element read once and written once per rank
        elif case == "rs_symm":
            outs = [torch.empty(n // W, device="cuda", dtype=dt) for _ in range(W)]
            t = _time(lambda: g.reduce_scatter(a, outs), args.launches)
            alg = W * (n * 2 + n // W * 2)
        elif case == "ag_symm":
            ins = [torch.randn(n // W, device="cuda").to(dt) for _ in range(W)]
            t = _time(lambda: g.allgatherv(ins, a, algo="symm"), args.launches)
            alg = W * (n // W * 2 + n * 2)
        else:
            ins = [torch.randn(n, device="cuda").to(dt) for _ in range(W)]
            t = _time(lambda: g.alltoall(ins, a), args.launches)
            alg = W * n * 2 * 2
        out.update(bytes_per_rank=n * 2, algorithmic_hbm_bytes=alg, seconds=t)
    elif case == "bcast":
        n = 16 << 20
        g = emu(64, staging_mb=48)
        xs = [torch.randn(n, device="cuda").to(dt) for _ in range(W)]
        t = _time(lambda: g.broadcast(xs, xs, root=0), args.launches)
        out.update(bytes_per_rank=n * 2, algorithmic_hbm_bytes=W * n * 2 * 2, seconds=t)
    elif case == "pack_fused":
        g = emu(160)
        tensors = [[torch.randn(2048, device="cuda").to(dt) for _ in range(W)] for _ in range(256)]
        t = _time(lambda: g.allreduce_fused(tensors), args.launches)
        out.update(tensors=256, bytes_each=4096, seconds=t)
    elif case == "sendrecv":
        n = 64 << 20  # bytes per message; even ranks send to the next odd rank
        g = emu(16)
        src = [torch.empty(n, dtype=torch.uint8, device="cuda").random_(0, 255) for _ in range(W)]
        dst = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in range(W)]
        peers = [r + 1 if r % 2 == 0 else r - 1 for r in range(W)]
        sends = [r % 2 == 0 for r in range(W)]
        t = _time(lambda: g.sendrecv(src, dst, peers, sends), args.launches)
        out.update(bytes_per_message=n, messages=W // 2, algorithmic_hbm_bytes=(W // 2) * n * 4, seconds=t)
    elif case == "moe_route":
        from oneccl_b200.parallel.ep import route_device

        T, E, k = 1 << 20, 8, 2
        logits = torch.randn(T, E, device="cuda")
        t = _time(lambda: route_device(logits, k), args.launches)
        out.update(tokens=T, experts=E, topk=k, algorithmic_hbm_bytes=T * (E * 4 + k * (8 + 4 + 8 + 8)), seconds=t)
    elif case == "gemm_rows":
        from oneccl_b200.ops.gemm import gemm_bf16

        M, N, Kd = 16384, 4096, 4096  # buffers for 16384 rows, 10000 of them valid (the count lives on the device)
        a = torch.randn(M, Kd, device="cuda").to(dt)
        w = torch.randn(N, Kd, device="cuda").to(dt)
        c = torch.empty(M, N, device="cuda", dtype=dt)
        rows = torch.tensor([10000], dtype=torch.int32, device="cuda")
        t = _time(lambda: gemm_bf16(a, w, out=c, rows=rows), args.launches)
        out.update(M_cap=M, rows=10000, N=N, K=Kd, flops=2.0 * 10000 * N * Kd, seconds=t,
                   tflops=2.0 * 10000 * N * Kd / t / 1e12)
    elif case == "moe_dispatch_combine":
        from oneccl_b200.parallel.ep import fused_combine, fused_dispatch

        T, H, topk = 1024, 4096, 2
        cap = T * topk * W
        g = emu((cap * H * 2 >> 20) + 192)  # the heap also holds the flag and staging regions
        xrecv = g.symm_empty((cap, H), dtype=dt)  # also stands in for the experts' output
        cnt = g.symm_empty((256 * W * W,), dtype=torch.int32)
        metas = [torch.zeros(2 * W + 2, dtype=torch.int32, device="cuda") for _ in range(W)]
        gen = torch.Generator(device="cuda").manual_seed(1)
        xs = [torch.randn(T, H, generator=gen, device="cuda").to(dt) for _ in range(W)]
        idx = [torch.topk(torch.randn(T, W, generator=gen, device="cuda"), topk, dim=-1)[1] for _ in range(W)]
        flat = [i.reshape(-1) for i in idx]
        order = [torch.argsort(f, stable=True) for f in flat]
        counts = [torch.bincount(f, minlength=W) for f in flat]
        wts = [torch.full((T * topk,), 0.5, device="cuda") for _ in range(W)]
        pos = []
        for r in range(W):
            p = torch.empty_like(order[r])
            p[order[r]] = torch.arange(order[r].numel(), device="cuda")
            pos.append(p)
        outs = [torch.empty(T, H, dtype=dt, device="cuda") for _ in range(W)]

        def step():
            fused_dispatch(g, xs, order, counts, metas, xrecv, cnt, topk)
            fused_combine(g, flat, pos, wts, outs, metas, xrecv, topk)

        t = _time(step, args.launches)
        out.update(tokens=T, hidden=H, topk=topk, algorithmic_hbm_bytes=W * T * topk * H * 2 * 4, seconds=t)
    elif case in ("ln_fwd_bwd", "colsum", "xent", "adamw"):
        from oneccl_b200.ops import nn as K
        from oneccl_b200.ops import train as T

        if case == "ln_fwd_bwd":
            rows, D = 131072, 1024  # 256 MB of activations
            x = torch.randn(rows, D, device="cuda").to(dt).requires_grad_(True)
            res = torch.randn(rows, D, device="cuda").to(dt).requires_grad_(True)
            w = torch.ones(D, device="cuda", dtype=dt, requires_grad=True)
            b = torch.zeros(D, device="cuda", dtype=dt, requires_grad=True)
            dy = torch.randn(rows, D, device="cuda").to(dt)

            def step():
                y, s = K.add_layer_norm(x, res, w, b)
                torch.autograd.backward([y, s], [dy, dy])

            t = _time(step, args.launches)
            out.update(rows=rows, width=D, algorithmic_hbm_bytes=rows * D * 2 * (4 + 5), seconds=t)
        elif case == "colsum":
            rows, N = 65536, 4096
            dy = torch.randn(rows, N, device="cuda").to(dt)
            t = _time(lambda: K.colsum(dy), args.launches)
            out.update(rows=rows, cols=N, algorithmic_hbm_bytes=rows * N * 2, seconds=t)
        elif case == "xent":
            rows, V = 4096, 50304
            tg = torch.randint(0, 50257, (rows,), device="cuda")
            lg = torch.randn(rows, V, device="cuda").to(dt)
            t = _time(lambda: T.softmax_cross_entropy(lg.clone(), tg, 50257), args.launches)
            out.update(rows=rows, vocab=V, algorithmic_hbm_bytes=rows * V * 2 * 2, seconds=t)
        else:
            n = 96 << 20
            flat = torch.randn(n, device="cuda").to(dt)
            grad = torch.randn(n, device="cuda").to(dt)
            opt = T.FlatAdamW(flat, n)
            t = _time(lambda: opt.step(grad), args.launches)
            out.update(params=n, algorithmic_hbm_bytes=n * 28 + n * 2, seconds=t)
    elif case == "gemm_2sm":
        from oneccl_b200.ops.gemm import gemm_bf16

        M = N = Kd = 8192
        a = torch.randn(M, Kd, device="cuda").to(dt)
        w = torch.randn(N, Kd, device="cuda").to(dt)
        c = torch.empty(M, N, device="cuda", dtype=dt)
        t = _time(lambda: gemm_bf16(a, w, out=c), args.launches)
        out.update(M=M, N=N, K=Kd, flops=2.0 * M * N * Kd, algorithmic_hbm_bytes=3 * M * N * 2, seconds=t,
                   tflops=2.0 * M * N * Kd / t / 1e12)
    elif case in ("ag_gemm", "gemm_rs"):
        from oneccl_b200.ops.gemm import FusedPlan

        W = out["world"] = min(W, 2)
        g = DeviceGroup.emulated(W, heap_bytes=512 << 20, staging_bytes=1 << 20)
        M, N, Kd = 8192, 4096, 4096
        ws = [(torch.randn(N, Kd, device="cuda") * 0.05).to(dt) for _ in range(W)]
        if case == "ag_gemm":
            plan = FusedPlan(g, "ag_gemm", M, N, Kd, epilogue="silu")
            for r in range(W):
                plan.x_shard(r).normal_()
            t = _time(lambda: plan.run(None, ws), args.launches)
        else:
            plan = FusedPlan(g, "gemm_rs", M, N, Kd)
            hs = [torch.randn(M, Kd, device="cuda").to(dt) for _ in range(W)]
            t = _time(lambda: plan.run(hs, ws), args.launches)
        out.update(M=M, N=N, K=Kd, flops_all_ranks=2.0 * M * N * Kd * W, seconds=t,
                   tflops_per_gpu_equivalent=2.0 * M * N * Kd * W / t / 1e12)
    else:
        raise SystemExit(f"unknown case {case}")
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
