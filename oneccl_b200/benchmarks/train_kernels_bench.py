"""Times the memory-bound training kernels on one GPU against their traffic floor.

    python -m oneccl_b200.benchmarks.train_kernels_bench [--rows 8192] [--vocab 50304] [--params 100M]
                                                          [--iters 10] [--hbm-gbs 6454.9]

Kernels: fused softmax cross-entropy (reads the bf16 logits once, writes the
gradient in place: 4 bytes per logit), flat AdamW with clipping (reads bf16
grad + fp32 master/m/v, writes fp32 master/m/v + bf16 model: 30 bytes per
parameter, plus 2 for the norm pass), squared norm (2 bytes per element).
Each is compared with the plain PyTorch ops that do the same work.  All
working sets are larger than the L2, timing uses CUDA events after 3 warm-up
calls, and the fraction is achieved bytes/s over the measured copy bandwidth
given by --hbm-gbs."""
from __future__ import annotations

import argparse
import json

import torch

from ..ops.train import FlatAdamW, softmax_cross_entropy, sq_norm


def _size(text: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(text[:-1]) * mult[text[-1]]) if text[-1] in mult else int(text)


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--params", default="100M")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--hbm-gbs", type=float, default=6454.9)
    args = ap.parse_args()
    dev = torch.device("cuda")
    out = []

    # ---- cross-entropy: loss + gradient in one pass
    rows, vocab = args.rows, args.vocab
    src = torch.randn(rows, vocab, device=dev).to(torch.bfloat16)
    tgt = torch.randint(0, vocab, (rows,), device=dev)
    work = torch.empty_like(src)

    def ours_xent():
        work.copy_(src)  # the kernel consumes its input; the copy is timed separately and subtracted
        # loss and gradient come out of the one kernel; backward only hands the buffer on, so there is
        # nothing else to time (a leaf tensor here would add autograd's defensive clone of the gradient)
        with torch.no_grad():
            softmax_cross_entropy(work, tgt)

    t_copy = timed(lambda: work.copy_(src), args.iters)
    t_ours = timed(ours_xent, args.iters) - t_copy

    def torch_xent():
        x = src.detach().requires_grad_(True)
        torch.nn.functional.cross_entropy(x.float(), tgt).backward()

    t_ref = timed(torch_xent, args.iters)
    bytes_x = rows * vocab * 4
    out.append({"kernel": "softmax_xent", "rows": rows, "vocab": vocab, "ours_ms": t_ours, "torch_ms": t_ref,
                "algorithmic_bytes": bytes_x, "ours_gbs": bytes_x / t_ours / 1e6,
                "fraction_of_measured_hbm": bytes_x / t_ours / 1e6 / args.hbm_gbs})
    print(json.dumps(out[-1]))
    del src, work

    # ---- AdamW (with global-norm clipping) and the squared norm
    n = _size(args.params)
    model = torch.randn(n, device=dev).to(torch.bfloat16)
    grad = (torch.randn(n, device=dev) * 1e-2).to(torch.bfloat16)
    opt = FlatAdamW(model, n_decay=n // 2, max_norm=1.0)
    t_ours = timed(lambda: opt.step(grad), args.iters)
    p32 = torch.nn.Parameter(model.float())
    p32.grad = grad.float()
    ref = torch.optim.AdamW([p32], lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def torch_adamw():
        p32.grad.copy_(grad)  # widen the bf16 gradient, as a mixed-precision loop must
        torch.nn.utils.clip_grad_norm_([p32], 1.0)
        ref.step()
        model.copy_(p32.detach())

    t_ref = timed(torch_adamw, args.iters)
    bytes_a = n * 32
    out.append({"kernel": "adamw_flat+sq_norm", "params": n, "ours_ms": t_ours, "torch_ms": t_ref,
                "algorithmic_bytes": bytes_a, "ours_gbs": bytes_a / t_ours / 1e6,
                "fraction_of_measured_hbm": bytes_a / t_ours / 1e6 / args.hbm_gbs})
    print(json.dumps(out[-1]))

    acc = torch.zeros(1, device=dev)
    t_ours = timed(lambda: sq_norm(grad, acc), args.iters)
    t_ref = timed(lambda: torch.linalg.vector_norm(grad, dtype=torch.float32), args.iters)
    out.append({"kernel": "sq_norm", "elements": n, "ours_ms": t_ours, "torch_ms": t_ref,
                "algorithmic_bytes": n * 2, "ours_gbs": n * 2 / t_ours / 1e6,
                "fraction_of_measured_hbm": n * 2 / t_ours / 1e6 / args.hbm_gbs})
    print(json.dumps(out[-1]))
    return out


if __name__ == "__main__":
    main()
