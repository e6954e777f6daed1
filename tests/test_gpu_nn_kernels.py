"""Fused LayerNorm (+ residual), bias-gradient column sums and the packed QKV gradient against PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [256, 768, 1024])
@pytest.mark.parametrize("rows", [1, 37, 4100])
@pytest.mark.parametrize("residual", [False, True])
def test_layer_norm_forward_backward(D, rows, residual):
    from oneccl_b200.ops.nn import add_layer_norm, layer_norm

    g = torch.Generator(device="cuda").manual_seed(D + rows)
    x = torch.randn(rows, D, generator=g, device="cuda").to(torch.bfloat16)
    r = torch.randn(rows, D, generator=g, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).to(torch.bfloat16)
    b = (0.1 * torch.randn(D, generator=g, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(rows, D, generator=g, device="cuda").to(torch.bfloat16)
    dsum = torch.randn(rows, D, generator=g, device="cuda").to(torch.bfloat16)

    xs = [t.clone().requires_grad_(True) for t in (x, r, w, b)]
    if residual:
        y, s = add_layer_norm(xs[0], xs[1], xs[2], xs[3])
        torch.autograd.backward([y, s], [dy, dsum])
    else:
        y = layer_norm(xs[0], xs[2], xs[3])
        y.backward(dy)
    # fp32 reference on the same bf16 inputs (the residual sum is rounded to bf16, as the kernel keeps it)
    ref = [t.float().clone().requires_grad_(True) for t in (x, r, w, b)]
    tot = (ref[0] + ref[1]).to(torch.bfloat16).float() if residual else ref[0]
    if residual:
        tot = ref[0] + ref[1] + ((ref[0] + ref[1]).to(torch.bfloat16).float() - (ref[0] + ref[1])).detach()
    yr = torch.nn.functional.layer_norm(tot, (D,), ref[2], ref[3])
    if residual:
        torch.autograd.backward([yr, tot], [dy.float(), dsum.float()])
    else:
        yr.backward(dy.float())
    torch.cuda.synchronize()
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(xs[0].grad.float(), ref[0].grad, rtol=2e-2, atol=3e-2)
    if residual:
        assert torch.equal(xs[0].grad, xs[1].grad)
        torch.testing.assert_close(s.float(), tot, rtol=0, atol=0)
    scale = max(1.0, rows ** 0.5)
    torch.testing.assert_close(xs[2].grad.float(), ref[2].grad, rtol=2e-2, atol=2e-2 * scale)
    torch.testing.assert_close(xs[3].grad.float(), ref[3].grad, rtol=2e-2, atol=2e-2 * scale)


def test_layer_norm_falls_back_for_other_widths():
    from oneccl_b200.ops.nn import layer_norm

    x = torch.randn(5, 128, device="cuda").to(torch.bfloat16)
    w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(128, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(layer_norm(x, w, b), torch.nn.functional.layer_norm(x, (128,), w, b))


@pytest.mark.parametrize("rows,N", [(1, 8), (33, 264), (8192, 3072)])
def test_linear_bias_gradient(rows, N):
    from oneccl_b200.ops.nn import linear

    g = torch.Generator(device="cuda").manual_seed(rows)
    K = 64
    x = torch.randn(rows, K, generator=g, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (0.1 * torch.randn(N, K, generator=g, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = torch.zeros(N, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    dy = torch.randn(rows, N, generator=g, device="cuda").to(torch.bfloat16)
    linear(x, w, b).backward(dy)
    xr, wr, br = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    torch.nn.functional.linear(xr, wr, br).backward(dy)
    torch.cuda.synchronize()
    torch.testing.assert_close(b.grad.float(), dy.float().sum(0), rtol=1e-2, atol=1e-2 * max(1.0, rows ** 0.5))
    torch.testing.assert_close(x.grad, xr.grad)
    torch.testing.assert_close(w.grad, wr.grad)


def test_split_qkv_gradient_matches_unbind():
    from oneccl_b200.ops.nn import split_qkv

    B, S, H, dh = 2, 128, 4, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(B, S, 3 * H * dh, generator=g, device="cuda").to(torch.bfloat16)
    outs = []
    for fused in (True, False):
        t = qkv.clone().requires_grad_(True)
        if fused:
            q, k, v = split_qkv(t, H)
        else:
            q, k, v = t.view(B, S, 3, H, dh).permute(2, 0, 3, 1, 4)
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        a.sum().backward()
        outs.append((a.detach(), t.grad))
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0])
    torch.testing.assert_close(outs[0][1], outs[1][1], rtol=0, atol=0)


def test_gpt2_fused_ops_match_stock_modules():
    from oneccl_b200.models.gpt2 import GPT2, GPT2Config

    cfg = GPT2Config(2, 4, 256, 64, 1000)
    torch.manual_seed(0)
    m = GPT2(cfg, fused_ops=True).cuda().to(torch.bfloat16)
    idx = torch.randint(0, cfg.vocab, (4, 64), device="cuda")
    tgt = torch.randint(0, cfg.vocab, (4, 64), device="cuda")
    grads = []
    losses = []
    for fused in (True, False):
        m.fused_ops = fused
        m.zero_grad(set_to_none=True)
        loss = m(idx, tgt)
        loss.backward()
        losses.append(float(loss.detach()))
        grads.append(torch.cat([p.grad.float().flatten() for p in m.parameters()]))
    assert abs(losses[0] - losses[1]) < 2e-2
    cos = torch.nn.functional.cosine_similarity(grads[0], grads[1], dim=0).item()
    assert cos > 0.99, cos


def test_data_parallel_gradient_sinks_match_autograd():
    """Linear layers accumulate their weight gradients straight into DataParallel's flat buffer (GEMM with
    beta = 1, no autograd accumulation): same gradients as the plain module, every bucket still fires."""
    from oneccl_b200.models.gpt2 import GPT2, GPT2Config
    from oneccl_b200.ops.device_group import DeviceGroup
    from oneccl_b200.parallel.ddp import DataParallel

    cfg = GPT2Config(2, 4, 256, 64, 1000)
    torch.manual_seed(0)
    plain = GPT2(cfg, fused_ops=True).cuda().to(torch.bfloat16)
    torch.manual_seed(0)
    wrapped = GPT2(cfg, fused_ops=True).cuda().to(torch.bfloat16)
    group = DeviceGroup.emulated(1, heap_bytes=64 << 20, staging_bytes=1 << 20)
    ddp = DataParallel(wrapped, group, bucket_mb=0.5)
    idx = torch.randint(0, cfg.vocab, (4, 64), device="cuda")
    tgt = torch.randint(0, cfg.vocab, (4, 64), device="cuda")
    for _ in range(2):  # the second pass checks that zero_grad re-arms everything
        plain.zero_grad(set_to_none=True)
        plain(idx, tgt).backward()
        ddp.zero_grad()
        ddp(idx, tgt).backward()
        ddp.finish()
        torch.cuda.synchronize()
        assert all(b.pending == 0 for b in ddp.buckets)
        for (n, a), (_, b) in zip(plain.named_parameters(), wrapped.named_parameters()):
            torch.testing.assert_close(b.grad.float(), a.grad.float(), rtol=2e-2, atol=2e-3, msg=n)
    group.close()
