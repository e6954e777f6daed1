"""tcgen05 GEMM (plain and fused with a collective) against torch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, w, silu=False):
    y = a.float() @ w.float().t()
    if silu:
        y = torch.nn.functional.silu(y)
    return y


def _check(out, ref, K):
    # bf16 output of an fp32 accumulation: one rounding of the result
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 1.0e-2 * scale + 1e-3, f"max err {err} vs scale {scale} (K={K})"


@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (1024, 1792, 1024),
                                   (384, 128, 192), (200, 264, 136)])
@pytest.mark.parametrize("kernel", ["1sm", "2sm", "auto"])
def test_gemm_plain(shape, kernel):
    """One CTA per 128 x 256 tile, CTA pairs on 256 x 256 tiles (cta_group::2), and the library's choice."""
    from oneccl_b200.ops.gemm import gemm_bf16

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    out = gemm_bf16(a, w, check=True, kernel=kernel)
    torch.cuda.synchronize()
    _check(out, _ref(a, w), K)


@pytest.mark.parametrize("kernel", ["1sm", "2sm"])
def test_gemm_silu_and_persistence(kernel):
    """More tiles than CTAs (each CTA loops, both TMEM accumulators are reused) + SiLU epilogue."""
    from oneccl_b200.ops.gemm import gemm_bf16

    M, N, K = 2048, 1024, 512
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm_bf16(a, w, epilogue="silu", ctas=8, check=True, kernel=kernel)
    torch.cuda.synchronize()
    _check(out, _ref(a, w, silu=True), K)


def _set_pairs(monkeypatch, on):
    """CTA pairs (cta_group::2) on or off for the fused kernels; the knob is read when a plan is created."""
    from oneccl_b200 import _lib

    monkeypatch.setenv("CCL_CUDA_GEMM_2SM", "1" if on else "0")
    _lib.load().cclx_env_reload()


@pytest.mark.parametrize("pairs", [False, True], ids=["one-cta", "cta-pairs"])
@pytest.mark.parametrize("world,shape", [(2, (1024, 1024, 512)), (4, (2048, 512, 448)), (2, (512, 256, 64))])
@pytest.mark.parametrize("mode", ["ag_gemm", "gemm_rs_ring", "gemm_rs_owner"])
def test_fused_gemm_larger_shapes_both_main_loops(monkeypatch, pairs, world, shape, mode):
    """Several 256 x 256 tiles per shard, more K steps than pipeline stages, with the single-CTA main loop and
    with CTA pairs, against the fp32 product."""
    from oneccl_b200.ops.device_group import DeviceGroup
    from oneccl_b200.ops.gemm import FusedPlan

    _set_pairs(monkeypatch, pairs)
    M, N, K = shape
    grp = DeviceGroup.emulated(world, heap_bytes=128 << 20, staging_bytes=1 << 20)
    g = torch.Generator(device="cuda").manual_seed(7)
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(world)]
    per = M // world
    if mode == "ag_gemm":
        plan = FusedPlan(grp, "ag_gemm", M, N, K, n_comm=2)
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        for it in range(2):
            for r in range(world):
                plan.x_shard(r).copy_(x[r * per:(r + 1) * per] * (it + 1))
            outs = plan.run(None, ws)
            torch.cuda.synchronize()
            grp.check()
            for r in range(world):
                assert plan.error(r) == 0
                _check(outs[r], _ref(x * (it + 1), ws[r]), K)
    else:
        plan = FusedPlan(grp, "gemm_rs", M, N, K, n_comm=-2 if mode == "gemm_rs_ring" else -1)
        hs = [torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        full = sum(_ref(h, w) for h, w in zip(hs, ws))
        for it in range(2):
            outs = plan.run(hs, ws)
            torch.cuda.synchronize()
            grp.check()
            for r in range(world):
                assert plan.error(r) == 0
                ref = full[r * per:(r + 1) * per]
                err = (outs[r].float() - ref).abs().max().item()
                assert err <= 2.0e-2 * ref.abs().max().item() + 1e-3, (mode, err)
    plan.close()
    grp.close()
    monkeypatch.delenv("CCL_CUDA_GEMM_2SM")
    from oneccl_b200 import _lib

    _lib.load().cclx_env_reload()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("n_comm", [2, -1], ids=["copy-ctas", "copy-engines"])
def test_ag_gemm_emulated(world, n_comm):
    """The gather runs on dedicated copy CTAs of the kernel, or on the copy engines of a side stream
    with one flag kernel per shard while every CTA computes."""
    from oneccl_b200.ops.device_group import DeviceGroup
    from oneccl_b200.ops.gemm import FusedPlan

    M, N, K = world * 256, 512, 256
    grp = DeviceGroup.emulated(world, heap_bytes=64 << 20, staging_bytes=1 << 20)
    plan = FusedPlan(grp, "ag_gemm", M, N, K, epilogue="silu", n_comm=n_comm)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(world)]
    per = M // world
    for it in range(2):  # twice: flags and sequence numbers are reused
        for r in range(world):
            plan.x_shard(r).copy_(x[r * per:(r + 1) * per] * (it + 1))
        outs = plan.run(None, ws)
        torch.cuda.synchronize()
        grp.check()
        for r in range(world):
            assert plan.error(r) == 0
            assert torch.equal(plan.x_full(r), x * (it + 1))
            _check(outs[r], _ref(x * (it + 1), ws[r], silu=True), K)
    plan.close()
    grp.close()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("variant", ["ring", "owner-reduce"])
@pytest.mark.parametrize("rows_per_rank", [128, 256])
def test_gemm_rs_emulated(world, variant, rows_per_rank):
    """GEMM -> reduce-scatter: partial sums passed down a ring inside the epilogues (bf16 on the wire,
    one rounding per hop), or stored at the owner and summed in fp32 after the GEMM."""
    from oneccl_b200.ops.device_group import DeviceGroup
    from oneccl_b200.ops.gemm import FusedPlan

    M, N, K = world * rows_per_rank, 768, 192
    grp = DeviceGroup.emulated(world, heap_bytes=64 << 20, staging_bytes=1 << 20)
    plan = FusedPlan(grp, "gemm_rs", M, N, K, n_comm=-2 if variant == "ring" else -1)
    g = torch.Generator(device="cuda").manual_seed(3)
    hs = [torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(world)]
    full = sum(_ref(h, w) for h, w in zip(hs, ws))
    per = M // world
    for it in range(2):
        outs = plan.run(hs, ws)
        torch.cuda.synchronize()
        grp.check()
        for r in range(world):
            assert plan.error(r) == 0
            ref = full[r * per:(r + 1) * per]
            err = (outs[r].float() - ref).abs().max().item()
            # one bf16 rounding per contribution (owner-reduce) or per hop (ring)
            assert err <= 2.0e-2 * ref.abs().max().item() + 1e-3, (variant, err)
    plan.close()
    grp.close()


@pytest.mark.parametrize("rows", [0, 1, 300, 700, 5000])
def test_gemm_row_count_read_on_the_device(rows):
    """The product over the first min(M, rows) rows of A, the count taken from device memory by the kernel: rows
    behind it keep what the output held."""
    from oneccl_b200.ops.gemm import gemm_bf16

    M, N, K = 700, 384, 320
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    n_dev = torch.tensor([rows, 0], dtype=torch.int32, device="cuda")
    gemm_bf16(a, w, out=out, epilogue="silu", rows=n_dev, check=True)
    torch.cuda.synchronize()
    n = min(rows, M)
    ref = torch.nn.functional.silu(a[:n].float() @ w.float().t())
    assert (out[:n].float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item()) if n else True
    assert bool((out[n:] == 7.0).all())
