"""Tensor / sequence parallel MLP block with the collectives fused into the GEMMs.

    X [tokens, d_model] is sharded over tokens (sequence parallel),
    W_up [d_model, d_ff] over columns, W_down [d_ff, d_model] over rows.
    H_r = silu(all_gather(X) @ W_up_r)          one kernel (ag_gemm, SiLU in the epilogue)
    Y_r = reduce_scatter(H_r @ W_down_r)        one kernel (gemm_rs)

Weights are kept in ``nn.Linear`` layout ([out, in]), which is the K-major
operand layout of the tcgen05 kernel.  ``forward_unfused`` is the same math
with separate collectives and cuBLAS GEMMs (the baseline shape of the block).
"""
from __future__ import annotations

import torch

from ..ops.device_group import DeviceGroup
from ..ops.gemm import FusedPlan


class TensorParallelMLP:
    def __init__(self, group: DeviceGroup, tokens: int, d_model: int, d_ff: int, seed: int = 0, n_comm: int = 0):
        assert not group.emulated_mode, "one rank per process"
        W = group.world
        assert tokens % (W * 128) == 0 and d_ff % W == 0
        self.group, self.world, self.rank = group, W, group.rank
        self.tokens, self.d_model, self.d_ff = tokens, d_model, d_ff
        self.ff_local = d_ff // W
        g = torch.Generator(device="cuda").manual_seed(seed + 31 * group.rank)
        self.w_up = (torch.randn(self.ff_local, d_model, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.w_down = (torch.randn(d_model, self.ff_local, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.up = FusedPlan(group, "ag_gemm", tokens, self.ff_local, d_model, epilogue="silu", n_comm=n_comm)
        self.down = FusedPlan(group, "gemm_rs", tokens, d_model, self.ff_local)
        self.h = torch.empty((tokens, self.ff_local), dtype=torch.bfloat16, device="cuda")
        self.y = torch.empty((tokens // W, d_model), dtype=torch.bfloat16, device="cuda")

    @property
    def x_shard(self) -> torch.Tensor:
        """[tokens/world, d_model] slot the caller fills with this rank's rows of X."""
        return self.up.x_shard(0 if not self.group.emulated_mode else self.rank)

    def forward(self) -> torch.Tensor:
        """Uses the contents of ``x_shard``; returns this rank's rows of Y."""
        self.up.run(None, self.w_up, out=self.h)
        self.down.run(self.h, self.w_down, out=self.y)
        return self.y

    def forward_unfused(self, x_local: torch.Tensor) -> torch.Tensor:
        xf = torch.empty((self.tokens, self.d_model), dtype=torch.bfloat16, device="cuda")
        self.group.allgatherv(x_local, xf)
        h = torch.nn.functional.silu(xf @ self.w_up.t())
        part = h @ self.w_down.t()
        y = torch.empty((self.tokens // self.world, self.d_model), dtype=torch.bfloat16, device="cuda")
        self.group.reduce_scatter(part, y)
        return y

    def close(self):
        self.up.close()
        self.down.close()
