"""GPT-2 (124M ... 1.5B) decoder used by the data-parallel benchmark.

cuBLAS GEMMs and fused SDPA attention; with ``fused_ops`` (the default on CUDA bf16) the
LayerNorms (with the residual addition in front of them), the bias gradients and the
packed QKV gradient use the kernels of ``oneccl_b200.ops.nn``; the loss goes through the
fused softmax cross-entropy kernel.  ``fused_ops=False`` is the same network on stock
PyTorch modules.  The vocabulary dimension of
the tied embedding / output matrix is padded to a multiple of 64 so that the
logit rows are 16-byte aligned; the padding columns take no part in the
softmax."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    seq_len: int = 1024
    vocab: int = 50257

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + 63) // 64 * 64

    @staticmethod
    def named(name: str) -> "GPT2Config":
        table = {
            "gpt2-small": GPT2Config(12, 12, 768),
            "gpt2-medium": GPT2Config(24, 16, 1024),
            "gpt2-large": GPT2Config(36, 20, 1280),
            "gpt2-xl": GPT2Config(48, 25, 1600),
            "gpt2-tiny": GPT2Config(2, 4, 128, 64, 1000),
        }
        return table[name]


class Block(nn.Module):
    def __init__(self, c: GPT2Config):
        super().__init__()
        self.n_head = c.n_head
        self.ln1 = nn.LayerNorm(c.d_model)
        self.qkv = nn.Linear(c.d_model, 3 * c.d_model)
        self.proj = nn.Linear(c.d_model, c.d_model)
        self.ln2 = nn.LayerNorm(c.d_model)
        self.fc = nn.Linear(c.d_model, 4 * c.d_model)
        self.fc2 = nn.Linear(4 * c.d_model, c.d_model)

    def forward(self, x):
        B, S, D = x.shape
        h = self.ln1(x)
        q, k, v = self.qkv(h).view(B, S, 3, self.n_head, D // self.n_head).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, D))
        h = self.ln2(x)
        x = x + self.fc2(F.gelu(self.fc(h), approximate="tanh"))
        return x

    def forward_fused(self, x, delta):
        """``x`` is the residual stream without the previous block's MLP output ``delta`` (None for
        the first block): the addition happens inside the LayerNorm kernel.  Returns (x, delta)."""
        from ..ops import nn as K

        B, S, D = x.shape
        h, x = K.add_layer_norm(x, delta, self.ln1.weight, self.ln1.bias, self.ln1.eps)
        q, k, v = K.split_qkv(K.linear(h, self.qkv.weight, self.qkv.bias), self.n_head)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        attn = K.linear(a.transpose(1, 2).reshape(B, S, D), self.proj.weight, self.proj.bias)
        h, x = K.add_layer_norm(x, attn, self.ln2.weight, self.ln2.bias, self.ln2.eps)
        delta = K.linear(F.gelu(K.linear(h, self.fc.weight, self.fc.bias), approximate="tanh"), self.fc2.weight,
                         self.fc2.bias)
        return x, delta


class GPT2(nn.Module):
    def __init__(self, c: GPT2Config, fused_ops: bool = True):
        super().__init__()
        self.cfg = c
        self.fused_ops = fused_ops
        self.wte = nn.Embedding(c.vocab_padded, c.d_model)
        self.wpe = nn.Embedding(c.seq_len, c.d_model)
        self.blocks = nn.ModuleList([Block(c) for _ in range(c.n_layer)])
        self.ln_f = nn.LayerNorm(c.d_model)
        self.apply(self._init)
        for b in self.blocks:  # scaled init of the residual projections
            for lin in (b.proj, b.fc2):
                nn.init.normal_(lin.weight, mean=0.0, std=0.02 / math.sqrt(2 * c.n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def hidden(self, idx):
        B, S = idx.shape
        pos = torch.arange(S, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        if self.fused_ops and x.is_cuda and x.dtype == torch.bfloat16:
            from ..ops import nn as K

            delta = None
            for b in self.blocks:
                x, delta = b.forward_fused(x, delta)
            h, _ = K.add_layer_norm(x, delta, self.ln_f.weight, self.ln_f.bias, self.ln_f.eps)
            return h
        for b in self.blocks:
            x = b(x)
        return self.ln_f(x)

    def logits(self, idx):
        x = self.hidden(idx)
        return F.linear(x.view(-1, x.shape[-1]), self.wte.weight)  # [B*S, vocab_padded]

    def forward(self, idx, targets=None, fused_loss: bool = True):
        lg = self.logits(idx)
        if targets is None:
            return lg[:, : self.cfg.vocab]
        if fused_loss and lg.is_cuda and lg.dtype == torch.bfloat16:
            from ..ops.train import softmax_cross_entropy

            return softmax_cross_entropy(lg, targets.reshape(-1), self.cfg.vocab)
        return F.cross_entropy(lg[:, : self.cfg.vocab].float(), targets.reshape(-1))

    def decay_split(self):
        """Parameters that receive weight decay (matrices) and those that do not."""
        decay, no_decay = [], []
        for _, p in self.named_parameters():
            (decay if p.dim() >= 2 else no_decay).append(p)
        return decay, no_decay
