"""Decoder-only transformers used by the data-parallel and sharded-optimizer
paths: a GPT-2 style block (LayerNorm, GELU MLP, learned positions) and a
Llama style block (RMSNorm, SwiGLU, rotary positions).  GEMMs and attention go
to the vendor libraries through PyTorch; this library's kernels are the
collectives and the fused optimizer / gradient steps around them."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPTConfig:
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    vocab: int = 50257
    seq_len: int = 1024
    ffn: int = 0            # 0: 4 * d_model (GPT-2); Llama style uses an explicit SwiGLU width
    style: str = "gpt2"     # "gpt2" | "llama"

    @staticmethod
    def gpt2_medium():
        return GPTConfig(24, 1024, 16, 50257, 1024, 0, "gpt2")

    @staticmethod
    def llama_1p3b():
        return GPTConfig(24, 2048, 16, 32000, 2048, 5504, "llama")

    @staticmethod
    def tiny(style="gpt2"):
        return GPTConfig(2, 64, 4, 257, 32, 0 if style == "gpt2" else 176, style)


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def _rope(q, k, base=10000.0):
    # q, k: [B, H, T, D]
    T, D = q.shape[-2], q.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, device=q.device, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(T, device=q.device, dtype=torch.float32), inv)
    cos, sin = ang.cos().to(q.dtype), ang.sin().to(q.dtype)

    def rot(x):
        x1, x2 = x[..., 0::2], x[..., 1::2]
        return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)

    return rot(q), rot(k)


class Block(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        d = cfg.d_model
        self.cfg = cfg
        llama = cfg.style == "llama"
        self.ln1 = RMSNorm(d) if llama else nn.LayerNorm(d)
        self.ln2 = RMSNorm(d) if llama else nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d, bias=not llama)
        self.proj = nn.Linear(d, d, bias=not llama)
        if llama:
            self.gate_up = nn.Linear(d, 2 * cfg.ffn, bias=False)
            self.down = nn.Linear(cfg.ffn, d, bias=False)
        else:
            self.fc = nn.Linear(d, 4 * d)
            self.down = nn.Linear(4 * d, d)

    def forward(self, x):
        B, T, d = x.shape
        H = self.cfg.n_head
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, H, d // H).permute(2, 0, 3, 1, 4)
        if self.cfg.style == "llama":
            q, k = _rope(q, k)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, d))
        h = self.ln2(x)
        if self.cfg.style == "llama":
            g, u = self.gate_up(h).chunk(2, dim=-1)
            x = x + self.down(F.silu(g) * u)
        else:
            x = x + self.down(F.gelu(self.fc(h), approximate="tanh"))
        return x


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq_len, cfg.d_model) if cfg.style == "gpt2" else None
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = RMSNorm(cfg.d_model) if cfg.style == "llama" else nn.LayerNorm(cfg.d_model)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets=None):
        B, T = idx.shape
        x = self.wte(idx)
        if self.wpe is not None:
            x = x + self.wpe(torch.arange(T, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)    # tied output embedding
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.view(-1))

    def num_params(self):
        return sum(p.numel() for p in self.parameters())
