"""Llama-3 style decoder (RMSNorm, rotary embeddings, grouped-query attention, SwiGLU) used by the data-parallel
training benchmark and the examples.  Plain PyTorch: the model is the workload whose gradients the library
reduces, not part of the communication library itself."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    vocab: int = 128256
    dim: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads

    def num_params(self) -> int:
        attn = self.dim * self.dim * 2 + 2 * self.dim * self.kv_heads * self.head_dim
        mlp = 3 * self.dim * self.ffn
        return self.layers * (attn + mlp + 2 * self.dim) + 2 * self.vocab * self.dim + self.dim


CONFIGS = {
    "llama3_8b": LlamaConfig(),
    "llama3_70b": LlamaConfig(dim=8192, layers=80, heads=64, kv_heads=8, ffn=28672),
    "tiny": LlamaConfig(vocab=512, dim=128, layers=2, heads=4, kv_heads=2, ffn=256),
    "small": LlamaConfig(vocab=32000, dim=1024, layers=4, heads=16, kv_heads=4, ffn=4096),
}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(seq: int, head_dim: int, theta: float, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):
    # x [B, H, S, D]; rotate pairs (even, odd halves)
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.wq = nn.Linear(cfg.dim, cfg.heads * cfg.head_dim, bias=False)
        self.wk = nn.Linear(cfg.dim, cfg.kv_heads * cfg.head_dim, bias=False)
        self.wv = nn.Linear(cfg.dim, cfg.kv_heads * cfg.head_dim, bias=False)
        self.wo = nn.Linear(cfg.heads * cfg.head_dim, cfg.dim, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        c = self.cfg
        q = self.wq(x).view(b, s, c.heads, c.head_dim).transpose(1, 2)
        k = self.wk(x).view(b, s, c.kv_heads, c.head_dim).transpose(1, 2)
        v = self.wv(x).view(b, s, c.kv_heads, c.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.wo(o.transpose(1, 2).reshape(b, s, -1))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w1 = nn.Linear(cfg.dim, cfg.ffn, bias=False)
        self.w3 = nn.Linear(cfg.dim, cfg.ffn, bias=False)
        self.w2 = nn.Linear(cfg.ffn, cfg.dim, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm, self.attn = RMSNorm(cfg.dim, cfg.eps), Attention(cfg)
        self.mlp_norm, self.mlp = RMSNorm(cfg.dim, cfg.eps), MLP(cfg)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.attn_norm(x), cos, sin)
        return x + self.mlp(self.mlp_norm(x))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab, cfg.dim)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.layers)])
        self.norm = RMSNorm(cfg.dim, cfg.eps)
        self.head = nn.Linear(cfg.dim, cfg.vocab, bias=False)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, tokens, targets=None):
        b, s = tokens.shape
        x = self.embed(tokens)
        cos, sin = rope_tables(s, self.cfg.head_dim, self.cfg.rope_theta, x.device, x.dtype)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
