"""Llama-style decoder (RMSNorm, rotary embeddings, grouped-query attention,
SwiGLU) used as the flagship training workload.

The model is written as separate stages - embedding, N identical blocks, head -
so that a sharded-data-parallel engine can gather, run and free one stage at a
time.  Norms, rotary embedding, SwiGLU and the loss use the hand-written
kernels of ``torchcomms_b200.ops``; projections are plain GEMMs and attention
is PyTorch's fused scaled-dot-product attention.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused


@dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    vocab_size: int = 128256
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 4096

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(dim=256, n_layers=2, n_heads=8, n_kv_heads=4, ffn_dim=512, vocab_size=1024, max_seq_len=256)

    def param_count(self) -> int:
        per_block = (
            2 * self.dim
            + (self.n_heads + 2 * self.n_kv_heads) * self.head_dim * self.dim
            + self.dim * self.n_heads * self.head_dim
            + 3 * self.ffn_dim * self.dim
        )
        return 2 * self.vocab_size * self.dim + self.dim + self.n_layers * per_block

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (forward + backward), attention included."""
        matmul_params = self.param_count() - self.vocab_size * self.dim  # the embedding lookup is not a GEMM
        attn = 2 * 2 * self.n_layers * seq_len * self.dim / 2  # causal QK^T and PV
        return 3 * (2 * matmul_params + attn)


class Embedding(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return F.embedding(tokens, self.weight)


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        hd = cfg.head_dim
        self.attn_norm = nn.Parameter(torch.ones(cfg.dim))
        self.wqkv = nn.Parameter(torch.empty((cfg.n_heads + 2 * cfg.n_kv_heads) * hd, cfg.dim))
        self.wo = nn.Parameter(torch.empty(cfg.dim, cfg.n_heads * hd))
        self.ffn_norm = nn.Parameter(torch.ones(cfg.dim))
        self.w13 = nn.Parameter(torch.empty(2 * cfg.ffn_dim, cfg.dim))  # gate rows first, then up rows
        self.w2 = nn.Parameter(torch.empty(cfg.dim, cfg.ffn_dim))
        for w in (self.wqkv, self.wo, self.w13, self.w2):
            nn.init.normal_(w, std=0.02)

    def forward(self, x: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        b, s, d = x.shape
        hd, nh, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        h = fused.rms_norm(x.reshape(b * s, d), self.attn_norm, cfg.norm_eps)
        qkv = F.linear(h, self.wqkv)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q = fused.apply_rope(q.reshape(b * s, nh, hd), pos, cos_t, sin_t).view(b, s, nh, hd)
        k = fused.apply_rope(k.reshape(b * s, nkv, hd), pos, cos_t, sin_t).view(b, s, nkv, hd)
        v = v.reshape(b, s, nkv, hd)
        o = F.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=(nkv != nh)
        )
        o = o.transpose(1, 2).reshape(b * s, nh * hd)
        x = x + F.linear(o, self.wo).view(b, s, d)
        h = fused.rms_norm(x.reshape(b * s, d), self.ffn_norm, cfg.norm_eps)
        h = fused.swiglu(F.linear(h, self.w13))
        return x + F.linear(h, self.w2).view(b, s, d)


class Head(nn.Module):
    """Final norm + vocabulary projection + mean token cross-entropy."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.norm = nn.Parameter(torch.ones(cfg.dim))
        self.weight = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        h = fused.rms_norm(x.reshape(b * s, d), self.norm, self.cfg.norm_eps)
        return fused.linear_cross_entropy(h, self.weight, targets.reshape(-1))


def build_stages(cfg: LlamaConfig, seed: int = 0) -> list[nn.Module]:
    """[Embedding, Block x n_layers, Head], random-initialised identically on every rank."""
    gen_state = torch.random.get_rng_state()
    torch.manual_seed(seed)
    stages: list[nn.Module] = [Embedding(cfg)]
    stages += [Block(cfg) for _ in range(cfg.n_layers)]
    stages.append(Head(cfg))
    torch.random.set_rng_state(gen_state)
    return stages


def reference_loss(stages, cfg: LlamaConfig, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Unsharded forward of the same stages (for tests)."""
    dev = tokens.device
    b, s = tokens.shape
    cos_t, sin_t = fused.rope_tables(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta, dev)
    pos = torch.arange(s, dtype=torch.int32, device=dev).repeat(b)
    x = stages[0](tokens)
    for blk in stages[1:-1]:
        x = blk(x, pos, cos_t, sin_t)
    return stages[-1](x, targets)
