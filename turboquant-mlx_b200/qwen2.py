"""Random-init decoder with the Qwen2 attention layout (grouped-query attention,
head_dim 128, RoPE, RMSNorm, gated MLP): the model that drives the caches and the
attention hook end to end when no checkpoint is available.  It plays the part of the
mlx-lm model in the reference's demo loop (demo_7b.py:13-34, README.md:28-47): every
layer calls `cache.update_and_fetch(keys, values)` and the
`scaled_dot_product_attention` symbol of `base`, which `patch.apply_patch` swaps.
Weights are synthetic; the attention path does not depend on them."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import base


@dataclass
class Qwen2Config:
    n_layers: int = 28
    hidden: int = 3584
    n_q_heads: int = 28
    n_kv_heads: int = 4
    head_dim: int = 128
    ffn: int = 18944
    vocab: int = 152064
    rope_theta: float = 1_000_000.0
    rms_eps: float = 1e-6
    init_std: float = 0.02

    def describe(self) -> dict:
        return dict(self.__dict__)


def rope_tables(pos: torch.Tensor, head_dim: int, theta: float, dtype):
    """(cos, sin) of shape (1, 1, L, head_dim / 2) for the positions `pos` (L,): computed once per
    forward pass and shared by all layers."""
    half = head_dim // 2
    freqs = 1.0 / (theta ** (torch.arange(half, device=pos.device, dtype=torch.float32) / half))
    ang = pos[:, None].float() * freqs[None]
    return ang.cos()[None, None].to(dtype), ang.sin()[None, None].to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding, half-split layout: x (B, H, L, D)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    cos, sin = rope_tables(pos, x.shape[-1], theta, x.dtype)
    return apply_rope(x, cos, sin)


class Qwen2Model:
    def __init__(self, cfg: Qwen2Config, device, dtype=torch.bfloat16, seed: int = 0):
        self.cfg = cfg
        self.dtype = dtype
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape):
            return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * cfg.init_std).to(dtype)

        qd, kvd = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        self.emb = w(cfg.vocab, cfg.hidden)
        self.layers = [dict(wq=w(cfg.hidden, qd), wk=w(cfg.hidden, kvd), wv=w(cfg.hidden, kvd), wo=w(qd, cfg.hidden),
                            w1=w(cfg.hidden, cfg.ffn), w3=w(cfg.hidden, cfg.ffn), w2=w(cfg.ffn, cfg.hidden))
                       for _ in range(cfg.n_layers)]
        self.head = w(cfg.hidden, cfg.vocab)

    def n_params(self) -> int:
        n = self.emb.numel() + self.head.numel()
        return n + sum(t.numel() for lw in self.layers for t in lw.values())

    def forward(self, tokens: torch.Tensor, caches, last_only: bool = True) -> torch.Tensor:
        """tokens (B, L) -> logits (B, 1 or L, vocab); appends to `caches` (one per layer)."""
        cfg = self.cfg
        B, L = tokens.shape
        D = cfg.head_dim
        x = self.emb[tokens]
        pos = torch.arange(caches[0].offset, caches[0].offset + L, device=x.device)
        mask = caches[0].make_mask(L)
        scale = 1.0 / math.sqrt(D)
        cos, sin = rope_tables(pos, D, cfg.rope_theta, x.dtype)
        for lw, cache in zip(self.layers, caches):
            h = F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps)
            q = apply_rope((h @ lw["wq"]).view(B, L, cfg.n_q_heads, D).transpose(1, 2), cos, sin)
            k = apply_rope((h @ lw["wk"]).view(B, L, cfg.n_kv_heads, D).transpose(1, 2), cos, sin)
            v = (h @ lw["wv"]).view(B, L, cfg.n_kv_heads, D).transpose(1, 2)
            keys, values = cache.update_and_fetch(k, v)
            att = base.scaled_dot_product_attention(q, keys, values, cache, scale, mask)
            x = x + att.transpose(1, 2).reshape(B, L, cfg.n_q_heads * D) @ lw["wo"]
            h = F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps)
            x = x + (F.silu(h @ lw["w1"]) * (h @ lw["w3"])) @ lw["w2"]
        if last_only:
            x = x[:, -1:]
        return F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps) @ self.head
