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
        self.layers = []
        for _ in range(cfg.n_layers):
            wq, wk, wv, wo = w(cfg.hidden, qd), w(cfg.hidden, kvd), w(cfg.hidden, kvd), w(qd, cfg.hidden)
            w1, w3, w2 = w(cfg.hidden, cfg.ffn), w(cfg.hidden, cfg.ffn), w(cfg.ffn, cfg.hidden)
            # the projections that share an input are stored side by side (one GEMM in the decode step);
            # the separate names are views of the same memory
            wqkv = torch.cat([wq, wk, wv], dim=1)
            w13 = torch.cat([w1, w3], dim=1)
            del wq, wk, wv, w1, w3
            self.layers.append(dict(wqkv=wqkv, wq=wqkv[:, :qd], wk=wqkv[:, qd:qd + kvd], wv=wqkv[:, qd + kvd:],
                                    wo=wo, w13=w13, w1=w13[:, :cfg.ffn], w3=w13[:, cfg.ffn:], w2=w2))
        self.head = w(cfg.hidden, cfg.vocab)
        half = cfg.head_dim // 2
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(half, device=device, dtype=torch.float32) / half))

    def n_params(self) -> int:
        n = self.emb.numel() + self.head.numel()
        return n + sum(lw[k].numel() for lw in self.layers for k in ("wqkv", "wo", "w13", "w2"))

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
            qd, kvd = cfg.n_q_heads * D, cfg.n_kv_heads * D
            qkv = h @ lw["wqkv"]
            q = apply_rope(qkv[..., :qd].view(B, L, cfg.n_q_heads, D).transpose(1, 2), cos, sin)
            k = apply_rope(qkv[..., qd:qd + kvd].view(B, L, cfg.n_kv_heads, D).transpose(1, 2), cos, sin)
            v = qkv[..., qd + kvd:].view(B, L, cfg.n_kv_heads, D).transpose(1, 2)
            keys, values = cache.update_and_fetch(k, v)
            att = base.scaled_dot_product_attention(q, keys, values, cache, scale, mask)
            x = x + att.transpose(1, 2).reshape(B, L, cfg.n_q_heads * D) @ lw["wo"]
            h = F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps)
            gu = h @ lw["w13"]
            x = x + (F.silu(gu[..., :cfg.ffn]) * gu[..., cfg.ffn:]) @ lw["w2"]
        if last_only:
            x = x[:, -1:]
        return F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps) @ self.head

    def decode_step(self, tok: torch.Tensor, caches, position: torch.Tensor) -> torch.Tensor:
        """One token per sequence, tok (B, 1), at the position held in the int32 device tensor
        `position` (1,): logits (B, vocab).  Nothing here depends on a host-side length, so with caches
        in static decode mode (`enable_static_decode`) the whole step can be captured in a CUDA graph
        and replayed while the position advances on the device.  Same layer structure as `forward`,
        with the projections that share an input fused (17 launches per layer instead of ~35)."""
        cfg = self.cfg
        B = tok.shape[0]
        D, nq, nkv = cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads
        half = D // 2
        x = self.emb[tok[:, 0]]
        ang = position.to(torch.float32) * self.inv_freq
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        scale = 1.0 / math.sqrt(D)
        for lw, cache in zip(self.layers, caches):
            h = F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps)
            qkv = h @ lw["wqkv"]
            qk = qkv[:, :(nq + nkv) * D].view(B, nq + nkv, D)
            x1, x2 = qk[..., :half], qk[..., half:]
            rot = torch.empty_like(qk)
            torch.mul(x1, cos, out=rot[..., :half])
            rot[..., :half].addcmul_(x2, sin, value=-1)
            torch.mul(x2, cos, out=rot[..., half:])
            rot[..., half:].addcmul_(x1, sin)
            q, k = rot[:, :nq].unsqueeze(2), rot[:, nq:].unsqueeze(2)
            v = qkv[:, (nq + nkv) * D:].view(B, nkv, D).unsqueeze(2)
            if B > 1:
                k, v = k.contiguous(), v.contiguous()
            keys, values = cache.update_and_fetch(k, v)
            att = base.scaled_dot_product_attention(q, keys, values, cache, scale, None)
            x = torch.addmm(x, att.reshape(B, nq * D), lw["wo"])
            h = F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps)
            gu = h @ lw["w13"]
            x = torch.addmm(x, F.silu(gu[:, :cfg.ffn]) * gu[:, cfg.ffn:], lw["w2"])
        return F.rms_norm(x, (cfg.hidden,), eps=cfg.rms_eps) @ self.head


class StaticDecoder:
    """Greedy decoding with one CUDA-graph replay per token.  The caches (MixedQuantKVCache) are put
    into static decode mode with one shared device counter [position, lengths]; a step = embedding
    of the token in `tok`, all layers (append at the device-side position, decode attention over the
    device-side length), logits, argmax into `tok`, counter += 1.  The first step runs eagerly (it
    warms the library's host-side parameter caches), the graph is captured once and replayed."""

    def __init__(self, model: Qwen2Model, caches, max_len: int):
        self.model, self.caches = model, caches
        counters = None
        for c in caches:
            counters = c.enable_static_decode(max_len, counters)
        self.counters = counters
        self.max_len = max_len
        B = caches[0].k_codes.shape[0]
        self.tok = torch.zeros((B, 1), dtype=torch.long, device=counters.device)
        self.graph = None

    def _step(self):
        logits = self.model.decode_step(self.tok, self.caches, self.counters[:1])
        self.tok.copy_(logits.argmax(-1, keepdim=True))
        self.counters += 1

    def generate(self, first_tok: torch.Tensor, n: int, use_graph: bool = True) -> torch.Tensor:
        """n further tokens after `first_tok` (B, 1): (B, n).  use_graph=False runs every step eagerly
        (the comparison the test makes)."""
        if int(self.counters[0].item()) + n > self.max_len:
            raise ValueError("the caches were sized for fewer positions")
        self.tok.copy_(first_tok)
        out = []
        if n > 0 and (self.graph is None or not use_graph):
            self._step()                                  # eager: also the warm-up before a capture
            out.append(self.tok.clone())
        if use_graph and self.graph is None and len(out) < n:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            keep = [self.tok.clone(), self.counters.clone()]
            with torch.cuda.graph(g):
                self._step()
            self.tok.copy_(keep[0])                       # a capture runs nothing, but keep the state explicit
            self.counters.copy_(keep[1])
            self.graph = g
        while len(out) < n:
            if use_graph:
                self.graph.replay()
            else:
                self._step()
            out.append(self.tok.clone())
        pos = int(self.counters[0].item())    # replays do not run the host code: read the position back once
        for c in self.caches:
            c.offset = pos
        return torch.cat(out, dim=1)

    def close(self):
        for c in self.caches:
            c.disable_static_decode()
