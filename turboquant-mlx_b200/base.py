"""Host-side stand-ins for the two mlx-lm pieces the reference plugs into
(`mlx_lm.models.cache.KVCache` and the `scaled_dot_product_attention` symbol of
`mlx_lm.models.base`): a plain concatenating KV cache and the attention entry
point that `patch.apply_patch` swaps.  mlx-lm itself is not a dependency."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def create_causal_mask(N: int, offset: int = 0, window_size=None, device=None) -> torch.Tensor:
    """Boolean (N, offset + N) mask, True where query i may attend key j."""
    rinds = torch.arange(offset + N, device=device)
    linds = torch.arange(offset, offset + N, device=device)[:, None]
    mask = linds >= rinds[None]
    if window_size is not None:
        mask = mask & (linds < rinds[None] + window_size)
    return mask


class KVCache:
    """Un-quantized KV cache growing in steps of 256 positions."""

    step = 256

    def __init__(self, keys_only: bool = False):
        self.keys = None
        self.values = None
        self.offset = 0
        # keys_only: the values live elsewhere (a V-only TurboQuant cache keeps
        # them packed), so no full-precision copy of V is stored here
        self.keys_only = keys_only

    def update_and_fetch(self, keys, values):
        B, H, S, Dk = keys.shape
        Dv = 0 if self.keys_only else values.shape[3]
        prev = self.offset
        if self.keys is None or prev + S > self.keys.shape[2]:
            n = ((prev + S + self.step - 1) // self.step) * self.step
            if self.keys is not None:
                n = max(n, 2 * self.keys.shape[2])
            new_k = torch.zeros((B, H, n, Dk), dtype=keys.dtype, device=keys.device)
            new_v = torch.zeros((B, H, n, Dv), dtype=keys.dtype, device=keys.device)
            if self.keys is not None:
                new_k[..., :prev, :] = self.keys[..., :prev, :]
                new_v[..., :prev, :] = self.values[..., :prev, :]
            self.keys, self.values = new_k, new_v
        self.keys[..., prev:prev + S, :] = keys
        if not self.keys_only:
            self.values[..., prev:prev + S, :] = values
        self.offset = prev + S
        return self.keys[..., :self.offset, :], self.values[..., :self.offset, :]

    @property
    def state(self):
        if self.keys is None:
            return []
        return [self.keys[..., :self.offset, :], self.values[..., :self.offset, :]]

    @state.setter
    def state(self, v):
        if v:
            self.keys, self.values = v
            self.offset = self.keys.shape[2]

    def to_quantized(self, group_size: int = 64, bits: int = 8, v_bits: int | None = None):
        """Group-affine quantized copy of this cache (keys at `bits`, values at `v_bits`)."""
        from .mixed_cache import MixedQuantKVCache
        return MixedQuantKVCache.from_kvcache(self, k_bits=bits, v_bits=bits if v_bits is None else v_bits,
                                              group_size=group_size)

    def make_mask(self, N, return_array: bool = False, window_size=None):
        if N == 1:
            return None
        if return_array or (window_size is not None and N > window_size):
            dev = self.keys.device if self.keys is not None else None
            return create_causal_mask(N, offset=self.offset, window_size=window_size, device=dev)
        return "causal"

    def empty(self):
        return self.keys is None

    def is_trimmable(self):
        return True

    def trim(self, n):
        n = min(self.offset, n)
        self.offset -= n
        return n

    def size(self):
        return self.offset


def _dense_sdpa(queries, keys, values, scale, mask):
    """Library attention for caches that are not quantized (not the hot path)."""
    B, n_q, L, D = queries.shape
    n_kv = keys.shape[1]
    if n_kv != n_q:
        rep = n_q // n_kv
        keys = keys.repeat_interleave(rep, dim=1)
        values = values.repeat_interleave(rep, dim=1)
    if isinstance(mask, str):
        S = keys.shape[2]
        mask = create_causal_mask(L, offset=S - L, device=queries.device)
    if mask is not None and mask.dtype != torch.bool:
        mask = mask.to(queries.dtype)
    return F.scaled_dot_product_attention(queries, keys, values, attn_mask=mask, scale=scale)


def scaled_dot_product_attention(queries, keys, values, cache, scale, mask, sinks=None):
    """Default attention entry point: models import this symbol, and
    `patch.apply_patch` replaces it with the TurboQuant-aware router."""
    return _dense_sdpa(queries, keys, values, scale, mask)


_dense_sdpa_entry = scaled_dot_product_attention
