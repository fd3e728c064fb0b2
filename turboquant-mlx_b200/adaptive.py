"""Layer-adaptive cache list (reference turboquant_mlx/adaptive.py:13-57):
plain caches for the first and last `fp16_layers` layers, TurboQuant caches in
between.  Unlike the reference, `k_bits` / `v_bits` take effect."""

from __future__ import annotations

from .base import KVCache
from .cache import TurboQuantKVCache


def make_adaptive_cache(num_layers: int, bits: int = 3, fp16_layers: int = 4, seed: int = 42,
                        fused: bool = False, k_bits: int | None = None, v_bits: int | None = None,
                        model=None):
    if model is not None and hasattr(model, "make_cache"):
        raise ValueError("model provides its own make_cache(); adaptive caches need uniform layers")
    caches = []
    for i in range(num_layers):
        if i < fp16_layers or i >= num_layers - fp16_layers:
            caches.append(KVCache())
        else:
            caches.append(TurboQuantKVCache(bits=bits, seed=seed + 2 * i, fused=fused,
                                            k_bits=k_bits, v_bits=v_bits))
    return caches
