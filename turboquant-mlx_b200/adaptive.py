"""Layer-adaptive cache list (reference turboquant_mlx/adaptive.py:13-57):
plain caches for the first and last `fp16_layers` layers, TurboQuant caches in
between.  Same positional order and the same model check as the reference;
unlike the reference, `k_bits` / `v_bits` take effect (its cache has one width)."""

from __future__ import annotations

from .base import KVCache
from .cache import TurboQuantKVCache


def make_adaptive_cache(num_layers: int, bits: int = 3, k_bits: int | None = None, v_bits: int | None = None,
                        fp16_layers: int = 4, seed: int = 42, fused: bool = False, model=None):
    """One cache per layer.  `model`: optional, checked for an architecture whose own
    `make_cache()` does not hand out plain KV caches (adaptive.py:38-46).  Every compressed
    layer uses `seed` (K) and `seed + 1` (V), as the reference does."""
    if model is not None and hasattr(model, "make_cache"):
        default_cache = model.make_cache()
        if default_cache and not isinstance(default_cache[0], KVCache):
            cache_type = type(default_cache[0]).__name__
            raise ValueError(
                f"[TurboQuant] Incompatible cache type: {cache_type}. "
                f"TurboQuant only works with standard multi-head attention "
                f"(KVCache). MLA, SSM, and hybrid architectures are not supported.")
    caches = []
    for i in range(num_layers):
        if i < fp16_layers or i >= num_layers - fp16_layers:
            caches.append(KVCache())
        else:
            caches.append(TurboQuantKVCache(bits=bits, seed=seed, fused=fused, k_bits=k_bits, v_bits=v_bits))
    return caches
