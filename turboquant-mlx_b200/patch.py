"""Attention hook (reference turboquant_mlx/patch.py:14-81): replaces the
`scaled_dot_product_attention` symbol of `base` and of every loaded module that
imported it, so decode over a fused TurboQuant cache runs on the packed
storage.  `remove_patch` restores every binding it replaced."""

from __future__ import annotations

import sys

from . import base as _base

_original_sdpa = None
_patched = False
_replaced: list = []   # (module, attribute) pairs that now point at _patched_sdpa


def _prefill_sdpa(queries, keys, values, scale, mask):
    """Multi-token attention over dense keys / values: the tensor-core prefill
    kernel when it covers the call, the library attention otherwise."""
    from .kernels import prefill_attention, prefill_supported
    if queries.shape[2] > 1 and prefill_supported(queries, keys, values, mask):
        return prefill_attention(queries, keys, values, scale, causal=mask is not None)
    return _base._dense_sdpa(queries, keys, values, scale, mask)


def _patched_sdpa(queries, keys, values, cache, scale, mask, sinks=None):
    """Fused TurboQuant decode, affine-quantized decode, or the original attention."""
    from .cache import TurboQuantKVCache
    from .v_only_cache import VOnlyTurboQuantCache

    is_decode = queries.shape[2] == 1
    if isinstance(cache, TurboQuantKVCache) and cache.offset > 0 and cache.fused and not cache.v_only:
        from .fused_attention import short_step_supported
        if is_decode or short_step_supported(queries, cache.k_packed.shape[1], mask):
            from .fused_attention import turboquant_attention
            return turboquant_attention(queries, cache, scale, mask,
                                        sparse_v_threshold=cache.sparse_v_threshold)
        # multi-token step on a fused cache: the placeholders returned by
        # update_and_fetch hold no data, so attend over the dequantized storage
        k, v = cache.dequantized(queries.dtype)
        return _prefill_sdpa(queries, k, v, scale, mask)
    if isinstance(cache, VOnlyTurboQuantCache) and cache.fused and cache.offset > 0:
        from .fused_attention import short_step_supported
        if is_decode or short_step_supported(queries, cache._v_tq.v_packed.shape[1], mask):
            from .v_only_cache import v_only_attention
            return v_only_attention(queries, cache, scale, mask)
        _, v = cache._v_tq.dequantized(queries.dtype)
        return _prefill_sdpa(queries, keys, v, scale, mask)
    if hasattr(cache, "bits") and getattr(cache, "bits", None) is not None and hasattr(cache, "quantized_attention"):
        return cache.quantized_attention(queries, scale, mask)
    if not is_decode and sinks is None and _original_sdpa in (None, _base._dense_sdpa_entry):
        return _prefill_sdpa(queries, keys, values, scale, mask)       # dense cache, prompt step
    return (_original_sdpa or _base._dense_sdpa_entry)(queries, keys, values, cache, scale, mask, sinks=sinks)


def apply_patch():
    """Route attention through the TurboQuant-aware function."""
    global _patched, _original_sdpa
    if _patched:
        return
    _original_sdpa = _base.scaled_dot_product_attention
    for name, mod in list(sys.modules.items()):
        if mod is None or not hasattr(mod, "scaled_dot_product_attention"):
            continue
        if getattr(mod, "scaled_dot_product_attention") is _original_sdpa:
            setattr(mod, "scaled_dot_product_attention", _patched_sdpa)
            _replaced.append((mod, "scaled_dot_product_attention"))
    _patched = True


def remove_patch():
    """Undo apply_patch on every module it touched."""
    global _patched, _original_sdpa
    if not _patched:
        return
    for mod, attr in _replaced:
        if getattr(mod, attr, None) is _patched_sdpa:
            setattr(mod, attr, _original_sdpa)
    _replaced.clear()
    _original_sdpa = None
    _patched = False
