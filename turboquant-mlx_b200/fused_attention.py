"""Decode attention straight from the packed cache (reference
turboquant_mlx/fused_attention.py:20-125).

The reference loops over the batch in Python and launches prerotate_query,
prerot_fused_qk_scores, softmax and sparse_v_matvec per element.  Here the
default route is one split-K flash-decode launch for the whole batch, also with
`sparse_v_threshold > 0`: the kernel then drops value tiles whose weights are
certain to end below the threshold (a subset of what the reference's exact rule
`w < threshold` drops, sparse_v.py:61).  The composed route is kept for
`v_buffer`, and for thresholds on calls the tensor-core kernel does not cover."""

from __future__ import annotations

import torch

from .kernels import flash_decode, prerot_fused_qk_scores, prerotate_query, sparse_v_matvec


def _mask_for_batch(mask, b, n_q_heads, total):
    m = mask
    if m.ndim == 4:
        m = m[min(b, m.shape[0] - 1)]
        if m.ndim == 3:
            m = m[:, 0, :]
            if m.shape[0] == 1:
                m = m.expand(n_q_heads, total)
    elif m.ndim == 3:
        m = m[min(b, m.shape[0] - 1), 0, :]
        m = m.reshape(1, -1).expand(n_q_heads, total)
    return m


def _mask_3d(mask, B, n_q_heads, total):
    """Additive mask broadcastable to (B, n_q, total), following the indexing
    rules of fused_attention.py:81-92."""
    m = mask
    if m.ndim == 4:
        m = m[:, :, 0, :]
    elif m.ndim == 3:
        m = m[:, 0, :].unsqueeze(1)
    elif m.ndim == 2:
        m = m.unsqueeze(0)
    elif m.ndim == 1:
        m = m.reshape(1, 1, -1)
    if m.shape[0] not in (1, B):
        idx = torch.clamp(torch.arange(B, device=m.device), max=m.shape[0] - 1)
        m = m[idx]
    return m


def cache_kv_descriptors(cache):
    """K / V descriptors of a TurboQuantKVCache for `kernels.flash_decode`."""
    total = cache.offset
    k = dict(format="polar", packed=cache.k_packed[:, :, :total, :], norms=cache.k_norms[:, :, :total],
             centroids=cache._k_q.centroids, signs=cache._k_q.signs, bits=cache._k_q.bits,
             boundaries=cache._k_q.boundaries)
    v = dict(format="polar", packed=cache.v_packed[:, :, :total, :], norms=cache.v_norms[:, :, :total],
             centroids=cache._v_q.centroids, signs=cache._v_q.signs, bits=cache._v_q.bits,
             boundaries=cache._v_q.boundaries)
    return k, v


def short_step_supported(queries, n_kv_heads: int, mask) -> bool:
    """A multi-token step the decode kernel takes as it is: the T new tokens (already stored) attend
    causally, and their n_rep * T (token, head) rows fit the eight rows of the kernel's MMA tile."""
    B, n_q_heads, T, dim = queries.shape
    n_rep = n_q_heads // max(1, n_kv_heads)
    return (T > 1 and isinstance(mask, str) and mask == "causal" and dim == 128 and n_rep * T <= 8
            and queries.dtype in (torch.float16, torch.bfloat16, torch.float32))


def turboquant_attention(queries, cache, attn_scale: float, mask=None, v_buffer=None,
                         sparse_v_threshold: float | None = None) -> torch.Tensor:
    """queries (B, n_heads, 1, dim) -> (B, n_heads, 1, dim) in queries.dtype; also a short causal
    multi-token step (B, n_heads, T, dim) with n_rep * T <= 8 (`short_step_supported`), which the
    reference leaves to dense attention (patch.py:19-21)."""
    B, n_q_heads, S_q, dim = queries.shape
    n_kv_heads = cache.k_packed.shape[1]
    n_rep = n_q_heads // n_kv_heads
    thr = sparse_v_threshold if (sparse_v_threshold is not None and sparse_v_threshold >= 0.0) else 0.0
    if S_q > 1:
        if v_buffer is not None or not short_step_supported(queries, n_kv_heads, mask):
            raise ValueError("a multi-token step needs mask='causal', dim 128, n_rep * tokens <= 8 and no v_buffer")
        if hasattr(cache, "flush_pending"):
            cache.flush_pending()
        k, v = cache_kv_descriptors(cache)
        return flash_decode(queries, k=k, v=v, attn_scale=attn_scale, out_dtype=queries.dtype,
                            sparse_v_threshold=thr)
    has_mask = mask is not None and not isinstance(mask, str)
    pending = getattr(cache, "_pending", None) is not None
    fused_ok = v_buffer is None and (thr == 0.0 or not (has_mask or n_rep > 8 or dim != 128))
    if pending and (not fused_ok or has_mask or n_rep > 8 or dim != 128):
        cache.flush_pending()          # the in-launch insert needs the tensor-core decode kernel
    total = cache.offset

    if fused_ok:
        k, v = cache_kv_descriptors(cache)
        m3 = None
        if has_mask:
            if mask.dtype == torch.bool:
                mask = torch.where(mask, 0.0, float("-inf"))
            m3 = _mask_3d(mask, B, n_q_heads, total)
        rows = cache.take_pending() if hasattr(cache, "take_pending") else None
        new_k, new_v = rows if rows is not None else (None, None)
        stable = bool(getattr(cache, "inputs_stable", False))
        # a workspace of the cache's own: decode launches of different layers overlap end to end
        owner = cache if (stable and m3 is None) else None
        active = None
        if thr > 0.0 and getattr(cache, "track_active_positions", False):
            active = torch.empty((B, n_kv_heads), dtype=torch.int32, device=queries.device)
            cache.last_active_positions = active
        out = flash_decode(queries[:, :, 0, :], k=k, v=v, attn_scale=attn_scale, mask=m3,
                           out_dtype=queries.dtype, kv_stable=stable, q_stable=stable,
                           new_k=new_k, new_v=new_v, sparse_v_threshold=thr, active_out=active, workspace_owner=owner)
        return out.unsqueeze(2)

    outputs = []
    for b in range(B):
        kp = cache.k_packed[b, :, :total, :]
        kn = cache.k_norms[b, :, :total]
        q = queries[b, :, 0, :]
        q_rot = prerotate_query(q, cache._k_q.signs)
        scores = prerot_fused_qk_scores(q_rot, kp, kn, cache._k_q.centroids, dim,
                                        cache._k_q.bits, n_rep=n_rep)
        scores = scores * attn_scale
        if mask is not None and not isinstance(mask, str):
            scores = scores + _mask_for_batch(mask, b, n_q_heads, total)
        weights = torch.softmax(scores, dim=-1)
        v_dim = cache._v_dim
        if v_buffer is not None:
            v_deq = v_buffer[b]
            if n_rep > 1:
                v_deq = v_deq.repeat_interleave(n_rep, dim=0)
            out = weights[:, None, :].to(queries.dtype) @ v_deq.to(queries.dtype)
        else:
            vp = cache.v_packed[b, :, :total, :]
            vn = cache.v_norms[b, :, :total]
            matvec = sparse_v_matvec(weights, vp, vn, cache._v_q.centroids, cache._v_q.signs,
                                     v_dim, cache._v_q.bits, threshold=thr, n_rep=n_rep)
            out = matvec[:, None, :].to(queries.dtype)
        outputs.append(out)
    return torch.stack(outputs, dim=0)
