"""V-only TurboQuant cache: keys stay fp16/bf16, values are PolarQuant-packed
(reference turboquant_mlx/v_only_cache.py:24-127).

With `fused=False` (the reference's behaviour) values are dequantized into an
incremental buffer and attention runs on plain tensors.  With `fused=True`
decode attention reads the dense keys and the packed values in one
flash-decode launch (`v_only_attention`), and no dequantized V buffer exists."""

from __future__ import annotations

import torch

from .base import KVCache
from .cache import TurboQuantKVCache
from .kernels import flash_decode


class VOnlyTurboQuantCache:
    """KV cache with un-quantized keys and TurboQuant-compressed values.

    Does not expose `.bits` / `.group_size`, so an attention router treats it
    as a plain cache unless `fused` is set."""

    def __init__(self, bits: int = 3, seed: int = 42, no_v_buffer: bool = False,
                 fused: bool = False, defer_append: bool = False, inputs_stable: bool = False):
        """`defer_append` (fused caches only, an addition to the reference's arguments): a
        one-token `update_and_fetch` only records the new rows; the decode attention that
        follows stores the key row and quantizes the value row inside its own launch, so a
        decode step is one kernel per layer.  The rows handed to `update_and_fetch` must stay
        unchanged until that attention call (or until anything else reads the cache, which
        materialises them first).  `inputs_stable`: the caller promises that neither the queries and
        new rows of a decode step nor this cache's storage are written by a kernel that may
        still be running when the step's attention kernel starts (see `kv_stable` / `q_stable`
        of `kernels.flash_decode`); the decode launches of consecutive layers then overlap."""
        self._k_cache = KVCache(keys_only=True)
        self._v_tq = TurboQuantKVCache(bits=bits, seed=seed, v_only=True, fused=fused)
        self._v_bits = bits
        self._no_v_buffer = no_v_buffer
        self.fused = fused
        self.defer_append = defer_append and fused
        self.inputs_stable = inputs_stable
        self._pending = None      # (new K rows, new V rows) (B, H, D) awaiting the attention launch
        self._decode_ws = None    # this cache's own decode workspace (inputs_stable: launches of different layers overlap)

    def reserve(self, B, H, n_positions, k_dim, v_dim, dtype=torch.float16, device=None):
        """Pre-size K and V storage for `n_positions` so inserts never reallocate."""
        self._v_tq.reserve(B, H, n_positions, k_dim, v_dim, device)
        kc = self._k_cache
        if kc.keys is None or kc.keys.shape[2] < n_positions:
            new_k = torch.zeros((B, H, n_positions, k_dim), dtype=dtype, device=self._v_tq.v_packed.device)
            if kc.keys is not None:
                new_k[..., :kc.offset, :] = kc.keys[..., :kc.offset, :]
            kc.keys = new_k
            kc.values = torch.zeros((B, H, n_positions, 0), dtype=dtype, device=new_k.device)

    def _append_fused(self, keys, values):
        """Decode-step append in one launch (`tq_quantize_append`): the K rows are copied and the V
        rows quantized by the same kernel.  Only when nothing has to grow and every view is
        row-uniform and 16-byte friendly; returns None otherwise."""
        kc, tq = self._k_cache, self._v_tq
        B, H, S, Dk = keys.shape
        if not (self.fused and keys.is_cuda and S <= 4 and kc.keys is not None and tq.v_packed is not None):
            return None
        prev = kc.offset
        if prev != tq.offset or prev + S > kc.keys.shape[2] or prev + S > tq.v_packed.shape[2]:
            return None
        if kc.keys.dtype != keys.dtype or kc.keys.shape[:2] != (B, H) or kc.keys.shape[3] != Dk:
            return None
        Dv = values.shape[3]
        if tq._v_q is None or tq._v_q.dim != Dv or not values.is_contiguous() or not keys.is_contiguous():
            return None
        es = keys.element_size()
        if (S * Dk * es) % 16 or (kc.keys.shape[2] * Dk * es) % 16 or (prev * Dk * es) % 16 or keys.data_ptr() % 16:
            return None
        src = keys.view(B * H, S * Dk)
        dst = kc.keys.view(B * H, kc.keys.shape[2] * Dk)[:, prev * Dk:(prev + S) * Dk]
        from .kernels import quantize_append
        q = tq._v_q
        tq._dtype = keys.dtype
        quantize_append(values.view(B * H, S, Dv), q.signs, q.boundaries, Dv, q.bits,
                        tq.v_packed.view(B * H, tq.v_packed.shape[2], tq.v_packed.shape[3]),
                        tq.v_norms.view(B * H, tq.v_norms.shape[2]), prev, src, dst)
        kc.offset = prev + S
        tq.offset = prev + S
        from .cache import _zero
        return kc.keys[..., :kc.offset, :], _zero(values.dtype, values.device).expand(B, H, kc.offset, Dv)

    def _defer(self, keys, values):
        """Record a one-token append for the next decode attention; None when it does not qualify
        (storage must exist with room, fp16 keys of the cache's type, head_dim 128)."""
        kc, tq = self._k_cache, self._v_tq
        B, H, S, Dk = keys.shape
        if not (self.defer_append and S == 1 and keys.is_cuda and kc.keys is not None and tq.v_packed is not None):
            return None
        prev = kc.offset
        if prev != tq.offset or prev + 1 > kc.keys.shape[2] or prev + 1 > tq.v_packed.shape[2]:
            return None
        if kc.keys.dtype != torch.float16 or keys.dtype != torch.float16 or values.dtype != torch.float16:
            return None
        if kc.keys.shape[:2] != (B, H) or Dk != 128 or values.shape[3] != 128 or tq._v_q is None:
            return None
        if tq._v_q.bits not in (3, 4) or keys.data_ptr() % 16 or any(st % 8 for st in keys.stride()[:2]):
            return None
        tq._dtype = keys.dtype
        self._pending = (keys[:, :, 0, :], values[:, :, 0, :])
        kc.offset = prev + 1
        tq.offset = prev + 1
        from .cache import _zero
        return kc.keys[..., :kc.offset, :], _zero(values.dtype, values.device).expand(B, H, kc.offset, values.shape[3])

    def flush_pending(self):
        """Materialise a deferred append with the ordinary append kernel (anything that reads the
        storage other than the decode attention calls this first)."""
        if self._pending is None:
            return
        k_row, v_row = self._pending
        self._pending = None
        self._k_cache.offset -= 1
        self._v_tq.offset -= 1
        defer, self.defer_append = self.defer_append, False
        try:
            self.update_and_fetch(k_row.unsqueeze(2), v_row.unsqueeze(2))
        finally:
            self.defer_append = defer

    def take_pending(self):
        """The deferred rows (or None), handing responsibility for them to the caller."""
        rows, self._pending = self._pending, None
        return rows

    def update_and_fetch(self, keys, values):
        """Store K as is, compress V, return (K, V_dequant)."""
        self.flush_pending()
        deferred = self._defer(keys, values)
        if deferred is not None:
            return deferred
        fused = self._append_fused(keys, values)
        if fused is not None:
            return fused
        k_out, _ = self._k_cache.update_and_fetch(keys, values)
        if self._no_v_buffer and not self.fused:
            # quantize, then re-dequantize everything from packed storage each call
            tq = self._v_tq
            B, H, S, v_dim = values.shape
            tq._dtype = keys.dtype
            tq._ensure_quantizer(keys.shape[-1], v_dim, values.device)
            tq._ensure_storage(B, H, S, values.device)
            tq._insert(values, tq._v_q, tq.v_packed, tq.v_norms, tq.offset)
            tq.offset += S
            _, v_out = tq.dequantized(values.dtype)
        else:
            _, v_out = self._v_tq.update_and_fetch(keys, values)
        return k_out, v_out

    @property
    def offset(self):
        return self._k_cache.offset

    @property
    def state(self):
        self.flush_pending()
        k_state = list(self._k_cache.state) if self._k_cache.state else []
        v_state = list(self._v_tq.state) if self._v_tq.state else []
        return k_state + v_state

    @property
    def state_with_signs(self):
        """`state` followed by the V sign vector (see TurboQuantKVCache.state_with_signs)."""
        return self.state + [self._v_tq._v_q.signs]

    @property
    def meta_state(self):
        return f"VOnlyTQ,{self._v_bits},{self._v_tq.seed},{self._v_tq.meta_state}"

    @classmethod
    def from_state(cls, state, meta_state):
        parts = meta_state.split(",", 3)
        obj = cls(bits=int(parts[1]), seed=int(parts[2]))
        if len(state) >= 2:
            obj._k_cache.keys = state[0].contiguous()
            obj._k_cache.values = state[1].contiguous()
            obj._k_cache.offset = state[0].shape[2]
        if len(state) > 2:
            obj._v_tq.meta_state = parts[3]
            obj._v_tq.state = state[2:]          # 2 arrays, or 3 with the saved V sign vector
            obj._v_tq._v_pdim = obj._v_tq.v_packed.shape[-1]
            if obj._v_tq._v_dim:
                obj._v_tq._ensure_quantizer(state[0].shape[-1], obj._v_tq._v_dim, obj._v_tq.v_packed.device)
        return obj

    def make_mask(self, *args, **kwargs):
        return self._k_cache.make_mask(*args, **kwargs)

    def empty(self):
        return self._k_cache.offset == 0

    def is_trimmable(self):
        return True

    def trim(self, n):
        self.flush_pending()
        self._k_cache.trim(n)
        return self._v_tq.trim(n)

    def size(self):
        return self._k_cache.offset


def v_only_attention(queries, cache: VOnlyTurboQuantCache, attn_scale: float, mask=None,
                     kv_stable: bool = False, out=None, q_stable: bool | None = None):
    """Decode attention for a fused V-only cache: queries (B, n_q, 1, dim),
    dense K and packed V read once per KV head -> (B, n_q, 1, dim).  A deferred
    one-token append of the cache is carried out by the same launch.  A short multi-token step
    (queries (B, n_q, T, dim), `short_step_supported`) attends causally over the same packed rows."""
    tq = cache._v_tq
    if queries.shape[2] > 1:
        from .fused_attention import short_step_supported
        if not short_step_supported(queries, tq.v_packed.shape[1], mask):
            raise ValueError("a multi-token step needs mask='causal', dim 128 and n_rep * tokens <= 8")
        cache.flush_pending()
        total = cache.offset
        k = dict(format="dense", data=cache._k_cache.keys[:, :, :total, :])
        v = dict(format="polar", packed=tq.v_packed[:, :, :total, :], norms=tq.v_norms[:, :, :total],
                 centroids=tq._v_q.centroids, signs=tq._v_q.signs, bits=tq._v_q.bits)
        return flash_decode(queries, k=k, v=v, attn_scale=attn_scale, out_dtype=queries.dtype, out=out)
    if q_stable is None:
        q_stable = cache.inputs_stable
    m3 = None
    if mask is not None and not isinstance(mask, str):
        from .fused_attention import _mask_3d
        if mask.dtype == torch.bool:
            mask = torch.where(mask, 0.0, float("-inf"))
        m3 = _mask_3d(mask, queries.shape[0], queries.shape[1], cache.offset)
    n_rep = queries.shape[1] // max(1, tq.v_packed.shape[1])
    if cache._pending is not None and (m3 is not None or n_rep > 8 or queries.shape[-1] != 128):
        cache.flush_pending()       # the in-launch append needs the tensor-core kernel
    total = cache.offset
    k = dict(format="dense", data=cache._k_cache.keys[:, :, :total, :])
    v = dict(format="polar", packed=tq.v_packed[:, :, :total, :], norms=tq.v_norms[:, :, :total],
             centroids=tq._v_q.centroids, signs=tq._v_q.signs, bits=tq._v_q.bits, boundaries=tq._v_q.boundaries)
    rows = cache.take_pending()
    new_k, new_v = rows if rows is not None else (None, None)
    # a workspace of the cache's own: decode launches of different layers overlap end to end
    owner = cache if (q_stable and (kv_stable or cache.inputs_stable) and m3 is None) else None
    res = flash_decode(queries[:, :, 0, :], k=k, v=v, attn_scale=attn_scale, mask=m3,
                       out_dtype=queries.dtype, kv_stable=kv_stable or q_stable,
                       q_stable=q_stable, new_k=new_k, new_v=new_v, workspace_owner=owner,
                       out=None if out is None else out[:, :, 0, :])
    return res.unsqueeze(2)
