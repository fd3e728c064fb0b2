"""Hybrid cache: 8-bit group-affine keys + PolarQuant-packed values (reference
turboquant_mlx/hybrid_cache.py:25-100) and its attention (hybrid_attention.py:21-88).

Until `maybe_quantize_k()` is called the cache behaves like the reference's: keys are
kept as they arrive, values are packed and dequantized on fetch, attention runs on plain
tensors.  After it the keys are group-affine codes (group 64, this library's own format,
see affine.py - the reference delegates to `KVCache.to_quantized` of mlx-lm), the cache
exposes `bits` / `group_size`, and the attention hook runs decode steps on the stored
codes and packed words in one split-K launch (tensor-core kernel for 8-bit keys with
3- or 4-bit values): neither K nor V is ever expanded in memory."""

from __future__ import annotations

import torch

from .affine import affine_dequantize, affine_quantize, affine_quantize_rows_into
from .base import KVCache
from .cache import TurboQuantKVCache, _zero
from .kernels import flash_decode, sparse_v_matvec


class HybridQuantCache:
    step = 256

    def __init__(self, k_bits: int = 8, k_group_size: int = 64, v_bits: int = 3, v_seed: int = 42):
        if k_bits != 8:
            raise ValueError(f"keys are stored at 8 bits, got k_bits={k_bits}")
        self._k_cache = KVCache(keys_only=True)
        self._v_tq = TurboQuantKVCache(bits=v_bits, seed=v_seed, v_only=True)
        self._k_bits = k_bits
        self._k_group_size = k_group_size
        self._v_bits = v_bits
        self._quantized_k = False
        self.k_codes = self.k_scales = self.k_biases = None
        self._k_offset = 0

    # ---- inserts --------------------------------------------------------------
    def update_and_fetch(self, keys, values):
        """Before `maybe_quantize_k`: store K as is, compress V, return (K, V dequantized).
        After it: quantize the new K rows into the code storage, pack V, return shape-only
        placeholders (attention reads the stored codes)."""
        if not self._quantized_k:
            k_out, _ = self._k_cache.update_and_fetch(keys, values)
            _, v_out = self._v_tq.update_and_fetch(keys, values)
            return k_out, v_out
        B, H, S, dk = keys.shape
        self._ensure_k(B, H, S, dk, keys.device)
        p = self._k_offset
        done = False
        if S == 1:            # one decode step: straight into the storage rows
            kx = keys[:, :, 0]
            if kx.stride(2) == 1 and (B == 1 or kx.stride(0) == H * kx.stride(1)) and not (H > 1 and kx.stride(1) == 0):
                rows = lambda t: t[:, :, p].as_strided((B * H, t.shape[3]), (t.stride(1), 1))  # noqa: E731
                done = affine_quantize_rows_into(kx.as_strided((B * H, dk), (kx.stride(1), 1)), rows(self.k_codes),
                                                 rows(self.k_scales), rows(self.k_biases), self._k_group_size,
                                                 self._k_bits)
        if not done:
            kc, ks, kb = affine_quantize(keys, self._k_group_size, self._k_bits)
            self.k_codes[:, :, p:p + S], self.k_scales[:, :, p:p + S], self.k_biases[:, :, p:p + S] = kc, ks, kb
        self._k_offset = p + S
        self._v_tq.update_and_fetch(keys, values)
        total = self._k_offset
        return (_zero(keys.dtype, keys.device).expand(B, H, total, dk),
                _zero(values.dtype, values.device).expand(B, H, total, values.shape[3]))

    def _ensure_k(self, B, H, n_new, dk, device):
        need = self._k_offset + n_new
        cur = 0 if self.k_codes is None else self.k_codes.shape[2]
        if need <= cur:
            return
        n = max(((need + self.step - 1) // self.step) * self.step, 2 * cur)
        g = self._k_group_size

        def grow(old, width, dtype):
            new = torch.zeros((B, H, n, width), dtype=dtype, device=device)
            if old is not None and self._k_offset:
                new[:, :, :self._k_offset] = old[:, :, :self._k_offset]
            return new

        self.k_codes = grow(self.k_codes, dk, torch.uint8)
        self.k_scales = grow(self.k_scales, dk // g, torch.float16)
        self.k_biases = grow(self.k_biases, dk // g, torch.float16)

    def maybe_quantize_k(self):
        """Convert the keys to 8-bit group-affine codes (after prefill) and stop keeping a
        dequantized copy of V (hybrid_cache.py:57-63)."""
        if self._quantized_k or self._k_cache.offset == 0:
            return
        kc = self._k_cache
        keys = kc.keys[..., :kc.offset, :]
        B, H, S, dk = keys.shape
        self._ensure_k(B, H, S, dk, keys.device)
        c, s, b = affine_quantize(keys, self._k_group_size, self._k_bits)
        self.k_codes[:, :, :S], self.k_scales[:, :, :S], self.k_biases[:, :, :S] = c, s, b
        self._k_offset = S
        self._k_dtype = keys.dtype
        kc.keys = kc.values = None
        tq = self._v_tq
        tq.fused = True                       # inserts stop maintaining the dequantized V buffer
        tq._k_deq_buf = tq._v_deq_buf = None
        tq._deq_offset = tq._deq_alloc = 0
        self._quantized_k = True

    # ---- attention ------------------------------------------------------------
    def descriptors(self):
        t, tq = self.offset, self._v_tq
        k = dict(format="affine", codes=self.k_codes[:, :, :t], scales=self.k_scales[:, :, :t],
                 biases=self.k_biases[:, :, :t], bits=self._k_bits, group=self._k_group_size)
        v = dict(format="polar", packed=tq.v_packed[:, :, :t], norms=tq.v_norms[:, :, :t],
                 centroids=tq._v_q.centroids, signs=tq._v_q.signs, bits=tq._v_q.bits)
        return k, v

    def dequantized(self, dtype=None):
        dtype = dtype or getattr(self, "_k_dtype", torch.float16)
        t = self.offset
        k = affine_dequantize(self.k_codes[:, :, :t], self.k_scales[:, :, :t], self.k_biases[:, :, :t],
                              self._k_group_size, self._k_bits, dtype)
        _, v = self._v_tq.dequantized(dtype)
        return k, v

    def quantized_attention(self, queries, scale, mask=None):
        """What the attention hook calls once `bits` is set: queries (B, n_q, L, dim) ->
        (B, n_q, L, dim); L == 1 is one decode launch over the codes and packed words."""
        if queries.shape[2] == 1:
            k, v = self.descriptors()
            m3 = None
            if mask is not None and not isinstance(mask, str):
                from .fused_attention import _mask_3d
                if mask.dtype == torch.bool:
                    mask = torch.where(mask, 0.0, float("-inf"))
                m3 = _mask_3d(mask, queries.shape[0], queries.shape[1], self.offset)
            out = flash_decode(queries[:, :, 0, :], k=k, v=v, attn_scale=scale, mask=m3, out_dtype=queries.dtype)
            return out.unsqueeze(2)
        from .patch import _prefill_sdpa
        k, v = self.dequantized(queries.dtype)
        return _prefill_sdpa(queries, k, v, scale, mask)

    # ---- cache protocol -------------------------------------------------------
    @property
    def offset(self):
        return self._k_offset if self._quantized_k else self._k_cache.offset

    @property
    def state(self):
        if self._quantized_k:
            t = self.offset
            return [self.k_codes[:, :, :t], self.k_scales[:, :, :t], self.k_biases[:, :, :t]]
        return self._k_cache.state

    @property
    def bits(self):
        """Set only once K is quantized: attention routers key on it."""
        return self._k_bits if self._quantized_k else None

    @property
    def group_size(self):
        return self._k_group_size if self._quantized_k else None

    @property
    def nbytes(self):
        k = 0
        if self._quantized_k:
            B, H = self.k_codes.shape[:2]
            k = B * H * self.offset * (self.k_codes.shape[3] + 2 * 2 * self.k_scales.shape[3])
        elif self._k_cache.keys is not None:
            B, H, _, dk = self._k_cache.keys.shape
            k = B * H * self.offset * dk * self._k_cache.keys.element_size()
        return k + self._v_tq.nbytes

    def make_mask(self, N, return_array: bool = False, window_size=None):
        from .base import create_causal_mask
        if N == 1:
            return None
        if return_array or (window_size is not None and N > window_size):
            dev = self._v_tq.v_packed.device if self._v_tq.v_packed is not None else None
            return create_causal_mask(N, offset=self.offset, window_size=window_size, device=dev)
        return "causal"

    def empty(self):
        return self.offset == 0

    def is_trimmable(self):
        return True

    def trim(self, n):
        n = min(self.offset, n)
        if self._quantized_k:
            self._k_offset -= n
        else:
            self._k_cache.trim(n)
        self._v_tq.trim(n)
        return n

    def size(self):
        return self.offset


def hybrid_quantized_attention(queries, q_keys, v_packed, v_norms, v_centroids, v_signs, scale: float, mask,
                               k_group_size: int = 64, k_bits: int = 8, v_dim: int = 128, v_bits: int = 3,
                               sparse_v_threshold: float = 0.0):
    """queries (B, n_q, L, D); q_keys = (codes, scales, biases) of the group-affine keys
    (B, n_kv, S, .); packed values (B, n_kv, S, pdim) + norms (B, n_kv, S) -> (B, n_q, L, v_dim)
    in queries.dtype (hybrid_attention.py:21-88).  One decode launch when L == 1 and no value
    is skipped; otherwise the reference's composition (scores on dequantized keys, softmax,
    packed-V weighted sum per batch element and query position).  The reference reshapes its
    (batch, position, head) stack as (batch, head, position), which is only right for L == 1;
    here the result is transposed properly."""
    B, n_q, L, D = queries.shape
    codes, scales, biases = q_keys
    n_kv, S = codes.shape[1], codes.shape[2]
    n_rep = n_q // n_kv
    bool_or_array = mask is not None and not isinstance(mask, str)
    if L == 1 and sparse_v_threshold <= 0.0:
        k = dict(format="affine", codes=codes, scales=scales, biases=biases, bits=k_bits, group=k_group_size)
        v = dict(format="polar", packed=v_packed, norms=v_norms, centroids=v_centroids, signs=v_signs, bits=v_bits)
        m3 = None
        if bool_or_array:
            from .fused_attention import _mask_3d
            m = torch.where(mask, 0.0, float("-inf")) if mask.dtype == torch.bool else mask
            m3 = _mask_3d(m, B, n_q, S)
        return flash_decode(queries[:, :, 0, :], k=k, v=v, attn_scale=scale, mask=m3,
                            out_dtype=queries.dtype).unsqueeze(2)
    kd = affine_dequantize(codes, scales, biases, k_group_size, k_bits, torch.float32)
    if n_rep > 1:
        kd = kd.repeat_interleave(n_rep, dim=1)
    scores = torch.matmul(queries.float() * scale, kd.transpose(-1, -2))          # (B, n_q, L, S)
    if mask is not None:
        if isinstance(mask, str):
            qi = torch.arange(S - L, S, device=scores.device)
            mask = qi[:, None] >= torch.arange(S, device=scores.device)[None]
        if mask.dtype == torch.bool:
            scores = torch.where(mask, scores, torch.finfo(scores.dtype).min)
        else:
            scores = scores + mask
    weights = torch.softmax(scores, dim=-1)
    outs = []
    for b in range(B):
        for l in range(L):
            outs.append(sparse_v_matvec(weights[b, :, l, :], v_packed[b], v_norms[b], v_centroids, v_signs,
                                        v_dim, v_bits, threshold=sparse_v_threshold, n_rep=n_rep))
    return torch.stack(outs, dim=0).reshape(B, L, n_q, v_dim).transpose(1, 2).to(queries.dtype)
