"""Mixed-precision group-affine KV cache: keys at `k_bits` (8), values at `v_bits`
(4 or 8), group size 64.

This is the cache the reference's README recommends (`MixedQuantKVCache.from_kvcache(
cache, k_bits=8, v_bits=4)` of its mlx-lm fork, README.md:28-47) and the format
`KVCache.to_quantized` produces in hybrid_cache.py:57-63.  Neither implementation
is part of the reference tree, so the number format is this library's own (see
affine.py).  Usage follows the README: prefill into a plain `KVCache`, convert once,
then decode; the attention hook recognises the cache by its `bits` attribute and
runs the quantized decode kernel on the stored codes (no dequantized copy)."""

from __future__ import annotations

import torch

from .affine import affine_dequantize, affine_quantize
from .cache import _zero
from .kernels import flash_decode


def H_stride_zero(rows_view) -> bool:
    """A (B * H, W) row view whose rows coincide (broadcast input): not a valid source."""
    return rows_view.shape[0] > 1 and rows_view.stride(0) == 0


class MixedQuantKVCache:
    step = 256

    def __init__(self, k_bits: int = 8, v_bits: int = 4, group_size: int = 64):
        if k_bits != 8:
            raise ValueError(f"keys are stored at 8 bits, got k_bits={k_bits}")
        if v_bits not in (4, 8):
            raise ValueError(f"values are stored at 4 or 8 bits, got v_bits={v_bits}")
        self.k_bits, self.v_bits, self.group_size = k_bits, v_bits, group_size
        self.bits = k_bits                 # what an attention router looks at
        self.offset = 0
        self.k_codes = self.k_scales = self.k_biases = None
        self.v_codes = self.v_scales = self.v_biases = None
        self._dtype = torch.float16
        self._static = None                # device-side length / position of the static decode mode

    # ---- static decode: lengths on the device, steps replayable from a CUDA graph -----------
    def enable_static_decode(self, max_len: int, counters: torch.Tensor | None = None) -> torch.Tensor:
        """Pre-size the storage for `max_len` positions and keep the sequence length on the device:
        one-token `update_and_fetch` calls then write at the device-side position and the decode
        kernel reads the device-side length, so a whole decode step can be captured once in a CUDA
        graph and replayed while the sequence grows (host-side `offset` goes stale during replays;
        `sync_offset()` reads it back).  `counters`: int32 (1 + B,) tensor [position, length per
        sequence] shared by the caches of all layers (made here when None); the caller advances it
        once per step with `counters += 1` after the last layer.  Returns the counters."""
        if self.k_codes is None:
            raise ValueError("static decode starts from a filled cache (prefill or convert first)")
        B, H = self.k_codes.shape[:2]
        dk = self.k_codes.shape[3]
        dv = self.v_codes.shape[3] * (1 if self.v_bits == 8 else 2)
        if max_len > self.k_codes.shape[2]:
            self._ensure(B, H, max_len - self.offset, dk, dv, self.k_codes.device)
        if counters is None:
            counters = torch.tensor([self.offset] + [self.offset + 1] * B, dtype=torch.int32,
                                    device=self.k_codes.device)
        elif counters.dtype != torch.int32 or counters.numel() != 1 + B:
            raise ValueError(f"counters must be an int32 tensor of {1 + B} elements")
        self._static = counters
        return counters

    def disable_static_decode(self):
        self.sync_offset()
        self._static = None

    def sync_offset(self) -> int:
        """Static decode: read the device-side position back into `offset` (synchronises)."""
        if self._static is not None:
            self.offset = int(self._static[0].item())
        return self.offset

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_kvcache(cls, cache, k_bits: int = 8, v_bits: int = 4, group_size: int = 64):
        """Quantize the contents of a plain KVCache (after prefill)."""
        obj = cls(k_bits, v_bits, group_size)
        if cache.keys is not None and cache.offset > 0:
            obj.update_and_fetch(cache.keys[..., :cache.offset, :], cache.values[..., :cache.offset, :])
        return obj

    def _ensure(self, B, H, n_new, dk, dv, device):
        need = self.offset + n_new
        cur = 0 if self.k_codes is None else self.k_codes.shape[2]
        if need <= cur:
            return
        n = max(((need + self.step - 1) // self.step) * self.step, 2 * cur)
        g = self.group_size
        vw = dv if self.v_bits == 8 else dv // 2

        def grow(old, width, dtype):
            new = torch.zeros((B, H, n, width), dtype=dtype, device=device)
            if old is not None and self.offset:
                new[:, :, :self.offset] = old[:, :, :self.offset]
            return new

        self.k_codes = grow(self.k_codes, dk, torch.uint8)
        self.k_scales = grow(self.k_scales, dk // g, torch.float16)
        self.k_biases = grow(self.k_biases, dk // g, torch.float16)
        self.v_codes = grow(self.v_codes, vw, torch.uint8)
        self.v_scales = grow(self.v_scales, dv // g, torch.float16)
        self.v_biases = grow(self.v_biases, dv // g, torch.float16)

    def update_and_fetch(self, keys, values):
        """Quantize and append; returns shape-only placeholders (attention reads the codes)."""
        B, H, S, dk = keys.shape
        dv = values.shape[3]
        self._dtype = keys.dtype
        self._ensure(B, H, S, dk, dv, keys.device)
        p = self.offset
        if self._static is not None:
            if S != 1 or not self._append_one(keys, values, 0, self._static):
                raise ValueError("static decode takes one token per step with row-uniform views")
            self.offset = p + 1            # host copy; the device counter is what the kernels read
            return (_zero(keys.dtype, keys.device).expand(B, H, self.offset, dk),
                    _zero(values.dtype, values.device).expand(B, H, self.offset, dv))
        if S == 1 and self._append_one(keys, values, p):
            self.offset = p + 1
            return (_zero(keys.dtype, keys.device).expand(B, H, self.offset, dk),
                    _zero(values.dtype, values.device).expand(B, H, self.offset, dv))
        kc, ks, kb = affine_quantize(keys, self.group_size, self.k_bits)
        vc, vs, vb = affine_quantize(values, self.group_size, self.v_bits)
        self.k_codes[:, :, p:p + S], self.k_scales[:, :, p:p + S], self.k_biases[:, :, p:p + S] = kc, ks, kb
        self.v_codes[:, :, p:p + S], self.v_scales[:, :, p:p + S], self.v_biases[:, :, p:p + S] = vc, vs, vb
        self.offset = p + S
        zk = _zero(keys.dtype, keys.device).expand(B, H, self.offset, dk)
        zv = _zero(values.dtype, values.device).expand(B, H, self.offset, dv)
        return zk, zv

    def _append_one(self, keys, values, p, position=None) -> bool:
        """One decode step: the (batch, head) rows are quantized straight into position p of the
        storage (two launches, no intermediate tensors).  False when a view is not row-uniform.
        With `position` (device counter) the rows go to p + position[0], read on the device."""
        from .affine import affine_quantize_rows_into

        def rows(t):            # (B, H, 1 or n, W) at position -> (B * H, W) view, or None
            v = t[:, :, 0] if t.shape[2] == 1 else t[:, :, p]
            B, H, W = v.shape
            if v.stride(2) != 1 or (B > 1 and v.stride(0) != H * v.stride(1)):
                return None
            return v.as_strided((B * H, W), (v.stride(1), 1))

        views = [rows(keys), rows(self.k_codes), rows(self.k_scales), rows(self.k_biases),
                 rows(values), rows(self.v_codes), rows(self.v_scales), rows(self.v_biases)]
        if any(v is None for v in views):
            return False
        kx, kc, ks, kb, vx, vc, vs, vb = views
        if H_stride_zero(kx) or H_stride_zero(vx):
            return False
        kps = (self.k_codes.stride(2), self.k_scales.stride(2))
        vps = (self.v_codes.stride(2), self.v_scales.stride(2))
        return (affine_quantize_rows_into(kx, kc, ks, kb, self.group_size, self.k_bits, position, kps) and
                affine_quantize_rows_into(vx, vc, vs, vb, self.group_size, self.v_bits, position, vps))

    # ---- attention --------------------------------------------------------------
    def descriptors(self):
        # static decode: the whole allocation, the valid length comes from the device counter
        t = self.offset if self._static is None else self.k_codes.shape[2]
        k = dict(format="affine", codes=self.k_codes[:, :, :t], scales=self.k_scales[:, :, :t],
                 biases=self.k_biases[:, :, :t], bits=self.k_bits, group=self.group_size)
        v = dict(format="affine", codes=self.v_codes[:, :, :t], scales=self.v_scales[:, :, :t],
                 biases=self.v_biases[:, :, :t], bits=self.v_bits, group=self.group_size)
        return k, v

    def dequantized(self, dtype=None):
        dtype = dtype or self._dtype
        t = self.offset
        k = affine_dequantize(self.k_codes[:, :, :t], self.k_scales[:, :, :t], self.k_biases[:, :, :t],
                              self.group_size, self.k_bits, dtype)
        v = affine_dequantize(self.v_codes[:, :, :t], self.v_scales[:, :, :t], self.v_biases[:, :, :t],
                              self.group_size, self.v_bits, dtype)
        return k, v

    def quantized_attention(self, queries, scale, mask=None):
        """queries (B, n_q, L, dim) -> (B, n_q, L, dim).  L == 1 runs the quantized
        decode kernel; longer steps attend over the dequantized tensors."""
        if queries.shape[2] == 1:
            k, v = self.descriptors()
            m3 = None
            if mask is not None and not isinstance(mask, str):
                from .fused_attention import _mask_3d
                if mask.dtype == torch.bool:
                    mask = torch.where(mask, 0.0, float("-inf"))
                m3 = _mask_3d(mask, queries.shape[0], queries.shape[1], self.offset)
            lens = None
            if self._static is not None:
                if m3 is not None:
                    raise ValueError("static decode does not take a mask")
                lens = self._static[1:]
            out = flash_decode(queries[:, :, 0, :], k=k, v=v, attn_scale=scale, mask=m3, out_dtype=queries.dtype,
                               seq_lens=lens)
            return out.unsqueeze(2)
        from .base import _dense_sdpa
        k, v = self.dequantized(queries.dtype)
        return _dense_sdpa(queries, k, v, scale, mask)

    # ---- cache protocol ------------------------------------------------------------
    @property
    def nbytes(self):
        if self.k_codes is None:
            return 0
        B, H = self.k_codes.shape[:2]
        per_row = sum(t.shape[3] * t.element_size() for t in
                      (self.k_codes, self.k_scales, self.k_biases, self.v_codes, self.v_scales, self.v_biases))
        return B * H * self.offset * per_row

    @property
    def state(self):
        if self.k_codes is None:
            return []
        t = self.offset
        return [x[:, :, :t] for x in (self.k_codes, self.k_scales, self.k_biases,
                                      self.v_codes, self.v_scales, self.v_biases)]

    @property
    def meta_state(self):
        return f"MixedQuant,{self.offset},{self.k_bits},{self.v_bits},{self.group_size}"

    def make_mask(self, N, return_array: bool = False, window_size=None):
        from .base import create_causal_mask
        if N == 1:
            return None
        if return_array or (window_size is not None and N > window_size):
            dev = self.k_codes.device if self.k_codes is not None else None
            return create_causal_mask(N, offset=self.offset, window_size=window_size, device=dev)
        return "causal"

    def empty(self):
        return self.k_codes is None

    def is_trimmable(self):
        return True

    def trim(self, n):
        n = min(self.offset, n)
        self.offset -= n
        return n

    def size(self):
        return self.offset
