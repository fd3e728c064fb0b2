"""TurboQuantKVCache: PolarQuant KV cache with packed uint32 storage (reference
turboquant_mlx/cache.py:42-369), on CUDA tensors.

Storage: k_packed / v_packed (B, H, n_alloc, packed_dim) uint32 and k_norms /
v_norms (B, H, n_alloc) float32, n_alloc a multiple of `step` = 256; valid rows
are [:offset].  Inserts are quantized by the fused kernel directly into the
storage rows (no temporary, no slice-assign), and the optional dequantized
fp16/bf16 buffers are filled in place for the new rows only.

Differences from the reference, all additive:
  * `k_bits` / `v_bits` allow different widths for K and V (`bits` sets both);
  * storage grows geometrically and `reserve(n)` pre-sizes it;
  * `state` can carry the sign vectors (see `state_with_signs`), because the
    reference regenerates them from the seed with a PRNG that other libraries
    cannot reproduce.
"""

from __future__ import annotations

import torch

from .kernels import dequantize_into, quantize_into
from .packing import packed_dim
from .quantizer import _compute_gaussian_boundaries, _compute_gaussian_codebook
from .rotation import random_diagonal_sign


class _Quantizer:
    def __init__(self, dim, bits, seed, device=None):
        self.dim = dim
        self.bits = bits
        self.signs = random_diagonal_sign(dim, seed=seed, device=device)
        self.centroids = _compute_gaussian_codebook(bits, device=self.signs.device)
        self.boundaries = _compute_gaussian_boundaries(self.centroids)


_DTYPE_MAP = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
_DTYPE_NAME = {v: k for k, v in _DTYPE_MAP.items()}


_ZEROS: dict = {}


def _zero(dtype, device) -> torch.Tensor:
    """One zero element per (dtype, device), made once: placeholders are stride-0 views of it, so
    handing them out launches nothing."""
    key = (dtype, str(device))
    z = _ZEROS.get(key)
    if z is None:
        z = torch.zeros((1,), dtype=dtype, device=device)
        _ZEROS[key] = z
    return z


class TurboQuantKVCache:
    """TurboQuant KV cache, drop-in for a plain KVCache."""

    step = 256

    def __init__(self, bits: int = 3, seed: int = 42, fused: bool = False,
                 sparse_v_threshold: float | None = None, v_only: bool = False,
                 k_bits: int | None = None, v_bits: int | None = None,
                 defer_append: bool = False, inputs_stable: bool = False):
        """`defer_append` / `inputs_stable` (fused caches, additions to the reference's
        arguments): see `VOnlyTurboQuantCache` - a one-token insert is recorded and carried out
        by the decode attention's own launch; consecutive decode launches may overlap."""
        self.defer_append = defer_append and fused and not v_only
        self.inputs_stable = inputs_stable
        self._pending = None
        self._decode_ws = None
        self.quant_bits = bits
        self.k_bits = bits if k_bits is None else k_bits
        self.v_bits = bits if v_bits is None else v_bits
        self.seed = seed
        self.offset = 0
        self.fused = fused
        self.sparse_v_threshold = sparse_v_threshold
        self.v_only = v_only

        self.k_packed = None
        self.k_norms = None
        self.v_packed = None
        self.v_norms = None

        self._k_deq_buf = None
        self._v_deq_buf = None
        self._deq_offset = 0
        self._deq_alloc = 0

        self._k_q = None
        self._v_q = None
        self._k_dim = None
        self._v_dim = None
        self._k_pdim = None
        self._v_pdim = None
        self._dtype = None

    # ---- set-up -----------------------------------------------------------
    def _ensure_quantizer(self, k_dim, v_dim, device=None):
        if not self.v_only and self._k_q is None:
            self._k_q = _Quantizer(k_dim, self.k_bits, self.seed, device)
            self._k_dim = k_dim
            self._k_pdim = packed_dim(k_dim, self.k_bits)
        if self._v_q is None:
            self._v_q = _Quantizer(v_dim, self.v_bits, self.seed + 1, device)
            self._v_dim = v_dim
            self._v_pdim = packed_dim(v_dim, self.v_bits)
        self._adopt_loaded_signs()

    @staticmethod
    def _grow(old_p, old_n, B, H, n, pdim, prev, device):
        new_p = torch.zeros((B, H, n, pdim), dtype=torch.uint32, device=device)
        new_n = torch.zeros((B, H, n), dtype=torch.float32, device=device)
        if old_p is not None and prev > 0:
            new_p[..., :prev, :] = old_p[..., :prev, :]
            new_n[..., :prev] = old_n[..., :prev]
        return new_p, new_n

    def _ensure_storage(self, B, H, num_new, device=None):
        prev = self.offset
        needed = prev + num_new
        cur = 0 if self.v_packed is None else self.v_packed.shape[2]
        if needed > cur:
            n = ((needed + self.step - 1) // self.step) * self.step
            if cur:
                n = max(n, 2 * cur)      # amortised growth; reserve() avoids it entirely
            if not self.v_only:
                self.k_packed, self.k_norms = self._grow(self.k_packed, self.k_norms, B, H, n,
                                                         self._k_pdim, prev, device)
            self.v_packed, self.v_norms = self._grow(self.v_packed, self.v_norms, B, H, n,
                                                     self._v_pdim, prev, device)

    def reserve(self, B, H, n_positions, k_dim, v_dim, device=None):
        """Pre-size storage for `n_positions` so later inserts never reallocate."""
        self._ensure_quantizer(k_dim, v_dim, device)
        self._ensure_storage(B, H, max(0, n_positions - self.offset), self._v_q.signs.device)

    # ---- quantize on insert -------------------------------------------------
    def _insert(self, x, q, packed, norms, prev):
        B, H, S, D = x.shape
        x3 = x.reshape(B * H, S, D)
        if not x3.is_contiguous():
            x3 = x3.contiguous()
        quantize_into(x3, q.signs, q.boundaries, D, q.bits,
                      packed.view(B * H, packed.shape[2], packed.shape[3]),
                      norms.view(B * H, norms.shape[2]), row_offset=prev)

    def _dequant_rows(self, packed, norms, q, buf, start, count):
        B, H = packed.shape[0], packed.shape[1]
        dequantize_into(packed.view(B * H, packed.shape[2], packed.shape[3]),
                        norms.view(B * H, norms.shape[2]), q.centroids, q.signs, q.dim, q.bits,
                        buf.view(B * H, buf.shape[2], buf.shape[3]), count,
                        src_row=start, dst_row=start)

    def _full_dequant(self, packed, norms, q, dim, B, H, total, dtype):
        alloc = ((total + self.step - 1) // self.step) * self.step
        buf = torch.zeros((B, H, alloc, dim), dtype=dtype, device=packed.device)
        self._dequant_rows(packed, norms, q, buf, 0, total)
        return buf, alloc

    def dequantized(self, dtype=None):
        """(K, V) (B, H, offset, D) dequantized from storage (K is None in v_only mode)."""
        self.flush_pending()
        dtype = dtype or self._dtype or torch.float16
        B, H = self.v_packed.shape[0], self.v_packed.shape[1]
        total = self.offset
        k = None
        if not self.v_only:
            k, _ = self._full_dequant(self.k_packed, self.k_norms, self._k_q, self._k_dim, B, H, total, dtype)
            k = k[..., :total, :]
        v, _ = self._full_dequant(self.v_packed, self.v_norms, self._v_q, self._v_dim, B, H, total, dtype)
        return k, v[..., :total, :]

    def flush_pending(self):
        """Materialise a deferred one-token insert with the ordinary quantize kernels."""
        if getattr(self, "_pending", None) is None:
            return
        k_row, v_row = self._pending
        self._pending = None
        self.offset -= 1
        defer, self.defer_append = self.defer_append, False
        try:
            self.update_and_fetch(k_row.unsqueeze(2), v_row.unsqueeze(2))
        finally:
            self.defer_append = defer

    def take_pending(self):
        rows, self._pending = getattr(self, "_pending", None), None
        return rows

    def update_and_fetch(self, keys, values):
        self.flush_pending()
        B, H, S, k_dim = keys.shape
        v_dim = values.shape[3]
        self._dtype = keys.dtype
        if (getattr(self, "defer_append", False) and S == 1 and keys.is_cuda and self.k_packed is not None
                and self.offset + 1 <= self.v_packed.shape[2] and k_dim == 128 and v_dim == 128
                and self.k_packed.shape[:2] == (B, H) and keys.dtype == values.dtype
                and self.k_bits in (3, 4) and self.v_bits in (3, 4)):
            self._pending = (keys[:, :, 0, :], values[:, :, 0, :])
            self.offset += 1
            return (_zero(keys.dtype, keys.device).expand(B, H, self.offset, k_dim),
                    _zero(values.dtype, values.device).expand(B, H, self.offset, v_dim))
        self._ensure_quantizer(k_dim, v_dim, values.device)
        self._ensure_storage(B, H, S, values.device)
        prev = self.offset

        self._insert(values, self._v_q, self.v_packed, self.v_norms, prev)
        if not self.v_only:
            self._insert(keys, self._k_q, self.k_packed, self.k_norms, prev)
        self.offset += S
        total = self.offset

        if self.fused:
            # attention reads the packed storage directly; hand back shape-only
            # placeholders (stride-0 views, no memory)
            zk = _zero(keys.dtype, keys.device).expand(B, H, total, k_dim)
            zv = _zero(values.dtype, values.device).expand(B, H, total, v_dim)
            return zk, zv

        incremental = S <= 4 and self._v_deq_buf is not None and self._deq_offset == prev
        if incremental and total > self._deq_alloc:
            na = max(((total + self.step - 1) // self.step) * self.step, 2 * self._deq_alloc)
            grow = lambda buf, d, dt: torch.cat(  # noqa: E731
                [buf[..., :prev, :], torch.zeros((B, H, na - prev, d), dtype=dt, device=buf.device)], dim=2)
            if self._k_deq_buf is not None:
                self._k_deq_buf = grow(self._k_deq_buf, k_dim, keys.dtype)
            self._v_deq_buf = grow(self._v_deq_buf, v_dim, values.dtype)
            self._deq_alloc = na

        if incremental:
            self._dequant_rows(self.v_packed, self.v_norms, self._v_q, self._v_deq_buf, prev, S)
            if not self.v_only:
                self._dequant_rows(self.k_packed, self.k_norms, self._k_q, self._k_deq_buf, prev, S)
        else:
            self._v_deq_buf, alloc = self._full_dequant(self.v_packed, self.v_norms, self._v_q,
                                                        v_dim, B, H, total, values.dtype)
            if not self.v_only:
                self._k_deq_buf, _ = self._full_dequant(self.k_packed, self.k_norms, self._k_q,
                                                        k_dim, B, H, total, keys.dtype)
            self._deq_alloc = alloc
        self._deq_offset = total
        v_out = self._v_deq_buf[..., :total, :]
        if self.v_only:
            # K is handled by the caller; the K return is a placeholder
            zk = _zero(keys.dtype, keys.device).expand(B, H, total, k_dim)
            return zk, v_out
        return self._k_deq_buf[..., :total, :], v_out

    # ---- bookkeeping ----------------------------------------------------------
    def empty(self):
        return self.v_packed is None if self.v_only else self.k_packed is None

    @property
    def nbytes(self):
        total = 0
        for p, n in ((self.k_packed, self.k_norms), (self.v_packed, self.v_norms)):
            if p is not None:
                B, H = p.shape[0], p.shape[1]
                total += B * H * self.offset * (p.shape[3] * 4 + 4)
        return total

    @property
    def compression_ratio(self) -> float:
        """FP16 bytes of the uncompressed K+V divided by packed + norm bytes."""
        total = self.nbytes
        if total == 0:
            return 1.0
        ref = self.v_packed if self.v_only else self.k_packed
        if ref is None:
            return 1.0
        B, H = ref.shape[0], ref.shape[1]
        fp16_bytes = B * H * self.offset * ((self._k_dim or 0) + (self._v_dim or 0)) * 2
        return fp16_bytes / total

    @property
    def state(self):
        self.flush_pending()
        if self.v_packed is None and self.k_packed is None:
            return []
        parts = []
        if self.k_packed is not None:
            parts += [self.k_packed[..., :self.offset, :], self.k_norms[..., :self.offset]]
        if self.v_packed is not None:
            parts += [self.v_packed[..., :self.offset, :], self.v_norms[..., :self.offset]]
        return parts

    @state.setter
    def state(self, v):
        """2 (v_only) or 4 arrays as the reference stores them (cache.py:262-274), or the
        `state_with_signs` form: the same followed by the sign vectors (one for v_only, K then V
        otherwise).  Saved sign vectors replace the ones this process would derive from the seed,
        so a cache written by a library with a different generator decodes correctly."""
        if not v:
            return
        v = [t.contiguous() for t in v]
        if len(v) in (3, 6):
            n_signs = 1 if len(v) == 3 else 2
            signs = [self._check_signs(t) for t in v[-n_signs:]]
            self._loaded_signs = (None, signs[0]) if n_signs == 1 else (signs[0], signs[1])
            v = v[:-n_signs]
            self._adopt_loaded_signs()
        if len(v) == 4:
            self.k_packed, self.k_norms, self.v_packed, self.v_norms = v
            self.offset = self.k_packed.shape[2]
        elif len(v) == 2:
            self.v_packed, self.v_norms = v
            self.offset = self.v_packed.shape[2]
        else:
            raise ValueError(f"Expected 2 (v_only) or 4 arrays in state (plus 1 or 2 sign vectors), got {len(v)}")

    @staticmethod
    def _check_signs(t):
        t = t.to(torch.float32).reshape(-1)
        if t.numel() == 0 or t.numel() & (t.numel() - 1) or not bool(((t == 1.0) | (t == -1.0)).all()):
            raise ValueError("a saved sign vector must hold +1 / -1 values and have a power-of-two length")
        return t

    def _adopt_loaded_signs(self):
        """Put sign vectors that came with a saved state into the quantizers (once they exist)."""
        loaded = getattr(self, "_loaded_signs", None)
        if loaded is None:
            return
        for q, sg in ((self._k_q, loaded[0]), (self._v_q, loaded[1])):
            if q is not None and sg is not None:
                if sg.numel() != q.dim:
                    raise ValueError(f"saved sign vector has {sg.numel()} entries, the cache dimension is {q.dim}")
                q.signs = sg.to(q.signs.device)

    def signs_match_seed(self) -> bool:
        """True when the sign vectors in use are the ones this library derives from `seed`
        (False after loading a state saved by a library with another generator)."""
        from .rotation import sign_values
        for q, sd in ((self._k_q, self.seed), (self._v_q, self.seed + 1)):
            if q is not None and q.signs.cpu().tolist() != sign_values(q.dim, sd):
                return False
        return True

    @property
    def state_with_signs(self):
        """`state` followed by the K and V sign vectors, so a saved cache can be
        reloaded by a process whose sign generator differs."""
        extra = [q.signs for q in (self._k_q, self._v_q) if q is not None]
        return self.state + extra

    @property
    def meta_state(self):
        dtype_str = _DTYPE_NAME.get(self._dtype, "float16")
        base = f"{self.offset},{self.quant_bits},{self.seed},{self._k_dim or 0},{self._v_dim or 0},{dtype_str}"
        if self.k_bits != self.quant_bits or self.v_bits != self.quant_bits:
            base += f",{self.k_bits},{self.v_bits}"
        return base

    @meta_state.setter
    def meta_state(self, v):
        parts = v.split(",")
        self.offset, self.quant_bits, self.seed = int(parts[0]), int(parts[1]), int(parts[2])
        self._k_dim = int(parts[3]) or None
        self._v_dim = int(parts[4]) or None
        self._dtype = _DTYPE_MAP.get(parts[5], torch.float16) if len(parts) > 5 else torch.float16
        self.k_bits = int(parts[6]) if len(parts) > 7 else self.quant_bits
        self.v_bits = int(parts[7]) if len(parts) > 7 else self.quant_bits

    def is_trimmable(self):
        return True

    def trim(self, n):
        self.flush_pending()
        n = min(self.offset, n)
        self.offset -= n
        self._k_deq_buf = None
        self._v_deq_buf = None
        self._deq_offset = 0
        self._deq_alloc = 0
        return n

    def size(self):
        return self.offset

    def make_mask(self, N, return_array: bool = False, window_size=None):
        """None for single-token decode, "causal" for multi-token, or an explicit
        offset-aware causal array when asked for one (cache.py:311-334)."""
        from .base import create_causal_mask

        if N == 1:
            return None
        if return_array or (window_size is not None and N > window_size):
            dev = self.v_packed.device if self.v_packed is not None else None
            return create_causal_mask(N, offset=self.offset, window_size=window_size, device=dev)
        return "causal"

    @classmethod
    def from_state(cls, state, meta_state):
        obj = cls.__new__(cls)
        cls.__init__(obj)
        obj.meta_state = meta_state
        obj.state = state
        if obj.k_packed is None and obj.v_packed is not None:
            obj.v_only = True      # a values-only state (the reference leaves v_only False here and then
                                   # reports such a cache as empty, cache.py:354-356 with :220-221)
        if obj.k_packed is not None:
            obj._k_pdim = obj.k_packed.shape[-1]
        if obj.v_packed is not None:
            obj._v_pdim = obj.v_packed.shape[-1]
        if obj._v_dim is not None and (obj._k_dim is not None or obj.v_only):
            dev = obj.v_packed.device if obj.v_packed is not None else None
            obj._ensure_quantizer(obj._k_dim or obj._v_dim, obj._v_dim, dev)
        return obj
