"""PolarQuantizer (reference turboquant_mlx/quantizer.py): per-vector norm,
randomized Hadamard rotation, Lloyd-Max scalar quantisation.  quantize() and
dequantize() run the library's fused kernels and convert to / from the
reference's unpacked uint8 index layout."""

from __future__ import annotations

import math
import struct

import torch

from . import _lib
from .packing import pack_indices, packed_dim, unpack_indices
from .rotation import random_diagonal_sign

_CODEBOOKS = {  # Lloyd-Max centroids for N(0,1), quantizer.py:27-36
    1: [-0.7979, 0.7979],
    2: [-1.5104, -0.4528, 0.4528, 1.5104],
    3: [-2.1520, -1.3440, -0.7560, -0.2451, 0.2451, 0.7560, 1.3440, 2.1520],
    4: [-2.7326, -2.0690, -1.6180, -1.2562, -0.9423, -0.6568, -0.3881, -0.1284,
        0.1284, 0.3881, 0.6568, 0.9423, 1.2562, 1.6180, 2.0690, 2.7326],
}


def _f32(v: float) -> float:
    return struct.unpack("f", struct.pack("f", v))[0]


def codebook_values(bits: int) -> list:
    if bits not in _CODEBOOKS:
        raise ValueError(f"Unsupported bit width: {bits}. Use 1-4.")
    return [_f32(c) for c in _CODEBOOKS[bits]]


def boundary_values(centroids: list) -> list:
    """float32 midpoints (quantizer.py:42-44)."""
    return [_f32((_f32(a) + _f32(b)) / 2.0) for a, b in zip(centroids[:-1], centroids[1:])]


def _device_param(vals, device) -> torch.Tensor:
    t = torch.tensor(vals, dtype=torch.float32, device=device)
    _lib.register_host_values(t, vals)
    return t


def _compute_gaussian_codebook(bits: int, device=None) -> torch.Tensor:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    return _device_param(codebook_values(bits), device)


def _compute_gaussian_boundaries(centroids: torch.Tensor) -> torch.Tensor:
    vals = boundary_values(list(_lib.host_floats(centroids)))
    return _device_param(vals, centroids.device)


class PolarQuantizer:
    """PolarQuant quantizer for a fixed dimension and bit width."""

    def __init__(self, dim: int, bits: int = 3, seed: int = 42, device=None):
        self.dim = dim
        self.bits = bits
        self.n_levels = 2 ** bits
        self.signs = random_diagonal_sign(dim, seed=seed, device=device)
        self.centroids = _compute_gaussian_codebook(bits, device=self.signs.device)
        self.boundaries = _compute_gaussian_boundaries(self.centroids)
        self.scale = 1.0 / math.sqrt(dim)

    def quantize_packed(self, x: torch.Tensor):
        """(..., dim) -> packed (..., packed_dim) uint32, norms (...,) float32."""
        from .kernels import fused_quantize
        lead = x.shape[:-1]
        packed, norms = fused_quantize(x.reshape(-1, self.dim), self.signs, self.boundaries,
                                       self.dim, self.bits)
        return packed.reshape(*lead, -1), norms.reshape(lead)

    def quantize(self, x: torch.Tensor):
        """(..., dim) -> indices (..., dim) uint8, norms (...,) (quantizer.py:75-106)."""
        packed, norms = self.quantize_packed(x)
        return unpack_indices(packed, self.bits, self.dim), norms

    def dequantize(self, indices: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        """indices + norms -> (..., dim) float32 (quantizer.py:108-132)."""
        from .kernels import packed_dequantize
        lead = indices.shape[:-1]
        packed = pack_indices(indices, self.bits).reshape(-1, packed_dim(self.dim, self.bits))
        out = packed_dequantize(packed, norms.reshape(-1).to(torch.float32), self.centroids,
                                self.signs, self.dim, self.bits)
        return out.reshape(*lead, self.dim)
