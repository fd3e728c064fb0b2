"""Bit-packing of codebook indices into uint32 words (reference
turboquant_mlx/packing.py:16-87): 1-bit 32/word, 2-bit 16/word, 3-bit 10/word
(30 of 32 bits used), 4-bit 8/word; element j sits in word j // vpw at bit
(j % vpw) * bits.  These two helpers are layout utilities on torch tensors;
the hot path packs inside the quantize kernel and never calls them."""

from __future__ import annotations

import torch

VALS_PER_WORD = {1: 32, 2: 16, 3: 10, 4: 8}
BIT_MASK = {1: 0x1, 2: 0x3, 3: 0x7, 4: 0xF}


def packed_dim(dim: int, bits: int) -> int:
    """Number of uint32 words needed to pack `dim` values at `bits` each."""
    vpw = VALS_PER_WORD[bits]
    return (dim + vpw - 1) // vpw


def pack_indices(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """(..., dim) uint8 -> (..., packed_dim) uint32 (packing.py:26-56)."""
    vpw = VALS_PER_WORD[bits]
    shape = indices.shape
    dim = shape[-1]
    pd = packed_dim(dim, bits)
    flat = indices.reshape(-1, dim).to(torch.int64)
    if dim % vpw:
        pad = torch.zeros((flat.shape[0], vpw - dim % vpw), dtype=torch.int64, device=flat.device)
        flat = torch.cat([flat, pad], dim=1)
    flat = flat.reshape(-1, pd, vpw)
    shifts = torch.arange(vpw, device=flat.device, dtype=torch.int64) * bits
    words = (flat << shifts).sum(dim=-1)            # fields do not overlap: sum == OR
    return words.to(torch.uint32).reshape(*shape[:-1], pd)


def unpack_indices(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """(..., packed_dim) uint32 -> (..., dim) uint8 (packing.py:59-87)."""
    vpw = VALS_PER_WORD[bits]
    shape = packed.shape
    flat = packed.reshape(-1, shape[-1]).to(torch.int64)
    shifts = torch.arange(vpw, device=flat.device, dtype=torch.int64) * bits
    vals = (flat.unsqueeze(-1) >> shifts) & BIT_MASK[bits]
    vals = vals.reshape(flat.shape[0], shape[-1] * vpw)[:, :dim]
    return vals.to(torch.uint8).reshape(*shape[:-1], dim)
