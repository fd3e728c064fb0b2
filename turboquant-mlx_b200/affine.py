"""Group-wise affine quantisation helpers (K8 / V4) over libtqb200.

Format: per group of `group` consecutive elements scale = fp16((max - min) /
(2^bits - 1)) and bias = fp16(min); code = clip(rint((x - bias) / scale), 0,
2^bits - 1); 4-bit codes are packed two per byte, low nibble first.  This stands
in for `KVCache.to_quantized(group_size, bits)` as the reference uses it
(turboquant_mlx/hybrid_cache.py:57-63); the reference's arithmetic lives in the
mlx library, so the format is this library's own."""

from __future__ import annotations

import torch

from . import _lib


def affine_quantize(x: torch.Tensor, group: int = 64, bits: int = 8):
    """(..., dim) -> codes (..., dim or dim/2) uint8, scales, biases (..., dim/group) fp16."""
    _lib.require_cuda(x)
    dim = x.shape[-1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, dim).contiguous()
    n = x2.shape[0]
    width = dim if bits == 8 else dim // 2
    codes = torch.empty((n, width), dtype=torch.uint8, device=x.device)
    scales = torch.empty((n, dim // group), dtype=torch.float16, device=x.device)
    biases = torch.empty((n, dim // group), dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().tq_affine_quantize(_lib.ptr(x2), _lib.dtype_code(x2.dtype), n, dim, group,
                                             bits, _lib.ptr(codes), _lib.ptr(scales),
                                             _lib.ptr(biases), _lib.stream_ptr(x.device)))
    return (codes.reshape(*lead, width), scales.reshape(*lead, dim // group),
            biases.reshape(*lead, dim // group))


def affine_quantize_rows_into(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                              group: int, bits: int, position: torch.Tensor | None = None,
                              pos_strides: tuple[int, int] = (0, 0)) -> bool:
    """Quantize the rows of x (n, dim) straight into codes / scales / biases (n, width), views whose
    rows may be far apart (one decode step's rows inside a pre-sized cache).  Returns False, writing
    nothing, when a view does not have unit-stride rows at one uniform row distance.
    `position`: an int32 device tensor whose first element, read when the kernel runs, moves the
    destination by `pos_strides` = (bytes of codes, halfs of scales / biases) per unit: the views
    then name position 0, and a CUDA graph of the step appends where the device counter points."""
    for t in (x, codes, scales, biases):
        if t.ndim != 2 or t.stride(1) != 1:
            return False
    if scales.stride(0) != biases.stride(0) or not x.is_cuda:
        return False
    if position is not None and (position.dtype != torch.int32 or not position.is_cuda):
        raise ValueError("position must be an int32 CUDA tensor")
    n, dim = x.shape
    _lib.check(_lib.lib().tq_affine_quantize_rows_at(
        _lib.ptr(x), _lib.dtype_code(x.dtype), n, dim, group, bits, x.stride(0), _lib.ptr(codes), codes.stride(0),
        _lib.ptr(scales), _lib.ptr(biases), scales.stride(0), _lib.ptr(position), int(pos_strides[0]),
        int(pos_strides[1]), _lib.stream_ptr(x.device)))
    return True


def affine_dequantize(codes, scales, biases, group: int = 64, bits: int = 8,
                      dtype=torch.float16) -> torch.Tensor:
    _lib.require_cuda(codes, scales, biases)
    dim = codes.shape[-1] * (1 if bits == 8 else 2)
    lead = codes.shape[:-1]
    c2 = codes.reshape(-1, codes.shape[-1]).contiguous()
    # the contiguous copies must outlive the launch call: a temporary dropped right after its
    # pointer is taken hands its block to the next temporary of the same size
    s2, b2 = scales.contiguous(), biases.contiguous()
    n = c2.shape[0]
    out = torch.empty((n, dim), dtype=dtype, device=codes.device)
    _lib.check(_lib.lib().tq_affine_dequantize(_lib.ptr(c2), _lib.ptr(s2), _lib.ptr(b2), n, dim, group, bits,
                                               _lib.ptr(out), _lib.dtype_code(dtype),
                                               _lib.stream_ptr(codes.device)))
    del s2, b2
    return out.reshape(*lead, dim)
