"""Walsh-Hadamard rotation helpers (reference turboquant_mlx/rotation.py),
running on the library's butterfly kernel."""

from __future__ import annotations

import torch

from . import _lib


def _splitmix64(state: int):
    state = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return state, z ^ (z >> 31)


def sign_values(d: int, seed: int = 42) -> list:
    """Host list of +/-1.  The reference draws these from the mlx PRNG
    (rotation.py:37-49), which cannot be regenerated elsewhere; this library's
    generator is splitmix64 seeded with `seed`, element i = +1 when the top bit
    of the i-th output is set."""
    state = seed & 0xFFFFFFFFFFFFFFFF
    out = []
    for _ in range(d):
        state, z = _splitmix64(state)
        out.append(1.0 if (z >> 63) else -1.0)
    return out


def random_diagonal_sign(d: int, seed: int = 42, device=None) -> torch.Tensor:
    """(d,) float32 tensor of +/-1 on the current CUDA device."""
    vals = sign_values(d, seed)
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    t = torch.tensor(vals, dtype=torch.float32, device=device)
    _lib.register_host_values(t, vals)
    return t


def _hadamard(x: torch.Tensor, pre, post, normalize: bool) -> torch.Tensor:
    d = x.shape[-1]
    assert d > 0 and (d & (d - 1)) == 0, f"Dimension must be power of 2, got {d}"
    _lib.require_cuda(x)
    dtype = x.dtype
    x32 = x.to(torch.float32).contiguous()
    out = torch.empty_like(x32)
    n_rows = x32.numel() // d
    _lib.check(_lib.lib().tq_hadamard(_lib.ptr(x32), n_rows, d, _lib.host_floats(pre),
                                      _lib.host_floats(post), int(normalize), _lib.ptr(out),
                                      _lib.stream_ptr(x.device)))
    return out.to(dtype)


def walsh_hadamard_transform(x: torch.Tensor) -> torch.Tensor:
    """Normalised WHT on the last dimension (rotation.py:7-34)."""
    return _hadamard(x, None, None, True)


def randomized_hadamard_transform(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """WHT(x * signs) (rotation.py:52-64)."""
    return _hadamard(x, signs, None, True)


def inverse_randomized_hadamard(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """WHT(x) * signs (rotation.py:67-80)."""
    return _hadamard(x, None, signs, True)
