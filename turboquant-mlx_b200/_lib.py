"""ctypes binding of libtqb200.so and the tensor <-> pointer marshalling.

The shared library is the product; this module only loads it, turns
`torch.Tensor`s (CUDA) into raw pointers, sizes and strides, and maps status
codes to exceptions.  There is no CPU implementation behind it: a missing
library or a non-CUDA tensor raises.
"""

from __future__ import annotations

import ctypes
import os
import weakref
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TQB200_LIB", os.path.join(_HERE, "libtqb200.so"))   # override: alternate builds

TQ_F32, TQ_F16, TQ_BF16 = 0, 1, 2
TQ_KV_POLAR, TQ_KV_DENSE, TQ_KV_AFFINE = 0, 1, 2
_DTYPES = {torch.float32: TQ_F32, torch.float16: TQ_F16, torch.bfloat16: TQ_BF16}

# status codes that mean "the caller passed something invalid" -> ValueError
_VALUE_ERRORS = {-1, -2, -3, -4, -5, -7, -8}


class FlashParams(ctypes.Structure):
    """Mirror of `tq_flash_params` (include/tqb200.h)."""

    _fields_ = [
        ("struct_bytes", c_int32),
        ("batch", c_int32), ("n_q_heads", c_int32), ("n_kv_heads", c_int32), ("dim", c_int32),
        ("seq_len", c_int64),
        ("q", c_void_p), ("q_dtype", c_int32), ("q_prerotated", c_int32),
        ("q_batch_stride", c_int64), ("q_head_stride", c_int64),
        ("k_format", c_int32), ("k_bits", c_int32), ("k_dtype", c_int32), ("k_group", c_int32),
        ("k_data", c_void_p), ("k_batch_stride", c_int64), ("k_head_stride", c_int64),
        ("k_norms", c_void_p), ("kn_batch_stride", c_int64), ("kn_head_stride", c_int64),
        ("k_scales", c_void_p), ("k_biases", c_void_p),
        ("ks_batch_stride", c_int64), ("ks_head_stride", c_int64),
        ("k_centroids_host", POINTER(c_float)), ("k_signs_host", POINTER(c_float)),
        ("v_format", c_int32), ("v_bits", c_int32), ("v_group", c_int32), ("kv_stable", c_int32),
        ("v_data", c_void_p), ("v_batch_stride", c_int64), ("v_head_stride", c_int64),
        ("v_norms", c_void_p), ("vn_batch_stride", c_int64), ("vn_head_stride", c_int64),
        ("v_scales", c_void_p), ("v_biases", c_void_p),
        ("vs_batch_stride", c_int64), ("vs_head_stride", c_int64),
        ("v_centroids_host", POINTER(c_float)), ("v_signs_host", POINTER(c_float)),
        ("attn_scale", c_float), ("num_splits", c_int32),
        ("mask", c_void_p), ("mask_batch_stride", c_int64), ("mask_head_stride", c_int64),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("out_mode", c_int32), ("out_dtype", c_int32),
        ("out", c_void_p), ("out_batch_stride", c_int64), ("out_head_stride", c_int64),
        ("part_m", c_void_p), ("part_l", c_void_p), ("part_acc", c_void_p),
        ("stream", c_void_p),
        ("n_peers", c_int32), ("peer_slots_exclusive", c_int32),
        ("peer_m", c_void_p * 8), ("peer_l", c_void_p * 8), ("peer_acc", c_void_p * 8),
        ("peer_counter", c_void_p * 8),
        ("q_stable", c_int32), ("new_dtype", c_int32),
        ("new_k", c_void_p), ("new_v", c_void_p),
        ("new_k_batch_stride", c_int64), ("new_k_head_stride", c_int64),
        ("new_v_batch_stride", c_int64), ("new_v_head_stride", c_int64),
        ("k_boundaries_host", POINTER(c_float)), ("v_boundaries_host", POINTER(c_float)),
        ("sparse_v_threshold", c_float), ("sparse_reserved", c_int32), ("active_positions", c_void_p),
        ("seq_lens_dev", c_void_p),
        ("workspace_exclusive", c_int32), ("gather_ranks", c_int32),
        ("gather_m", c_void_p), ("gather_l", c_void_p), ("gather_acc", c_void_p),
        ("gather_part_stride", c_int64), ("gather_flags", c_void_p),
        ("q_tokens", c_int32), ("q_tokens_reserved", c_int32), ("q_token_stride", c_int64), ("out_token_stride", c_int64),
    ]


_lib = None

_FP = POINTER(c_float)
_SIGNATURES = {
    "tq_version": (c_int, []),
    "tq_last_error_string": (c_char_p, []),
    "tq_quantize": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, _FP, _FP,
                            c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "tq_quantize_append": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, _FP, _FP,
                                   c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                   c_int64, c_int64, c_void_p]),
    "tq_dequantize": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                              _FP, _FP, c_void_p, c_int, c_int64, c_void_p]),
    "tq_prerotate_query": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, _FP, c_void_p, c_void_p]),
    "tq_hadamard": (c_int, [c_void_p, c_int64, c_int, _FP, _FP, c_int, c_void_p, c_void_p]),
    "tq_prerot_qk_scores": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64,
                                    _FP, c_int, c_int, c_int, c_void_p, c_void_p]),
    "tq_packed_qk_scores": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64,
                                    _FP, _FP, c_int, c_int, c_void_p, c_void_p]),
    "tq_sparse_v_workspace_bytes": (c_size_t, [c_int, c_int64, c_int]),
    "tq_sparse_v_matvec": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                   c_int64, _FP, _FP, c_int, c_int, c_float, c_int, c_void_p,
                                   c_void_p, c_size_t, c_void_p]),
    "tq_sparse_v_noalloc_max_bytes": (c_size_t, []),
    "tq_sparse_v_matvec_noalloc": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                           c_int64, _FP, _FP, c_int, c_int, c_float, c_int, c_void_p,
                                           c_void_p]),
    "tq_flash_decode_header_bytes": (c_int64, [c_int, c_int]),
    "tq_flash_decode_workspace_bytes": (c_int64, [POINTER(FlashParams)]),
    "tq_flash_decode": (c_int, [POINTER(FlashParams)]),
    "tq_flash_decode_last_kernel": (c_int, []),
    "tq_flash_decode_resident_ctas_per_sm": (c_int, []),
    "tq_merge_partials": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int,
                                  c_int64, c_int, _FP, c_void_p, c_int, c_int64, c_void_p]),
    "tq_affine_quantize": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p]),
    "tq_affine_quantize_rows": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int64, c_void_p, c_int64,
                                        c_void_p, c_void_p, c_int64, c_void_p]),
    "tq_affine_quantize_rows_at": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int64, c_void_p, c_int64,
                                           c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "tq_affine_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                     c_void_p, c_int, c_void_p]),
    "tq_merge_partials_after_peers": (c_int, [c_void_p, c_int, c_uint32, c_void_p, c_int, c_void_p, c_int64, c_void_p,
                                              c_int64, c_void_p, c_int64, c_int, c_int64, c_int, _FP, c_void_p,
                                              c_int, c_int64, c_void_p]),
    "tq_set_peer_wait_limit_ms": (c_int, [c_int]),
    "tq_peer_push": (c_int, [c_void_p, c_int64, POINTER(c_void_p), POINTER(c_void_p), c_int, c_uint32, c_void_p]),
    "tq_peer_wait": (c_int, [c_void_p, c_int, c_uint32, c_void_p, c_void_p]),
    "tq_prefill_sdpa": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int64, c_int64, c_int] + [c_int64] * 12 + [c_float, c_int, c_void_p, c_void_p]),
}


def lib() -> ctypes.CDLL:
    """Load libtqb200.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {_HERE}` "
                "(nvcc, sm_100a).  There is no fallback implementation.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def check(status: int) -> None:
    if status == 0:
        return
    msg = lib().tq_last_error_string().decode("utf-8", "replace")
    if status in _VALUE_ERRORS:
        raise ValueError(msg)
    raise RuntimeError(f"libtqb200 error {status}: {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; use float32, float16 or bfloat16") from None


def ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise RuntimeError("libtqb200 operates on CUDA tensors only (no CPU path)")
    return c_void_p(t.data_ptr())


def stream_ptr(device=None) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


# ---------------------------------------------------------------------------
# codebook-sized parameters: the C ABI takes them as host float arrays
# ---------------------------------------------------------------------------
_host_cache: dict = {}     # id(tensor) -> (weak reference, tensor version, ctypes array)


def _remember(t: torch.Tensor, arr) -> None:
    key = id(t)

    def _evict(_ref, key=key):
        _host_cache.pop(key, None)

    _host_cache[key] = (weakref.ref(t, _evict), t._version, arr)


def register_host_values(t: torch.Tensor, values) -> None:
    """Remember the host copy of a small device tensor (signs, centroids,
    boundaries) so that passing the tensor later costs no device read."""
    _remember(t, (c_float * len(values))(*[float(v) for v in values]))


def host_floats(x):
    """ctypes float array for a codebook-sized parameter given as a tensor,
    numpy array or sequence.  A device tensor seen for the first time is read
    back once (this synchronises) and the copy is kept for as long as that tensor
    object lives and is not modified in place: the entry is keyed on the object
    itself (not its address, which the allocator hands to the next tensor of the
    same size) and dropped when the tensor is freed."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        hit = _host_cache.get(id(x))
        if hit is not None and hit[0]() is x and hit[1] == x._version:
            return hit[2]
        vals = x.detach().to(torch.float32).reshape(-1).cpu().tolist()
        arr = (c_float * len(vals))(*vals)
        _remember(x, arr)
        return arr
    vals = [float(v) for v in x]
    return (c_float * len(vals))(*vals)


# ---------------------------------------------------------------------------
# scratch memory: allocated by torch (the library never allocates), cached per
# (device, stream) so stream-ordered reuse is safe
# ---------------------------------------------------------------------------
_workspaces: dict = {}


def workspace(nbytes: int, device, tag: str = "flash") -> torch.Tensor | None:
    """Zero-filled scratch tensor for one kind of call (`tag`): the flash-decode
    workspace starts with counters that must stay zero between calls, so other
    kernels never share it."""
    if nbytes <= 0:
        return None
    key = (tag, str(device), torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libtqb200 operates on CUDA tensors only (no CPU path)")
