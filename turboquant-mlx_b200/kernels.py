"""Kernel-level API with the reference's names and argument meaning, on CUDA
`torch.Tensor`s.  Each function marshals pointers, sizes and strides into the
C ABI of libtqb200.so and raises the reference's `ValueError`s.

Reference entry points mirrored here (paths inside the reference project):
  fused_quantize, dequant_fp16           turboquant_mlx/metal.py:147-232
  packed_dequantize, packed_fused_qk_scores   turboquant_mlx/kernels.py:123-196
  prerotate_query, prerot_fused_qk_scores     turboquant_mlx/metal_kernels_v4.py:119-221
  sparse_v_matvec, count_active_positions     turboquant_mlx/sparse_v.py:94-191
  flash_attention_turboquant                  turboquant_mlx/flash_attention.py:168-274
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .packing import VALS_PER_WORD, packed_dim

__all__ = [
    "fused_quantize", "dequant_fp16", "packed_dequantize", "packed_fused_qk_scores",
    "prerotate_query", "prerot_fused_qk_scores", "prerot_packed_dequantize",
    "sparse_v_matvec", "count_active_positions", "flash_attention_turboquant",
    "flash_decode", "merge_partials", "FlashDecodePlan", "MergePlan",
    "prefill_attention", "prefill_supported", "prefill_status", "flash_status", "decode_workspace",
    "workspace_status",
]


def _check_bits(bits: int) -> None:
    if bits not in VALS_PER_WORD:
        raise ValueError(f"Unsupported bit width: {bits}. Use 1-4.")


# ---------------------------------------------------------------------------
# quantize / dequantize
# ---------------------------------------------------------------------------
def quantize_into(x: torch.Tensor, signs, boundaries, dim: int, bits: int,
                  packed_out: torch.Tensor, norms_out: torch.Tensor, row_offset: int = 0) -> None:
    """Quantize x (n_outer, n_inner, dim) straight into rows
    [row_offset, row_offset + n_inner) of packed_out (n_outer, n_alloc, pdim) /
    norms_out (n_outer, n_alloc): the append a cache insert needs, with no
    temporary and no copy."""
    _check_bits(bits)
    _lib.require_cuda(x, packed_out, norms_out)
    n_outer, n_inner, d = x.shape
    assert d == dim and x.is_contiguous()
    assert packed_out.stride(-1) == 1 and packed_out.stride(-2) == packed_out.shape[-1]
    pd = packed_out.shape[-1]
    p_ptr = ctypes.c_void_p(packed_out.data_ptr() + row_offset * pd * 4)
    n_ptr = ctypes.c_void_p(norms_out.data_ptr() + row_offset * 4)
    _lib.check(_lib.lib().tq_quantize(
        _lib.ptr(x), _lib.dtype_code(x.dtype), n_outer, n_inner, n_inner * dim, dim, bits,
        _lib.host_floats(signs), _lib.host_floats(boundaries),
        p_ptr, packed_out.stride(0), n_ptr, norms_out.stride(0), _lib.stream_ptr(x.device)))


def quantize_append(x: torch.Tensor, signs, boundaries, dim: int, bits: int, packed_out: torch.Tensor,
                    norms_out: torch.Tensor, row_offset: int, copy_src: torch.Tensor, copy_dst: torch.Tensor) -> None:
    """`quantize_into` plus, in the same launch, the row copy copy_src (rows, n) -> copy_dst (rows, n)
    (views with unit-stride rows at uniform row distances whose byte sizes are multiples of 16):
    one step's cache append for dense keys + packed values."""
    _check_bits(bits)
    _lib.require_cuda(x, packed_out, norms_out, copy_src, copy_dst)
    n_outer, n_inner, d = x.shape
    assert d == dim and x.is_contiguous()
    assert packed_out.stride(-1) == 1 and packed_out.stride(-2) == packed_out.shape[-1]
    assert copy_src.shape == copy_dst.shape and copy_src.dtype == copy_dst.dtype and copy_src.ndim == 2
    assert copy_src.stride(1) == 1 and copy_dst.stride(1) == 1
    es = copy_src.element_size()
    pd = packed_out.shape[-1]
    p_ptr = ctypes.c_void_p(packed_out.data_ptr() + row_offset * pd * 4)
    n_ptr = ctypes.c_void_p(norms_out.data_ptr() + row_offset * 4)
    _lib.check(_lib.lib().tq_quantize_append(
        _lib.ptr(x), _lib.dtype_code(x.dtype), n_outer, n_inner, n_inner * dim, dim, bits,
        _lib.host_floats(signs), _lib.host_floats(boundaries),
        p_ptr, packed_out.stride(0), n_ptr, norms_out.stride(0),
        _lib.ptr(copy_src), _lib.ptr(copy_dst), copy_src.shape[0], copy_src.shape[1] * es,
        copy_src.stride(0) * es, copy_dst.stride(0) * es, _lib.stream_ptr(x.device)))


def fused_quantize(vectors: torch.Tensor, signs, boundaries, dim: int, bits: int):
    """Raw vectors (n_vecs, dim) fp16/bf16/fp32 -> (packed (n_vecs, packed_dim)
    uint32, norms (n_vecs,) float32) in one kernel."""
    _check_bits(bits)
    _lib.require_cuda(vectors)
    n_vecs = vectors.shape[0]
    x = vectors.reshape(n_vecs, dim).contiguous()
    packed = torch.empty((1, n_vecs, packed_dim(dim, bits)), dtype=torch.uint32, device=x.device)
    norms = torch.empty((1, n_vecs), dtype=torch.float32, device=x.device)
    quantize_into(x.unsqueeze(0), signs, boundaries, dim, bits, packed, norms)
    return packed[0], norms[0]


def dequantize_into(packed: torch.Tensor, norms: torch.Tensor, centroids, signs, dim: int,
                    bits: int, out: torch.Tensor, n_inner: int, src_row: int = 0,
                    dst_row: int = 0) -> None:
    """Dequantize rows [src_row, src_row + n_inner) of packed (n_outer, n_alloc,
    pdim) into rows [dst_row, ...) of out (n_outer, n_alloc_out, dim)."""
    _check_bits(bits)
    _lib.require_cuda(packed, norms, out)
    n_outer = packed.shape[0]
    pd = packed.shape[-1]
    p_ptr = ctypes.c_void_p(packed.data_ptr() + src_row * pd * 4)
    n_ptr = ctypes.c_void_p(norms.data_ptr() + src_row * 4)
    o_ptr = ctypes.c_void_p(out.data_ptr() + dst_row * dim * out.element_size())
    _lib.check(_lib.lib().tq_dequantize(
        p_ptr, packed.stride(0), n_ptr, norms.stride(0), n_outer, n_inner, dim, bits,
        _lib.host_floats(centroids), _lib.host_floats(signs), o_ptr, _lib.dtype_code(out.dtype),
        out.stride(0), _lib.stream_ptr(out.device)))


def _dequant(packed, norms, centroids, signs, dim, bits, dtype):
    n = norms.shape[0]
    packed = packed.reshape(n, -1).contiguous()
    norms = norms.reshape(n).to(torch.float32).contiguous()
    out = torch.empty((1, n, dim), dtype=dtype, device=packed.device)
    dequantize_into(packed.unsqueeze(0), norms.unsqueeze(0), centroids, signs, dim, bits, out, n)
    return out[0]


def dequant_fp16(packed, norms, centroids, signs, dim: int, bits: int) -> torch.Tensor:
    """Packed rows -> (n, dim) float16."""
    return _dequant(packed, norms, centroids, signs, dim, bits, torch.float16)


def packed_dequantize(packed, norms, centroids, signs, dim: int, bits: int) -> torch.Tensor:
    """Packed rows -> (n, dim) float32."""
    return _dequant(packed, norms, centroids, signs, dim, bits, torch.float32)


prerot_packed_dequantize = packed_dequantize


# ---------------------------------------------------------------------------
# scores
# ---------------------------------------------------------------------------
def prerotate_query(q: torch.Tensor, signs) -> torch.Tensor:
    """(n_heads, dim) -> raw_butterfly(q * signs), float32, no 1/sqrt(dim)."""
    if q.ndim != 2:
        raise ValueError(f"prerotate_query expects (n_heads, dim), got {tuple(q.shape)}")
    _lib.require_cuda(q)
    n_heads, dim = q.shape
    if q.stride(-1) != 1:
        q = q.contiguous()
    out = torch.empty((n_heads, dim), dtype=torch.float32, device=q.device)
    _lib.check(_lib.lib().tq_prerotate_query(_lib.ptr(q), _lib.dtype_code(q.dtype), n_heads,
                                             q.stride(0), dim, _lib.host_floats(signs),
                                             _lib.ptr(out), _lib.stream_ptr(q.device)))
    return out


def _rows_view(t: torch.Tensor) -> torch.Tensor:
    """(heads, seq, width) with contiguous rows; the head stride may be anything."""
    if t.stride(-1) != 1 or t.stride(-2) != t.shape[-1]:
        t = t.contiguous()
    return t


def _vec_view(t: torch.Tensor) -> torch.Tensor:
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def prerot_fused_qk_scores(q_rot, k_packed, k_norms, centroids, dim: int, bits: int,
                           n_rep: int = 1) -> torch.Tensor:
    """(n_q, dim) x packed K (n_kv, seq, pdim) -> (n_q, seq) float32 raw scores."""
    _check_bits(bits)
    _lib.require_cuda(q_rot, k_packed, k_norms)
    n_q = q_rot.shape[0]
    n_kv, seq = k_norms.shape
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    q_rot = q_rot.to(torch.float32).contiguous()
    kp = _rows_view(k_packed)
    kn = _vec_view(k_norms.to(torch.float32))
    out = torch.empty((n_q, seq), dtype=torch.float32, device=q_rot.device)
    _lib.check(_lib.lib().tq_prerot_qk_scores(
        _lib.ptr(q_rot), _lib.ptr(kp), kp.stride(0), _lib.ptr(kn), kn.stride(0), n_kv, seq,
        _lib.host_floats(centroids), dim, bits, n_rep, _lib.ptr(out),
        _lib.stream_ptr(q_rot.device)))
    return out


def packed_fused_qk_scores(query, k_packed, k_norms, centroids, signs, dim: int,
                           bits: int) -> torch.Tensor:
    """Per-position dequant then dot with the un-rotated query (multi-head)."""
    _check_bits(bits)
    _lib.require_cuda(query, k_packed, k_norms)
    n_heads, seq = k_norms.shape
    query = query.to(torch.float32).contiguous()
    kp = _rows_view(k_packed)
    kn = _vec_view(k_norms.to(torch.float32))
    out = torch.empty((n_heads, seq), dtype=torch.float32, device=query.device)
    _lib.check(_lib.lib().tq_packed_qk_scores(
        _lib.ptr(query), _lib.ptr(kp), kp.stride(0), _lib.ptr(kn), kn.stride(0), n_heads, seq,
        _lib.host_floats(centroids), _lib.host_floats(signs), dim, bits, _lib.ptr(out),
        _lib.stream_ptr(query.device)))
    return out


# ---------------------------------------------------------------------------
# weighted V sum
# ---------------------------------------------------------------------------
def sparse_v_matvec(weights, v_packed, v_norms, centroids, signs, dim: int, bits: int,
                    threshold: float = 1e-5, n_rep: int = 1) -> torch.Tensor:
    """Weighted sum of dequantized V rows, (n_q, seq) x packed V -> (n_q, dim)
    float32; positions with weight < threshold are skipped."""
    if dim & (dim - 1):
        raise ValueError(f"dim must be a power of 2, got {dim}")
    if dim > 256:
        raise ValueError(f"dim > 256 not supported by threadgroup layout, got {dim}")
    _check_bits(bits)
    _lib.require_cuda(weights, v_packed, v_norms)
    n_q, seq = weights.shape
    n_kv = v_packed.shape[0]
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    w = _vec_view(weights.to(torch.float32))
    vp = _rows_view(v_packed)
    vn = _vec_view(v_norms.to(torch.float32))
    out = torch.empty((n_q, dim), dtype=torch.float32, device=w.device)
    L = _lib.lib()
    need = L.tq_sparse_v_workspace_bytes(n_q, seq, dim)
    ws = _lib.workspace(need, w.device, tag="sparse_v")
    _lib.check(L.tq_sparse_v_matvec(
        _lib.ptr(w), w.stride(0), _lib.ptr(vp), vp.stride(0), _lib.ptr(vn), vn.stride(0), n_kv,
        seq, _lib.host_floats(centroids), _lib.host_floats(signs), dim, bits, float(threshold),
        n_rep, _lib.ptr(out), _lib.ptr(ws), need, _lib.stream_ptr(w.device)))
    return out


def count_active_positions(weights: torch.Tensor, threshold: float = 1e-5) -> int:
    """Positions whose weight exceeds `threshold` (diagnostics only)."""
    return int((weights > threshold).sum().item())


# ---------------------------------------------------------------------------
# flash decode
# ---------------------------------------------------------------------------
def _strides3(t: torch.Tensor, batched: bool):
    """(batch_stride, head_stride) of a (B, H, ...) or (H, ...) tensor."""
    if batched:
        return t.stride(0), t.stride(1)
    return 0, t.stride(0)


def flash_decode(q: torch.Tensor, *, k=None, v=None, attn_scale: float, q_prerotated: bool = False,
                 mask: torch.Tensor | None = None, num_splits: int = 0, out_dtype=None,
                 partials: bool = False, partial_out=None, kv_stable: bool = False, out=None, peers=None,
                 q_stable: bool = False, new_k: torch.Tensor | None = None, new_v: torch.Tensor | None = None,
                 sparse_v_threshold: float = 0.0, active_out: torch.Tensor | None = None,
                 seq_lens: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                 workspace_owner=None, gather=None, _prepare_only: bool = False):
    """Split-K flash decoding for one query token per sequence (or a few, see below).

    q: (B, n_q, dim), or (B, n_q, T, dim) with n_rep * T <= 8 for a short multi-token step: the T
    queries are the last T positions of the sequence (their K / V rows are already stored, S counts
    them) and attend causally; the result is (B, n_q, T, dim).  The reference sends such steps to
    dense attention over the dequantized cache (patch.py:19-21); here they read the packed rows once.
    k / v: dicts describing the stored keys / values:
      polar : dict(format="polar", packed (B, n_kv, S, pdim) uint32, norms (B, n_kv, S),
                   centroids, signs, bits)
      dense : dict(format="dense", data (B, n_kv, S, dim) fp16/bf16/fp32)       [keys only]
      affine: dict(format="affine", codes (B, n_kv, S, bytes) uint8, scales, biases
                   (B, n_kv, S, dim/group) fp16, bits, group)
    The sequence dimension may be a view of a longer allocation (head and batch
    strides are passed through).  mask: optional additive float mask
    broadcastable to (B, n_q, S).  Returns (B, n_q, dim) in out_dtype (default
    q.dtype), or with partials=True the merged state (m (B, n_q), l (B, n_q),
    acc (B, n_q, dim)) before the final butterfly / normalisation; `partial_out`
    optionally names the three tensors to write (e.g. slices of a send buffer).
    `out` optionally names the (B, n_q, dim) tensor to write.  `peers` (partials only, see
    distributed.PeerExchange.targets) makes the kernel also store the merged state into the
    given peer buffers and bump their counters.

    kv_stable=True promises that no kernel that may still be running when this call's kernel
    starts (the decode kernel is launched with programmatic stream serialization, so the
    kernels in front of it on the stream may still be draining) writes a K / V row this call
    reads; q_stable=True promises the same for q (and new_k / new_v).  With both the kernel
    reads its inputs at once and consecutive decode calls overlap on the GPU.

    new_k / new_v (B, n_kv, dim): the step's own token.  The K / V descriptors must already
    span it (S counts it, its row is the last one); the kernel stores / quantizes the two rows
    into that position and attends over them in the same launch, replacing the separate cache
    append.  The descriptors need "boundaries" (and polar keys "signs") for this.  Raises
    ValueError when the call does not qualify for the tensor-core kernel.

    sparse_v_threshold > 0 (tensor-core kernel only, ValueError otherwise): values of positions
    whose softmax weight is certain to end below the threshold are not accumulated (decided per
    16-position tile and kv-head group from the running softmax state and the largest score the
    group's CTAs have seen so far, so nothing is dropped that the reference's `sparse_v_matvec`
    would keep); `active_out`, an int32 (B, n_kv) tensor, receives the number of positions whose
    values were accumulated (it is zeroed here with a launch of its own: leave it out where decode
    launches are meant to overlap).

    seq_lens (tensor-core kernel only): int32 (B,) device tensor with the number of valid positions
    of each sequence (<= S), read by the kernel when it runs: ragged batches without a mask, and
    decode steps replayed from a CUDA graph whose lengths advance on the device.  With new_k /
    new_v the rows go to position seq_lens[b] - 1.

    workspace: a zero-initialised uint8 CUDA tensor owned by the caller and used by no other call
    that may be in flight together with this one (`decode_workspace` makes one; e.g. one per
    layer).  With kv_stable and q_stable such a call depends on nothing that is still running, so
    consecutive decode launches overlap from start to end.  Without it the calls of a stream share
    one workspace and each waits for its predecessor before writing it.  `workspace_owner`: any
    object (a cache, say); its attribute `_decode_ws` holds such a workspace, made or grown here.

    gather (with partials=True and peers; see distributed.PeerExchange.gather_spec): after the
    push the same launch waits (bounded) for every rank's rows in this GPU's own receive slot,
    merges them and writes the final (B, n_q, dim) result to `out`, which is returned: the
    sequence-sharded decode step in one launch per layer.
    """
    _lib.require_cuda(q)
    q_tokens = 1
    if q.ndim == 4:                       # (B, n_q, T, dim): the last T positions of each sequence, causal
        q_tokens = q.shape[2]
        if q_tokens == 1:
            q = q[:, :, 0]
        elif partials or new_k is not None or mask is not None:
            raise ValueError("several query tokens: no partials, no in-launch append, no mask (causal is implied)")
    if q.stride(-1) != 1:
        q = q.contiguous()
    B, n_q, dim = q.shape[0], q.shape[1], q.shape[-1]
    P = _lib.FlashParams()
    P.struct_bytes = ctypes.sizeof(_lib.FlashParams)
    P.batch, P.n_q_heads, P.dim = B, n_q, dim
    P.q, P.q_dtype, P.q_prerotated = q.data_ptr(), _lib.dtype_code(q.dtype), int(q_prerotated)
    P.q_batch_stride, P.q_head_stride = q.stride(0), q.stride(1)
    if q_tokens > 1:
        P.q_tokens, P.q_token_stride = q_tokens, q.stride(2)
    out_shape = (B, n_q, dim) if q_tokens == 1 else (B, n_q, q_tokens, dim)
    keep = []  # keeps converted tensors / host arrays alive until the launch returns

    def rows(t):
        t = _rows_view(t)
        keep.append(t)
        return t

    kf = k["format"]
    if kf == "polar":
        kp, kn = rows(k["packed"]), k["norms"]
        if kn.stride(-1) != 1:
            kn = kn.contiguous()
        keep.append(kn)
        n_kv, S = kn.shape[1], kn.shape[2]
        P.k_format, P.k_bits = _lib.TQ_KV_POLAR, int(k["bits"])
        _check_bits(P.k_bits)
        P.k_data, P.k_batch_stride, P.k_head_stride = kp.data_ptr(), kp.stride(0), kp.stride(1)
        P.k_norms, P.kn_batch_stride, P.kn_head_stride = kn.data_ptr(), kn.stride(0), kn.stride(1)
        kc = _lib.host_floats(k["centroids"])
        ks = _lib.host_floats(k.get("signs"))
        keep += [kc, ks]
        P.k_centroids_host = kc
        if ks is not None:
            P.k_signs_host = ks
    elif kf == "dense":
        kd = rows(k["data"])
        n_kv, S = kd.shape[1], kd.shape[2]
        P.k_format, P.k_dtype = _lib.TQ_KV_DENSE, _lib.dtype_code(kd.dtype)
        P.k_data, P.k_batch_stride, P.k_head_stride = kd.data_ptr(), kd.stride(0), kd.stride(1)
    elif kf == "affine":
        kc_, ksc, kbi = rows(k["codes"]), rows(k["scales"]), rows(k["biases"])
        n_kv, S = kc_.shape[1], kc_.shape[2]
        P.k_format, P.k_bits, P.k_group = _lib.TQ_KV_AFFINE, int(k["bits"]), int(k["group"])
        P.k_data, P.k_batch_stride, P.k_head_stride = kc_.data_ptr(), kc_.stride(0), kc_.stride(1)
        P.k_scales, P.k_biases = ksc.data_ptr(), kbi.data_ptr()
        P.ks_batch_stride, P.ks_head_stride = ksc.stride(0), ksc.stride(1)
    else:
        raise ValueError(f"unknown key format {kf!r}")

    vf = v["format"]
    if vf == "polar":
        vp, vn = rows(v["packed"]), v["norms"]
        if vn.stride(-1) != 1:
            vn = vn.contiguous()
        keep.append(vn)
        P.v_format, P.v_bits = _lib.TQ_KV_POLAR, int(v["bits"])
        _check_bits(P.v_bits)
        P.v_data, P.v_batch_stride, P.v_head_stride = vp.data_ptr(), vp.stride(0), vp.stride(1)
        P.v_norms, P.vn_batch_stride, P.vn_head_stride = vn.data_ptr(), vn.stride(0), vn.stride(1)
        vc, vs = _lib.host_floats(v["centroids"]), _lib.host_floats(v["signs"])
        keep += [vc, vs]
        P.v_centroids_host, P.v_signs_host = vc, vs
        v_heads, v_seq = vn.shape[1], vn.shape[2]
    elif vf == "affine":
        vc_, vsc, vbi = rows(v["codes"]), rows(v["scales"]), rows(v["biases"])
        P.v_format, P.v_bits, P.v_group = _lib.TQ_KV_AFFINE, int(v["bits"]), int(v["group"])
        P.v_data, P.v_batch_stride, P.v_head_stride = vc_.data_ptr(), vc_.stride(0), vc_.stride(1)
        P.v_scales, P.v_biases = vsc.data_ptr(), vbi.data_ptr()
        P.vs_batch_stride, P.vs_head_stride = vsc.stride(0), vsc.stride(1)
        v_heads, v_seq = vc_.shape[1], vc_.shape[2]
    else:
        raise ValueError(f"unknown value format {vf!r}")
    if v_heads != n_kv or v_seq != S:
        raise ValueError(f"K ({n_kv} heads, {S} positions) and V ({v_heads}, {v_seq}) disagree")
    if n_q % n_kv:
        raise ValueError(f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep")
    P.n_kv_heads, P.seq_len = n_kv, S
    P.attn_scale, P.num_splits = float(attn_scale), int(num_splits)
    P.kv_stable = int(kv_stable)
    P.q_stable = int(q_stable)
    P.sparse_v_threshold = max(float(sparse_v_threshold), 0.0)
    if seq_lens is not None:
        _lib.require_cuda(seq_lens)
        if seq_lens.dtype != torch.int32 or tuple(seq_lens.shape) != (B,) or not seq_lens.is_contiguous():
            raise ValueError(f"seq_lens must be a contiguous int32 ({B},) tensor")
        keep.append(seq_lens)
        P.seq_lens_dev = seq_lens.data_ptr()
    if active_out is not None:
        _lib.require_cuda(active_out)
        if active_out.dtype != torch.int32 or tuple(active_out.shape) != (B, n_kv) or not active_out.is_contiguous():
            raise ValueError(f"active_out must be a contiguous int32 ({B}, {n_kv}) tensor")
        active_out.zero_()
        keep.append(active_out)
        P.active_positions = active_out.data_ptr()
    if (new_k is None) != (new_v is None):
        raise ValueError("new_k and new_v must be given together")
    if new_k is not None:
        _lib.require_cuda(new_k, new_v)
        if new_k.shape != (B, n_kv, dim) or new_v.shape != (B, n_kv, dim) or new_k.dtype != new_v.dtype:
            raise ValueError(f"new_k / new_v must be ({B}, {n_kv}, {dim}) tensors of one dtype")
        if new_k.stride(-1) != 1:
            new_k = new_k.contiguous()
        if new_v.stride(-1) != 1:
            new_v = new_v.contiguous()
        keep += [new_k, new_v]
        P.new_dtype = _lib.dtype_code(new_k.dtype)
        P.new_k, P.new_v = new_k.data_ptr(), new_v.data_ptr()
        P.new_k_batch_stride, P.new_k_head_stride = new_k.stride(0), new_k.stride(1)
        P.new_v_batch_stride, P.new_v_head_stride = new_v.stride(0), new_v.stride(1)
        vb = _lib.host_floats(v.get("boundaries"))
        kb = _lib.host_floats(k.get("boundaries")) if kf == "polar" else None
        keep += [vb, kb]
        if vb is not None:
            P.v_boundaries_host = vb
        if kb is not None:
            P.k_boundaries_host = kb

    if mask is not None:
        m = mask.to(torch.float32)
        while m.ndim < 3:
            m = m.unsqueeze(0)
        if m.shape[-1] != S or m.shape[0] not in (1, B) or m.shape[1] not in (1, n_q):
            raise ValueError(f"mask shape {tuple(mask.shape)} does not broadcast to ({B}, {n_q}, {S})")
        if m.stride(-1) != 1:
            m = m.contiguous()
        keep.append(m)
        P.mask = m.data_ptr()
        P.mask_batch_stride = 0 if m.shape[0] == 1 else m.stride(0)
        P.mask_head_stride = 0 if m.shape[1] == 1 else m.stride(1)

    dev = q.device
    if gather is not None and (not partials or peers is None):
        raise ValueError("gather needs partials=True and peers")
    if partials:
        P.out_mode = 1 if gather is None else 2
        if gather is not None:
            if out is None:
                out = torch.empty((B, n_q, dim), dtype=out_dtype or q.dtype, device=dev)
            elif tuple(out.shape) != (B, n_q, dim) or out.stride(-1) != 1:
                raise ValueError(f"out must be ({B}, {n_q}, {dim}) with a contiguous last dimension")
            P.out, P.out_dtype = out.data_ptr(), _lib.dtype_code(out.dtype)
            P.out_batch_stride, P.out_head_stride = out.stride(0), out.stride(1)
            P.gather_ranks = int(gather["n_ranks"])
            P.gather_m, P.gather_l, P.gather_acc = int(gather["m"]), int(gather["l"]), int(gather["acc"])
            P.gather_part_stride, P.gather_flags = int(gather["part_stride"]), int(gather["flags"])
        if partial_out is not None:     # contiguous float32 views (B, n_q), (B, n_q), (B, n_q, dim)
            pm, pl, pa = partial_out
            assert pm.is_contiguous() and pl.is_contiguous() and pa.is_contiguous()
        else:
            pm = torch.empty((B, n_q), dtype=torch.float32, device=dev)
            pl = torch.empty((B, n_q), dtype=torch.float32, device=dev)
            pa = torch.empty((B, n_q, dim), dtype=torch.float32, device=dev)
        P.part_m, P.part_l, P.part_acc = pm.data_ptr(), pl.data_ptr(), pa.data_ptr()
        if peers is not None:           # the merged state also goes to these (peer GPU) addresses
            n_peers = len(peers["acc"])
            if not (1 <= n_peers <= 8) or any(len(peers[key]) != n_peers for key in ("m", "l", "counter")):
                raise ValueError("peers: 1..8 entries in each of m, l, acc, counter")
            P.n_peers = n_peers
            P.peer_slots_exclusive = int(bool(peers.get("exclusive", False)))
            for i in range(n_peers):
                P.peer_m[i], P.peer_l[i] = int(peers["m"][i]), int(peers["l"][i])
                P.peer_acc[i], P.peer_counter[i] = int(peers["acc"][i]), int(peers["counter"][i])
    else:
        P.out_mode = 0
        if out is None:
            out = torch.empty(out_shape, dtype=out_dtype or q.dtype, device=dev)
        elif tuple(out.shape) != out_shape or out.stride(-1) != 1:
            raise ValueError(f"out must be {out_shape} with a contiguous last dimension")
        P.out, P.out_dtype = out.data_ptr(), _lib.dtype_code(out.dtype)
        P.out_batch_stride, P.out_head_stride = out.stride(0), out.stride(1)
        if q_tokens > 1:
            P.out_token_stride = out.stride(2)
    P.stream = torch.cuda.current_stream(dev).cuda_stream
    L = _lib.lib()
    need = L.tq_flash_decode_workspace_bytes(ctypes.byref(P))
    if need < 0:
        _lib.check(int(need))
    if workspace is None and workspace_owner is not None:
        workspace = getattr(workspace_owner, "_decode_ws", None)
        if workspace is None or workspace.numel() < need or workspace.device != dev:
            workspace = decode_workspace(dev, max(int(need), 1 << 20))
            workspace_owner._decode_ws = workspace
    if workspace is not None:
        _lib.require_cuda(workspace)
        if workspace.dtype != torch.uint8 or not workspace.is_contiguous() or workspace.numel() < need:
            raise ValueError(f"workspace must be a contiguous uint8 tensor of at least {need} bytes")
        ws = workspace
        P.workspace_exclusive = 1
    else:
        ws = _lib.workspace(need, dev, tag=f"flash{B * n_kv}")   # counters: one layout per batch * n_kv
    if ws is not None:
        P.workspace, P.workspace_bytes = ws.data_ptr(), ws.numel()
    result = out if (not partials or gather is not None) else (pm, pl, pa)
    if _prepare_only:
        keep += [q, ws, result]
        return P, keep, result, dev
    _lib.check(L.tq_flash_decode(ctypes.byref(P)))
    del keep
    return result


class FlashDecodePlan:
    """A flash_decode call with its arguments marshalled once.  The tensors named
    at construction (q, K/V storage, outputs) are read / written in place on every
    `run()`, which costs a single C call: use it in decode loops where the host
    time per layer matters.  Same keyword arguments as `flash_decode`."""

    def __init__(self, q, **kwargs):
        self._keep_ws = kwargs.get("workspace")          # a caller-owned workspace, if any (status word in front)
        self._P, self._keep, self.result, self._dev = flash_decode(q, _prepare_only=True, **kwargs)
        self._fn = _lib.lib().tq_flash_decode
        self._ref = ctypes.byref(self._P)

    def run(self):
        self._P.stream = torch.cuda.current_stream(self._dev).cuda_stream
        rc = self._fn(self._ref)
        if rc:
            _lib.check(rc)
        return self.result


def decode_workspace(device, nbytes: int = 4 << 20) -> torch.Tensor:
    """A zero-filled workspace for `flash_decode(..., workspace=...)`: give every call that may
    overlap with others (one per layer, say) its own.  4 MiB covers 96 splits of 64 heads."""
    return torch.zeros((int(nbytes),), dtype=torch.uint8, device=device)


def workspace_status(ws: torch.Tensor) -> int:
    """Status word of a caller-owned decode workspace (synchronises; resets the word): 0 unless
    a bounded wait inside the kernel gave up."""
    word = ws[:4].view(torch.int32)
    code = int(word.item())
    if code:
        word.zero_()
    return code


def flash_status(device, batch_kv_groups: int) -> int:
    """Status word of the tensor-core decode kernel's workspace for calls with
    batch * n_kv_heads == `batch_kv_groups` on this device and stream (synchronises):
    0 unless a bounded wait inside the kernel gave up, in which case the outputs of
    the calls since the last check are invalid.  Resets the word."""
    key = (f"flash{batch_kv_groups}", str(torch.device(device)), torch.cuda.current_stream(device).cuda_stream)
    ws = _lib._workspaces.get(key)
    if ws is None:
        return 0
    word = ws[:4].view(torch.int32)
    code = int(word.item())
    if code:
        word.zero_()
    return code


def flash_attention_turboquant(q_rot, k_packed, k_norms, v_packed, v_norms, k_centroids,
                               v_centroids, v_signs, dim: int, bits: int, attn_scale: float,
                               block_size: int = 16, n_rep: int = 1, v_bits: int | None = None):
    """Fused SDPA over packed K/V for one pre-rotated query per head:
    (n_q, dim) -> (n_q, dim) float32.  `block_size` is validated for
    compatibility; the kernel picks its own tiling and splits the sequence
    across CTAs.  `v_bits` (default: bits) allows a different width for V."""
    if dim > 128 or dim & (dim - 1):
        raise ValueError(f"dim must be a power of 2 and <= 128, got {dim}")
    if block_size < 1 or block_size > 32:
        raise ValueError(f"block_size must be in 1..32, got {block_size}")
    n_q = q_rot.shape[0]
    n_kv, seq = k_norms.shape
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    k = dict(format="polar", packed=k_packed.unsqueeze(0), norms=k_norms.to(torch.float32).unsqueeze(0),
             centroids=k_centroids, bits=bits)
    v = dict(format="polar", packed=v_packed.unsqueeze(0), norms=v_norms.to(torch.float32).unsqueeze(0),
             centroids=v_centroids, signs=v_signs, bits=bits if v_bits is None else v_bits)
    out = flash_decode(q_rot.to(torch.float32).unsqueeze(0), k=k, v=v, attn_scale=attn_scale,
                       q_prerotated=True, out_dtype=torch.float32)
    return out[0]


def merge_partials(part_m, part_l, part_acc, v_signs, out_dtype=torch.float32) -> torch.Tensor:
    """Merge (n_parts, rows) / (n_parts, rows, dim) partial states from sequence
    chunks or ranks into the final (rows, dim) output.  The three tensors may be
    views into one gathered buffer: only the part stride (dim 0) is free."""
    _lib.require_cuda(part_m, part_l, part_acc)
    n_parts, rows, dim = part_acc.shape

    def rows_contiguous(t, inner):
        ok = t.stride(-1) == 1 and (t.ndim == 2 or t.stride(1) == inner)
        return t if ok else t.contiguous()

    pm, pl, pa = rows_contiguous(part_m, 1), rows_contiguous(part_l, 1), rows_contiguous(part_acc, dim)
    out = torch.empty((rows, dim), dtype=out_dtype, device=pa.device)
    _lib.check(_lib.lib().tq_merge_partials(
        _lib.ptr(pm), pm.stride(0), _lib.ptr(pl), pl.stride(0), _lib.ptr(pa), pa.stride(0), n_parts,
        rows, dim, _lib.host_floats(v_signs), _lib.ptr(out), _lib.dtype_code(out_dtype), dim,
        _lib.stream_ptr(pa.device)))
    return out


class MergePlan:
    """`merge_partials` with its arguments marshalled once (see FlashDecodePlan)."""

    def __init__(self, part_m, part_l, part_acc, v_signs, out):
        _lib.require_cuda(part_m, part_l, part_acc, out)
        n_parts, rows, dim = part_acc.shape
        assert part_m.stride(-1) == 1 and part_l.stride(-1) == 1 and part_acc.stride(-1) == 1
        assert part_acc.stride(1) == dim and out.is_contiguous()
        self._keep = (part_m, part_l, part_acc, out, _lib.host_floats(v_signs))
        self._args = (_lib.ptr(part_m), part_m.stride(0), _lib.ptr(part_l), part_l.stride(0),
                      _lib.ptr(part_acc), part_acc.stride(0), n_parts, rows, dim, self._keep[4],
                      _lib.ptr(out), _lib.dtype_code(out.dtype), dim)
        self._fn = _lib.lib().tq_merge_partials
        self._dev = out.device
        self.result = out

    def run(self):
        rc = self._fn(*self._args, _lib.stream_ptr(self._dev))
        if rc:
            _lib.check(rc)
        return self.result

    def run_after_peers(self, flags_ptr, n_ranks: int, epoch: int, status_ptr, reset_flags: bool = False,
                        exclusive_flags: bool = False):
        """The same merge, gated inside the kernel on the peers' flags (see PeerExchange).  With
        `reset_flags` the kernel zeroes the flags once it is past the gate (graph-replayable);
        `exclusive_flags`: no other merge waits on these flag words (a slot per layer), so this one
        need not wait for the launch in front of it."""
        rc = _lib.lib().tq_merge_partials_after_peers(flags_ptr, n_ranks, epoch, status_ptr,
                                                      (2 if exclusive_flags else 1) if reset_flags else 0,
                                                      *self._args, _lib.stream_ptr(self._dev))
        if rc:
            _lib.check(rc)
        return self.result


# ---------------------------------------------------------------------------
# prefill attention (dense 16-bit Q, K, V on the tcgen05 tensor cores)
# ---------------------------------------------------------------------------
def prefill_supported(queries, keys, values, mask) -> bool:
    """True when tq_prefill_sdpa covers the call: CUDA f16 / bf16 tensors of one
    dtype, head_dim 128, no mask or the "causal" mask, rows of 128 contiguous
    elements and strides that are multiples of 8 elements."""
    if not (queries.is_cuda and keys.is_cuda and values.is_cuda):
        return False
    if queries.dtype not in (torch.float16, torch.bfloat16):
        return False
    if keys.dtype != queries.dtype or values.dtype != queries.dtype:
        return False
    if queries.ndim != 4 or keys.ndim != 4 or values.ndim != 4:
        return False
    if queries.shape[-1] != 128 or keys.shape[-1] != 128 or values.shape[-1] != 128:
        return False
    if not (mask is None or (isinstance(mask, str) and mask == "causal")):
        return False
    if mask is not None and keys.shape[2] < queries.shape[2]:
        return False
    if keys.shape[2] != values.shape[2] or queries.shape[1] % keys.shape[1]:
        return False
    for t in (queries, keys, values):
        if t.stride(-1) != 1 or any(st % 8 for st in t.stride()[:-1]) or t.data_ptr() % 16:
            return False
    return True


def prefill_attention(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, scale: float,
                      causal: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(scale * Q K^T [+ causal]) V for (B, n_q, L, 128) queries and
    (B, n_kv, S, 128) keys / values of one 16-bit dtype (GQA without replication).
    The call the reference leaves to its array library for every step that is not
    a single-token decode (turboquant_mlx/patch.py:37)."""
    _lib.require_cuda(queries, keys, values)
    if queries.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("prefill_attention takes float16 or bfloat16 tensors")
    if keys.dtype != queries.dtype or values.dtype != queries.dtype:
        raise ValueError("queries, keys and values must share one dtype")
    B, n_q, L, D = queries.shape
    Bk, n_kv, S, Dk = keys.shape
    if D != 128 or Dk != 128 or values.shape[-1] != 128:
        raise ValueError(f"prefill_attention supports head_dim 128, got {D}")
    if n_q % n_kv:
        raise ValueError(f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_q // max(n_kv, 1)})")
    if values.shape[:3] != keys.shape[:3] or Bk != B:
        raise ValueError("keys and values must have the same (batch, heads, length)")

    def usable(t):
        ok = t.stride(-1) == 1 and not any(st % 8 for st in t.stride()[:-1]) and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()

    q, k, v = usable(queries), usable(keys), usable(values)
    if out is None:
        out = torch.empty((B, n_q, L, D), dtype=q.dtype, device=q.device)
    status = _lib.workspace(16, q.device, tag="prefill")
    _lib.check(_lib.lib().tq_prefill_sdpa(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.dtype_code(q.dtype), B, n_q, n_kv, L, S, D,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
        float(scale), 1 if causal else 0, _lib.ptr(status), _lib.stream_ptr(q.device)))
    return out


def prefill_status(device) -> int:
    """Status word of the prefill kernel on this device and stream (synchronises):
    0 unless a bounded wait inside the kernel gave up."""
    status = _lib.workspace(16, device, tag="prefill")
    return int(status[:4].view(torch.int32).item())
