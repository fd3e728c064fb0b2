"""CPU oracle for the TurboQuant / PolarQuant packed-KV path (numpy, float32).

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is
compared against.  Nothing in the product package imports it; only the test
suite, the smoke check and the CPU-baseline leg of the benchmark do.

It restates, operation by operation and in float32, the reference's pure
array-math path (paths are relative to the reference project root):

  turboquant_mlx/rotation.py:7-34     walsh_hadamard_transform
  turboquant_mlx/rotation.py:52-80    randomized / inverse randomized Hadamard
  turboquant_mlx/quantizer.py:18-44   Lloyd-Max codebooks and midpoint boundaries
  turboquant_mlx/quantizer.py:75-132  PolarQuantizer.quantize / dequantize
  turboquant_mlx/packing.py:16-87     pack_indices / unpack_indices / packed_dim
  turboquant_mlx/metal_kernels_v4.py:37-113   prerotate_query, prerot scores
  turboquant_mlx/sparse_v.py:32-88    butterfly-pulled-out weighted V sum
  turboquant_mlx/flash_attention.py:36-163    online-softmax SDPA over packed K/V
  turboquant_mlx/fused_attention.py:50-125    composed decode attention
  turboquant_mlx/hybrid_attention.py:45-88    affine-K + PolarQuant-V composition

PARITY STATUS: parity unpinned against a live run of the reference.  The
reference executes on the `mlx` array library (dependency `mlx>=0.20.0`, no
upper pin), which is not installable where this code is built, and the
reference's tests store no golden vectors.  The oracle is therefore pinned
against (i) known-answer vectors that follow from the arithmetic itself
(zero vector, x == signs, Sylvester-Hadamard matrix entries, the float32 bit
patterns of the boundaries) and (ii) the relational tests of the reference
(WHT self-inverse, norm preservation, composed-vs-fused equalities).

Two quantities depend on `mlx` internals and are defined here instead:
  * the +/-1 sign diagonal: `mlx.random.bernoulli` cannot be regenerated, so
    signs are an explicit input everywhere and `signs_from_seed` documents
    this build's own seed -> signs generator (splitmix64);
  * the reduction order of the L2 norm (`mx.linalg.norm`): `sumsq_tree`
    fixes it to a pairwise tree in natural index order.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32

VALS_PER_WORD = {1: 32, 2: 16, 3: 10, 4: 8}  # packing.py:16
BIT_MASK = {1: 0x1, 2: 0x3, 3: 0x7, 4: 0xF}  # packing.py:17

_CODEBOOKS = {  # quantizer.py:27-36 (the same table is repeated in cache.py:16-25)
    1: [-0.7979, 0.7979],
    2: [-1.5104, -0.4528, 0.4528, 1.5104],
    3: [-2.1520, -1.3440, -0.7560, -0.2451, 0.2451, 0.7560, 1.3440, 2.1520],
    4: [-2.7326, -2.0690, -1.6180, -1.2562, -0.9423, -0.6568, -0.3881, -0.1284,
        0.1284, 0.3881, 0.6568, 0.9423, 1.2562, 1.6180, 2.0690, 2.7326],
}


# --------------------------------------------------------------------------
# codebooks, signs
# --------------------------------------------------------------------------
def codebook(bits: int) -> np.ndarray:
    """Lloyd-Max centroids for N(0,1), float32 (quantizer.py:18-39)."""
    if bits not in _CODEBOOKS:
        raise ValueError(f"Unsupported bit width: {bits}. Use 1-4.")
    return np.asarray(_CODEBOOKS[bits], dtype=F32)


def boundaries(centroids: np.ndarray) -> np.ndarray:
    """Midpoints between adjacent centroids, float32 (quantizer.py:42-44)."""
    c = np.asarray(centroids, dtype=F32)
    return ((c[:-1] + c[1:]) / F32(2.0)).astype(F32)


def _splitmix64(state: int):
    state = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return state, z ^ (z >> 31)


def signs_from_seed(d: int, seed: int = 42) -> np.ndarray:
    """+/-1 diagonal of length d.

    Stands in for rotation.py:37-49, whose values come from the `mlx` PRNG and
    cannot be regenerated.  Generator of this build: splitmix64 seeded with
    `seed`; element i is +1 when the top bit of the i-th output is set.
    """
    state = seed & 0xFFFFFFFFFFFFFFFF
    out = np.empty(d, dtype=F32)
    for i in range(d):
        state, z = _splitmix64(state)
        out[i] = 1.0 if (z >> 63) else -1.0
    return out


# --------------------------------------------------------------------------
# rotation (rotation.py)
# --------------------------------------------------------------------------
def raw_butterfly(x: np.ndarray) -> np.ndarray:
    """Un-normalised Walsh-Hadamard butterfly on the last axis, float32.

    Stages h = 1, 2, 4, ...: each block of 2h splits into halves (a, b) and
    becomes (a + b, a - b) (rotation.py:22-32).
    """
    x = np.asarray(x, dtype=F32)
    d = x.shape[-1]
    assert d > 0 and (d & (d - 1)) == 0, f"Dimension must be power of 2, got {d}"
    lead = x.shape[:-1]
    h = 1
    while h < d:
        xr = x.reshape(*lead, d // (2 * h), 2, h)
        even = xr[..., 0, :]
        odd = xr[..., 1, :]
        x = np.stack([even + odd, even - odd], axis=-2).reshape(*lead, d)
        h *= 2
    return x


def wht_scale(d: int) -> np.float32:
    """float32(1/sqrt(d)): the Python double meets a float32 array (rotation.py:34)."""
    return F32(1.0 / math.sqrt(d))


def walsh_hadamard_transform(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=F32)
    return (raw_butterfly(x) * wht_scale(x.shape[-1])).astype(F32)


def randomized_hadamard_transform(x, signs):  # rotation.py:52-64
    return walsh_hadamard_transform(np.asarray(x, F32) * np.asarray(signs, F32))


def inverse_randomized_hadamard(x, signs):  # rotation.py:67-80
    return (walsh_hadamard_transform(x) * np.asarray(signs, F32)).astype(F32)


# --------------------------------------------------------------------------
# quantize / dequantize (quantizer.py)
# --------------------------------------------------------------------------
def sumsq_tree(x32: np.ndarray) -> np.ndarray:
    """Sum of squares over the last axis: float32 squares, then a pairwise
    tree in natural index order (level k adds s[2i] + s[2i+1])."""
    s = (x32 * x32).astype(F32)
    while s.shape[-1] > 1:
        s = (s[..., 0::2] + s[..., 1::2]).astype(F32)
    return s[..., 0]


def quantize_scaled(x, signs):
    """Steps 1-7 of PolarQuantizer.quantize (quantizer.py:85-97).

    Returns (z, norms): z is the value compared with the boundaries,
    z = (bfly(x/max(n,1e-8) * signs) * s) / s with s = float32(1/sqrt(d)).
    """
    x32 = np.asarray(x).astype(F32)
    d = x32.shape[-1]
    n = np.sqrt(sumsq_tree(x32)).astype(F32)
    safe = np.maximum(n, F32(1e-8)).astype(F32)
    u = (x32 / safe[..., None]).astype(F32)
    t = (u * np.asarray(signs, F32)).astype(F32)
    r = (raw_butterfly(t) * wht_scale(d)).astype(F32)
    z = (r / wht_scale(d)).astype(F32)
    return z, n


def quantize(x, signs, bits: int):
    """PolarQuantizer.quantize (quantizer.py:75-106): (indices uint8, norms f32)."""
    z, n = quantize_scaled(x, signs)
    b = boundaries(codebook(bits))
    idx = np.zeros(z.shape, dtype=np.uint8)
    for bi in b.tolist():
        idx = idx + (z > F32(bi)).astype(np.uint8)  # strict compare, quantizer.py:104
    return idx, n


def dequantize(indices, norms, signs, bits: int) -> np.ndarray:
    """PolarQuantizer.dequantize (quantizer.py:108-132), float32 result."""
    c = codebook(bits)
    idx = np.asarray(indices)
    d = idx.shape[-1]
    y = (c[idx.astype(np.int64)] * wht_scale(d)).astype(F32)
    xu = inverse_randomized_hadamard(y, signs)
    return (xu * np.asarray(norms, F32)[..., None]).astype(F32)


def tie_distance_ulps(z: np.ndarray, bits: int) -> np.ndarray:
    """Distance, in float32 ulps of the boundary, from each z to its nearest
    boundary.  An index mismatch with distance <= 2 is classed as a tie."""
    b = boundaries(codebook(bits))
    diff = np.abs(z[..., None].astype(np.float64) - b.astype(np.float64))
    ulp = np.maximum(np.spacing(np.abs(b)).astype(np.float64), np.spacing(F32(1e-30)))
    return (diff / ulp).min(axis=-1)


# --------------------------------------------------------------------------
# packing (packing.py)
# --------------------------------------------------------------------------
def packed_dim(dim: int, bits: int) -> int:
    vpw = VALS_PER_WORD[bits]
    return (dim + vpw - 1) // vpw


def pack_indices(indices, bits: int) -> np.ndarray:
    """packing.py:26-56: element j -> word j // vpw, bit (j % vpw) * bits, LSB first."""
    vpw = VALS_PER_WORD[bits]
    idx = np.asarray(indices)
    shape = idx.shape
    dim = shape[-1]
    flat = idx.reshape(-1, dim).astype(np.uint32)
    pd = packed_dim(dim, bits)
    if dim % vpw:
        pad = np.zeros((flat.shape[0], vpw - dim % vpw), dtype=np.uint32)
        flat = np.concatenate([flat, pad], axis=1)
    flat = flat.reshape(-1, pd, vpw)
    out = np.zeros((flat.shape[0], pd), dtype=np.uint32)
    for i in range(vpw):
        out |= flat[:, :, i] << np.uint32(i * bits)
    return out.reshape(*shape[:-1], pd)


def unpack_indices(packed, bits: int, dim: int) -> np.ndarray:
    """packing.py:59-87."""
    vpw = VALS_PER_WORD[bits]
    mask = np.uint32(BIT_MASK[bits])
    p = np.asarray(packed, dtype=np.uint32)
    shape = p.shape
    flat = p.reshape(-1, shape[-1])
    vals = [(flat >> np.uint32(i * bits)) & mask for i in range(vpw)]
    res = np.stack(vals, axis=-1).reshape(flat.shape[0], shape[-1] * vpw)[:, :dim]
    return res.reshape(*shape[:-1], dim).astype(np.uint8)


def quantize_packed(x, signs, bits: int):
    """quantize followed by pack_indices: the stored form (packed u32, norms f32)."""
    idx, n = quantize(x, signs, bits)
    return pack_indices(idx, bits), n


def packed_dequantize(packed, norms, centroids, signs, dim: int, bits: int) -> np.ndarray:
    """kernels.py:14-55: unpack -> c*s -> raw butterfly -> *s *signs *norm, float32."""
    s = wht_scale(dim)
    idx = unpack_indices(packed, bits, dim).astype(np.int64)
    y = (np.asarray(centroids, F32)[idx] * s).astype(F32)
    r = raw_butterfly(y)
    r = (r * s).astype(F32)
    r = (r * np.asarray(signs, F32)).astype(F32)
    return (r * np.asarray(norms, F32)[..., None]).astype(F32)


def metal_fused_quantize_indices(x, signs, bits: int):
    """Variant used by the reference's fused kernel (metal.py:66-77): the raw
    butterfly is compared with the boundaries directly, without the multiply
    and divide by s.  Kept to report how often the two conventions differ;
    the parity target is `quantize`."""
    x32 = np.asarray(x).astype(F32)
    n = np.sqrt(sumsq_tree(x32)).astype(F32)
    u = (x32 / np.maximum(n, F32(1e-8))[..., None]).astype(F32)
    raw = raw_butterfly((u * np.asarray(signs, F32)).astype(F32))
    b = boundaries(codebook(bits))
    idx = np.zeros(raw.shape, dtype=np.uint8)
    for bi in b.tolist():
        idx = idx + (raw > F32(bi)).astype(np.uint8)
    return idx, n


# --------------------------------------------------------------------------
# attention-side kernels
# --------------------------------------------------------------------------
def prerotate_query(q, signs) -> np.ndarray:
    """metal_kernels_v4.py:37-62: raw butterfly of q * signs, no 1/sqrt(d)."""
    q = np.asarray(q).astype(F32)
    if q.ndim != 2:
        raise ValueError(f"prerotate_query expects (n_heads, dim), got {q.shape}")
    return raw_butterfly((q * np.asarray(signs, F32)).astype(F32))


def prerot_fused_qk_scores(q_rot, k_packed, k_norms, centroids, dim, bits, n_rep=1):
    """metal_kernels_v4.py:71-113: score[h,p] = (sum_e c[idx]*q_rot[h,e]) * norm * (1/dim)."""
    q_rot = np.asarray(q_rot, F32)
    n_q = q_rot.shape[0]
    n_kv, seq = np.asarray(k_norms).shape
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    cvals = np.asarray(centroids, F32)[unpack_indices(k_packed, bits, dim).astype(np.int64)]
    kv = np.arange(n_q) // n_rep
    dots = np.einsum("hpe,he->hp", cvals[kv].astype(np.float64), q_rot.astype(np.float64))
    out = dots.astype(F32) * np.asarray(k_norms, F32)[kv] * F32(1.0 / dim)
    return out.astype(F32)


def packed_fused_qk_scores(query, k_packed, k_norms, centroids, signs, dim, bits):
    """kernels.py:58-117: per-position dequant then dot with the raw query (MHA)."""
    deq = packed_dequantize(k_packed, k_norms, centroids, signs, dim, bits)
    return np.einsum("hpe,he->hp", deq.astype(np.float64),
                     np.asarray(query, F32).astype(np.float64)).astype(F32)


def sparse_v_matvec(weights, v_packed, v_norms, centroids, signs, dim, bits,
                    threshold=1e-5, n_rep=1):
    """sparse_v.py:32-88: out[h] = signs * bfly(sum_{p: w>=thr} w*norm*c[idx]) * (1/dim)."""
    if dim & (dim - 1):
        raise ValueError(f"dim must be a power of 2, got {dim}")
    if dim > 256:
        raise ValueError(f"dim > 256 not supported by threadgroup layout, got {dim}")
    w = np.asarray(weights, F32)
    n_q, seq = w.shape
    n_kv = np.asarray(v_packed).shape[0]
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    thr = F32(max(threshold, 0.0))
    cvals = np.asarray(centroids, F32)[unpack_indices(v_packed, bits, dim).astype(np.int64)]
    kv = np.arange(n_q) // n_rep
    wn = np.where(w < thr, F32(0), w).astype(np.float64) * np.asarray(v_norms, F32)[kv]
    S = np.einsum("hp,hpe->he", wn, cvals[kv].astype(np.float64)).astype(F32)
    out = raw_butterfly(S) * np.asarray(signs, F32) * F32(1.0 / dim)
    return out.astype(F32)


def count_active_positions(weights, threshold=1e-5) -> int:  # sparse_v.py:189-191
    return int((np.asarray(weights) > threshold).sum())


def softmax(x, axis=-1):
    x = np.asarray(x, dtype=np.float64)
    m = x.max(axis=axis, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.exp(x - m)
    return (e / e.sum(axis=axis, keepdims=True)).astype(F32)


def prefill_sdpa(q, k, v, scale, causal=True):
    """Dense attention of a multi-token step: the call the reference leaves to its
    array library (patch.py:37, `mx.fast.scaled_dot_product_attention(queries, keys,
    values, scale=scale, mask=mask)`), restated from the published definition
    softmax(scale * Q K^T + mask) V.  q (B, n_q, L, D), k / v (B, n_kv, S, D); query
    head h reads kv head h // (n_q // n_kv); with `causal` query row i sees keys
    0 .. i + (S - L), which is what create_causal_mask(L, offset=S - L) masks
    (cache.py:328).  float64 accumulation, float32 result."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    B, n_q, L, D = q.shape
    n_kv, S = k.shape[1], k.shape[2]
    rep = n_q // n_kv
    out = np.empty((B, n_q, L, D), dtype=F32)
    allowed = None
    if causal:
        allowed = np.arange(S)[None, :] <= (np.arange(L)[:, None] + (S - L))
    for b in range(B):
        for h in range(n_q):
            s = (q[b, h] @ k[b, h // rep].T) * scale
            if allowed is not None:
                s = np.where(allowed, s, -np.inf)
            out[b, h] = softmax(s, axis=-1).astype(np.float64) @ v[b, h // rep]
    return out


def flash_attention_turboquant(q_rot, k_packed, k_norms, v_packed, v_norms,
                               k_centroids, v_centroids, v_signs, dim, bits,
                               attn_scale, block_size=16, n_rep=1, v_bits=None):
    """flash_attention.py:36-163 restated block by block (online softmax, the
    accumulator stays in the rotated domain, one butterfly at the end).
    `v_bits` (default: bits) is this build's extension for asymmetric K/V widths."""
    if dim > 128 or dim & (dim - 1):
        raise ValueError(f"dim must be a power of 2 and <= 128, got {dim}")
    if block_size < 1 or block_size > 32:
        raise ValueError(f"block_size must be in 1..32, got {block_size}")
    v_bits = bits if v_bits is None else v_bits
    q_rot = np.asarray(q_rot, F32)
    n_q = q_rot.shape[0]
    n_kv, seq = np.asarray(k_norms).shape
    if n_q != n_kv * n_rep:
        raise ValueError(
            f"n_q_heads ({n_q}) must equal n_kv_heads ({n_kv}) * n_rep ({n_rep})")
    kc = np.asarray(k_centroids, F32)[unpack_indices(k_packed, bits, dim).astype(np.int64)]
    vc = np.asarray(v_centroids, F32)[unpack_indices(v_packed, v_bits, dim).astype(np.int64)]
    kn = np.asarray(k_norms, F32)
    vn = np.asarray(v_norms, F32)
    out = np.zeros((n_q, dim), dtype=F32)
    inv_dim = F32(1.0 / dim)
    for h in range(n_q):
        kvh = h // n_rep
        m = -np.inf
        l = 0.0
        S = np.zeros(dim, dtype=np.float64)
        for b0 in range(0, seq, block_size):
            b1 = min(b0 + block_size, seq)
            sc = (kc[kvh, b0:b1].astype(np.float64) @ q_rot[h].astype(np.float64))
            sc = sc * kn[kvh, b0:b1] * inv_dim * F32(attn_scale)
            m_new = max(m, sc.max())
            alpha = math.exp(m - m_new) if np.isfinite(m) else 0.0
            p = np.exp(sc - m_new)
            l = l * alpha + p.sum()
            S = S * alpha + (p * vn[kvh, b0:b1]) @ vc[kvh, b0:b1].astype(np.float64)
            m = m_new
        o = raw_butterfly(S.astype(F32)) * np.asarray(v_signs, F32) * inv_dim / F32(l)
        out[h] = o
    return out


def decode_attention(q, k_polar=None, k_dense=None, v_polar=None, *, attn_scale,
                     n_rep=1, mask=None, sparse_v_threshold=0.0):
    """Composed decode attention for one batch element (fused_attention.py:56-121).

    q: (n_q, d) raw query.
    k_polar: dict(packed, norms, centroids, signs, bits) for PolarQuant K, or
    k_dense: (n_kv, S, d) float K (fp16 keys of the V-only cache; scores are
             plain q.k, the composition hybrid_attention.py:45-73 uses).
    v_polar: dict(packed, norms, centroids, signs, bits).
    Returns (out (n_q, d) float32, weights (n_q, S) float32).
    """
    q = np.asarray(q).astype(F32)
    n_q, d = q.shape
    if k_polar is not None:
        q_rot = prerotate_query(q, k_polar["signs"])
        scores = prerot_fused_qk_scores(q_rot, k_polar["packed"], k_polar["norms"],
                                        k_polar["centroids"], d, k_polar["bits"], n_rep)
    else:
        kd = np.asarray(k_dense).astype(np.float64)
        kv = np.arange(n_q) // n_rep
        scores = np.einsum("hpe,he->hp", kd[kv], q.astype(np.float64)).astype(F32)
    scores = (scores * F32(attn_scale)).astype(F32)
    if mask is not None:
        scores = scores + np.asarray(mask, F32)
    w = softmax(scores, axis=-1)
    out = sparse_v_matvec(w, v_polar["packed"], v_polar["norms"], v_polar["centroids"],
                          v_polar["signs"], d, v_polar["bits"],
                          threshold=sparse_v_threshold, n_rep=n_rep)
    return out, w


# --------------------------------------------------------------------------
# split-K / cross-rank partial merge (rotated-domain accumulator)
# --------------------------------------------------------------------------
def decode_partials(scores, v_packed, v_norms, centroids, dim, bits, n_rep=1):
    """Partial state of one sequence chunk: m (n_q,), l (n_q,), S (n_q, d) with
    S = sum_p exp(score-m) * norm * c[idx] kept before the final butterfly."""
    sc = np.asarray(scores, dtype=np.float64)
    n_q = sc.shape[0]
    kv = np.arange(n_q) // n_rep
    m = sc.max(axis=-1)
    p = np.exp(sc - m[:, None])
    l = p.sum(axis=-1)
    cvals = np.asarray(centroids, F32)[unpack_indices(v_packed, bits, dim).astype(np.int64)]
    S = np.einsum("hp,hpe->he", p * np.asarray(v_norms, F32)[kv], cvals[kv].astype(np.float64))
    return m.astype(F32), l.astype(F32), S.astype(F32)


def merge_partials(ms, ls, Ss, v_signs, dim):
    """Merge chunk partials: m* = max m_i, l* = sum l_i e^(m_i-m*), S* likewise,
    out = signs * bfly(S*) * (1/dim) / l*.  A chunk with l == 0 merges as a no-op."""
    ms = np.asarray(ms, dtype=np.float64)      # (n_parts, n_q)
    ls = np.asarray(ls, dtype=np.float64)
    Ss = np.asarray(Ss, dtype=np.float64)      # (n_parts, n_q, d)
    ms = np.where(ls > 0, ms, -np.inf)
    m_star = ms.max(axis=0)
    m_safe = np.where(np.isfinite(m_star), m_star, 0.0)
    w = np.where(ls > 0, np.exp(ms - m_safe[None]), 0.0)
    l_star = (ls * w).sum(axis=0)
    S_star = (Ss * w[..., None]).sum(axis=0).astype(F32)
    o = raw_butterfly(S_star) * np.asarray(v_signs, F32) * F32(1.0 / dim)
    return (o / np.maximum(l_star, 1e-38)[:, None]).astype(F32)


# --------------------------------------------------------------------------
# group-wise affine quantisation (K8 / V4).  The reference's arithmetic for
# this lives in `mlx` (mx.quantize / mx.quantized_matmul, used at
# hybrid_cache.py:57-63 and hybrid_attention.py:52-55) and in an un-vendored
# mlx-lm fork; neither is available, so the format below is this build's own:
#   per group of `group` consecutive elements: lo = min, hi = max (float32),
#   scale = float16((hi - lo) / (2^bits - 1)), bias = float16(lo),
#   code = clip(rint((x - bias) / scale), 0, 2^bits - 1)  (scale == 0 -> code 0),
#   dequant = scale * code + bias.
# 8-bit codes are one byte each; 4-bit codes are two per byte, low nibble first.
# --------------------------------------------------------------------------
def affine_quantize(x, group: int = 64, bits: int = 8):
    x32 = np.asarray(x).astype(F32)
    d = x32.shape[-1]
    assert d % group == 0
    g = x32.reshape(*x32.shape[:-1], d // group, group)
    lo = g.min(axis=-1)
    hi = g.max(axis=-1)
    qmax = F32((1 << bits) - 1)
    scale = ((hi - lo) / qmax).astype(np.float16)
    bias = lo.astype(np.float16)
    s32 = scale.astype(F32)[..., None]
    b32 = bias.astype(F32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        code = np.rint((g - b32) / s32)
    code = np.where(s32 > 0, code, 0.0)
    code = np.clip(code, 0, qmax).astype(np.uint8).reshape(*x32.shape[:-1], d)
    if bits == 4:
        code = (code[..., 0::2] | (code[..., 1::2] << 4)).astype(np.uint8)
    return code, scale, bias


def affine_dequantize(code, scale, bias, group: int = 64, bits: int = 8):
    code = np.asarray(code, dtype=np.uint8)
    if bits == 4:
        lo = code & 0xF
        hi = code >> 4
        code = np.stack([lo, hi], axis=-1).reshape(*code.shape[:-1], code.shape[-1] * 2)
    d = code.shape[-1]
    g = code.reshape(*code.shape[:-1], d // group, group).astype(F32)
    out = g * np.asarray(scale).astype(F32)[..., None] + np.asarray(bias).astype(F32)[..., None]
    return out.reshape(*code.shape[:-1], d).astype(F32)
