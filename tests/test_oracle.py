"""CPU tests of the oracle: spec-derived known-answer vectors, the relational
properties the reference's own tests pin (tests/test_core.py, test_prerot.py,
test_sparse_v.py, test_flash_attention.py of the reference), and the frozen
golden fixtures."""

import math

import numpy as np
import pytest


def test_boundary_bit_patterns(oracle):
    b3 = oracle.boundaries(oracle.codebook(3)).view(np.uint32)
    assert [f"{v:08x}" for v in b3] == ["bfdfbe76", "bf866666", "bf00240b", "00000000",
                                        "3f00240b", "3f866666", "3fdfbe76"]
    b4 = oracle.boundaries(oracle.codebook(4)).view(np.uint32)
    assert [f"{v:08x}" for v in b4[:8]] == ["c019a6b5", "bfebf7cf", "bfb7f2e4", "bf8cb439",
                                            "bf4caf4f", "bf05bf48", "be843958", "00000000"]
    with pytest.raises(ValueError):
        oracle.codebook(5)


def test_kat_zero_vector(oracle):
    s = oracle.signs_from_seed(128, 43)
    p, n = oracle.quantize_packed(np.zeros((1, 128), np.float16), s, 3)
    assert n[0] == 0.0
    assert list(p[0]) == [0x1B6DB6DB] * 12 + [0x006DB6DB]
    idx4, _ = oracle.quantize(np.zeros((1, 128), np.float32), s, 4)
    assert (idx4 == 7).all()


def test_kat_x_equals_signs(oracle):
    s = oracle.signs_from_seed(128, 42)
    idx, n = oracle.quantize(s[None], s, 3)
    assert n[0] == np.float32(math.sqrt(128.0))
    assert idx[0, 0] == 7 and (idx[0, 1:] == 3).all()


def test_hadamard_matrix_is_sylvester(oracle):
    d = 64
    H = oracle.raw_butterfly(np.eye(d, dtype=np.float32))
    i, j = np.meshgrid(np.arange(d), np.arange(d), indexing="ij")
    pop = np.vectorize(lambda v: bin(v).count("1"))(i & j)
    assert np.array_equal(H, np.where(pop % 2 == 0, 1.0, -1.0).astype(np.float32))


def test_wht_self_inverse_and_norm_preserving(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((10, 128)).astype(np.float32)
    y = oracle.walsh_hadamard_transform(x)
    assert np.abs(oracle.walsh_hadamard_transform(y) - x).max() < 1e-5
    assert np.abs(np.linalg.norm(x, axis=-1) - np.linalg.norm(y, axis=-1)).max() < 1e-4
    s = oracle.signs_from_seed(128, 42)
    z = oracle.inverse_randomized_hadamard(oracle.randomized_hadamard_transform(x, s), s)
    assert np.abs(z - x).max() < 1e-4


def test_rotation_gaussianises(oracle):
    rng = np.random.default_rng(1)
    d = 256
    x = rng.standard_normal((1000, d)).astype(np.float32)
    x[:, :10] *= 10.0
    s = oracle.signs_from_seed(d, 42)
    y = oracle.randomized_hadamard_transform(x, s).reshape(-1)
    m, sd = y.mean(), y.std()
    kurt = (((y - m) / sd) ** 4).mean()
    assert 1.5 < kurt < 6.0


def test_roundtrip_quality_monotone_in_bits(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((100, 128)).astype(np.float32)
    s = oracle.signs_from_seed(128, 42)
    cos = []
    for bits in (2, 3, 4):
        idx, n = oracle.quantize(x, s, bits)
        xh = oracle.dequantize(idx, n, s, bits)
        c = (x * xh).sum(-1) / (np.linalg.norm(x, axis=-1) * np.linalg.norm(xh, axis=-1) + 1e-8)
        cos.append(c.mean())
    assert cos[1] > 0.7 and cos[0] < cos[1] < cos[2]


@pytest.mark.parametrize("bits,dim", [(1, 128), (2, 32), (3, 128), (4, 64), (3, 100)])
def test_pack_unpack_roundtrip(oracle, bits, dim):
    rng = np.random.default_rng(3)
    idx = rng.integers(0, 1 << bits, size=(7, 5, dim)).astype(np.uint8)
    p = oracle.pack_indices(idx, bits)
    assert p.shape == (7, 5, oracle.packed_dim(dim, bits)) and p.dtype == np.uint32
    assert np.array_equal(oracle.unpack_indices(p, bits, dim), idx)
    # element j sits in word j // vpw at bit (j % vpw) * bits
    vpw = oracle.VALS_PER_WORD[bits]
    j = dim - 1
    assert ((p[0, 0, j // vpw] >> ((j % vpw) * bits)) & ((1 << bits) - 1)) == idx[0, 0, j]


def test_mul_div_by_scale_is_not_identity(oracle):
    """(raw * s) / s differs from raw for a noticeable share of float32 values,
    which is why the index compare has to replay both operations."""
    rng = np.random.default_rng(4)
    raw = rng.standard_normal(200000).astype(np.float32)
    s = oracle.wht_scale(128)
    z = ((raw * s).astype(np.float32) / s).astype(np.float32)
    frac = (z != raw).mean()
    assert 0.05 < frac < 0.3


@pytest.mark.parametrize("H,S,D,bits", [(4, 64, 128, 3), (8, 256, 128, 3), (2, 16, 64, 4), (1, 128, 32, 2)])
def test_prerot_scores_match_per_position_dequant(oracle, H, S, D, bits):
    rng = np.random.default_rng(5)
    s = oracle.signs_from_seed(D, 42)
    c = oracle.codebook(bits)
    kp = oracle.pack_indices(rng.integers(0, 1 << bits, (H, S, D)).astype(np.uint8), bits)
    kn = (rng.random((H, S)) * 5 + 0.1).astype(np.float32)
    q = rng.standard_normal((H, D)).astype(np.float32)
    a = oracle.prerot_fused_qk_scores(oracle.prerotate_query(q, s), kp, kn, c, D, bits)
    b = oracle.packed_fused_qk_scores(q, kp, kn, c, s, D, bits)
    assert np.abs(a - b).max() < 1e-4 * max(1.0, np.abs(b).max())


@pytest.mark.parametrize("n_kv,n_rep", [(4, 2), (2, 4), (4, 7)])
def test_gqa_equals_repeat(oracle, n_kv, n_rep):
    rng = np.random.default_rng(6)
    S, D, bits = 128, 128, 3
    s = oracle.signs_from_seed(D, 42)
    c = oracle.codebook(bits)
    vp = oracle.pack_indices(rng.integers(0, 8, (n_kv, S, D)).astype(np.uint8), bits)
    vn = (rng.random((n_kv, S)) + 0.1).astype(np.float32)
    w = oracle.softmax(rng.standard_normal((n_kv * n_rep, S)) * 3)
    g = oracle.sparse_v_matvec(w, vp, vn, c, s, D, bits, threshold=0.0, n_rep=n_rep)
    r = oracle.sparse_v_matvec(w, np.repeat(vp, n_rep, 0), np.repeat(vn, n_rep, 0), c, s, D, bits,
                               threshold=0.0, n_rep=1)
    assert np.abs(g - r).max() < 1e-4
    with pytest.raises(ValueError):
        oracle.sparse_v_matvec(w, vp, vn, c, s, D, bits, n_rep=n_rep + 1)


def test_sparse_v_threshold_semantics(oracle):
    rng = np.random.default_rng(7)
    H, S, D, bits = 4, 512, 128, 3
    s = oracle.signs_from_seed(D, 42)
    c = oracle.codebook(bits)
    vp = oracle.pack_indices(rng.integers(0, 8, (H, S, D)).astype(np.uint8), bits)
    vn = (rng.random((H, S)) + 0.1).astype(np.float32)
    w = oracle.softmax(rng.standard_normal((H, S)) * 3)
    dense = np.einsum("hp,hpe->he", w, oracle.packed_dequantize(vp, vn, c, s, D, bits))
    out0 = oracle.sparse_v_matvec(w, vp, vn, c, s, D, bits, threshold=0.0)
    assert np.abs(out0 - dense).max() / np.abs(dense).max() < 1e-5
    out1 = oracle.sparse_v_matvec(w, vp, vn, c, s, D, bits, threshold=1e-5)
    cos = (out1 * dense).sum() / (np.linalg.norm(out1) * np.linalg.norm(dense))
    assert cos > 0.999
    assert np.abs(oracle.sparse_v_matvec(w, vp, vn, c, s, D, bits, threshold=w.max() * 2 + 1)).max() == 0.0


@pytest.mark.parametrize("H,S,D,bits,bc,n_rep", [(4, 32, 128, 3, 8, 1), (4, 96, 128, 3, 32, 1),
                                                  (2, 64, 64, 4, 8, 1), (4, 128, 128, 3, 16, 2)])
def test_flash_equals_composed(oracle, H, S, D, bits, bc, n_rep):
    rng = np.random.default_rng(8)
    ks, vs = oracle.signs_from_seed(D, 42), oracle.signs_from_seed(D, 43)
    c = oracle.codebook(bits)
    kp = oracle.pack_indices(rng.integers(0, 1 << bits, (H, S, D)).astype(np.uint8), bits)
    vp = oracle.pack_indices(rng.integers(0, 1 << bits, (H, S, D)).astype(np.uint8), bits)
    kn = (rng.random((H, S)) * 5 + 0.1).astype(np.float32)
    vn = (rng.random((H, S)) * 5 + 0.1).astype(np.float32)
    q = rng.standard_normal((H * n_rep, D)).astype(np.float32)
    scale = 1.0 / math.sqrt(D)
    q_rot = oracle.prerotate_query(q, ks)
    flash = oracle.flash_attention_turboquant(q_rot, kp, kn, vp, vn, c, c, vs, D, bits, scale,
                                              block_size=bc, n_rep=n_rep)
    comp, _ = oracle.decode_attention(
        q, k_polar=dict(packed=kp, norms=kn, centroids=c, signs=ks, bits=bits),
        v_polar=dict(packed=vp, norms=vn, centroids=c, signs=vs, bits=bits),
        attn_scale=scale, n_rep=n_rep)
    assert np.abs(flash - comp).max() / np.abs(comp).max() < 1e-3
    with pytest.raises(ValueError):
        oracle.flash_attention_turboquant(q_rot, kp, kn, vp, vn, c, c, vs, D, bits, scale, block_size=33)


def test_merge_of_chunks_equals_whole(oracle):
    rng = np.random.default_rng(9)
    n_kv, n_rep, S, D, bits = 2, 4, 300, 128, 3
    vs = oracle.signs_from_seed(D, 43)
    c = oracle.codebook(bits)
    vp = oracle.pack_indices(rng.integers(0, 8, (n_kv, S, D)).astype(np.uint8), bits)
    vn = (rng.random((n_kv, S)) + 0.1).astype(np.float32)
    scores = (rng.standard_normal((n_kv * n_rep, S)) * 2).astype(np.float32)
    whole = oracle.sparse_v_matvec(oracle.softmax(scores), vp, vn, c, vs, D, bits, 0.0, n_rep)
    cuts = [0, 100, 101, 300]
    parts = [oracle.decode_partials(scores[:, a:b], vp[:, a:b], vn[:, a:b], c, D, bits, n_rep)
             for a, b in zip(cuts[:-1], cuts[1:])]
    # an empty chunk (l = 0) must merge as a no-op
    parts.append((np.zeros(n_kv * n_rep, np.float32), np.zeros(n_kv * n_rep, np.float32),
                  np.zeros((n_kv * n_rep, D), np.float32)))
    m, l, S_ = (np.stack(t) for t in zip(*parts))
    merged = oracle.merge_partials(m, l, S_, vs, D)
    assert np.abs(merged - whole).max() / np.abs(whole).max() < 1e-5


def test_affine_roundtrip(oracle):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((50, 128)).astype(np.float16)
    for bits, tol in ((8, 0.02), (4, 0.3)):
        code, sc, bi = oracle.affine_quantize(x, 64, bits)
        assert code.shape == (50, 128 if bits == 8 else 64) and sc.shape == (50, 2)
        xh = oracle.affine_dequantize(code, sc, bi, 64, bits)
        assert np.abs(xh - x.astype(np.float32)).max() < tol
    z = np.zeros((2, 64), np.float32)
    code, sc, bi = oracle.affine_quantize(z, 64, 8)
    assert (code == 0).all() and (oracle.affine_dequantize(code, sc, bi, 64, 8) == 0).all()


def test_prefill_sdpa_definition(oracle):
    """The dense prompt-step attention: causal rows see keys 0 .. i + (S - L), query head h reads
    kv head h // n_rep, a single visible key returns that key's value row, and the last query row of
    a causal call equals a one-token decode over all keys."""
    rng = np.random.default_rng(21)
    B, n_q, n_kv, L, S, D = 2, 4, 2, 5, 9, 16
    q = rng.standard_normal((B, n_q, L, D)).astype(np.float32)
    k = rng.standard_normal((B, n_kv, S, D)).astype(np.float32)
    v = rng.standard_normal((B, n_kv, S, D)).astype(np.float32)
    scale = 0.3
    out = oracle.prefill_sdpa(q, k, v, scale, causal=True)
    for b in range(B):
        for h in range(n_q):
            for i in range(L):
                vis = i + (S - L) + 1
                s_ = (k[b, h // 2, :vis].astype(np.float64) @ q[b, h, i].astype(np.float64)) * scale
                w = np.exp(s_ - s_.max())
                ref = (w / w.sum()) @ v[b, h // 2, :vis].astype(np.float64)
                assert np.allclose(out[b, h, i], ref, rtol=1e-5, atol=1e-6)
    one = oracle.prefill_sdpa(q[:, :, :1], k[:, :, :1], v[:, :, :1], scale, causal=True)
    assert np.allclose(one[:, :, 0], np.repeat(v[:, :, 0], 2, axis=1), atol=1e-6)
    full = oracle.prefill_sdpa(q[:, :, -1:], k, v, scale, causal=False)
    assert np.allclose(full[:, :, 0], out[:, :, -1], rtol=1e-5, atol=1e-6)


def test_golden_fixtures_match_oracle(oracle, golden):
    g = golden
    assert np.array_equal(oracle.signs_from_seed(128, 42), g["signs_42"])
    assert np.array_equal(oracle.signs_from_seed(128, 43), g["signs_43"])
    for bits in (1, 2, 3, 4):
        p, n = oracle.quantize_packed(g["x_f16"], g["signs_43"], bits)
        assert np.array_equal(p, g[f"packed_b{bits}"])
        assert np.array_equal(n, g["norms"])
        deq = oracle.packed_dequantize(p, n, oracle.codebook(bits), g["signs_43"], 128, bits)
        assert np.array_equal(deq, g[f"deq_b{bits}"])
    assert list(g["packed_b3"][0]) == [0x1B6DB6DB] * 12 + [0x006DB6DB]
    vdesc = dict(packed=g["att_vp"], norms=g["att_vn"], centroids=oracle.codebook(3),
                 signs=g["signs_43"], bits=3)
    out, _ = oracle.decode_attention(g["att_q"], k_dense=g["att_kd"], v_polar=vdesc,
                                     attn_scale=1 / math.sqrt(128), n_rep=7)
    assert np.allclose(out, g["att_out_dense"], rtol=0, atol=1e-6)
