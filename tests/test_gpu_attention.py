"""GPU parity of the attention-side kernels against the oracle: re-expression
of the reference's tests/test_prerot.py, test_sparse_v.py and
test_flash_attention.py with the oracle as the comparator, plus the cases the
reference lacks (dense and affine keys, batch, masks, split-K partials, ragged
lengths).  Tolerance for attention outputs: 2e-3 max relative error."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ATT_TOL = 2e-3


def _rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


def _t(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def _packed(rng, oracle, shape, bits):
    return oracle.pack_indices(rng.integers(0, 1 << bits, shape).astype(np.uint8), bits)


@pytest.mark.parametrize("n_heads,dim", [(4, 128), (8, 64), (1, 32), (32, 128)])
def test_prerotate_query(tq, oracle, dev, n_heads, dim):
    rng = np.random.default_rng(0)
    q = rng.standard_normal((n_heads, dim)).astype(np.float32)
    s = tq.random_diagonal_sign(dim, 42, device=dev)
    out = tq.prerotate_query(_t(q, dev), s)
    assert np.array_equal(out.cpu().numpy(), oracle.prerotate_query(q, s.cpu().numpy()))
    with pytest.raises(ValueError):
        tq.prerotate_query(_t(q, dev).unsqueeze(0), s)


@pytest.mark.parametrize("H,S,D,bits", [(4, 64, 128, 3), (8, 256, 128, 3), (2, 16, 64, 4), (1, 128, 32, 2),
                                        (3, 77, 128, 4)])
def test_prerot_scores(tq, oracle, dev, H, S, D, bits):
    rng = np.random.default_rng(1)
    pq = tq.PolarQuantizer(D, bits, seed=42, device=dev)
    signs, c = pq.signs.cpu().numpy(), oracle.codebook(bits)
    kp = _packed(rng, oracle, (H, S, D), bits)
    kn = (rng.random((H, S)) * 5 + 0.1).astype(np.float32)
    q = rng.standard_normal((H, D)).astype(np.float32)
    q_rot = tq.prerotate_query(_t(q, dev), pq.signs)
    got = tq.prerot_fused_qk_scores(q_rot, _t(kp, dev), _t(kn, dev), pq.centroids, D, bits)
    ref = oracle.prerot_fused_qk_scores(oracle.prerotate_query(q, signs), kp, kn, c, D, bits)
    assert np.abs(got.cpu().numpy() - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    legacy = tq.packed_fused_qk_scores(_t(q, dev), _t(kp, dev), _t(kn, dev), pq.centroids, pq.signs, D, bits)
    assert np.abs(legacy.cpu().numpy() - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("n_kv,n_rep", [(4, 2), (2, 4), (4, 7), (2, 9)])
def test_prerot_scores_gqa(tq, oracle, dev, n_kv, n_rep):
    rng = np.random.default_rng(2)
    S, D, bits = 128, 128, 3
    pq = tq.PolarQuantizer(D, bits, seed=42, device=dev)
    kp = _packed(rng, oracle, (n_kv, S, D), bits)
    kn = (rng.random((n_kv, S)) * 5 + 0.1).astype(np.float32)
    q_rot = rng.standard_normal((n_kv * n_rep, D)).astype(np.float32) * 10
    got = tq.prerot_fused_qk_scores(_t(q_rot, dev), _t(kp, dev), _t(kn, dev), pq.centroids, D, bits, n_rep=n_rep)
    ref = oracle.prerot_fused_qk_scores(q_rot, kp, kn, oracle.codebook(bits), D, bits, n_rep)
    assert np.abs(got.cpu().numpy() - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    with pytest.raises(ValueError, match="must equal n_kv_heads"):
        tq.prerot_fused_qk_scores(_t(q_rot, dev), _t(kp, dev), _t(kn, dev), pq.centroids, D, bits, n_rep=n_rep + 1)


@pytest.mark.parametrize("H,S,D,bits", [(4, 128, 128, 3), (2, 512, 128, 3), (8, 64, 64, 4), (2, 1000, 128, 3),
                                        (1, 40, 256, 2)])
def test_sparse_v_threshold_zero_matches_dense(tq, oracle, dev, H, S, D, bits):
    rng = np.random.default_rng(3)
    pq = tq.PolarQuantizer(D, bits, seed=42, device=dev)
    vp = _packed(rng, oracle, (H, S, D), bits)
    vn = (rng.random((H, S)) + 0.1).astype(np.float32)
    w = oracle.softmax(rng.standard_normal((H, S)) * 3)
    got = tq.sparse_v_matvec(_t(w, dev), _t(vp, dev), _t(vn, dev), pq.centroids, pq.signs, D, bits, threshold=0.0)
    dense = np.einsum("hp,hpe->he", w.astype(np.float64),
                      oracle.packed_dequantize(vp, vn, oracle.codebook(bits), pq.signs.cpu().numpy(), D, bits))
    assert _rel(got.cpu().numpy(), dense) < 1e-5


def test_sparse_v_threshold_and_gqa(tq, oracle, dev):
    rng = np.random.default_rng(4)
    S, D, bits = 512, 128, 3
    pq = tq.PolarQuantizer(D, bits, seed=42, device=dev)
    signs, c = pq.signs.cpu().numpy(), oracle.codebook(bits)
    for n_kv, n_rep in ((4, 1), (4, 2), (2, 4), (4, 7), (1, 12)):
        vp = _packed(rng, oracle, (n_kv, S, D), bits)
        vn = (rng.random((n_kv, S)) + 0.1).astype(np.float32)
        w = oracle.softmax(rng.standard_normal((n_kv * n_rep, S)) * 3)
        for thr in (0.0, 1e-5, 1e-3):
            got = tq.sparse_v_matvec(_t(w, dev), _t(vp, dev), _t(vn, dev), pq.centroids, pq.signs, D, bits,
                                     threshold=thr, n_rep=n_rep)
            ref = oracle.sparse_v_matvec(w, vp, vn, c, signs, D, bits, threshold=thr, n_rep=n_rep)
            assert _rel(got.cpu().numpy(), ref) < 1e-5
        zero = tq.sparse_v_matvec(_t(w, dev), _t(vp, dev), _t(vn, dev), pq.centroids, pq.signs, D, bits,
                                  threshold=float(w.max()) * 2 + 1, n_rep=n_rep)
        assert float(zero.abs().max()) == 0.0
    assert tq.count_active_positions(_t(w, dev), 1e-5) == oracle.count_active_positions(w, 1e-5)
    with pytest.raises(ValueError, match="power of 2"):
        tq.sparse_v_matvec(_t(w, dev), _t(vp, dev), _t(vn, dev), pq.centroids, pq.signs, 100, bits)
    with pytest.raises(ValueError, match="dim > 256"):
        tq.sparse_v_matvec(_t(w, dev), _t(vp, dev), _t(vn, dev), pq.centroids, pq.signs, 512, bits)


@pytest.mark.parametrize("n_kv,n_rep,S,D,bits,bc", [(4, 1, 32, 128, 3, 8), (4, 1, 128, 128, 3, 16),
                                                   (8, 1, 256, 128, 3, 16), (2, 1, 64, 64, 4, 8),
                                                   (4, 1, 96, 128, 3, 32), (4, 2, 128, 128, 3, 16),
                                                   (2, 4, 128, 128, 3, 16), (4, 7, 1000, 128, 3, 16),
                                                   (2, 8, 4099, 128, 4, 16), (1, 12, 300, 128, 2, 16)])
def test_flash_matches_composed(tq, oracle, dev, n_kv, n_rep, S, D, bits, bc):
    rng = np.random.default_rng(5)
    kq = tq.PolarQuantizer(D, bits, seed=42, device=dev)
    vq = tq.PolarQuantizer(D, bits, seed=43, device=dev)
    c = oracle.codebook(bits)
    kp, vp = _packed(rng, oracle, (n_kv, S, D), bits), _packed(rng, oracle, (n_kv, S, D), bits)
    kn = (rng.random((n_kv, S)) * 5 + 0.1).astype(np.float32)
    vn = (rng.random((n_kv, S)) * 5 + 0.1).astype(np.float32)
    q = rng.standard_normal((n_kv * n_rep, D)).astype(np.float32)
    scale = 1.0 / math.sqrt(D)
    q_rot = tq.prerotate_query(_t(q, dev), kq.signs)
    got = tq.flash_attention_turboquant(q_rot, _t(kp, dev), _t(kn, dev), _t(vp, dev), _t(vn, dev),
                                        kq.centroids, vq.centroids, vq.signs, D, bits, scale,
                                        block_size=bc, n_rep=n_rep)
    ref, _ = oracle.decode_attention(
        q, k_polar=dict(packed=kp, norms=kn, centroids=c, signs=kq.signs.cpu().numpy(), bits=bits),
        v_polar=dict(packed=vp, norms=vn, centroids=c, signs=vq.signs.cpu().numpy(), bits=bits),
        attn_scale=scale, n_rep=n_rep)
    assert got.shape == (n_kv * n_rep, D) and got.dtype == torch.float32
    assert _rel(got.cpu().numpy(), ref) < 1e-3
    # composed GPU path (scores -> softmax -> sparse_v) agrees too
    sc = tq.prerot_fused_qk_scores(q_rot, _t(kp, dev), _t(kn, dev), kq.centroids, D, bits, n_rep=n_rep)
    w = torch.softmax(sc * scale, dim=-1)
    comp = tq.sparse_v_matvec(w, _t(vp, dev), _t(vn, dev), vq.centroids, vq.signs, D, bits, threshold=0.0, n_rep=n_rep)
    assert _rel(got.cpu().numpy(), comp.cpu().numpy()) < 1e-3


def test_flash_argument_errors(tq, dev):
    z = torch.zeros((4, 128), device=dev)
    zp = torch.zeros((4, 8, 13), dtype=torch.uint32, device=dev)
    zn = torch.ones((4, 8), device=dev)
    c = [0.0] * 8
    s = [1.0] * 128
    with pytest.raises(ValueError, match="<= 128"):
        tq.flash_attention_turboquant(z, zp, zn, zp, zn, c, c, s, 256, 3, 1.0)
    with pytest.raises(ValueError, match="block_size"):
        tq.flash_attention_turboquant(z, zp, zn, zp, zn, c, c, s, 128, 3, 1.0, block_size=0)
    with pytest.raises(ValueError, match="must equal n_kv_heads"):
        tq.flash_attention_turboquant(z, zp, zn, zp, zn, c, c, s, 128, 3, 1.0, n_rep=2)


def _golden_dense_case(tq, golden, dev):
    g = golden
    vq = tq.PolarQuantizer(128, 3, seed=43, device=dev)
    k = dict(format="dense", data=_t(g["att_kd"], dev).unsqueeze(0))
    v = dict(format="polar", packed=_t(g["att_vp"], dev).unsqueeze(0), norms=_t(g["att_vn"], dev).unsqueeze(0),
             centroids=vq.centroids, signs=vq.signs, bits=3)
    return k, v


def test_flash_decode_golden_dense_and_polar(tq, golden, dev):
    g = golden
    scale = 1.0 / math.sqrt(128)
    q = _t(g["att_q"], dev).unsqueeze(0)
    k, v = _golden_dense_case(tq, golden, dev)
    out = tq.flash_decode(q, k=k, v=v, attn_scale=scale, out_dtype=torch.float32)
    assert _rel(out[0].cpu().numpy(), g["att_out_dense"]) < ATT_TOL
    out16 = tq.flash_decode(q, k=k, v=v, attn_scale=scale)
    assert out16.dtype == torch.float16
    assert _rel(out16[0].float().cpu().numpy(), g["att_out_dense"]) < ATT_TOL
    kq = tq.PolarQuantizer(128, 4, seed=42, device=dev)
    kpol = dict(format="polar", packed=_t(g["att_kp"], dev).unsqueeze(0), norms=_t(g["att_kn"], dev).unsqueeze(0),
                centroids=kq.centroids, signs=kq.signs, bits=4)
    out2 = tq.flash_decode(q, k=kpol, v=v, attn_scale=scale, out_dtype=torch.float32)
    assert _rel(out2[0].cpu().numpy(), g["att_out_polar"]) < ATT_TOL
    q_rot = tq.prerotate_query(q[0], kq.signs)
    assert np.array_equal(q_rot.cpu().numpy(), g["q_rot"])
    sc = tq.prerot_fused_qk_scores(q_rot, kpol["packed"][0], kpol["norms"][0], kq.centroids, 128, 4, n_rep=7)
    assert np.abs(sc.cpu().numpy() - g["scores_polar"]).max() < 1e-4 * np.abs(g["scores_polar"]).max()


@pytest.mark.parametrize("splits", [0, 1, 3, 16])
def test_flash_decode_batch_splits_mask_strides(tq, oracle, dev, splits):
    """Batch of 3, K/V are views of a longer allocation (stride != length), an
    additive mask hides a ragged tail per sequence, bf16 dense keys."""
    rng = np.random.default_rng(6)
    B, n_kv, n_rep, n_alloc, S, D = 3, 2, 4, 768, 531, 128
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    signs = vq.signs.cpu().numpy()
    kd = torch.from_numpy(rng.standard_normal((B, n_kv, n_alloc, D)).astype(np.float32)).to(torch.bfloat16)
    vraw = (rng.standard_normal((B, n_kv, n_alloc, D)) * rng.lognormal(0, 0.5, (B, n_kv, n_alloc, 1))).astype(np.float16)
    vp, vn = oracle.quantize_packed(vraw, signs, 3)
    q = rng.standard_normal((B, n_kv * n_rep, D)).astype(np.float16)
    lens = [531, 200, 17]
    mask = np.zeros((B, 1, S), np.float32)
    for b, L in enumerate(lens):
        mask[b, 0, L:] = -np.inf
    scale = 1.0 / math.sqrt(D)
    k = dict(format="dense", data=kd.to(dev)[:, :, :S])
    v = dict(format="polar", packed=_t(vp, dev)[:, :, :S], norms=_t(vn, dev)[:, :, :S],
             centroids=vq.centroids, signs=vq.signs, bits=3)
    out = tq.flash_decode(_t(q, dev), k=k, v=v, attn_scale=scale, mask=_t(mask, dev), num_splits=splits,
                          out_dtype=torch.float32)
    for b in range(B):
        ref, _ = oracle.decode_attention(
            q[b], k_dense=kd[b, :, :S].float().numpy(),
            v_polar=dict(packed=vp[b, :, :S], norms=vn[b, :, :S], centroids=oracle.codebook(3), signs=signs, bits=3),
            attn_scale=scale, n_rep=n_rep, mask=np.broadcast_to(mask[b], (n_kv * n_rep, S)))
        assert _rel(out[b].cpu().numpy(), ref) < ATT_TOL


def test_partials_merge_across_chunks_equals_whole(tq, oracle, golden, dev):
    """Sequence chunks processed separately (as ranks would) and merged with
    tq_merge_partials equal the single-pass output; an empty chunk is a no-op."""
    g = golden
    scale = 1.0 / math.sqrt(128)
    q = _t(g["att_q"], dev).unsqueeze(0)
    k, v = _golden_dense_case(tq, golden, dev)
    whole = tq.flash_decode(q, k=k, v=v, attn_scale=scale, out_dtype=torch.float32)
    cuts = [0, 64, 65, 160]
    ms, ls, accs = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        kk = dict(k, data=k["data"][:, :, a:b])
        vv = dict(v, packed=v["packed"][:, :, a:b], norms=v["norms"][:, :, a:b])
        m, l, acc = tq.flash_decode(q, k=kk, v=vv, attn_scale=scale, partials=True)
        ms.append(m[0]); ls.append(l[0]); accs.append(acc[0])
    ms.append(torch.zeros_like(ms[0])); ls.append(torch.zeros_like(ls[0])); accs.append(torch.zeros_like(accs[0]))
    merged = tq.merge_partials(torch.stack(ms), torch.stack(ls), torch.stack(accs), v["signs"])
    # `whole` ran on the tensor-core kernel (f16 operands), the ragged chunks on the float32 one
    assert _rel(merged.cpu().numpy(), whole[0].cpu().numpy()) < 1e-3
    assert _rel(merged.cpu().numpy(), g["att_out_dense"]) < ATT_TOL
    ref = oracle.merge_partials(torch.stack(ms).cpu().numpy(), torch.stack(ls).cpu().numpy(),
                                torch.stack(accs).cpu().numpy(), g["signs_43"], 128)
    assert _rel(merged.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("v_bits", [4, 8])
def test_affine_k8_with_polar_and_affine_values(tq, oracle, dev, v_bits):
    rng = np.random.default_rng(7)
    B, n_kv, n_rep, S, D, G = 2, 2, 4, 300, 128, 64
    kraw = rng.standard_normal((B, n_kv, S, D)).astype(np.float16)
    vraw = rng.standard_normal((B, n_kv, S, D)).astype(np.float16)
    q = rng.standard_normal((B, n_kv * n_rep, D)).astype(np.float16)
    kc, ks, kb = oracle.affine_quantize(kraw, G, 8)
    vc, vs, vb = oracle.affine_quantize(vraw, G, v_bits)
    from turboquant_mlx_b200 import affine
    gkc, gks, gkb = affine.affine_quantize(_t(kraw, dev), G, 8)
    assert np.array_equal(gkc.cpu().numpy(), kc) and np.array_equal(gks.cpu().numpy(), ks)
    assert np.array_equal(gkb.cpu().numpy(), kb)
    gvc, gvs, gvb = affine.affine_quantize(_t(vraw, dev), G, v_bits)
    assert np.array_equal(gvc.cpu().numpy(), vc)
    deq = affine.affine_dequantize(gvc, gvs, gvb, G, v_bits, torch.float32)
    assert np.array_equal(deq.cpu().numpy(), oracle.affine_dequantize(vc, vs, vb, G, v_bits))
    scale = 1.0 / math.sqrt(D)
    k = dict(format="affine", codes=gkc, scales=gks, biases=gkb, bits=8, group=G)
    v = dict(format="affine", codes=gvc, scales=gvs, biases=gvb, bits=v_bits, group=G)
    out = tq.flash_decode(_t(q, dev), k=k, v=v, attn_scale=scale, out_dtype=torch.float32)
    kd = oracle.affine_dequantize(kc, ks, kb, G, 8)
    vd = oracle.affine_dequantize(vc, vs, vb, G, v_bits)
    # K8 / V4 (group 64) runs on the tensor-core kernel, 8-bit values on the general one
    assert tq._lib.lib().tq_flash_decode_last_kernel() == (1 if v_bits == 4 else 0)
    for b in range(B):
        kv = np.arange(n_kv * n_rep) // n_rep
        sc = np.einsum("hpe,he->hp", kd[b][kv].astype(np.float64), q[b].astype(np.float64)) * scale
        w = oracle.softmax(sc)
        ref = np.einsum("hp,hpe->he", w.astype(np.float64), vd[b][kv].astype(np.float64))
        assert _rel(out[b].cpu().numpy(), ref) < ATT_TOL
    # affine K8 + PolarQuant V3 (the long-context sharded layout)
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    vp, vn = oracle.quantize_packed(vraw, vq.signs.cpu().numpy(), 3)
    vpol = dict(format="polar", packed=_t(vp, dev), norms=_t(vn, dev), centroids=vq.centroids, signs=vq.signs, bits=3)
    out2 = tq.flash_decode(_t(q, dev), k=k, v=vpol, attn_scale=scale, out_dtype=torch.float32)
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1      # K8 affine + V3 polar runs on tensor cores
    for b in range(B):
        ref, _ = oracle.decode_attention(q[b], k_dense=kd[b], attn_scale=scale, n_rep=n_rep,
                                         v_polar=dict(packed=vp[b], norms=vn[b], centroids=oracle.codebook(3),
                                                      signs=vq.signs.cpu().numpy(), bits=3))
        assert _rel(out2[b].cpu().numpy(), ref) < ATT_TOL


@pytest.mark.parametrize("k_format", ["affine", "dense"])
@pytest.mark.parametrize("S,n_rep", [(4100, 7), (40004, 2)])   # row strides stay 16-byte multiples
def test_affine_v4_tensor_core_path(tq, oracle, dev, k_format, S, n_rep):
    """4-bit group-affine values on the tensor-core kernel: values with a large common offset and
    per-row spread (so that bias and scale terms both matter), ragged lengths, many splits
    (two merge levels at 40000 positions), fp16 output."""
    rng = np.random.default_rng(S)
    n_kv, D, G = 2, 128, 64
    kraw = rng.standard_normal((1, n_kv, S, D)).astype(np.float16)
    vraw = (3.0 + rng.standard_normal((1, n_kv, S, D)) * rng.lognormal(0, 0.7, (1, n_kv, S, 1))).astype(np.float16)
    q = (1.5 * rng.standard_normal((1, n_kv * n_rep, D))).astype(np.float16)
    from turboquant_mlx_b200 import affine
    gvc, gvs, gvb = affine.affine_quantize(_t(vraw, dev), G, 4)
    vd = oracle.affine_dequantize(gvc.cpu().numpy(), gvs.cpu().numpy(), gvb.cpu().numpy(), G, 4)
    v = dict(format="affine", codes=gvc, scales=gvs, biases=gvb, bits=4, group=G)
    if k_format == "affine":
        gkc, gks, gkb = affine.affine_quantize(_t(kraw, dev), G, 8)
        k = dict(format="affine", codes=gkc, scales=gks, biases=gkb, bits=8, group=G)
        kd = oracle.affine_dequantize(gkc.cpu().numpy(), gks.cpu().numpy(), gkb.cpu().numpy(), G, 8)
    else:
        k = dict(format="dense", data=_t(kraw, dev))
        kd = kraw.astype(np.float32)
    scale = 1.0 / math.sqrt(D)
    out = tq.flash_decode(_t(q, dev), k=k, v=v, attn_scale=scale, out_dtype=torch.float16)
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
    kv = np.arange(n_kv * n_rep) // n_rep
    sc = np.einsum("hpe,he->hp", kd[0][kv].astype(np.float64), q[0].astype(np.float64)) * scale
    ref = np.einsum("hp,hpe->he", oracle.softmax(sc).astype(np.float64), vd[0][kv].astype(np.float64))
    assert _rel(out[0].float().cpu().numpy(), ref) < ATT_TOL


def test_tensor_core_path_is_taken_and_accurate(tq, oracle, dev):
    """Shapes that qualify (dim 128, n_rep <= 8, aligned rows, no mask) must run
    the tensor-core kernel; its result stays within tolerance of the oracle for
    fp16 keys and for 3/4-bit packed keys, including a ragged last tile and
    large / tiny V norms."""
    L = tq._lib.lib()
    rng = np.random.default_rng(21)
    n_kv, n_rep, S, D = 2, 7, 1531, 128
    scale = 1.0 / math.sqrt(D)
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    vs = vq.signs.cpu().numpy()
    vraw = (rng.standard_normal((n_kv, S, D)) * rng.lognormal(0, 1.5, (n_kv, S, 1))).astype(np.float32)
    vraw[0, 5] = 0.0
    vraw[1, 7] *= 3000.0
    vp, vn = oracle.quantize_packed(vraw, vs, 3)

    def alloc(x, n_alloc=1536):   # rows live in a longer allocation, as in a cache (16-byte aligned heads)
        full = np.zeros((x.shape[0], n_alloc) + x.shape[2:], x.dtype)
        full[:, :S] = x
        return _t(full, dev)[:, :S].unsqueeze(0)

    v = dict(format="polar", packed=alloc(vp), norms=alloc(vn), centroids=vq.centroids, signs=vq.signs, bits=3)
    vdesc = dict(packed=vp, norms=vn, centroids=oracle.codebook(3), signs=vs, bits=3)
    q = rng.standard_normal((n_kv * n_rep, D)).astype(np.float16)
    kd = rng.standard_normal((n_kv, S, D)).astype(np.float16)
    out = tq.flash_decode(_t(q, dev).unsqueeze(0), k=dict(format="dense", data=_t(kd, dev).unsqueeze(0)), v=v,
                          attn_scale=scale, out_dtype=torch.float32)
    assert L.tq_flash_decode_last_kernel() == 1
    ref, _ = oracle.decode_attention(q, k_dense=kd, v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
    assert _rel(out[0].cpu().numpy(), ref) < ATT_TOL
    for kbits in (3, 4):
        kq = tq.PolarQuantizer(D, kbits, seed=42, device=dev)
        ks = kq.signs.cpu().numpy()
        kraw = (rng.standard_normal((n_kv, S, D)) * rng.lognormal(0, 0.5, (n_kv, S, 1))).astype(np.float16)
        kp, kn = oracle.quantize_packed(kraw, ks, kbits)
        kpol = dict(format="polar", packed=alloc(kp), norms=alloc(kn), centroids=kq.centroids, signs=kq.signs,
                    bits=kbits)
        out = tq.flash_decode(_t(q, dev).unsqueeze(0), k=kpol, v=v, attn_scale=scale, out_dtype=torch.float32)
        assert L.tq_flash_decode_last_kernel() == 1
        ref, _ = oracle.decode_attention(
            q, k_polar=dict(packed=kp, norms=kn, centroids=oracle.codebook(kbits), signs=ks, bits=kbits),
            v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
        assert _rel(out[0].cpu().numpy(), ref) < ATT_TOL
    # a mask sends the same call down the general path
    out = tq.flash_decode(_t(q, dev).unsqueeze(0), k=kpol, v=v, attn_scale=scale, out_dtype=torch.float32,
                          mask=torch.zeros((1, 1, S), device=dev))
    assert L.tq_flash_decode_last_kernel() == 0
    assert _rel(out[0].cpu().numpy(), ref) < ATT_TOL
    ws = tq._lib.workspace(16, dev, tag=f"flash{n_kv}")
    hdr = L.tq_flash_decode_header_bytes(1, n_kv)
    assert int(ws[:hdr].view(torch.int32).abs().sum()) == 0   # no bounded wait gave up, counters back at zero


def test_prepared_calls_match_direct_calls(tq, golden, dev):
    """FlashDecodePlan / MergePlan (arguments marshalled once) give the same result as the direct
    calls, also when run repeatedly and with kv_stable / out set."""
    g = golden
    scale = 1.0 / math.sqrt(128)
    q = _t(g["att_q"], dev).unsqueeze(0)
    k, v = _golden_dense_case(tq, golden, dev)
    want = tq.flash_decode(q, k=k, v=v, attn_scale=scale, out_dtype=torch.float32)
    out = torch.empty_like(want)
    plan = tq.FlashDecodePlan(q, k=k, v=v, attn_scale=scale, out=out, kv_stable=True)
    for _ in range(3):
        res = plan.run()
    assert res.data_ptr() == out.data_ptr()
    assert _rel(out[0].cpu().numpy(), want[0].cpu().numpy()) < 1e-6
    m, l, acc = tq.flash_decode(q, k=k, v=v, attn_scale=scale, partials=True)
    pm, pl, pa = torch.stack([m[0], m[0]]), torch.stack([l[0], l[0]]), torch.stack([acc[0], acc[0]])
    merged = torch.empty((14, 128), dtype=torch.float32, device=dev)
    mp = tq.MergePlan(pm, pl, pa, v["signs"], merged)
    mp.run()
    assert _rel(merged.cpu().numpy(), want[0].cpu().numpy()) < 1e-5   # two identical parts merge to the same result


def test_flash_decode_value_skipping_is_conservative(tq, oracle, dev):
    """sparse_v_threshold inside the decode kernel (sparse_v.py:59-65 semantics, conservative):
    peaked attention over 4096 positions.  The kernel drops a subset of what the exact rule drops
    (it only knows the running state of the chunk it has seen), so its result lies between the exact
    rule's and the un-thresholded one, the count of accumulated positions is never below the
    oracle's count of kept positions, a single chunk whose dominant keys come early drops most
    tiles, and a threshold of 0 changes nothing."""
    rng = np.random.default_rng(21)
    n_kv, n_rep, S, D = 2, 4, 4096, 128
    kq = tq.PolarQuantizer(D, 4, seed=42, device=dev)
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    ks, vs = kq.signs.cpu().numpy(), vq.signs.cpu().numpy()
    q = rng.standard_normal((n_kv * n_rep, D)).astype(np.float16)
    kraw = rng.standard_normal((n_kv, S, D)).astype(np.float16)
    # a few keys line up with the queries so that the softmax is peaked (as in a trained model)
    for h in range(n_kv):
        for j in range(6):
            kraw[h, 97 * (j + 1) + 300 * h] = (q[h * n_rep + (j % n_rep)] * 6).astype(np.float16)
    vraw = (rng.standard_normal((n_kv, S, D)) * rng.lognormal(0, 0.5, (n_kv, S, 1))).astype(np.float16)
    kp, kn = oracle.quantize_packed(kraw, ks, 4)
    vp, vn = oracle.quantize_packed(vraw, vs, 3)
    scale = 1.0 / math.sqrt(D)
    kdesc = dict(packed=kp, norms=kn, centroids=oracle.codebook(4), signs=ks, bits=4)
    vdesc = dict(packed=vp, norms=vn, centroids=oracle.codebook(3), signs=vs, bits=3)
    k = dict(format="polar", packed=_t(kp, dev).unsqueeze(0), norms=_t(kn, dev).unsqueeze(0), centroids=kq.centroids,
             signs=kq.signs, bits=4)
    v = dict(format="polar", packed=_t(vp, dev).unsqueeze(0), norms=_t(vn, dev).unsqueeze(0), centroids=vq.centroids,
             signs=vq.signs, bits=3)
    qd = _t(q, dev).unsqueeze(0)
    dense = tq.flash_decode(qd, k=k, v=v, attn_scale=scale, out_dtype=torch.float32)
    dense_ref, w = oracle.decode_attention(q, k_polar=kdesc, v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
    assert _rel(dense[0].cpu().numpy(), dense_ref) < ATT_TOL
    for thr in (1e-5, 1e-3):
        exact, _ = oracle.decode_attention(q, k_polar=kdesc, v_polar=vdesc, attn_scale=scale, n_rep=n_rep,
                                           sparse_v_threshold=thr)
        active = torch.empty((1, n_kv), dtype=torch.int32, device=dev)
        got = tq.flash_decode(qd, k=k, v=v, attn_scale=scale, out_dtype=torch.float32, sparse_v_threshold=thr,
                              active_out=active, num_splits=1)
        assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
        g0 = got[0].cpu().numpy()
        split = tq.flash_decode(qd, k=k, v=v, attn_scale=scale, out_dtype=torch.float32, sparse_v_threshold=thr)
        assert _rel(split[0].cpu().numpy(), dense_ref) <= _rel(exact, dense_ref) + ATT_TOL
        # the kernel drops a subset of what the exact rule drops: it is at least as close to the
        # un-thresholded result as the exact rule is
        assert _rel(g0, dense_ref) <= _rel(exact, dense_ref) + ATT_TOL
        if thr == 1e-5:                                            # the reference's own criterion at its default
            cos = (g0 * dense_ref).sum(-1) / (np.linalg.norm(g0, axis=-1) * np.linalg.norm(dense_ref, axis=-1))
            assert cos.min() > 0.999
        kept = (w >= thr).reshape(n_kv, n_rep, S).any(1).sum(-1)   # positions the exact rule keeps for some head
        act = active[0].cpu().numpy()
        print(f"thr {thr}: positions accumulated per kv head {act.tolist()}, kept by the exact rule {kept.tolist()}")
        assert (act >= kept).all() and (act <= S).all()
        if thr == 1e-3:
            assert (act < S // 2).all()                            # one chunk, dominant keys in its first quarter
            # four splits: the dominant keys sit in the first one; the others learn of them through the
            # group's hint words in the workspace (how much that lets them drop depends on how far they have
            # come by then: the CTAs run side by side), and the result stays on the safe side
            active4 = torch.empty((1, n_kv), dtype=torch.int32, device=dev)
            got4 = tq.flash_decode(qd, k=k, v=v, attn_scale=scale, out_dtype=torch.float32, sparse_v_threshold=thr,
                                   active_out=active4, num_splits=4)
            assert _rel(got4[0].cpu().numpy(), dense_ref) <= _rel(exact, dense_ref) + ATT_TOL
            act4 = active4[0].cpu().numpy()
            print(f"thr {thr}, 4 splits: positions accumulated per kv head {act4.tolist()}")
            assert (act4 >= kept).all() and (act4 <= S).all()
    same = tq.flash_decode(qd, k=k, v=v, attn_scale=scale, out_dtype=torch.float32, sparse_v_threshold=0.0)
    assert torch.equal(same, dense)
    with pytest.raises(ValueError, match="value skipping"):
        tq.flash_decode(qd, k=k, v=v, attn_scale=scale, sparse_v_threshold=1e-3, mask=torch.zeros((1, 1, S), device=dev))


def test_flash_decode_device_side_lengths(tq, dev):
    """seq_lens: a ragged batch in one launch equals per-sequence calls on the truncated views, for
    dense and packed keys; with new_k / new_v each row lands at its own sequence's end; and a CUDA
    graph replays with lengths that advance on the device."""
    g = torch.Generator(device=dev).manual_seed(31)
    B, n_kv, n_rep, S, D = 3, 2, 4, 1500, 128
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    kq = tq.PolarQuantizer(D, 4, seed=42, device=dev)
    lens = [1500, 777, 33]
    kd = torch.randn((B, n_kv, S, D), generator=g, device=dev).half()
    vraw = (torch.randn((B, n_kv, S, D), generator=g, device=dev) * 2).half()
    vp, vn = tq.fused_quantize(vraw.reshape(-1, D), vq.signs, vq.boundaries, D, 3)
    kp, kn = tq.fused_quantize(kd.reshape(-1, D), kq.signs, kq.boundaries, D, 4)
    v = dict(format="polar", packed=vp.reshape(B, n_kv, S, 13), norms=vn.reshape(B, n_kv, S), centroids=vq.centroids,
             signs=vq.signs, bits=3, boundaries=vq.boundaries)
    k_dense = dict(format="dense", data=kd)
    k_polar = dict(format="polar", packed=kp.reshape(B, n_kv, S, 16), norms=kn.reshape(B, n_kv, S),
                   centroids=kq.centroids, signs=kq.signs, bits=4, boundaries=kq.boundaries)
    q = torch.randn((B, n_kv * n_rep, D), generator=g, device=dev).half()
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    scale = 0.09

    def cut(desc, b, n):
        return {key: (val[b:b + 1, :, :n] if isinstance(val, torch.Tensor) and val.ndim >= 3 else val)
                for key, val in desc.items()}

    for k in (k_dense, k_polar):
        got = tq.flash_decode(q, k=k, v=v, attn_scale=scale, out_dtype=torch.float32, seq_lens=sl)
        assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
        for b, n in enumerate(lens):
            one = tq.flash_decode(q[b:b + 1], k=cut(k, b, n), v=cut(v, b, n), attn_scale=scale, out_dtype=torch.float32)
            assert _rel(got[b].cpu().numpy(), one[0].cpu().numpy()) < 1e-5
    # in-launch append at each sequence's own end
    kd2, vp2, vn2 = kd.clone(), v["packed"].clone(), v["norms"].clone()
    new_k = torch.randn((B, n_kv, D), generator=g, device=dev).half()
    new_v = torch.randn((B, n_kv, D), generator=g, device=dev).half()
    v2 = dict(v, packed=vp2, norms=vn2)
    got = tq.flash_decode(q, k=dict(format="dense", data=kd2), v=v2, attn_scale=scale, out_dtype=torch.float32,
                          seq_lens=sl, new_k=new_k, new_v=new_v)
    rp, rn = tq.fused_quantize(new_v.reshape(-1, D), vq.signs, vq.boundaries, D, 3)
    for b, n in enumerate(lens):
        assert torch.equal(kd2[b, :, n - 1], new_k[b]) and torch.equal(vp2[b, :, n - 1], rp.reshape(B, n_kv, 13)[b])
        assert torch.equal(vn2[b, :, n - 1], rn.reshape(B, n_kv)[b])
        assert torch.equal(kd2[b, :, :n - 1], kd[b, :, :n - 1]) and torch.equal(kd2[b, :, n:], kd[b, :, n:])
        one = tq.flash_decode(q[b:b + 1], k=dict(format="dense", data=kd2[b:b + 1, :, :n]), v=cut(v2, b, n),
                              attn_scale=scale, out_dtype=torch.float32)
        assert _rel(got[b].cpu().numpy(), one[0].cpu().numpy()) < 1e-5
    # graph replay with a device-side length that grows by one per replay
    out = torch.zeros((B, n_kv * n_rep, D), dtype=torch.float32, device=dev)
    sl2 = torch.tensor([100, 200, 300], dtype=torch.int32, device=dev)

    def step():
        sl2.add_(1)
        tq.flash_decode(q, k=k_dense, v=v, attn_scale=scale, out=out, seq_lens=sl2)

    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    n_now = sl2.tolist()
    assert n_now == [104, 204, 304]           # one eager run (capture itself runs nothing) + three replays
    for b in range(B):
        one = tq.flash_decode(q[b:b + 1], k=cut(k_dense, b, n_now[b]), v=cut(v, b, n_now[b]), attn_scale=scale,
                              out_dtype=torch.float32)
        assert _rel(out[b].cpu().numpy(), one[0].cpu().numpy()) < 1e-5
    with pytest.raises(ValueError, match="seq_lens"):
        tq.flash_decode(q, k=k_dense, v=v, attn_scale=scale, seq_lens=sl, mask=torch.zeros((1, 1, S), device=dev))


@pytest.mark.parametrize("n_rep,T,S,kind", [(2, 4, 1531, "polar4"), (4, 2, 700, "dense"), (1, 8, 2300, "polar3"),
                                            (2, 3, 5000, "dense"), (7, 1, 300, "dense")])
def test_short_multi_token_step_is_causal_and_matches_oracle(tq, oracle, dev, n_rep, T, S, kind):
    """T query tokens per sequence (the last T stored positions) in one launch over the packed rows:
    token t must equal a single-token decode over the first S - T + 1 + t positions (the oracle's
    composed path), for dense and packed keys, with several splits and a ragged last tile.  The
    reference sends such steps to dense attention (patch.py:19-21)."""
    L = tq._lib.lib()
    rng = np.random.default_rng(77 + T)
    B, n_kv, D = 2, 2, 128
    scale = 1.0 / math.sqrt(D)
    vq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    vs = vq.signs.cpu().numpy()
    vraw = (rng.standard_normal((B, n_kv, S, D)) * rng.lognormal(0, 0.5, (B, n_kv, S, 1))).astype(np.float32)
    vp, vn = oracle.quantize_packed(vraw, vs, 3)
    n_alloc = (S + 255) // 256 * 256

    def alloc(x):   # rows live in a longer allocation, as in a cache
        full = np.zeros(x.shape[:2] + (n_alloc,) + x.shape[3:], x.dtype)
        full[:, :, :S] = x
        return _t(full, dev)[:, :, :S]

    v = dict(format="polar", packed=alloc(vp), norms=alloc(vn), centroids=vq.centroids, signs=vq.signs, bits=3)
    if kind == "dense":
        kd = rng.standard_normal((B, n_kv, S, D)).astype(np.float16)
        k = dict(format="dense", data=alloc(kd))
    else:
        kbits = int(kind[-1])
        kq = tq.PolarQuantizer(D, kbits, seed=42, device=dev)
        ks = kq.signs.cpu().numpy()
        kraw = rng.standard_normal((B, n_kv, S, D)).astype(np.float16)
        kp, kn = oracle.quantize_packed(kraw, ks, kbits)
        k = dict(format="polar", packed=alloc(kp), norms=alloc(kn), centroids=kq.centroids, signs=kq.signs, bits=kbits)
    q = rng.standard_normal((B, n_kv * n_rep, T, D)).astype(np.float16)
    for splits in (0, 3):
        out = tq.flash_decode(_t(q, dev) if T > 1 else _t(q, dev)[:, :, 0], k=k, v=v, attn_scale=scale,
                              out_dtype=torch.float32, num_splits=splits)
        assert L.tq_flash_decode_last_kernel() == 1
        out = out.cpu().numpy().reshape(B, n_kv * n_rep, T, D)
        for b in range(B):
            for t in range(T):
                n = S - T + 1 + t
                vdesc = dict(packed=vp[b, :, :n], norms=vn[b, :, :n], centroids=oracle.codebook(3), signs=vs, bits=3)
                if kind == "dense":
                    ref, _ = oracle.decode_attention(q[b, :, t], k_dense=kd[b, :, :n], v_polar=vdesc,
                                                     attn_scale=scale, n_rep=n_rep)
                else:
                    ref, _ = oracle.decode_attention(
                        q[b, :, t], k_polar=dict(packed=kp[b, :, :n], norms=kn[b, :, :n],
                                                 centroids=oracle.codebook(kbits), signs=ks, bits=kbits),
                        v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
                assert _rel(out[b, :, t], ref) < ATT_TOL, (b, t, splits)
    # the small-CTA geometry (launches that overlap their neighbours) takes the same rows
    ws = tq.kernels.decode_workspace(dev)
    out4 = tq.flash_decode(_t(q, dev) if T > 1 else _t(q, dev)[:, :, 0], k=k, v=v, attn_scale=scale,
                           out_dtype=torch.float32, kv_stable=True, q_stable=True, workspace=ws)
    assert L.tq_flash_decode_last_kernel() == 1 and tq.kernels.workspace_status(ws) == 0
    assert _rel(out4.cpu().numpy().reshape(out.shape), out) < 1e-3
    assert tq.kernels.flash_status(dev, B * n_kv) == 0
    if T > 1:
        # device-side lengths: sequence 1 is 5 positions shorter, its T queries are the last T of those
        lens = torch.tensor([S, S - 5], dtype=torch.int32, device=dev)
        outl = tq.flash_decode(_t(q, dev), k=k, v=v, attn_scale=scale, out_dtype=torch.float32,
                               seq_lens=lens).cpu().numpy()
        assert _rel(outl[0], out[0]) < 1e-3          # sequence 0 at full length: the result above
        for t in range(T):
            n = S - 5 - T + 1 + t
            vdesc = dict(packed=vp[1, :, :n], norms=vn[1, :, :n], centroids=oracle.codebook(3), signs=vs, bits=3)
            if kind == "dense":
                ref, _ = oracle.decode_attention(q[1, :, t], k_dense=kd[1, :, :n], v_polar=vdesc, attn_scale=scale,
                                                 n_rep=n_rep)
            else:
                ref, _ = oracle.decode_attention(
                    q[1, :, t], k_polar=dict(packed=kp[1, :, :n], norms=kn[1, :, :n],
                                             centroids=oracle.codebook(kbits), signs=ks, bits=kbits),
                    v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
            assert _rel(outl[1, :, t], ref) < ATT_TOL, t
        with pytest.raises(ValueError):      # rows beyond the MMA tile: refused, not silently wrong
            tq.flash_decode(_t(np.zeros((B, n_kv * n_rep, 9 // n_rep + 1, D), np.float16), dev), k=k, v=v,
                            attn_scale=scale)
