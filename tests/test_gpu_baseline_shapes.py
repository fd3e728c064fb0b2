"""GPU parity against the oracle at the exact shapes of the benchmark configurations
(same seeded input distributions as bench.py), each through the public route the
benchmark itself uses, with the decode kernel's choice and its status word checked:

  C1  PolarQuant 3-bit encode + decode of [1, 4, 4096, 128] fp16
  C2  V-only decode, 28 q / 4 kv heads, ctx 32768, through VOnlyTurboQuantCache + the hooked SDPA
  C3  full TurboQuant cache (K 4-bit, V 3-bit), B = 32, 32 q / 8 kv heads, ctx 8192
  C5  per-GPU shard: 64 q / 8 kv heads, 131072 positions, K 8-bit affine + V 3-bit, two chunks merged
  and, at the C2 size, bf16 dense keys (tensor-core kernel) and a padding mask (general kernel).

Tolerances (reference tests/test_flash_attention.py:38-137, test_core.py:70-109 and the
stated targets): packed words bit-exact, norms <= 1e-6 relative, attention <= 2e-3 max
relative error."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ATT_TOL = 2e-3
D = 128


def _rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def _lognormal_vectors(rng, shape):
    return (rng.standard_normal(shape + (D,)) * rng.lognormal(0.0, 0.5, shape + (1,))).astype(np.float16)


def _oracle_dense_k(oracle, q, kd, vdesc, scale, n_rep, mask=None):
    """The oracle's composed decode attention (fused_attention.py:56-121) for dense keys, evaluated
    per kv head so that the float64 temporaries stay small at long context."""
    outs = []
    for h in range(kd.shape[0]):
        sub = dict(vdesc, packed=vdesc["packed"][h:h + 1], norms=vdesc["norms"][h:h + 1])
        m = None if mask is None else mask[h * n_rep:(h + 1) * n_rep]
        o, _ = oracle.decode_attention(q[h * n_rep:(h + 1) * n_rep], k_dense=kd[h:h + 1], v_polar=sub,
                                       attn_scale=scale, n_rep=n_rep, mask=m)
        outs.append(o)
    return np.concatenate(outs, 0)


def test_c1_exact_shape_bit_exact(tq, oracle, dev):
    rng = np.random.default_rng(101)
    x = _lognormal_vectors(rng, (1, 4, 4096))
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    signs = pq.signs.cpu().numpy()
    xd = torch.from_numpy(x).to(dev)
    packed, norms = tq.fused_quantize(xd.reshape(-1, D), pq.signs, pq.boundaries, D, 3)
    ref_p, ref_n = oracle.quantize_packed(x.reshape(-1, D), signs, 3)
    got_p, got_n = packed.cpu().numpy(), norms.cpu().numpy()
    differing_words = int((got_p != ref_p).sum())
    got_idx = oracle.unpack_indices(got_p, 3, D)
    ref_idx = oracle.unpack_indices(ref_p, 3, D)
    mism = got_idx != ref_idx
    # classify mismatches: a tie is a coordinate whose scaled value is within 2 ulps of a boundary
    z = oracle.quantize_scaled(x.reshape(-1, D), signs)[0] if mism.any() else None
    ties = int((oracle.tie_distance_ulps(z, 3)[mism] <= 2).sum()) if mism.any() else 0
    print(f"C1: {got_idx.size} indices, {int(mism.sum())} mismatches ({ties} ties, {int(mism.sum()) - ties} non-ties), "
          f"{differing_words} differing words")
    assert int(mism.sum()) - ties == 0
    assert differing_words == 0            # same norm reduction order as the oracle: not even ties differ
    assert np.array_equal(got_n, ref_n)
    assert np.abs(got_n - np.linalg.norm(x.reshape(-1, D).astype(np.float32), axis=-1)).max() <= 1e-6 * got_n.max()
    # decode back to fp16 (the round trip config 1 names): float32 result bit-exact, fp16 = its rounding
    deq32 = tq.packed_dequantize(packed, norms, pq.centroids, pq.signs, D, 3).cpu().numpy()
    ref32 = oracle.packed_dequantize(ref_p, ref_n, oracle.codebook(3), signs, D, 3)
    assert np.array_equal(deq32, ref32)
    deq16 = tq.dequant_fp16(packed, norms, pq.centroids, pq.signs, D, 3).cpu().numpy()
    assert np.array_equal(deq16, ref32.astype(np.float16))
    # the same through the cache (insert -> state): the stored words are the oracle's
    cache = tq.TurboQuantKVCache(bits=3, seed=42, fused=True)
    cache.update_and_fetch(xd, xd)
    vp = cache.v_packed[:, :, :4096, :].cpu().numpy().reshape(-1, 13)
    assert np.array_equal(vp, oracle.quantize_packed(x.reshape(-1, D), cache._v_q.signs.cpu().numpy(), 3)[0])


@pytest.mark.parametrize("deferred", [True, False])
def test_c2_exact_shape_through_cache_and_hook(tq, oracle, dev, deferred):
    """28 q / 4 kv heads, ctx 32768: 32767 prompt tokens inserted through the cache, the last
    token through a one-token update_and_fetch followed by the hooked SDPA (with `deferred` the
    decode launch itself appends it), compared with the oracle on all 32768 positions."""
    from turboquant_mlx_b200 import base
    from turboquant_mlx_b200.kernels import flash_status
    rng = np.random.default_rng(202)
    n_q, n_kv, S = 28, 4, 32768
    n_rep = n_q // n_kv
    k_all = rng.standard_normal((1, n_kv, S, D)).astype(np.float16)
    v_all = _lognormal_vectors(rng, (1, n_kv, S))
    q = (rng.standard_normal((1, n_q, 1, D))).astype(np.float16)
    scale = 1.0 / math.sqrt(D)
    cache = tq.VOnlyTurboQuantCache(bits=3, seed=42, fused=True, defer_append=deferred, inputs_stable=deferred)
    cache.reserve(1, n_kv, S + 256, D, D, torch.float16, dev)
    kd, vd = torch.from_numpy(k_all).to(dev), torch.from_numpy(v_all).to(dev)
    cache.update_and_fetch(kd[:, :, :S - 1], vd[:, :, :S - 1])
    tq.apply_patch()
    try:
        keys, values = cache.update_and_fetch(kd[:, :, S - 1:], vd[:, :, S - 1:])
        assert (cache._pending is not None) == deferred
        out = base.scaled_dot_product_attention(torch.from_numpy(q).to(dev), keys, values, cache, scale, None)
    finally:
        tq.remove_patch()
    torch.cuda.synchronize()
    assert cache._pending is None and cache.offset == S
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
    assert flash_status(dev, n_kv) == 0
    assert cache._decode_ws is None or tq.kernels.workspace_status(cache._decode_ws) == 0
    signs = cache._v_tq._v_q.signs.cpu().numpy()
    ref_p, ref_n = oracle.quantize_packed(v_all[0], signs, 3)
    # the stored rows (including the one appended by the decode launch) are the oracle's, bit for bit
    assert np.array_equal(cache._v_tq.v_packed[0, :, :S].cpu().numpy(), ref_p)
    assert np.array_equal(cache._v_tq.v_norms[0, :, :S].cpu().numpy(), ref_n)
    assert np.array_equal(cache._k_cache.keys[0, :, :S].cpu().numpy(), k_all[0])
    vdesc = dict(packed=ref_p, norms=ref_n, centroids=oracle.codebook(3), signs=signs, bits=3)
    ref = _oracle_dense_k(oracle, q[0, :, 0], k_all[0], vdesc, scale, n_rep)
    err = _rel(out[0, :, 0].float().cpu().numpy(), ref)
    print(f"C2 (deferred append: {deferred}): max rel err vs oracle {err:.2e}")
    assert err < ATT_TOL


@pytest.mark.parametrize("own_workspaces", [False, True])
def test_c2_pipelined_launches_match_serial(tq, dev, own_workspaces):
    """Six layers of the C2 shape replayed from one CUDA graph with kv_stable and q_stable: the
    launches overlap, sharing one workspace (each waits for its predecessor before writing it) or
    with a workspace each (nothing waits); every layer's output equals its stand-alone result."""
    from turboquant_mlx_b200.kernels import flash_status
    g = torch.Generator(device=dev).manual_seed(7)
    n_q, n_kv, S, layers = 28, 4, 32768, 6
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    ks, vs, qs = [], [], []
    for _ in range(layers):
        ks.append(dict(format="dense", data=torch.randn((1, n_kv, S, D), generator=g, device=dev).half()))
        vp = torch.randint(0, 2 ** 30, (1, n_kv, S, 13), generator=g, device=dev, dtype=torch.int64)
        vp[..., 12] &= 0x00FFFFFF
        vs.append(dict(format="polar", packed=vp.to(torch.uint32), centroids=pq.centroids, signs=pq.signs, bits=3,
                       norms=torch.exp(0.5 * torch.randn((1, n_kv, S), generator=g, device=dev)) * 11.3))
        qs.append(torch.randn((1, n_q, D), generator=g, device=dev).half())
    scale = 1.0 / math.sqrt(D)
    wss = [tq.kernels.decode_workspace(dev) if own_workspaces else None for _ in range(layers)]
    # the same launches (same flags, hence the same split plan) one at a time
    serial = []
    for l in range(layers):
        serial.append(tq.flash_decode(qs[l], k=ks[l], v=vs[l], attn_scale=scale, out_dtype=torch.float32,
                                      kv_stable=True, q_stable=True, workspace=wss[l]))
        torch.cuda.synchronize()
    alone = tq.flash_decode(qs[0], k=ks[0], v=vs[0], attn_scale=scale, out_dtype=torch.float32)
    assert _rel(alone.cpu().numpy(), serial[0].cpu().numpy()) < 1e-3     # another split plan: equal to fp16 rounding of P
    outs = [torch.zeros_like(o) for o in serial]

    def step():
        for l in range(layers):
            tq.flash_decode(qs[l], k=ks[l], v=vs[l], attn_scale=scale, kv_stable=True, q_stable=True, out=outs[l],
                            workspace=wss[l])

    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(5):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for l in range(layers):
            assert torch.equal(outs[l], serial[l])       # overlapping launches change nothing, bit for bit
    assert flash_status(dev, n_kv) == 0
    assert all(w is None or tq.kernels.workspace_status(w) == 0 for w in wss)


@pytest.mark.parametrize("deferred", [False, True])
def test_c3_exact_shape_batch32(tq, oracle, dev, deferred):
    """B = 32, 32 q / 8 kv heads, ctx 8192, K 4-bit + V 3-bit through TurboQuantKVCache and
    turboquant_attention: the oracle on batch elements 0, 19, 20 and 31 (first, two in the second
    wave of (batch, kv head) groups, last), the composed GPU route on all 32."""
    from turboquant_mlx_b200.kernels import flash_status
    B, n_q, n_kv, S = 32, 32, 8, 8192
    n_rep = n_q // n_kv
    g = torch.Generator(device=dev).manual_seed(303)
    cache = tq.TurboQuantKVCache(bits=3, k_bits=4, v_bits=3, fused=True, defer_append=deferred, inputs_stable=deferred)
    cache.reserve(B, n_kv, S + 256, D, D, dev)
    checked = (0, 19, 20, 31)
    kept = {}
    for s0 in range(0, S, 2048):
        n = min(2048, S - s0) - (1 if s0 + 2048 >= S else 0)     # the last token goes in separately
        k = (torch.randn((B, n_kv, n, D), generator=g, device=dev) *
             torch.exp(0.5 * torch.randn((B, n_kv, n, 1), generator=g, device=dev))).half()
        v = (torch.randn((B, n_kv, n, D), generator=g, device=dev) *
             torch.exp(0.5 * torch.randn((B, n_kv, n, 1), generator=g, device=dev))).half()
        cache.update_and_fetch(k, v)
        for b in checked:
            kept.setdefault(b, []).append((k[b].cpu().numpy(), v[b].cpu().numpy()))
    k1 = torch.randn((B, n_kv, 1, D), generator=g, device=dev).half()
    v1 = torch.randn((B, n_kv, 1, D), generator=g, device=dev).half()
    q = torch.randn((B, n_q, 1, D), generator=g, device=dev).half()
    cache.update_and_fetch(k1, v1)
    assert (cache._pending is not None) == deferred
    scale = 1.0 / math.sqrt(D)
    out = tq.turboquant_attention(q, cache, scale)
    torch.cuda.synchronize()
    assert cache.offset == S and cache._pending is None
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
    assert flash_status(dev, B * n_kv) == 0
    assert cache._decode_ws is None or tq.kernels.workspace_status(cache._decode_ws) == 0
    ks, vs = cache._k_q.signs.cpu().numpy(), cache._v_q.signs.cpu().numpy()
    for b in checked:
        kb = np.concatenate([a for a, _ in kept[b]] + [k1[b].cpu().numpy()], axis=1)
        vb = np.concatenate([a for _, a in kept[b]] + [v1[b].cpu().numpy()], axis=1)
        kp, kn = oracle.quantize_packed(kb, ks, 4)
        vp, vn = oracle.quantize_packed(vb, vs, 3)
        assert np.array_equal(cache.k_packed[b, :, :S].cpu().numpy(), kp)      # stored words = the oracle's
        assert np.array_equal(cache.v_packed[b, :, :S].cpu().numpy(), vp)
        assert np.array_equal(cache.k_norms[b, :, :S].cpu().numpy(), kn)
        assert np.array_equal(cache.v_norms[b, :, :S].cpu().numpy(), vn)
        ref, _ = oracle.decode_attention(
            q[b, :, 0].cpu().numpy(), k_polar=dict(packed=kp, norms=kn, centroids=oracle.codebook(4), signs=ks, bits=4),
            v_polar=dict(packed=vp, norms=vn, centroids=oracle.codebook(3), signs=vs, bits=3),
            attn_scale=scale, n_rep=n_rep)
        err = _rel(out[b, :, 0].float().cpu().numpy(), ref)
        print(f"C3 batch element {b}: max rel err vs oracle {err:.2e}")
        assert err < ATT_TOL
    # every batch element against the composed GPU route (scores -> softmax -> packed-V sum)
    worst = 0.0
    for b in range(B):
        q_rot = tq.prerotate_query(q[b, :, 0], cache._k_q.signs)
        sc = tq.prerot_fused_qk_scores(q_rot, cache.k_packed[b, :, :S], cache.k_norms[b, :, :S],
                                       cache._k_q.centroids, D, 4, n_rep=n_rep)
        w = torch.softmax(sc * scale, dim=-1)
        comp = tq.sparse_v_matvec(w, cache.v_packed[b, :, :S], cache.v_norms[b, :, :S], cache._v_q.centroids,
                                  cache._v_q.signs, D, 3, threshold=0.0, n_rep=n_rep)
        worst = max(worst, _rel(out[b, :, 0].float().cpu().numpy(), comp.cpu().numpy()))
    print(f"C3: worst max rel err vs composed GPU route over 32 batch elements {worst:.2e}")
    assert worst < ATT_TOL


def test_c5_per_gpu_shape_two_chunks_merged(tq, oracle, dev):
    """64 q / 8 kv heads, two chunks of 131072 positions (K 8-bit affine group 64, V 3-bit) decoded in
    partial mode and merged, against the oracle on kv heads 0 and 7 (16 of the 64 rows)."""
    from turboquant_mlx_b200.kernels import flash_status
    n_q, n_kv, S = 64, 8, 131072
    n_rep = n_q // n_kv
    g = torch.Generator(device=dev).manual_seed(505)
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    signs = pq.signs.cpu().numpy()
    q = torch.randn((1, n_q, D), generator=g, device=dev).half()
    scale = 1.0 / math.sqrt(D)
    chunks, parts = [], []
    for _ in range(2):
        kraw = torch.randn((1, n_kv, S, D), generator=g, device=dev).half()
        codes, scales, biases = tq.affine.affine_quantize(kraw, group=64, bits=8)
        vraw = (torch.randn((n_kv, S, D), generator=g, device=dev) *
                torch.exp(0.5 * torch.randn((n_kv, S, 1), generator=g, device=dev))).half()
        vp, vn = tq.fused_quantize(vraw.reshape(-1, D), pq.signs, pq.boundaries, D, 3)
        k = dict(format="affine", codes=codes, scales=scales, biases=biases, bits=8, group=64)
        v = dict(format="polar", packed=vp.reshape(1, n_kv, S, 13), norms=vn.reshape(1, n_kv, S),
                 centroids=pq.centroids, signs=pq.signs, bits=3)
        parts.append(tq.flash_decode(q, k=k, v=v, attn_scale=scale, partials=True))
        assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
        chunks.append((codes, scales, biases, vp.reshape(n_kv, S, 13), vn.reshape(n_kv, S)))
        del kraw, vraw
    m = torch.stack([p[0][0] for p in parts])
    l = torch.stack([p[1][0] for p in parts])
    acc = torch.stack([p[2][0] for p in parts])
    out = tq.merge_partials(m, l, acc, pq.signs, torch.float32).cpu().numpy()
    assert flash_status(dev, n_kv) == 0
    qn = q[0].cpu().numpy()
    for h in (0, 7):
        rows = slice(h * n_rep, (h + 1) * n_rep)
        kd = np.concatenate([oracle.affine_dequantize(c[0][0, h].cpu().numpy(), c[1][0, h].cpu().numpy(),
                                                      c[2][0, h].cpu().numpy(), 64, 8) for c in chunks], axis=0)
        vdesc = dict(packed=np.concatenate([c[3][h].cpu().numpy() for c in chunks], 0)[None],
                     norms=np.concatenate([c[4][h].cpu().numpy() for c in chunks], 0)[None],
                     centroids=oracle.codebook(3), signs=signs, bits=3)
        ref, _ = oracle.decode_attention(qn[rows], k_dense=kd[None], v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
        err = _rel(out[rows], ref)
        print(f"C5 kv head {h}: max rel err vs oracle {err:.2e}")
        assert err < ATT_TOL


@pytest.mark.parametrize("case", ["bf16_keys", "padding_mask"])
def test_c2_size_bf16_keys_and_padding_mask(tq, oracle, dev, case):
    """At the C2 size: bf16 dense keys (a bf16 model with the V-only cache) run on the tensor-core
    kernel through the bf16 MMA; an additive padding mask takes the general float32 kernel."""
    rng = np.random.default_rng(606)
    n_q, n_kv, S = 28, 4, 32768
    n_rep = n_q // n_kv
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    signs = pq.signs.cpu().numpy()
    kt = torch.from_numpy(rng.standard_normal((n_kv, S, D)).astype(np.float32))
    kt = kt.to(torch.bfloat16) if case == "bf16_keys" else kt.to(torch.float16)
    v_all = _lognormal_vectors(rng, (n_kv, S))
    vp, vn = oracle.quantize_packed(v_all, signs, 3)
    q = rng.standard_normal((n_q, D)).astype(np.float16)
    mask = None
    if case == "padding_mask":
        mask = np.zeros((1, 1, S), np.float32)
        mask[..., 30000:] = -np.inf
    scale = 1.0 / math.sqrt(D)
    k = dict(format="dense", data=kt.to(dev).unsqueeze(0))
    v = dict(format="polar", packed=torch.from_numpy(vp).to(dev).unsqueeze(0), norms=torch.from_numpy(vn).to(dev).unsqueeze(0),
             centroids=pq.centroids, signs=pq.signs, bits=3)
    out = tq.flash_decode(torch.from_numpy(q).to(dev).unsqueeze(0), k=k, v=v, attn_scale=scale, out_dtype=torch.float32,
                          mask=None if mask is None else torch.from_numpy(mask).to(dev))
    torch.cuda.synchronize()
    assert tq._lib.lib().tq_flash_decode_last_kernel() == (1 if case == "bf16_keys" else 0)
    vdesc = dict(packed=vp, norms=vn, centroids=oracle.codebook(3), signs=signs, bits=3)
    m2 = None if mask is None else np.broadcast_to(mask[0], (n_q, S))
    ref = _oracle_dense_k(oracle, q, kt.float().numpy(), vdesc, scale, n_rep, mask=m2)
    err = _rel(out[0].cpu().numpy(), ref)
    print(f"C2 size, {case}: max rel err vs oracle {err:.2e}")
    assert err < ATT_TOL


def test_in_launch_append_refused_outside_the_tensor_core_path(tq, dev):
    """new_k / new_v with a mask (general kernel) is refused, nothing is launched."""
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    S = 512
    k = dict(format="dense", data=torch.zeros((1, 2, S, D), dtype=torch.float16, device=dev))
    v = dict(format="polar", packed=torch.zeros((1, 2, S, 13), dtype=torch.uint32, device=dev),
             norms=torch.ones((1, 2, S), device=dev), centroids=pq.centroids, signs=pq.signs, bits=3,
             boundaries=pq.boundaries)
    q = torch.zeros((1, 4, D), dtype=torch.float16, device=dev)
    rows = torch.zeros((1, 2, D), dtype=torch.float16, device=dev)
    with pytest.raises(ValueError, match="in-launch append"):
        tq.flash_decode(q, k=k, v=v, attn_scale=1.0, mask=torch.zeros((1, 1, S), device=dev), new_k=rows, new_v=rows)
    with pytest.raises(ValueError, match="together"):
        tq.flash_decode(q, k=k, v=v, attn_scale=1.0, new_k=rows)
