"""GPU tests of the cache classes and the attention hook: re-expression of the
reference's tests/test_core.py (cache part), test_fused_attn.py and
test_v_only_cache.py on CUDA tensors."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().reshape(-1, a.shape[-1]),
                                                 b.float().reshape(-1, b.shape[-1]), dim=-1).mean().item()


def test_cache_shapes_offsets_and_quality(tq, dev):
    torch.manual_seed(0)
    c = tq.TurboQuantKVCache(bits=3)
    k = torch.randn(1, 4, 1, 128, device=dev, dtype=torch.float16)
    ko, vo = c.update_and_fetch(k, k)
    assert ko.shape == (1, 4, 1, 128) and c.offset == 1 and not c.empty()
    assert c.k_packed.dtype == torch.uint32 and c.k_packed.shape == (1, 4, 256, 13)
    k64 = torch.randn(1, 4, 64, 128, device=dev, dtype=torch.float16)
    v64 = torch.randn(1, 4, 64, 128, device=dev, dtype=torch.float16)
    ko, vo = c.update_and_fetch(k64, v64)
    assert ko.shape == (1, 4, 65, 128) and vo.dtype == torch.float16 and c.offset == 65
    assert _cos(ko[:, :, 1:], k64) > 0.7 and _cos(vo[:, :, 1:], v64) > 0.7
    assert c.compression_ratio > 1.5 and c.nbytes == 2 * 4 * 65 * 56
    for _ in range(3):   # incremental decode path (S <= 4)
        k1 = torch.randn(1, 4, 1, 128, device=dev, dtype=torch.float16)
        ko2, vo2 = c.update_and_fetch(k1, k1)
    assert ko2.shape[2] == 68 and torch.equal(ko2[:, :, :65], ko)
    assert _cos(ko2[:, :, -1:], k1) > 0.7
    assert c.trim(8) == 8 and c.offset == 60 and c.size() == 60


def test_cache_insert_matches_oracle_and_grows(tq, oracle, dev):
    rng = np.random.default_rng(1)
    c = tq.TurboQuantKVCache(bits=3, seed=42, fused=True, k_bits=4, v_bits=3)
    ks, vs = oracle.signs_from_seed(128, 42), oracle.signs_from_seed(128, 43)
    chunks, all_k, all_v = [200, 1, 1, 3, 300, 1], [], []
    for S in chunks:
        k = rng.standard_normal((2, 3, S, 128)).astype(np.float16)
        v = rng.standard_normal((2, 3, S, 128)).astype(np.float16)
        zk, zv = c.update_and_fetch(torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev))
        assert zk.shape == (2, 3, c.offset, 128) and float(zk.abs().max()) == 0.0
        all_k.append(k); all_v.append(v)
    K, V = np.concatenate(all_k, 2), np.concatenate(all_v, 2)
    total = sum(chunks)
    assert c.offset == total and c.k_packed.shape[2] % 256 == 0 and c.k_packed.shape[3] == 16
    kp, kn = oracle.quantize_packed(K, ks, 4)
    vp, vn = oracle.quantize_packed(V, vs, 3)
    assert np.array_equal(c.k_packed[:, :, :total].cpu().numpy(), kp)
    assert np.array_equal(c.v_packed[:, :, :total].cpu().numpy(), vp)
    assert np.array_equal(c.k_norms[:, :, :total].cpu().numpy(), kn)
    assert np.array_equal(c.v_norms[:, :, :total].cpu().numpy(), vn)


def test_state_round_trip_and_extend(tq, dev):
    torch.manual_seed(2)
    c = tq.TurboQuantKVCache(bits=3, seed=42)
    k = torch.randn(1, 4, 10, 128, device=dev, dtype=torch.float16)
    c.update_and_fetch(k, k)
    st, meta = c.state, c.meta_state
    assert len(st) == 4 and meta == "10,3,42,128,128,float16"
    assert len(c.state_with_signs) == 6
    r = tq.TurboQuantKVCache.from_state(st, meta)
    assert r.offset == 10 and torch.equal(r.k_packed.view(torch.int32), st[0].view(torch.int32))
    k2 = torch.randn(1, 4, 2, 128, device=dev, dtype=torch.float16)
    ko, vo = r.update_and_fetch(k2, k2)
    assert r.offset == 12 and ko.shape == (1, 4, 12, 128)
    assert torch.equal(r.k_packed[:, :, :10].view(torch.int32), st[0].view(torch.int32))


def test_state_with_signs_on_disk_round_trip(tq, oracle, dev, tmp_path):
    """A cache written with sign vectors that this library's generator would NOT derive from the seed
    (the situation of a file saved by the reference: its signs come from another PRNG) goes to disk as
    safetensors, comes back through `from_state`, decodes with the saved signs and can be extended
    (tests/test_v_only_cache.py:98-134 of the reference, plus the sign vectors)."""
    from safetensors.torch import load_file, save_file
    torch.manual_seed(21)
    B, n_kv, S = 1, 2, 40
    k = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    v = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    g = torch.Generator().manual_seed(77)
    foreign_k = (torch.randint(0, 2, (128,), generator=g) * 2 - 1).float()
    foreign_v = (torch.randint(0, 2, (128,), generator=g) * 2 - 1).float()
    # the writer: packed rows produced with the foreign signs (oracle arithmetic), as the other library would
    kp, kn = oracle.quantize_packed(k.cpu().numpy(), foreign_k.numpy(), 3)
    vp, vn = oracle.quantize_packed(v.cpu().numpy(), foreign_v.numpy(), 3)
    arrays = [torch.from_numpy(kp.view(np.int32)), torch.from_numpy(kn), torch.from_numpy(vp.view(np.int32)),
              torch.from_numpy(vn), foreign_k, foreign_v]
    path = str(tmp_path / "cache.safetensors")
    save_file({f"a{i}": t.contiguous() for i, t in enumerate(arrays)}, path,
              metadata={"meta_state": f"{S},3,42,128,128,float16"})
    loaded = load_file(path, device=str(dev))
    from safetensors import safe_open
    with safe_open(path, framework="pt") as f:
        meta = f.metadata()["meta_state"]
    state = [loaded[f"a{i}"] for i in range(6)]
    state[0], state[2] = state[0].view(torch.uint32), state[2].view(torch.uint32)
    r = tq.TurboQuantKVCache.from_state(state, meta)
    assert r.offset == S and not r.signs_match_seed()
    kd, vd = r.dequantized(dtype=torch.float32)
    want_k = oracle.packed_dequantize(kp, kn, oracle.codebook(3), foreign_k.numpy(), 128, 3)
    want_v = oracle.packed_dequantize(vp, vn, oracle.codebook(3), foreign_v.numpy(), 128, 3)
    assert np.array_equal(kd.cpu().numpy(), want_k) and np.array_equal(vd.cpu().numpy(), want_v)
    # the loaded cache keeps quantizing with the saved signs
    k2 = torch.randn(B, n_kv, 3, 128, device=dev, dtype=torch.float16)
    ko, vo = r.update_and_fetch(k2, k2)
    assert r.offset == S + 3 and ko.shape == (B, n_kv, S + 3, 128)
    kp2, kn2 = oracle.quantize_packed(k2.cpu().numpy(), foreign_k.numpy(), 3)
    assert np.array_equal(r.k_packed[:, :, S:S + 3].cpu().numpy().view(np.uint32), kp2)
    # its own state with signs survives a second trip through a file unchanged
    st2 = r.state_with_signs
    save_file({f"a{i}": (t.view(torch.int32) if t.dtype == torch.uint32 else t).contiguous().cpu()
               for i, t in enumerate(st2)}, path, metadata={"meta_state": r.meta_state})
    again = load_file(path, device=str(dev))
    st3 = [again[f"a{i}"] for i in range(6)]
    st3[0], st3[2] = st3[0].view(torch.uint32), st3[2].view(torch.uint32)
    r2 = tq.TurboQuantKVCache.from_state(st3, r.meta_state)
    assert r2.offset == S + 3 and torch.equal(r2.k_packed.view(torch.int32), r.k_packed[:, :, :S + 3].view(torch.int32))
    assert torch.equal(r2._v_q.signs.cpu(), foreign_v)


def _filled_cache(tq, dev, B, n_kv, S, fused=True, **kw):
    torch.manual_seed(3)
    c = tq.TurboQuantKVCache(bits=3, fused=fused, **kw)
    k = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    v = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    c.update_and_fetch(k, v)
    return c


@pytest.mark.parametrize("S,thr,B,n_rep", [(128, None, 1, 1), (512, 1e-5, 2, 4), (300, 0.0, 3, 7)])
def test_turboquant_attention_vs_dense_sdpa(tq, dev, S, thr, B, n_rep):
    n_kv = 4
    c = _filled_cache(tq, dev, B, n_kv, S)
    q = torch.randn(B, n_kv * n_rep, 1, 128, device=dev, dtype=torch.float16)
    scale = 1.0 / math.sqrt(128)
    out = tq.turboquant_attention(q, c, scale, sparse_v_threshold=thr)
    assert out.shape == q.shape and out.dtype == q.dtype
    kd, vd = c.dequantized(torch.float32)
    kd = kd.repeat_interleave(n_rep, 1); vd = vd.repeat_interleave(n_rep, 1)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), kd, vd, scale=scale)
    assert _cos(out, ref) > 0.999
    if thr is None or thr == 0.0:
        rel = (out.float() - ref).abs().max() / ref.abs().max()
        assert rel < 3e-3   # fp16 output rounding included
    # scores on cached K equal sum(dequant(K) * q)
    q_rot = tq.prerotate_query(q[0, :, 0, :], c._k_q.signs)
    sc = tq.prerot_fused_qk_scores(q_rot, c.k_packed[0, :, :S], c.k_norms[0, :, :S], c._k_q.centroids,
                                   128, c.quant_bits, n_rep=n_rep)
    ref_sc = torch.einsum("hpe,he->hp", kd[0], q[0, :, 0, :].float())
    assert ((sc - ref_sc).abs().max() / ref_sc.abs().max()) < 1e-3


def test_turboquant_attention_mask_and_v_buffer(tq, dev):
    B, n_kv, n_rep, S = 2, 2, 2, 200
    c = _filled_cache(tq, dev, B, n_kv, S)
    q = torch.randn(B, n_kv * n_rep, 1, 128, device=dev, dtype=torch.float16)
    scale = 1.0 / math.sqrt(128)
    mask = torch.zeros(B, 1, 1, S, device=dev)
    mask[0, :, :, 150:] = float("-inf")
    out = tq.turboquant_attention(q, c, scale, mask=mask)
    kd, vd = c.dequantized(torch.float32)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.float(), kd.repeat_interleave(n_rep, 1), vd.repeat_interleave(n_rep, 1), attn_mask=mask, scale=scale)
    assert ((out.float() - ref).abs().max() / ref.abs().max()) < 3e-3
    out_thr = tq.turboquant_attention(q, c, scale, mask=mask, sparse_v_threshold=1e-6)
    assert _cos(out_thr, ref) > 0.999
    out_vb = tq.turboquant_attention(q, c, scale, mask=mask, v_buffer=vd.half())
    assert _cos(out_vb, ref) > 0.999


def test_patched_sdpa_routes_fused_decode_and_prefill(tq, dev):
    from turboquant_mlx_b200 import base
    tq.apply_patch()
    try:
        B, n_kv, n_rep = 1, 2, 2
        c = tq.TurboQuantKVCache(bits=4, fused=True)
        k = torch.randn(B, n_kv, 40, 128, device=dev, dtype=torch.float16)
        q = torch.randn(B, n_kv * n_rep, 40, 128, device=dev, dtype=torch.float16)
        zk, zv = c.update_and_fetch(k, k)
        scale = 1.0 / math.sqrt(128)
        out = base.scaled_dot_product_attention(q, zk, zv, c, scale, "causal")   # prefill on fused cache
        kd, vd = c.dequantized(torch.float16)
        ref = base._dense_sdpa(q, kd, vd, scale, "causal")
        assert torch.allclose(out, ref, atol=1e-3, rtol=1e-2) and float(out.abs().max()) > 0
        q1 = torch.randn(B, n_kv * n_rep, 1, 128, device=dev, dtype=torch.float16)
        zk, zv = c.update_and_fetch(k[:, :, :1], k[:, :, :1])
        out1 = base.scaled_dot_product_attention(q1, zk, zv, c, scale, None)
        kd, vd = c.dequantized(torch.float32)
        ref1 = base._dense_sdpa(q1.float(), kd, vd, scale, None)
        assert ((out1.float() - ref1).abs().max() / ref1.abs().max()) < 3e-3
    finally:
        tq.remove_patch()


def test_v_only_cache(tq, dev):
    torch.manual_seed(4)
    for kwargs in ({}, {"no_v_buffer": True}):
        c = tq.VOnlyTurboQuantCache(bits=3, **kwargs)
        assert c.empty() and c.offset == 0
        k = torch.randn(1, 4, 10, 128, device=dev, dtype=torch.float16)
        v = torch.randn(1, 4, 10, 128, device=dev, dtype=torch.float16)
        ko, vo = c.update_and_fetch(k, v)
        assert _cos(ko, k) > 0.999 and _cos(vo, v) > 0.95 and c.offset == 10 and not c.empty()
        ko, vo = c.update_and_fetch(k[:, :, :1], v[:, :, :1])
        assert ko.shape == (1, 4, 11, 128) and vo.shape == (1, 4, 11, 128) and _cos(vo[:, :, :10], v) > 0.95
        assert len(c.state) >= 4 and c.meta_state.startswith("VOnlyTQ,3,")
        assert c.trim(1) == 1 and c.size() == 10
    c = tq.VOnlyTurboQuantCache(bits=3)
    c.update_and_fetch(k, v)
    r = tq.VOnlyTurboQuantCache.from_state(c.state, c.meta_state)
    assert r.offset == 10 and torch.equal(r._v_tq.v_packed.view(torch.int32), c.state[2].view(torch.int32))
    ko, vo = r.update_and_fetch(k[:, :, :2], v[:, :, :2])
    assert r.offset == 12 and vo.shape == (1, 4, 12, 128)


def test_v_only_fused_decode_attention(tq, dev):
    from turboquant_mlx_b200 import base
    torch.manual_seed(5)
    B, n_kv, n_rep, S = 2, 4, 7, 700
    c = tq.VOnlyTurboQuantCache(bits=3, fused=True)
    k = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    v = torch.randn(B, n_kv, S, 128, device=dev, dtype=torch.float16)
    ko, _ = c.update_and_fetch(k, v)
    q = torch.randn(B, n_kv * n_rep, 1, 128, device=dev, dtype=torch.float16)
    scale = 1.0 / math.sqrt(128)
    tq.apply_patch()
    try:
        out = base.scaled_dot_product_attention(q, ko, None, c, scale, None)
    finally:
        tq.remove_patch()
    _, vd = c._v_tq.dequantized(torch.float32)
    ref = base._dense_sdpa(q.float(), k.float(), vd, scale, None)
    assert ((out.float() - ref).abs().max() / ref.abs().max()) < 3e-3


def test_adaptive_cache_layout(tq):
    from turboquant_mlx_b200.base import KVCache
    caches = tq.make_adaptive_cache(12, bits=3, fp16_layers=2)
    assert len(caches) == 12
    assert all(isinstance(c, KVCache) for c in caches[:2] + caches[-2:])
    assert all(isinstance(c, tq.TurboQuantKVCache) for c in caches[2:-2])


def test_mixed_cache_single_step_append_matches_bulk(tq, dev):
    """One-token appends go straight into the storage rows (strided quantize); the stored codes,
    scales and biases must equal those of a bulk append of the same rows."""
    g = torch.Generator(device=dev).manual_seed(4)
    B, H, D = 2, 3, 128
    k = torch.randn((B, H, 7, D), generator=g, device=dev).half()
    v = (torch.randn((B, H, 7, D), generator=g, device=dev) * 2 + 1).half()
    bulk = tq.MixedQuantKVCache(8, 4, 64)
    bulk.update_and_fetch(k, v)
    step = tq.MixedQuantKVCache(8, 4, 64)
    step.update_and_fetch(k[:, :, :3], v[:, :, :3])
    for i in range(3, 7):
        # the layout a model produces: (B, 1, H, D) transposed to (B, H, 1, D)
        ki = k[:, :, i:i + 1].transpose(1, 2).contiguous().transpose(1, 2)
        vi = v[:, :, i:i + 1].transpose(1, 2).contiguous().transpose(1, 2)
        zk, zv = step.update_and_fetch(ki, vi)
        assert zk.shape == (B, H, i + 1, D) and zv.shape == (B, H, i + 1, D)
    assert step.offset == bulk.offset == 7
    for name in ("k_codes", "k_scales", "k_biases", "v_codes", "v_scales", "v_biases"):
        assert torch.equal(getattr(step, name)[:, :, :7], getattr(bulk, name)[:, :, :7]), name


def test_v_only_fused_append_matches_two_step_append(tq, dev):
    """Decode-step appends of the fused V-only cache take one launch (K copy + V quantize); the stored
    keys, packed values and norms must equal those of the plain two-step path."""
    g = torch.Generator(device=dev).manual_seed(8)
    B, H, D, n0 = 2, 4, 128, 37
    k0 = torch.randn((B, H, n0, D), generator=g, device=dev).half()
    v0 = torch.randn((B, H, n0, D), generator=g, device=dev).half()
    fast = tq.VOnlyTurboQuantCache(bits=3, seed=5, fused=True)
    fast.reserve(B, H, 512, D, D, torch.float16, dev)
    slow = tq.VOnlyTurboQuantCache(bits=3, seed=5, fused=True)         # grows on demand: never takes the one-launch path
    fast.update_and_fetch(k0, v0)
    slow.update_and_fetch(k0, v0)
    took_fast = 0
    for s in (1, 1, 2, 1):
        k = torch.randn((B, H, s, D), generator=g, device=dev).half()
        v = torch.randn((B, H, s, D), generator=g, device=dev).half()
        took_fast += fast._append_fused(k, v) is not None
        slow._k_cache.update_and_fetch(k, v)
        slow._v_tq.update_and_fetch(k, v)
    n = n0 + 5
    assert took_fast == 4 and fast.offset == slow.offset == n and fast._v_tq.offset == n
    assert torch.equal(fast._k_cache.keys[:, :, :n], slow._k_cache.keys[:, :, :n])
    assert torch.equal(fast._v_tq.v_packed[:, :, :n], slow._v_tq.v_packed[:, :, :n])
    assert torch.equal(fast._v_tq.v_norms[:, :, :n], slow._v_tq.v_norms[:, :, :n])
    # the public call takes the same path and hands back the key view plus a value placeholder
    k = torch.randn((B, H, 1, D), generator=g, device=dev).half()
    keys, vals = fast.update_and_fetch(k, k)
    assert keys.shape == (B, H, n + 1, D) and vals.shape == (B, H, n + 1, D)
    assert torch.equal(keys[:, :, n], k[:, :, 0])


def test_hybrid_cache_quantize_k_then_decode(tq, oracle, dev):
    """HybridQuantCache (hybrid_cache.py:25-100): plain K + packed V during the prompt, then
    `maybe_quantize_k()` and decode steps on 8-bit affine K + 3-bit packed V through the hook;
    compared with the oracle's composed attention over the dequantized affine keys."""
    import math
    from turboquant_mlx_b200 import base
    rng = np.random.default_rng(11)
    B, n_kv, n_rep, S, D = 2, 2, 4, 300, 128
    k_all = rng.standard_normal((B, n_kv, S + 2, D)).astype(np.float16)
    v_all = (rng.standard_normal((B, n_kv, S + 2, D)) * rng.lognormal(0, 0.5, (B, n_kv, S + 2, 1))).astype(np.float16)
    q = rng.standard_normal((B, n_kv * n_rep, 1, D)).astype(np.float16)
    kd, vd, qd = (torch.from_numpy(a).to(dev) for a in (k_all, v_all, q))
    scale = 1.0 / math.sqrt(D)
    c = tq.HybridQuantCache(k_bits=8, k_group_size=64, v_bits=3, v_seed=42)
    assert c.empty() and c.bits is None and c.group_size is None
    k_out, v_out = c.update_and_fetch(kd[:, :, :S], vd[:, :, :S])
    assert torch.equal(k_out, kd[:, :, :S]) and v_out.shape == (B, n_kv, S, D)     # reference behaviour before conversion
    c.maybe_quantize_k()
    assert c.bits == 8 and c.group_size == 64 and c.offset == S
    fp16_bytes = B * n_kv * S * 2 * D * 2
    assert 0.30 < c.nbytes / fp16_bytes < 0.40          # ~35 % of an fp16 cache (hybrid_cache.py:3-6)
    tq.apply_patch()
    try:
        for step in range(2):
            keys, values = c.update_and_fetch(kd[:, :, S + step:S + step + 1], vd[:, :, S + step:S + step + 1])
            out = base.scaled_dot_product_attention(qd, keys, values, c, scale, None)
    finally:
        tq.remove_patch()
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1 and c.offset == S + 2
    signs = c._v_tq._v_q.signs.cpu().numpy()
    codes, sc, bi = oracle.affine_quantize(k_all, 64, 8)
    assert np.array_equal(c.k_codes[:, :, :S + 2].cpu().numpy(), codes)
    k_deq = oracle.affine_dequantize(codes, sc, bi, 64, 8)
    fn_out = tq.hybrid_quantized_attention(qd, tuple(c.state), c._v_tq.v_packed[:, :, :S + 2], c._v_tq.v_norms[:, :, :S + 2],
                                           c._v_tq._v_q.centroids, c._v_tq._v_q.signs, scale, None)
    thr_out = tq.hybrid_quantized_attention(qd, tuple(c.state), c._v_tq.v_packed[:, :, :S + 2], c._v_tq.v_norms[:, :, :S + 2],
                                            c._v_tq._v_q.centroids, c._v_tq._v_q.signs, scale, None,
                                            sparse_v_threshold=1e-6)
    for b in range(B):
        vp, vn = oracle.quantize_packed(v_all[b], signs, 3)
        ref, _ = oracle.decode_attention(q[b, :, 0], k_dense=k_deq[b],
                                         v_polar=dict(packed=vp, norms=vn, centroids=oracle.codebook(3), signs=signs, bits=3),
                                         attn_scale=scale, n_rep=n_rep)
        for name, got in (("hook", out), ("function", fn_out), ("function with threshold", thr_out)):
            err = np.abs(got[b, :, 0].float().cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 2e-3, f"{name}, batch element {b}: max rel err {err:.3e}"
    assert c.trim(1) == 1 and c.offset == S + 1


def test_mixed_cache_static_append_matches_host_side_append(tq, dev):
    """One-token appends at a position read from a device counter (static decode mode) write the same
    codes, scales and biases as appends at the host-side offset, and the decode over the device-side
    length equals the decode over the sliced views."""
    torch.manual_seed(31)
    B, n_kv, n_q, S, D = 1, 2, 8, 70, 128
    k0 = torch.randn(B, n_kv, S, D, device=dev, dtype=torch.bfloat16)
    v0 = torch.randn(B, n_kv, S, D, device=dev, dtype=torch.bfloat16)
    steps = [(torch.randn(B, n_kv, 1, D, device=dev, dtype=torch.bfloat16),
              torch.randn(B, n_kv, 1, D, device=dev, dtype=torch.bfloat16)) for _ in range(5)]
    q = torch.randn(B, n_q, 1, D, device=dev, dtype=torch.bfloat16)
    a, b = tq.MixedQuantKVCache(), tq.MixedQuantKVCache()
    a.update_and_fetch(k0, v0)
    b.update_and_fetch(k0, v0)
    counters = b.enable_static_decode(S + 16)
    assert counters.tolist() == [S, S + 1]
    for ks, vs in steps:
        a.update_and_fetch(ks, vs)
        out_a = a.quantized_attention(q, 1.0 / math.sqrt(D))
        b.update_and_fetch(ks, vs)
        out_b = b.quantized_attention(q, 1.0 / math.sqrt(D))     # reads the length from the device counter
        counters += 1
        assert (out_a.float() - out_b.float()).abs().max().item() < 2e-3 * out_a.float().abs().max().item()
    t = S + len(steps)
    assert b.sync_offset() == t == a.offset
    for name in ("k_codes", "k_scales", "k_biases", "v_codes", "v_scales", "v_biases"):
        assert torch.equal(getattr(a, name)[:, :, :t], getattr(b, name)[:, :, :t]), name
    with pytest.raises(ValueError):
        b.update_and_fetch(k0[:, :, :2], v0[:, :, :2])           # static decode takes one token per step
    b.disable_static_decode()
    b.update_and_fetch(k0[:, :, :2], v0[:, :, :2])
    assert b.offset == t + 2
