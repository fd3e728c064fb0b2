"""Host-side logic that needs no GPU: packing utilities, codebooks, the sign
generator, the plain KV cache and the mask helpers."""

import numpy as np
import pytest
import torch


def test_packing_matches_oracle(tq, oracle):
    rng = np.random.default_rng(0)
    for bits, dim in ((1, 64), (2, 32), (3, 128), (4, 64), (3, 50)):
        idx = rng.integers(0, 1 << bits, size=(3, 9, dim)).astype(np.uint8)
        p = tq.pack_indices(torch.from_numpy(idx), bits)
        assert p.dtype == torch.uint32
        assert np.array_equal(p.numpy(), oracle.pack_indices(idx, bits))
        assert np.array_equal(tq.unpack_indices(p, bits, dim).numpy(), idx)
        assert tq.packed_dim(dim, bits) == oracle.packed_dim(dim, bits)


def test_codebooks_boundaries_and_signs_match_oracle(tq, oracle):
    from turboquant_mlx_b200 import quantizer, rotation
    for bits in (1, 2, 3, 4):
        c = quantizer.codebook_values(bits)
        assert np.array_equal(np.asarray(c, np.float32), oracle.codebook(bits))
        assert np.array_equal(np.asarray(quantizer.boundary_values(c), np.float32),
                              oracle.boundaries(oracle.codebook(bits)))
    with pytest.raises(ValueError, match="Unsupported bit width"):
        quantizer.codebook_values(5)
    for d, seed in ((128, 42), (128, 43), (64, 7)):
        assert np.array_equal(np.asarray(rotation.sign_values(d, seed), np.float32),
                              oracle.signs_from_seed(d, seed))


def test_plain_kv_cache_and_masks(tq):
    from turboquant_mlx_b200.base import KVCache, create_causal_mask
    c = KVCache()
    assert c.empty() and c.make_mask(1) is None and c.make_mask(5) == "causal"
    k = torch.randn(1, 2, 5, 8)
    ko, vo = c.update_and_fetch(k, k * 2)
    assert ko.shape == (1, 2, 5, 8) and c.offset == 5 and c.keys.shape[2] == 256
    ko, _ = c.update_and_fetch(k[:, :, :1], k[:, :, :1])
    assert ko.shape[2] == 6 and torch.equal(ko[:, :, :5], k)
    assert c.trim(2) == 2 and c.size() == 4
    m = create_causal_mask(3, offset=2)
    assert m.shape == (3, 5) and bool(m[0, 2]) and not bool(m[0, 3])
    m = c.make_mask(3, return_array=True)
    assert m.shape == (3, 7)


def test_mask_broadcast_rules(tq):
    from turboquant_mlx_b200.fused_attention import _mask_3d
    B, H, T = 3, 4, 10
    assert _mask_3d(torch.zeros(B, 1, 1, T), B, H, T).shape == (B, 1, T)
    assert _mask_3d(torch.zeros(1, H, 1, T), B, H, T).shape == (1, H, T)
    assert _mask_3d(torch.zeros(1, 1, T), B, H, T).shape == (1, 1, T)
    assert _mask_3d(torch.zeros(2, 1, 1, T), B, H, T).shape == (B, 1, T)  # index min(b, M-1)


def test_patch_swaps_and_restores_symbol(tq):
    from turboquant_mlx_b200 import base, patch
    orig = base.scaled_dot_product_attention
    tq.apply_patch()
    assert base.scaled_dot_product_attention is patch._patched_sdpa
    tq.apply_patch()  # idempotent
    tq.remove_patch()
    assert base.scaled_dot_product_attention is orig
    q = torch.randn(1, 4, 1, 8)
    k = torch.randn(1, 2, 6, 8)
    out = base.scaled_dot_product_attention(q, k, k, None, 0.3, None)
    assert out.shape == (1, 4, 1, 8)


def test_meta_state_format(tq):
    c = tq.TurboQuantKVCache(bits=3, seed=42)
    assert c.meta_state == "0,3,42,0,0,float16"
    c.meta_state = "12,3,42,128,128,bfloat16"
    assert c.offset == 12 and c._dtype == torch.bfloat16 and c._k_dim == 128
    c2 = tq.TurboQuantKVCache(bits=3, k_bits=4, v_bits=3)
    assert c2.meta_state.endswith(",4,3")
    v = tq.VOnlyTurboQuantCache(bits=3)
    assert v.meta_state.startswith("VOnlyTQ,3,")
    assert v.empty() and v.is_trimmable() and tq.TurboQuantKVCache().empty()
    with pytest.raises(ValueError, match="Expected 2"):
        c.state = [torch.zeros(1)] * 5


def test_qwen2_module_cache_consistency():
    """The random-init decoder that drives the caches: prompt + one decode step through a plain
    cache gives the logits of the full sequence's last position (CPU, library attention)."""
    import torch
    import __graft_entry__ as entry
    tq = entry.load_package()
    from turboquant_mlx_b200.qwen2 import Qwen2Config, Qwen2Model
    cfg = Qwen2Config(n_layers=2, hidden=64, n_q_heads=4, n_kv_heads=2, head_dim=16, ffn=96, vocab=50,
                      init_std=0.2)
    model = Qwen2Model(cfg, "cpu", torch.float32, seed=1)
    toks = torch.randint(0, cfg.vocab, (2, 9), generator=torch.Generator().manual_seed(0))
    full = model.forward(toks, [tq.KVCache() for _ in range(cfg.n_layers)], last_only=False)
    caches = [tq.KVCache() for _ in range(cfg.n_layers)]
    model.forward(toks[:, :8], caches)
    step = model.forward(toks[:, 8:], caches)
    assert caches[0].offset == 9
    assert torch.allclose(step[:, 0], full[:, -1], atol=1e-4, rtol=1e-4)
    per_layer = 2 * cfg.hidden * cfg.n_q_heads * cfg.head_dim + 2 * cfg.hidden * cfg.n_kv_heads * cfg.head_dim + \
        3 * cfg.hidden * cfg.ffn
    assert model.n_params() == cfg.n_layers * per_layer + 2 * cfg.vocab * cfg.hidden
    lw = model.layers[0]      # the separate projection names are views of the fused matrices
    assert lw["wq"].data_ptr() == lw["wqkv"].data_ptr() and lw["w3"].shape == (cfg.hidden, cfg.ffn)


def test_host_float_cache_follows_the_tensor_object(tq):
    """The host copy of a codebook-sized tensor is tied to the tensor object: a new tensor that
    lands at a freed tensor's address, or an in-place change, is read again."""
    from turboquant_mlx_b200 import _lib
    a = torch.tensor([1.0, -1.0, 1.0, 1.0])
    assert list(_lib.host_floats(a)) == [1.0, -1.0, 1.0, 1.0]
    assert _lib.host_floats(a) is _lib.host_floats(a)            # cached while it lives
    addr = a.data_ptr()
    del a
    for _ in range(8):                                           # the allocator reuses the block
        b = torch.tensor([-1.0, -1.0, 1.0, -1.0])
        assert list(_lib.host_floats(b)) == [-1.0, -1.0, 1.0, -1.0]
        if b.data_ptr() == addr:
            break
        del b
    c = torch.tensor([1.0, 1.0])
    first = _lib.host_floats(c)
    c.mul_(-1.0)
    assert list(_lib.host_floats(c)) == [-1.0, -1.0] and list(first) == [1.0, 1.0]
    n_before = len(_lib._host_cache)
    del c
    assert len(_lib._host_cache) == n_before - 1                 # evicted with the tensor


def test_state_with_saved_sign_vectors_loads(tq):
    """A saved state may carry its sign vectors (a library whose generator differs cannot rebuild
    them from the seed): they replace the seed-derived ones; malformed vectors are refused."""
    from turboquant_mlx_b200.rotation import sign_values
    B, H, S, D = 1, 2, 5, 128
    kp = torch.zeros((B, H, S, 16), dtype=torch.int32).view(torch.uint32)
    vp = torch.zeros((B, H, S, 13), dtype=torch.int32).view(torch.uint32)
    kn, vn = torch.ones((B, H, S)), torch.ones((B, H, S))
    ks = torch.tensor(sign_values(D, 42))
    vs = -torch.tensor(sign_values(D, 43))                       # not what seed 43 gives here
    meta = f"{S},3,42,{D},{D},float16,4,3"
    c = tq.TurboQuantKVCache.from_state([kp, kn, vp, vn, ks, vs], meta)
    assert c.offset == S and c.k_bits == 4 and c.v_bits == 3
    assert torch.equal(c._k_q.signs, ks) and torch.equal(c._v_q.signs, vs)
    assert not c.signs_match_seed()
    assert len(c.state) == 4 and len(c.state_with_signs) == 6
    plain = tq.TurboQuantKVCache.from_state([kp, kn, vp, vn], meta)
    assert plain.signs_match_seed()
    with pytest.raises(ValueError, match=r"\+1 / -1"):
        tq.TurboQuantKVCache.from_state([kp, kn, vp, vn, ks * 0.5, vs], meta)
    with pytest.raises(ValueError, match="cache dimension"):
        tq.TurboQuantKVCache.from_state([kp, kn, vp, vn, ks[:64], vs], meta)
    with pytest.raises(ValueError, match="Expected 2"):
        tq.TurboQuantKVCache.from_state([kp, kn, vp, vn, ks], meta)
    # values-only forms: 2 arrays, or 3 with the V sign vector
    v_only = tq.TurboQuantKVCache.from_state([vp, vn, vs], f"{S},3,42,0,{D},float16")
    assert v_only.v_only and not v_only.empty() and torch.equal(v_only._v_q.signs, vs)
    k16 = torch.zeros((B, H, S, D), dtype=torch.float16)
    vo = tq.VOnlyTurboQuantCache.from_state([k16, k16[..., :0], vp, vn, vs], f"VOnlyTQ,3,42,{S},3,42,0,{D},float16")
    assert vo.offset == S and torch.equal(vo._v_tq._v_q.signs, vs)
    assert len(vo.state_with_signs) == 5


def test_adaptive_cache_arguments_follow_the_reference(tq):
    from turboquant_mlx_b200.base import KVCache
    caches = tq.make_adaptive_cache(8, 3, 4, 3, 2)      # num_layers, bits, k_bits, v_bits, fp16_layers
    assert [isinstance(c, KVCache) for c in caches] == [True, True] + [False] * 4 + [True, True]
    mid = caches[3]
    assert (mid.k_bits, mid.v_bits, mid.seed) == (4, 3, 42)

    class Plain:
        def make_cache(self):
            return [KVCache()]

    class Other:
        def make_cache(self):
            return [object()]

    assert len(tq.make_adaptive_cache(4, model=Plain())) == 4
    with pytest.raises(ValueError, match="Incompatible cache type"):
        tq.make_adaptive_cache(4, model=Other())
