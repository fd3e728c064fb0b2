"""tq_prefill_sdpa (tcgen05 prefill attention) against the numpy oracle and, at
sizes the oracle would take too long for, against float32 torch math."""
import math

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tq():
    return entry.load_package()


@pytest.fixture(scope="module")
def oracle():
    return entry.load_oracle()


def _inputs(B, n_q, n_kv, L, S, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((B, n_q, L, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    k = torch.randn((B, n_kv, S, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    v = torch.randn((B, n_kv, S, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    return q, k, v


# tolerance: the path rounds P and the output to the 16-bit dtype (2^-11 / 2^-8 relative steps);
# outputs are averages of N(0,1) values, so absolute errors are compared on an O(1) scale
TOL = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,n_q,n_kv,L,S,causal", [
    (1, 1, 1, 128, 128, True),      # one tile, diagonal mask
    (1, 2, 1, 256, 256, True),      # two tiles, GQA pair
    (2, 4, 2, 200, 200, True),      # ragged tail in both directions
    (1, 7, 1, 130, 391, True),      # L < S: offset diagonal, n_rep 7
    (1, 2, 2, 77, 300, False),      # full attention, ragged keys
    (1, 1, 1, 1, 129, True),        # a single query row through the prefill path
])
def test_prefill_matches_oracle(tq, oracle, dtype, B, n_q, n_kv, L, S, causal):
    q, k, v = _inputs(B, n_q, n_kv, L, S, dtype, seed=L * 1000 + S)
    scale = 1.0 / math.sqrt(128)
    out = tq.prefill_attention(q, k, v, scale, causal=causal)
    torch.cuda.synchronize()
    assert tq.kernels.prefill_status(q.device) == 0
    ref = oracle.prefill_sdpa(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                              scale, causal=causal)
    err = np.abs(out.float().cpu().numpy() - ref).max()
    assert out.shape == (B, n_q, L, 128) and out.dtype == dtype
    assert err < TOL[dtype], err


def _torch_reference(q, k, v, scale, causal):
    B, n_q, L, D = q.shape
    n_kv, S = k.shape[1], k.shape[2]
    rep = n_q // n_kv
    qf = q.float()
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        allowed = torch.arange(S, device=q.device)[None, :] <= torch.arange(L, device=q.device)[:, None] + (S - L)
        s = s.masked_fill(~allowed, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_long_sequence(tq, dtype):
    # 28 q / 4 kv heads as in the headline attention shape, many K/V tiles per query tile,
    # large-magnitude scores so that the lazy rescale of the output accumulator triggers
    q, k, v = _inputs(1, 28, 4, 2048, 2048, dtype, seed=7)
    q = q * 3.0
    scale = 1.0 / math.sqrt(128)
    out = tq.prefill_attention(q, k, v, scale, causal=True)
    torch.cuda.synchronize()
    assert tq.kernels.prefill_status(q.device) == 0
    ref = _torch_reference(q, k, v, scale, True)
    err = (out.float() - ref).abs().max().item()
    assert err < 2 * TOL[dtype], err


def test_prefill_strided_views_and_out(tq):
    # keys / values as views into a larger pre-sized cache buffer (the cache's own layout)
    B, n_q, n_kv, L, cap = 2, 8, 2, 384, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    kbuf = torch.randn((B, n_kv, cap, 128), generator=g, device="cuda").half()
    vbuf = torch.randn((B, n_kv, cap, 128), generator=g, device="cuda").half()
    q = torch.randn((B, n_q, L, 128), generator=g, device="cuda").half()
    k, v = kbuf[:, :, :L], vbuf[:, :, :L]
    out = torch.empty((B, n_q, L, 128), device="cuda", dtype=torch.float16)
    res = tq.prefill_attention(q, k, v, 0.1, causal=True, out=out)
    assert res.data_ptr() == out.data_ptr()
    ref = _torch_reference(q, k, v, 0.1, True)
    assert (out.float() - ref).abs().max().item() < 2e-3


def test_prefill_argument_errors(tq):
    q = torch.zeros((1, 3, 16, 128), device="cuda", dtype=torch.float16)
    k = torch.zeros((1, 2, 16, 128), device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="n_q_heads"):
        tq.prefill_attention(q, k, k, 1.0)
    q64 = torch.zeros((1, 2, 16, 64), device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="head_dim 128"):
        tq.prefill_attention(q64, q64, q64, 1.0)
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        tq.prefill_attention(q.float(), k.float(), k.float(), 1.0)


def test_hook_routes_prompt_step_to_prefill_kernel(tq):
    # a prompt step through the patched attention symbol over a fused V-only cache
    tq.apply_patch()
    try:
        from turboquant_mlx_b200 import base
        cache = tq.VOnlyTurboQuantCache(bits=4, seed=5, fused=True)
        g = torch.Generator(device="cuda").manual_seed(11)
        keys = torch.randn((1, 2, 256, 128), generator=g, device="cuda").half()
        values = torch.randn((1, 2, 256, 128), generator=g, device="cuda").half()
        queries = torch.randn((1, 4, 256, 128), generator=g, device="cuda").half()
        k, v = cache.update_and_fetch(keys, values)
        out = base.scaled_dot_product_attention(queries, k, v, cache, 0.09, "causal")
        _, v_deq = cache._v_tq.dequantized(torch.float16)
        ref = _torch_reference(queries, keys, v_deq, 0.09, True)
        assert (out.float() - ref).abs().max().item() < 2e-3
    finally:
        tq.remove_patch()
