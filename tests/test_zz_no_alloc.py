"""The allocation-free variant of the weighted packed-V sum.

Some hosts of this library cannot give it a workspace: they run inside a serving
framework that owns all device memory and bans cudaMalloc from plugin code, or
bind the C ABI from a language that has no device allocator, or sit in a decode
loop where an allocation would stall the GPU.  For them
`tq_sparse_v_matvec_noalloc` keeps its scratch in a fixed 4 MiB array inside the
library.  This test calls it through the C ABI, twice in a row with different
inputs (the second call starts from the first call's leftovers in the shared
array), and checks each result against `tq_sparse_v_matvec` with an ordinary
workspace.  It also checks that an oversized request is refused, not truncated.

The file name sorts last on purpose: if this test fails under `-x`, every other
test has already run.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(oracle, rng, n_kv, n_rep, seq, dim, bits, dev):
    vp = oracle.pack_indices(rng.integers(0, 1 << bits, (n_kv, seq, dim)).astype(np.uint8), bits)
    vn = (rng.random((n_kv, seq)) * 3 + 0.1).astype(np.float32)
    w = oracle.softmax(rng.standard_normal((n_kv * n_rep, seq)) * 3)
    to = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)  # noqa: E731
    return to(w), to(vp), to(vn)


def _call_noalloc(tq, w, vp, vn, cent, signs, dim, bits, thr, n_rep, stream):
    L = tq._lib.lib()
    out = torch.full((w.shape[0], dim), float("nan"), dtype=torch.float32, device=w.device)
    rc = L.tq_sparse_v_matvec_noalloc(
        ctypes.c_void_p(w.data_ptr()), w.stride(0), ctypes.c_void_p(vp.data_ptr()), vp.stride(0),
        ctypes.c_void_p(vn.data_ptr()), vn.stride(0), vp.shape[0], w.shape[1],
        tq._lib.host_floats(cent), tq._lib.host_floats(signs), dim, bits, thr, n_rep,
        ctypes.c_void_p(out.data_ptr()), stream)
    return rc, out


def test_noalloc_matches_workspace_variant_twice_in_a_row(tq, oracle, dev):
    L = tq._lib.lib()
    assert L.tq_sparse_v_noalloc_max_bytes() == 4 << 20
    rng = np.random.default_rng(99)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    # two different shapes back to back: the second run reuses a dirty scratch array
    for n_kv, n_rep, seq, dim, bits, thr in ((4, 7, 3000, 128, 3, 0.0), (2, 4, 1500, 64, 4, 1e-5)):
        pq = tq.PolarQuantizer(dim, bits, seed=43, device=dev)
        w, vp, vn = _case(oracle, rng, n_kv, n_rep, seq, dim, bits, dev)
        rc, got = _call_noalloc(tq, w, vp, vn, pq.centroids, pq.signs, dim, bits, thr, n_rep, stream)
        assert rc == 0, L.tq_last_error_string()
        want = tq.sparse_v_matvec(w, vp, vn, pq.centroids, pq.signs, dim, bits, threshold=thr, n_rep=n_rep)
        torch.cuda.synchronize()
        ref = want.cpu().numpy()
        err = np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err < 1e-5, f"noalloc differs from the workspace variant: rel {err:.2e}"
        ora = oracle.sparse_v_matvec(w.cpu().numpy(), vp.cpu().numpy(), vn.cpu().numpy(), oracle.codebook(bits),
                                     pq.signs.cpu().numpy(), dim, bits, threshold=thr, n_rep=n_rep)
        assert np.abs(got.cpu().numpy() - ora).max() / np.abs(ora).max() < 1e-5


def test_noalloc_refuses_more_than_its_array_holds(tq, dev):
    L = tq._lib.lib()
    n_kv, n_rep, seq, dim = 8, 8, 200000, 256      # 256 chunks x 64 heads x 256 x 4 B = 16 MiB
    assert L.tq_sparse_v_workspace_bytes(n_kv * n_rep, seq, dim) > L.tq_sparse_v_noalloc_max_bytes()
    one = ctypes.c_void_p(256)
    cent = (ctypes.c_float * 8)(*([0.0] * 8))
    signs = (ctypes.c_float * 256)(*([1.0] * 256))
    rc = L.tq_sparse_v_matvec_noalloc(one, seq, one, seq * 26, one, seq, n_kv, seq, cent, signs, dim, 3,
                                      0.0, n_rep, one, ctypes.c_void_p(0))
    assert rc == -5
    assert b"built-in array" in L.tq_last_error_string()
