"""tq_peer_push / tq_peer_wait / tq_merge_partials_after_peers on one GPU: the "peers" are
buffers of the same device, which exercises the copy, the flag protocol, the gate inside the merge
kernel and the bounded wait (a flag that nothing sets: the wait gives up and reports which rank is
missing; no fault, no hang)."""
import ctypes
import time

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tq():
    return entry.load_package()


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def test_push_copies_block_and_raises_flags(tq):
    dev = torch.device("cuda", 0)
    L, st = tq._lib.lib(), tq._lib.stream_ptr(dev)
    n, world = 4 * 130 * 16, 3                       # three receive buffers on this device stand in for three ranks
    src = torch.randn(n, device=dev)
    recv = torch.zeros((world, 2, n), device=dev)    # [peer][slot of the sending rank][block]
    flags = torch.zeros((world, 2), dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    my_rank = 1
    dst = _ptr_array([recv[p, my_rank].data_ptr() for p in range(world)])
    flg = _ptr_array([flags[p, my_rank:].data_ptr() for p in range(world)])
    tq._lib.check(L.tq_peer_push(tq._lib.ptr(src), n * 4, dst, flg, world, 7, st))
    # each "rank" waits on its own flag array; only the sender's word was raised
    tq._lib.check(L.tq_peer_wait(flags[0, my_rank:].data_ptr(), 1, 7, tq._lib.ptr(status), st))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(flags[:, my_rank].cpu(), torch.full((world,), 7, dtype=torch.int32))
    assert torch.equal(flags[:, 0].cpu(), torch.zeros(world, dtype=torch.int32))
    for p in range(world):
        assert torch.equal(recv[p, my_rank], src) and not recv[p, 0].any()
    with pytest.raises(ValueError):
        tq._lib.check(L.tq_peer_push(tq._lib.ptr(src), n * 4 + 4, dst, flg, world, 8, st))   # not a multiple of 16


def test_wait_gives_up_and_names_the_missing_rank(tq):
    dev = torch.device("cuda", 0)
    L, st = tq._lib.lib(), tq._lib.stream_ptr(dev)
    flags = torch.tensor([5, 5, 4, 5], dtype=torch.int32, device=dev)      # rank 2 never reached epoch 5
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    prev = L.tq_set_peer_wait_limit_ms(100)          # the default limit is seconds; keep the test short
    assert prev == 2000 and L.tq_set_peer_wait_limit_ms(0) == 100
    try:
        t0 = time.perf_counter()
        tq._lib.check(L.tq_peer_wait(tq._lib.ptr(flags), 4, 5, tq._lib.ptr(status), st))
        torch.cuda.synchronize()
        assert 0.05 < time.perf_counter() - t0 < 10.0    # the time limit, not an iteration count, ended it
        assert int(status[0]) == 21 + 2
        # a merge gated on the same incomplete flags reports the rank and hands out NaN, not a partial merge
        status.zero_()
        g = torch.Generator(device=dev).manual_seed(3)
        m = torch.randn((4, 6), generator=g, device=dev)
        l = torch.rand((4, 6), generator=g, device=dev) + 0.1
        acc = torch.randn((4, 6, 128), generator=g, device=dev)
        out = torch.zeros((6, 128), dtype=torch.float32, device=dev)
        pq = tq.PolarQuantizer(128, 3, seed=43, device=dev)
        tq.MergePlan(m, l, acc, pq.signs, out).run_after_peers(tq._lib.ptr(flags), 4, 5, tq._lib.ptr(status))
        torch.cuda.synchronize()
        assert int(status[0]) == 21 + 2 and bool(torch.isnan(out).all())
    finally:
        L.tq_set_peer_wait_limit_ms(prev)
    # the context is still usable and a later epoch that is complete passes at once
    status.zero_()
    tq._lib.check(L.tq_peer_wait(tq._lib.ptr(flags), 4, 4, tq._lib.ptr(status), st))
    torch.cuda.synchronize()
    assert int(status[0]) == 0


def test_merge_gated_on_flags_equals_plain_merge(tq):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    parts, rows, D = 4, 14, 128
    m = torch.randn((parts, rows), generator=g, device=dev)
    l = torch.rand((parts, rows), generator=g, device=dev) + 0.1
    acc = torch.randn((parts, rows, D), generator=g, device=dev)
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    ref = tq.merge_partials(m, l, acc, pq.signs, torch.float32)
    out = torch.empty((rows, D), dtype=torch.float32, device=dev)
    flags = torch.full((parts,), 9, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    tq.MergePlan(m, l, acc, pq.signs, out).run_after_peers(tq._lib.ptr(flags), parts, 9, tq._lib.ptr(status))
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and torch.equal(out, ref)
    assert np.isfinite(out.cpu().numpy()).all()


def test_gated_merge_resets_its_flags_for_graph_replay(tq):
    """reset_flags: the launch zeroes the flag words once every block is past the gate, so the same
    call (constant expected count) can be replayed; counters pushed between replays gate each one."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    parts, rows, D = 2, 28, 128
    m = torch.randn((parts, rows), generator=g, device=dev)
    l = torch.rand((parts, rows), generator=g, device=dev) + 0.1
    acc = torch.randn((parts, rows, D), generator=g, device=dev)
    pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
    ref = tq.merge_partials(m, l, acc, pq.signs, torch.float32)
    out = torch.empty((rows, D), dtype=torch.float32, device=dev)
    flags = torch.zeros((parts,), dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    plan = tq.MergePlan(m, l, acc, pq.signs, out)
    for _ in range(3):
        flags.add_(4)                 # what the peers' decode kernels would add (4 groups each)
        out.zero_()
        plan.run_after_peers(tq._lib.ptr(flags), parts, 4, tq._lib.ptr(status), reset_flags=True)
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and int(status[1]) == 0 and torch.equal(out, ref)
        assert int(flags.abs().sum()) == 0
