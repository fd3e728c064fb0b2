"""World-size-2 gloo tests (CPU) of the multi-GPU plumbing: shard bookkeeping
and the all-gather of packed partial states, merged with the oracle.  Failures
are made on the host (an empty chunk, a malformed buffer), never on a GPU."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything(tq):
    from turboquant_mlx_b200.distributed import shard_range
    for n, world in ((32, 8), (4, 8), (7, 3), (1048576, 8), (0, 2)):
        spans = [shard_range(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans[:-1], spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def test_send_buffer_keeps_the_accumulator_on_a_16_byte_boundary(tq):
    """The decode kernel writes accumulator rows as 16-byte vectors: the send buffer of a rank must put
    `acc` on a 16-byte boundary for odd row counts too (one kv-head shard with 7 query heads, say)."""
    from turboquant_mlx_b200.distributed import partial_buffer, partial_views
    for rows in (1, 7, 8, 21, 28, 63, 64):
        buf = partial_buffer(rows, 128, "cpu")[0]
        m, l, acc = partial_views(buf, rows, 128)
        assert acc.data_ptr() % 16 == 0, rows
        assert m.shape == (rows,) and l.data_ptr() - m.data_ptr() == 4 * rows and acc.shape == (rows, 128)


def test_partial_views_layout(tq):
    from turboquant_mlx_b200.distributed import partial_buffer, partial_views
    rows, dim, world = 6, 32, 3
    buf = partial_buffer(rows, dim, "cpu", world)
    buf.copy_(torch.arange(buf.numel(), dtype=torch.float32).view_as(buf))
    m, l, acc = partial_views(buf, rows, dim)
    assert m.shape == (world, rows) and l.shape == (world, rows) and acc.shape == (world, rows, dim)
    assert m[1, 0] == rows * (dim + 2) and l[0, 0] == rows and acc[0, 0, 0] == 2 * rows
    assert acc[2, 1, 3] == 2 * rows * (dim + 2) + 2 * rows + dim + 3


def _worker(rank, world, port, empty_rank, ret):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    o = entry.load_oracle()
    from turboquant_mlx_b200.distributed import gather_partials, partial_views, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)          # same data on every rank
        n_kv, n_rep, S, D, bits = 2, 4, 301, 64, 3
        rows = n_kv * n_rep
        vs = o.signs_from_seed(D, 43)
        c = o.codebook(bits)
        vp = o.pack_indices(rng.integers(0, 8, (n_kv, S, D)).astype(np.uint8), bits)
        vn = (rng.random((n_kv, S)) + 0.1).astype(np.float32)
        scores = (rng.standard_normal((rows, S)) * 2).astype(np.float32)
        whole = o.sparse_v_matvec(o.softmax(scores), vp, vn, c, vs, D, bits, 0.0, n_rep)
        # positions are sharded over the ranks that hold data; `empty_rank` holds none
        holders = [r for r in range(world) if r != empty_rank]
        send = torch.zeros(rows * (D + 2), dtype=torch.float32)
        if rank in holders:
            a, b = shard_range(S, len(holders), holders.index(rank))
            m, l, acc = o.decode_partials(scores[:, a:b], vp[:, a:b], vn[:, a:b], c, D, bits, n_rep)
            send[:rows] = torch.from_numpy(m)
            send[rows:2 * rows] = torch.from_numpy(l)
            send[2 * rows:] = torch.from_numpy(acc.reshape(-1))
        recv = gather_partials(send)
        assert recv.shape == (world, rows * (D + 2))
        gm, gl, gacc = partial_views(recv, rows, D)
        merged = o.merge_partials(gm.numpy(), gl.numpy(), gacc.numpy(), vs, D)
        err = float(np.abs(merged - whole).max() / np.abs(whole).max())
        bad = False
        try:
            gather_partials(send.view(2, -1))
        except ValueError:
            bad = True
        ret[rank] = (err, bad)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("empty_rank", [None, 1])
def test_gloo_gather_and_merge_equals_whole(empty_rank):
    world = 2
    port = 29500 + (os.getpid() % 2000) + (0 if empty_rank is None else 1)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, empty_rank, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        err, bad = ret[r]
        assert err < 1e-5 and bad


def _failure_worker(rank, world, port, mode, ret):
    """Host-made failures: `nan` - rank 1 sends a partial state with NaN in it; `late` - rank 1
    joins the collective two seconds late; `dropped` - rank 1 never joins and rank 0's collective
    ends with an error after the short process-group timeout."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from turboquant_mlx_b200.distributed import check_partials, gather_partials, partial_views
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    try:
        rows, D = 4, 32
        send = torch.zeros(rows * (D + 2), dtype=torch.float32)
        send[:rows] = 0.5 + rank
        send[rows:2 * rows] = 1.0
        send[2 * rows:] = float(rank + 1)
        if mode == "nan" and rank == 1:
            send[2 * rows + 7] = float("nan")
        if mode == "late" and rank == 1:
            time.sleep(2.0)
        if mode == "dropped" and rank == 1:
            time.sleep(10.0)              # leaves between steps: never joins the gather
            ret[rank] = "left"
            return
        try:
            recv = gather_partials(send)
        except Exception as exc:          # the short timeout ended the collective
            ret[rank] = f"collective failed: {type(exc).__name__}"
            return
        try:
            check_partials(recv, rows, D)
            m, l, acc = partial_views(recv, rows, D)
            ret[rank] = ("ok", float(acc[1, 0, 0]), bool(torch.isfinite(acc).all()))
        except RuntimeError as exc:
            ret[rank] = str(exc)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("mode", ["nan", "late", "dropped"])
def test_gloo_host_side_failures(mode):
    world = 2
    port = 31500 + (os.getpid() % 2000) + {"nan": 0, "late": 1, "dropped": 2}[mode]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_failure_worker, args=(world, port, mode, ret), nprocs=world, join=True)
    if mode == "nan":          # every rank learns which rank sent the bad block
        assert all("rank 1 sent a non-finite" in ret[r] for r in range(world))
    elif mode == "late":       # a late rank only delays the step
        assert all(ret[r] == ("ok", 2.0, True) for r in range(world))
    else:                      # the remaining rank gets an error instead of hanging
        assert ret[1] == "left" and ret[0].startswith("collective failed")
