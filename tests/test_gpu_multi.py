"""Two-GPU test of sequence-parallel decode, over NCCL and over peer-to-peer stores (skipped on a one-GPU box).
Ranks are child processes; each attends over half of the positions and the
merged result must equal single-GPU decode over the whole sequence."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r'''
import os, sys, math
sys.path.insert(0, os.environ["TQ_ROOT"])
import torch, torch.distributed as dist
import __graft_entry__ as entry
tq = entry.load_package()
from turboquant_mlx_b200.distributed import sequence_parallel_decode, shard_range
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
g = torch.Generator().manual_seed(11)
B, n_kv, n_rep, S, D = 2, 2, 7, 2048, 128
kd = torch.randn((B, n_kv, S, D), generator=g).half().to(dev)
vraw = torch.randn((B, n_kv, S, D), generator=g).half().to(dev)
q = torch.randn((B, n_kv * n_rep, D), generator=g).half().to(dev)
pq = tq.PolarQuantizer(D, 3, seed=43, device=dev)
vp, vn = pq.quantize_packed(vraw)
scale = 1 / math.sqrt(D)
full = tq.flash_decode(q, k=dict(format="dense", data=kd),
                       v=dict(format="polar", packed=vp, norms=vn, centroids=pq.centroids, signs=pq.signs, bits=3),
                       attn_scale=scale, out_dtype=torch.float32)
a, b = shard_range(S, world, rank)
out = sequence_parallel_decode(
    q, k=dict(format="dense", data=kd[:, :, a:b]),
    v=dict(format="polar", packed=vp[:, :, a:b], norms=vn[:, :, a:b], centroids=pq.centroids, signs=pq.signs, bits=3),
    attn_scale=scale, out_dtype=torch.float32)
torch.cuda.synchronize()
err = float((out - full).abs().max() / full.abs().max())
print(f"rank {rank} rel err {err:.3e}")
# the same exchange through peer-to-peer stores and flags, several rounds (both slots, growing epochs)
from turboquant_mlx_b200.distributed import PeerExchange
ex = PeerExchange(B * n_kv * n_rep * (D + 2), dev)
err2 = 0.0
for it in range(5):
    out2 = sequence_parallel_decode(
        q, k=dict(format="dense", data=kd[:, :, a:b]),
        v=dict(format="polar", packed=vp[:, :, a:b], norms=vn[:, :, a:b], centroids=pq.centroids, signs=pq.signs, bits=3),
        attn_scale=scale, out_dtype=torch.float32, exchange=ex)
    err2 = max(err2, float((out2 - full).abs().max() / full.abs().max()))
# push + merge gated inside the merge kernel (one launch less)
from turboquant_mlx_b200.distributed import partial_buffer, partial_views
rows = B * n_kv * n_rep
send = partial_buffer(rows, D, dev)[0]
m_, l_, acc_ = partial_views(send, rows, D)
tq.flash_decode(q, k=dict(format="dense", data=kd[:, :, a:b]),
                v=dict(format="polar", packed=vp[:, :, a:b], norms=vn[:, :, a:b], centroids=pq.centroids,
                       signs=pq.signs, bits=3),
                attn_scale=scale, partials=True,
                partial_out=(m_.view(B, -1), l_.view(B, -1), acc_.view(B, -1, D)))
out3 = torch.empty((rows, D), dtype=torch.float32, device=dev)
for it in range(4):
    block, flags_ptr, epoch = ex.push(send)
    gm, gl, gacc = partial_views(block, rows, D)
    tq.MergePlan(gm, gl, gacc, pq.signs, out3).run_after_peers(flags_ptr, world, epoch, tq._lib.ptr(ex.status))
    err2 = max(err2, float((out3.view(B, -1, D) - full).abs().max() / full.abs().max()))
ex.check()
# the push done by the decode kernel's own final step (peer stores + counters), merge gated as above
ex2 = PeerExchange(rows * (D + 2), dev)
for it in range(4):
    slot, block, flags_ptr, want = ex2.next_fused(B * n_kv)
    tq.flash_decode(q, k=dict(format="dense", data=kd[:, :, a:b]),
                    v=dict(format="polar", packed=vp[:, :, a:b], norms=vn[:, :, a:b], centroids=pq.centroids,
                           signs=pq.signs, bits=3),
                    attn_scale=scale, partials=True, peers=ex2.targets(slot, rows, D),
                    partial_out=(m_.view(B, -1), l_.view(B, -1), acc_.view(B, -1, D)))
    assert tq._lib.lib().tq_flash_decode_last_kernel() == 1
    gm, gl, gacc = partial_views(block, rows, D)
    out4 = torch.empty((rows, D), dtype=torch.float32, device=dev)
    tq.MergePlan(gm, gl, gacc, pq.signs, out4).run_after_peers(flags_ptr, world, want, tq._lib.ptr(ex2.status))
    err2 = max(err2, float((out4.view(B, -1, D) - full).abs().max() / full.abs().max()))
ex2.check()
# one CUDA graph per step: four layers (different queries) of decode-with-push (stable inputs, a
# workspace each, so the launches overlap) + merges gated on the peers' counters, which they reset for
# the next replay; the receive slots are a ring of two (pushes wait for the merge in front) or one per
# layer (nothing waits)
kdesc = dict(format="dense", data=kd[:, :, a:b])
vdesc = dict(format="polar", packed=vp[:, :, a:b], norms=vn[:, :, a:b], centroids=pq.centroids, signs=pq.signs, bits=3)
kfull = dict(format="dense", data=kd)
vfull = dict(format="polar", packed=vp, norms=vn, centroids=pq.centroids, signs=pq.signs, bits=3)
n_layers = 6
qs = [(q.float() * (1.0 + 0.25 * l)).half() for l in range(n_layers)]
fulls = [tq.flash_decode(qs[l], k=kfull, v=vfull, attn_scale=scale, out_dtype=torch.float32) for l in range(n_layers)]
for ring in (True, False):
    ex3 = PeerExchange(rows * (D + 2), dev, slots=2 if ring else n_layers)
    plans, merges, outs5, slots = [], [], [], []
    for l in range(n_layers):
        slot = l & 1 if ring else l
        slots.append(slot)
        sb = partial_buffer(rows, D, dev)[0]
        m5, l5, a5 = partial_views(sb, rows, D)
        plans.append(tq.FlashDecodePlan(
            qs[l], k=kdesc, v=vdesc, attn_scale=scale, partials=True,
            peers=ex3.targets(slot, rows, D, exclusive=not ring), kv_stable=True, q_stable=True,
            workspace=tq.kernels.decode_workspace(dev),
            partial_out=(m5.view(B, -1), l5.view(B, -1), a5.view(B, -1, D))))
        gm, gl, gacc = partial_views(ex3.data[slot], rows, D)
        outs5.append(torch.zeros((rows, D), dtype=torch.float32, device=dev))
        merges.append(tq.MergePlan(gm, gl, gacc, pq.signs, outs5[-1]))
    def step():
        for l in range(n_layers):
            plans[l].run()
            merges[l].run_after_peers(tq._lib.ptr(ex3.flags[slots[l]]), world, B * n_kv, tq._lib.ptr(ex3.status),
                                      reset_flags=True, exclusive_flags=not ring)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(); step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for it in range(8):
        for o5 in outs5:
            o5.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for l in range(n_layers):
            err2 = max(err2, float((outs5[l].view(B, -1, D) - fulls[l]).abs().max() / fulls[l].abs().max()))
    ex3.check()
    assert int(ex3.flags.abs().sum()) == 0          # the merges left the counters at zero
    assert all(tq.kernels.workspace_status(p._keep_ws) == 0 for p in plans)
    dist.barrier()
# the whole exchange inside the decode launch (push, bounded wait for the other ranks' rows, merge):
# one launch per layer, a slot per layer, replayed from a graph
ex4 = PeerExchange(rows * (D + 2), dev, slots=n_layers)
plans, outs6 = [], []
for l in range(n_layers):
    sb = partial_buffer(rows, D, dev)[0]
    m5, l5, a5 = partial_views(sb, rows, D)
    outs6.append(torch.zeros((B, n_kv * n_rep, D), dtype=torch.float32, device=dev))
    plans.append(tq.FlashDecodePlan(
        qs[l], k=kdesc, v=vdesc, attn_scale=scale, partials=True, peers=ex4.targets(l, rows, D, exclusive=True),
        gather=ex4.gather_spec(l, rows, D), out=outs6[-1], kv_stable=True, q_stable=True,
        workspace=tq.kernels.decode_workspace(dev),
        partial_out=(m5.view(B, -1), l5.view(B, -1), a5.view(B, -1, D))))
def step2():
    for l in range(n_layers):
        plans[l].run()
side = torch.cuda.Stream(device=dev)
side.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(side):
    step2(); step2()
torch.cuda.current_stream().wait_stream(side)
torch.cuda.synchronize()
dist.barrier()
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph):
    step2()
for it in range(8):
    for o6 in outs6:
        o6.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for l in range(n_layers):
        err2 = max(err2, float((outs6[l] - fulls[l]).abs().max() / fulls[l].abs().max()))
assert int(ex4.flags.abs().sum()) == 0              # the kernels left their counters at zero
assert all(tq.kernels.workspace_status(p._keep_ws) == 0 for p in plans)
dist.barrier()
print(f"rank {rank} peer exchange rel err {err2:.3e}")
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if err < 1e-3 and err2 < 1e-3 else 1)
'''


def test_sequence_parallel_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, TQ_ROOT=ROOT, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
