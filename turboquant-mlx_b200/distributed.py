"""Multi-GPU sharding of the decode path, one process per GPU.

The path shards without any exchange by batch and by KV-head group (every
(sequence, kv head) pair is independent): `shard_range` gives a rank its slice.
At very long context the sequence axis is split instead: each rank attends over
its own chunk of positions with `flash_decode(..., partials=True)`, the ranks
`all_gather` their (m, l, acc) states (rows * (dim + 2) floats per rank, 33 KB at
64 heads) and every rank merges them locally with `tq_merge_partials`.  The
accumulator travels in the rotated domain, so the single butterfly happens after
the merge.  The reference has no multi-device code; this module is new.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib, kernels


def shard_range(n_items: int, world: int, rank: int):
    """Contiguous [start, stop) of `n_items` (sequences, kv heads or positions)
    owned by `rank`; the first n_items % world ranks get one extra item."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def partial_buffer(rows: int, dim: int, device, world: int = 1) -> torch.Tensor:
    """(world, rows * (dim + 2)) float32: per rank [m (rows) | l (rows) | acc (rows * dim)].
    The decode kernel stores accumulator rows as 16-byte vectors; acc starts 8 * rows bytes into a
    block, so a one-block buffer (a rank's send buffer) with an odd row count is placed 8 bytes into
    its allocation, which puts acc on a 16-byte boundary."""
    n = rows * (dim + 2)
    if world == 1 and rows % 2:
        return torch.empty((n + 2,), dtype=torch.float32, device=device)[2:].view(1, n)
    return torch.empty((world, n), dtype=torch.float32, device=device)


def partial_views(buf: torch.Tensor, rows: int, dim: int):
    """(m, l, acc) views of a partial buffer: (..., rows), (..., rows), (..., rows, dim)."""
    lead = buf.shape[:-1]
    m = buf[..., :rows]
    l = buf[..., rows:2 * rows]
    acc = buf[..., 2 * rows:].reshape(*lead, rows, dim) if buf.is_contiguous() else \
        buf[..., 2 * rows:].unflatten(-1, (rows, dim))
    return m, l, acc


def gather_partials(send: torch.Tensor, group=None, recv: torch.Tensor | None = None) -> torch.Tensor:
    """all_gather of one rank's packed partial state (rows * (dim + 2),) ->
    (world, rows * (dim + 2)).  Works on CUDA tensors (NCCL) and CPU tensors (gloo).
    `recv` optionally names a persistent receive buffer."""
    world = dist.get_world_size(group)
    if send.ndim != 1:
        raise ValueError(f"expected a flat partial buffer, got shape {tuple(send.shape)}")
    if recv is None:
        recv = torch.empty((world, send.numel()), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(recv.view(-1), send.contiguous(), group=group)
    return recv


def check_partials(recv: torch.Tensor, rows: int, dim: int) -> None:
    """Host-side guard for a gathered (world, rows * (dim + 2)) block (synchronises): raises
    RuntimeError naming the first rank whose partial state holds a non-finite value where one
    cannot occur (l or acc anywhere, m on a row with l > 0; m = -inf marks an empty chunk)."""
    m, l, acc = partial_views(recv, rows, dim)
    bad = (~torch.isfinite(l)).any(-1) | (~torch.isfinite(acc)).flatten(1).any(-1) | \
        ((l > 0) & ~torch.isfinite(m)).any(-1) | torch.isnan(m).any(-1)
    if bool(bad.any()):
        rank = int(torch.nonzero(bad)[0])
        raise RuntimeError(f"rank {rank} sent a non-finite partial attention state")


class PeerExchange:
    """All-gather of one flat float32 block per rank through peer-to-peer stores over
    NVLink instead of a library collective: `tq_peer_push` writes this rank's block into
    every rank's receive slot and raises a flag there, `tq_peer_wait` lets the stream
    continue once all ranks' flags show the current epoch.  The buffers are torch
    symmetric memory (one allocation per rank, mapped into every process of the group);
    two slots alternate so that a rank that is one exchange ahead never overwrites a
    block that is still being merged.  All ranks must call `exchange` the same number
    of times.  Multicast mappings are not used (and switched off before the rendezvous)."""

    def __init__(self, n_floats: int, device, group=None, slots: int = 2):
        """`slots`: receive slots per rank.  Two alternate by exchange (the default protocol of
        `exchange` / `push` / `next_fused`); a caller that addresses slots itself through `targets`
        (one per layer of a replayed decode step, say) may ask for more."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        if n_floats % 4:
            raise ValueError("the block must be a multiple of 4 floats (16 bytes)")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.n = n_floats
        self.device = torch.device(device)
        self.slots = max(2, int(slots))
        self.data = symm.empty((self.slots, self.world, n_floats), dtype=torch.float32, device=self.device)
        self.flags = symm.empty((self.slots, 64), dtype=torch.int32, device=self.device)
        self.data.zero_()
        self.flags.zero_()
        self._hd = symm.rendezvous(self.data, self.group)
        self._hf = symm.rendezvous(self.flags, self.group)
        self.status = torch.zeros((4,), dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)          # every rank's buffers are zeroed before anyone pushes
        self.epoch = 0
        self._slot_uses = [0, 0]
        vp = ctypes.c_void_p
        self._dst, self._flg = [], []
        for slot in range(2):
            d = (vp * self.world)(*[int(self._hd.buffer_ptrs[p]) + (slot * self.world + self.rank) * n_floats * 4
                                    for p in range(self.world)])
            f = (vp * self.world)(*[int(self._hf.buffer_ptrs[p]) + (slot * 64 + self.rank) * 4
                                    for p in range(self.world)])
            self._dst.append(d)
            self._flg.append(f)

    def exchange(self, send: torch.Tensor) -> torch.Tensor:
        """Push `send` (n_floats,) to all ranks; returns the (world, n_floats) block of this
        exchange, valid in stream order.  Nothing here synchronises with the host."""
        if send.numel() != self.n or send.dtype != torch.float32 or not send.is_contiguous():
            raise ValueError("send must be a contiguous float32 tensor of the size given at construction")
        self.epoch += 1
        slot = self.epoch & 1
        lib, stream = _lib.lib(), _lib.stream_ptr(self.device)
        _lib.check(lib.tq_peer_push(_lib.ptr(send), self.n * 4, self._dst[slot], self._flg[slot], self.world,
                                    self.epoch, stream))
        _lib.check(lib.tq_peer_wait(_lib.ptr(self.flags[slot]), self.world, self.epoch, _lib.ptr(self.status), stream))
        return self.data[slot]

    def push(self, send: torch.Tensor):
        """First half of `exchange`: push only.  Returns (block view, flags pointer, epoch) for a
        merge that waits inside its own kernel (`MergePlan.run_after_peers`)."""
        self.epoch += 1
        slot = self.epoch & 1
        _lib.check(_lib.lib().tq_peer_push(_lib.ptr(send), self.n * 4, self._dst[slot], self._flg[slot], self.world,
                                           self.epoch, _lib.stream_ptr(self.device)))
        return self.data[slot], _lib.ptr(self.flags[slot]), self.epoch

    # ---- push done by the decode kernel itself -------------------------------------------------
    def targets(self, slot: int, rows: int, dim: int, exclusive: bool = False) -> dict:
        """Peer addresses of this rank's block in `slot` for `flash_decode(..., peers=...)`: the block
        is laid out [m (rows) | l (rows) | acc (rows * dim)] as in `partial_buffer`.  The decode
        kernel adds 1 to every rank's flag word per (batch, kv head) group it completes, so an
        exchange object must be used either this way or through `push` / `exchange`, not both.
        `exclusive`: the slot is used by no other exchange that may be in flight at the same time
        (one slot per layer), so a decode call that waits for nothing may store into it at once."""
        if rows * (dim + 2) != self.n:
            raise ValueError("rows * (dim + 2) must equal the block size given at construction")
        base = [int(self._hd.buffer_ptrs[p]) + (slot * self.world + self.rank) * self.n * 4 for p in range(self.world)]
        return dict(m=base, l=[b + rows * 4 for b in base], acc=[b + 2 * rows * 4 for b in base],
                    counter=[int(self._hf.buffer_ptrs[p]) + (slot * 64 + self.rank) * 4 for p in range(self.world)],
                    exclusive=exclusive)

    def gather_spec(self, slot: int, rows: int, dim: int) -> dict:
        """This rank's own view of `slot` for `flash_decode(..., peers=..., gather=...)`: where the
        ranks' blocks arrive, and the counters their pushes add to (the decode kernel waits on them,
        merges the blocks and puts the counters back to zero)."""
        if rows * (dim + 2) != self.n:
            raise ValueError("rows * (dim + 2) must equal the block size given at construction")
        base = self.data[slot].data_ptr()
        return dict(m=base, l=base + rows * 4, acc=base + 2 * rows * 4, part_stride=self.n,
                    flags=self.flags[slot].data_ptr(), n_ranks=self.world)

    def next_fused(self, groups: int):
        """Bookkeeping of one exchange whose push is done by the decode kernel: returns (slot, block
        view, flags pointer, counter value to wait for).  `groups` = batch * n_kv_heads additions
        arrive from every rank per exchange."""
        self.epoch += 1
        slot = self.epoch & 1
        self._slot_uses[slot] += 1
        return slot, self.data[slot], _lib.ptr(self.flags[slot]), self._slot_uses[slot] * groups

    def check(self) -> None:
        """Synchronises; raises if a bounded wait gave up (a rank never pushed)."""
        code = int(self.status[0].item())
        if code:
            raise RuntimeError(f"peer exchange: no block from rank {code - 21} within the wait limit")


def sequence_parallel_decode(q, *, k, v, attn_scale: float, group=None, out_dtype=None,
                             q_prerotated: bool = False, mask=None, send_buf=None,
                             recv_buf=None, exchange: "PeerExchange | None" = None,
                             check: bool = False) -> torch.Tensor:
    """Decode attention with the sequence split across the ranks of `group`.

    q (B, n_q, dim) is replicated; `k` / `v` describe this rank's chunk of
    positions (formats as in `kernels.flash_decode`).  Returns (B, n_q, dim) on
    every rank.  A rank whose chunk is empty passes k = v = None.  With `exchange`
    (a PeerExchange sized rows * (dim + 2) floats) the partial states travel by peer
    stores instead of the all_gather; its waits are bounded, and a wait that gave up leaves NaN in
    the output and a code in `exchange.status`: call `exchange.check()` at your next host
    synchronisation point, or pass check=True here (which synchronises on every call and also
    validates the gathered block with `check_partials`)."""
    B, n_q, dim = q.shape
    rows = B * n_q
    dev = q.device
    if send_buf is None:
        send_buf = partial_buffer(rows, dim, dev)[0]
    m, l, acc = partial_views(send_buf, rows, dim)
    if k is None:
        send_buf.zero_()          # l == 0 marks an empty chunk; it merges as a no-op
    else:
        kernels.flash_decode(q, k=k, v=v, attn_scale=attn_scale, q_prerotated=q_prerotated, mask=mask,
                             partials=True,
                             partial_out=(m.view(B, n_q), l.view(B, n_q), acc.view(B, n_q, dim)))
    recv = exchange.exchange(send_buf) if exchange is not None else gather_partials(send_buf, group, recv_buf)
    if check:
        if exchange is not None:
            exchange.check()
        check_partials(recv, rows, dim)
    gm, gl, gacc = partial_views(recv, rows, dim)
    signs = v["signs"] if (v is not None and v.get("format") == "polar") else None
    out = kernels.merge_partials(gm, gl, gacc, signs, out_dtype or q.dtype)
    return out.view(B, n_q, dim)
