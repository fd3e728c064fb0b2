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

import torch
import torch.distributed as dist

from . import kernels


def shard_range(n_items: int, world: int, rank: int):
    """Contiguous [start, stop) of `n_items` (sequences, kv heads or positions)
    owned by `rank`; the first n_items % world ranks get one extra item."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def partial_buffer(rows: int, dim: int, device, world: int = 1) -> torch.Tensor:
    """(world, rows * (dim + 2)) float32: per rank [m (rows) | l (rows) | acc (rows * dim)]."""
    return torch.empty((world, rows * (dim + 2)), dtype=torch.float32, device=device)


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


def sequence_parallel_decode(q, *, k, v, attn_scale: float, group=None, out_dtype=None,
                             q_prerotated: bool = False, mask=None, send_buf=None,
                             recv_buf=None) -> torch.Tensor:
    """Decode attention with the sequence split across the ranks of `group`.

    q (B, n_q, dim) is replicated; `k` / `v` describe this rank's chunk of
    positions (formats as in `kernels.flash_decode`).  Returns (B, n_q, dim) on
    every rank.  A rank whose chunk is empty passes k = v = None."""
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
    recv = gather_partials(send_buf, group, recv_buf)
    gm, gl, gacc = partial_views(recv, rows, dim)
    signs = v["signs"] if (v is not None and v.get("format") == "polar") else None
    out = kernels.merge_partials(gm, gl, gacc, signs, out_dtype or q.dtype)
    return out.view(B, n_q, dim)
