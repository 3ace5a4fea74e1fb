"""Sharding layer: start rows split across ranks, one process per GPU.

Walks are independent, the CSR is replicated in every GPU's memory and read-only, so
the walk itself needs no collective. Two layouts: ``"block"`` -- rank ``r`` of ``G`` walks
the contiguous rows ``shard_range(n, G, r)``; ``"cyclic"`` -- rank ``r`` walks rows
``r, r + G, ...``. Cyclic is the default of the bench: on generated graphs node ids are
correlated with degree (R-MAT: low ids are hubs, high ids are often isolated), and block
shards then differ by a quarter in work. node2vec draws are indexed by the *global* row
(``walk_index_base``/``walk_index_stride``), so the union of the shards is bit-identical
to a single-GPU run whatever ``G`` and the layout are. The one
optional exchange is the gather of the walk matrix to one rank, done with point-to-point
sends posted as one batch (rows land at their global offset; the destination rank's own
walk kernel writes straight into its slice of the gathered matrix).

The reference has no counterpart: it is a single-device library.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib


def shard_range(num_walks: int, world_size: int, rank: int):
    """Rows ``[begin, end)`` of rank ``rank``: blocks of ``ceil(n / world_size)`` rows."""
    return _lib.shard_range(num_walks, world_size, rank)


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def shard_rows(num_walks: int, world_size: int, rank: int, layout: str = "block"):
    """The rows of rank ``rank`` as a ``slice`` (``start:stop:step``) and the
    ``(walk_index_base, walk_index_stride)`` of its first row."""
    if layout == "block":
        b, e = shard_range(num_walks, world_size, rank)
        return slice(b, e, 1), (b, 1)
    if layout == "cyclic":
        count = _lib.shard_count_cyclic(num_walks, world_size, rank)
        return slice(rank, rank + count * world_size if count else rank, world_size), (rank, world_size)
    raise ValueError(f"unknown layout {layout!r}")


def gather_rows_cyclic(shard: torch.Tensor, num_rows: int, *, group=None, dst: int = 0,
                       chunk_rows: int = 1 << 22):
    """Collect cyclic shards on ``dst``: rank r's rows land at ``r::world``. A received message is a
    contiguous run of one rank's rows, so the cyclic layout cannot be received in place: all shards
    arrive, in one batch of point-to-point messages, in a staging buffer and are interleaved by one
    strided copy per source. Costs a second copy of the matrix on ``dst``; the block layout
    (:func:`gather_rows`) needs neither the staging nor the interleave."""
    world, rank = _world(group)
    if world == 1:
        return shard
    width = shard.shape[1]
    peer = (lambda r: dist.get_global_rank(group, r)) if group else (lambda r: r)
    if rank != dst:
        ops = [dist.P2POp(dist.isend, shard[c0:min(shard.shape[0], c0 + chunk_rows)], peer(dst), group)
               for c0 in range(0, shard.shape[0], chunk_rows)]
        for req in (dist.batch_isend_irecv(ops) if ops else []):
            req.wait()
        return None
    counts = [_lib.shard_count_cyclic(num_rows, world, r) for r in range(world)]
    stage = torch.empty((sum(c for r, c in enumerate(counts) if r != dst), width), dtype=shard.dtype,
                        device=shard.device)
    ops, at, where = [], 0, {}
    for r in range(world):
        if r == dst or counts[r] == 0:
            continue
        where[r] = at
        for c0 in range(0, counts[r], chunk_rows):
            c1 = min(counts[r], c0 + chunk_rows)
            ops.append(dist.P2POp(dist.irecv, stage[at + c0:at + c1], peer(r), group))
        at += counts[r]
    reqs = dist.batch_isend_irecv(ops) if ops else []
    full = torch.empty((num_rows, width), dtype=shard.dtype, device=shard.device)
    full[rank::world].copy_(shard)  # overlaps the transfers
    for req in reqs:
        req.wait()
    for r, at in where.items():
        full[r::world].copy_(stage[at:at + counts[r]])
    return full


def gather_rows(shard: torch.Tensor, num_rows: int, *, group=None, dst: int = 0,
                out: Optional[torch.Tensor] = None, chunk_rows: int = 1 << 22, row_range=None):
    """Collect row shards (``shard_range`` layout) on rank ``dst``.

    Returns the ``[num_rows, width]`` matrix on ``dst`` and ``None`` elsewhere. When
    ``out`` is given on ``dst`` and ``shard`` already is the matching slice of ``out`` (the
    destination's own walk kernel wrote it there), no local copy is made. Every other rank's rows are
    received straight at their row offset; all messages (pieces of ``chunk_rows`` rows) are posted as one
    batch, so the transfers of all sources run at the same time and the destination's inbound link is
    the bound. ``row_range=(lo, hi)`` gathers only the global rows ``[lo, hi)`` into a
    ``[hi - lo, width]`` matrix: a walk matrix larger than one GPU's memory cannot be gathered whole.
    """
    world, rank = _world(group)
    width = shard.shape[1]
    lo, hi = (0, num_rows) if row_range is None else (int(row_range[0]), int(row_range[1]))
    if not 0 <= lo <= hi <= num_rows:
        raise ValueError(f"row_range {row_range} outside [0, {num_rows}]")
    if world == 1:
        part = shard[lo:hi]
        if out is None:
            return part
        if out.data_ptr() != part.data_ptr():
            out.copy_(part)
        return out
    peer = (lambda r: dist.get_global_rank(group, r)) if group else (lambda r: r)
    ops = []
    if rank == dst:
        if out is None:
            out = torch.empty((hi - lo, width), dtype=shard.dtype, device=shard.device)
        elif out.shape[0] != hi - lo:
            raise ValueError(f"out has {out.shape[0]} rows, the gathered range has {hi - lo}")
        for r in range(world):
            rb, re = shard_range(num_rows, world, r)
            b, e = max(rb, lo), min(re, hi)  # this rank's part of the range
            if b >= e:
                continue
            if r == dst:
                mine = shard[b - rb:e - rb]
                if out[b - lo:e - lo].data_ptr() != mine.data_ptr():
                    out[b - lo:e - lo].copy_(mine)
                continue
            for c0 in range(b, e, chunk_rows):
                c1 = min(e, c0 + chunk_rows)
                ops.append(dist.P2POp(dist.irecv, out[c0 - lo:c1 - lo], peer(r), group))
    else:
        rb, re = shard_range(num_rows, world, rank)
        assert shard.shape[0] == re - rb, "shard does not match shard_range"
        b, e = max(rb, lo), min(re, hi)
        for c0 in range(b, e, chunk_rows):
            c1 = min(e, c0 + chunk_rows)
            ops.append(dist.P2POp(dist.isend, shard[c0 - rb:c1 - rb], peer(dst), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out if rank == dst else None


def sharded_walk(op: Callable[..., torch.Tensor], start: torch.Tensor, walk_length: int, *,
                 rand: Optional[torch.Tensor] = None, group=None, gather: bool = False, dst: int = 0,
                 start_is_sharded: bool = False, num_walks: Optional[int] = None, layout: str = "block"):
    """Run ``op`` on this rank's share of the start rows.

    ``op(start_shard, rand_shard, walk_index_base, out)`` (block layout) or
    ``op(start_shard, rand_shard, (walk_index_base, walk_index_stride), out)`` (cyclic layout)
    must return the ``[rows, walk_length + 1]`` matrix (written into ``out`` when ``out`` is not
    None); the product callers pass a closure over :func:`random_walk` /
    :func:`rejection_sampling`. ``start`` (and ``rand``) are either the full arrays, replicated on
    every rank (default), or already this rank's share (``start_is_sharded=True`` with
    ``num_walks`` = global row count). Returns ``(shard, rows)`` -- ``rows`` is ``(begin, end)``
    for the block layout and the ``slice`` of global rows for the cyclic one -- or, with
    ``gather=True``, the full matrix on ``dst`` (None elsewhere) in place of the shard.
    """
    world, rank = _world(group)
    if start_is_sharded and num_walks is None:
        raise ValueError("num_walks is required when start is already sharded")
    n = int(num_walks) if start_is_sharded else start.shape[0]
    rows, (base, stride) = shard_rows(n, world, rank, layout)
    count = len(range(*rows.indices(n))) if layout == "cyclic" else rows.stop - rows.start
    if start_is_sharded:
        if start.shape[0] != count:
            raise ValueError(f"rank {rank} expects {count} start rows, got {start.shape[0]}")
        s_shard, r_shard = start, rand
    else:
        s_shard = start[rows].contiguous()
        r_shard = None if rand is None else rand.reshape(n, -1)[rows].contiguous()
    if layout == "cyclic":
        shard = op(s_shard, r_shard, (base, stride), None)
        if not gather:
            return shard, rows
        return gather_rows_cyclic(shard, n, group=group, dst=dst), rows
    b, e = rows.start, rows.stop
    out_view = None
    full = None
    if gather and rank == dst and world > 1:
        full = torch.empty((n, walk_length + 1), dtype=torch.int64, device=start.device)
        out_view = full[b:e]
    shard = op(s_shard, r_shard, b, out_view)
    if not gather:
        return shard, (b, e)
    return gather_rows(shard, n, group=group, dst=dst, out=full), (b, e)
