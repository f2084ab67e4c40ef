"""Batch sharding across the GPUs of one box.

The reference is single-device (no ``torch.distributed``, no NCCL anywhere in it).  Every
(path, window) unit of the signature is independent, so the natural multi-GPU form is one
process per GPU, each owning a contiguous slice of the batch, with **no collective on the hot
path**.  This module holds the two host-side helpers for that layout:

* :func:`shard_bounds` / :func:`shard_batch` — the slice of the batch a rank owns;
* :func:`gather_batch` — only for callers that want the full ``(B, D)`` output on every rank:
  an all-gather of the per-rank outputs (NCCL over NVLink on GPUs, gloo in the CPU tests).
  It is differentiable.  By default the backward of a gathered output is the local slice of the
  incoming gradient: that is the full gradient when every rank evaluates the SAME loss on the
  gathered tensor (replicated loss), which is the usual data-parallel case.  When ranks evaluate
  different losses on it (per-rank contrastive or metric terms), pass ``reduce_grads=True``: the
  backward then sums every rank's gradient for this rank's rows (a reduce-scatter).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(batch: int, rank: int, world_size: int) -> Tuple[int, int]:
    """[lo, hi) of ``rank``'s slice; the first ``batch % world_size`` ranks hold one extra path."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    base, extra = divmod(batch, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _rank_world(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def shard_batch(x: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's contiguous slice of ``x`` along dimension 0 (a view, no copy)."""
    rank, world = _rank_world(group)
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi]


class _GatherBatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, local: torch.Tensor, group, sizes: List[int], reduce_grads: bool):
        rank, world = _rank_world(group)
        ctx.lo = sum(sizes[:rank])
        ctx.n = sizes[rank]
        ctx.group, ctx.sizes, ctx.reduce_grads = group, list(sizes), bool(reduce_grads)
        local = local.contiguous()
        if len(set(sizes)) == 1:
            out = local.new_empty((sum(sizes),) + tuple(local.shape[1:]))
            dist.all_gather_into_tensor(out, local, group=group)
            return out
        # ragged shards: pad to the largest, gather, trim
        widest = max(sizes)
        padded = local.new_zeros((widest,) + tuple(local.shape[1:]))
        padded[: local.shape[0]] = local
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded, group=group)
        return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        if not ctx.reduce_grads:
            return grad_out[ctx.lo: ctx.lo + ctx.n].contiguous(), None, None, None
        # every rank holds a gradient for every row: sum them and keep this rank's rows
        sizes, world = ctx.sizes, len(ctx.sizes)
        grad_out = grad_out.contiguous()
        if len(set(sizes)) == 1:
            mine = grad_out.new_empty((ctx.n,) + tuple(grad_out.shape[1:]))
            dist.reduce_scatter_tensor(mine, grad_out, op=dist.ReduceOp.SUM, group=ctx.group)
            return mine, None, None, None
        # ragged shards: pad every rank's block to the largest, reduce-scatter, trim
        widest, offsets = max(sizes), [sum(sizes[:r]) for r in range(world)]
        padded = grad_out.new_zeros((world * widest,) + tuple(grad_out.shape[1:]))
        for r, (lo, n) in enumerate(zip(offsets, sizes)):
            padded[r * widest: r * widest + n] = grad_out[lo: lo + n]
        mine = grad_out.new_empty((widest,) + tuple(grad_out.shape[1:]))
        dist.reduce_scatter_tensor(mine, padded, op=dist.ReduceOp.SUM, group=ctx.group)
        return mine[: ctx.n].contiguous(), None, None, None


def gather_batch(local: torch.Tensor, group=None, sizes: Optional[List[int]] = None,
                 reduce_grads: bool = False) -> torch.Tensor:
    """All ranks' outputs concatenated along dimension 0, on every rank.

    ``sizes`` are the per-rank batch sizes; when omitted they are exchanged first (one small
    all-gather).  With a single process this is the identity.

    Gradient: with ``reduce_grads=False`` (default) each rank keeps the slice of its own incoming
    gradient that belongs to its rows -- correct when all ranks differentiate the same loss of the
    gathered tensor.  With ``reduce_grads=True`` the incoming gradients of all ranks are summed for
    these rows (one reduce-scatter), which is what rank-dependent losses need.
    """
    rank, world = _rank_world(group)
    if world == 1:
        return local
    if sizes is None:
        mine = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine, group=group)
        sizes = [int(t.item()) for t in every]
    if len(sizes) != world or sizes[rank] != local.shape[0]:
        raise ValueError("sizes must list every rank's batch size")
    return _GatherBatch.apply(local, group, list(sizes), reduce_grads)
