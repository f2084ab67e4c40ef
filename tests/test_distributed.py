"""Batch-sharding helpers on 2 CPU ranks (gloo).  The signature itself needs a GPU, so the
per-rank "operator" here is a differentiable stand-in with one row per path; what is tested is
the host-side sharding and the gather + its backward."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pathsig_b200.distributed import gather_batch, shard_batch, shard_bounds


def test_shard_bounds_cover_the_batch():
    for batch in (0, 1, 7, 8, 4096):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_single_process_is_identity():
    x = torch.arange(12.0).reshape(6, 2)
    assert shard_batch(x).data_ptr() == x.data_ptr()
    assert gather_batch(x) is x


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(batch, 5, 3, generator=g, dtype=torch.float64)
        weight = torch.randn(batch, 4, generator=g, dtype=torch.float64)
        mine = shard_batch(x).clone().requires_grad_(True)
        lo, hi = shard_bounds(batch, rank, world)
        assert mine.shape[0] == hi - lo
        local_out = torch.stack([mine.sum((1, 2)), (mine ** 2).sum((1, 2)), mine[:, -1, 0], mine[:, 0, 1]], dim=1)
        full = gather_batch(local_out)
        assert full.shape == (batch, 4)
        (full * weight).sum().backward()
        # single-process reference
        xr = x.clone().requires_grad_(True)
        ref_out = torch.stack([xr.sum((1, 2)), (xr ** 2).sum((1, 2)), xr[:, -1, 0], xr[:, 0, 1]], dim=1)
        (ref_out * weight).sum().backward()
        ok = torch.allclose(full, ref_out.detach()) and torch.allclose(mine.grad, xr.grad[lo:hi])
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 7])  # even and ragged shards
def test_gather_and_its_backward_on_two_ranks(batch):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {0: True, 1: True}


def _worker_rank_losses(rank, world, port, batch, q):
    """Each rank differentiates its OWN loss of the gathered tensor: the gradient of a rank's rows is the
    sum over all ranks' losses, which needs reduce_grads=True."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        x = torch.randn(batch, 3, generator=g, dtype=torch.float64)
        weights = [torch.randn(batch, 3, generator=g, dtype=torch.float64) for _ in range(world)]
        mine = shard_batch(x).clone().requires_grad_(True)
        lo, hi = shard_bounds(batch, rank, world)
        full = gather_batch(mine * 2.0, reduce_grads=True)
        (full * weights[rank]).sum().backward()                      # this rank's loss
        expect = 2.0 * sum(weights)[lo:hi]                            # d(sum of all ranks' losses) / d(mine)
        q.put((rank, bool(torch.allclose(mine.grad, expect))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 7])
def test_gather_with_rank_dependent_losses_reduces_the_gradients(batch):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_rank_losses, args=(r, world, port, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(q.get(timeout=10) for _ in range(world)) == {0: True, 1: True}
