"""Batch-sharded signature on two GPUs (NCCL): each rank computes its slice, the optional
all-gather returns the full output on every rank, and gradients flow back to the local slice.
Skipped on machines with a single GPU."""
from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    import pathsig_b200 as ps
    from pathsig_b200.distributed import gather_batch, shard_batch, shard_bounds

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(13, 30, 8, generator=g).cumsum(1)            # ragged shards: 7 + 6 paths
        w = torch.randn(13, 4680, generator=g)
        dev = torch.device("cuda", rank)
        mine = shard_batch(x).to(dev).requires_grad_(True)
        lo, hi = shard_bounds(13, rank, world)
        sig = ps.Signature(depth=4)
        full = gather_batch(sig(mine))                                 # (13, 4680) on every rank
        (full * w.to(dev)).sum().backward()
        xr = x.to(dev).requires_grad_(True)                            # single-GPU reference
        ref = sig(xr)
        (ref * w.to(dev)).sum().backward()
        ok = torch.allclose(full, ref.detach(), rtol=1e-5, atol=1e-6) and \
            torch.allclose(mine.grad, xr.grad[lo:hi], rtol=1e-4, atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_signature_with_gather_on_two_gpus():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert dict(q.get(timeout=10) for _ in range(world)) == {0: True, 1: True}
