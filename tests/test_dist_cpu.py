"""world_size-2 gloo tests (CPU) of the batch / head shard + all-gather logic."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernel_collections_b200 import dist as xdist


def test_shard_bounds_cover_and_balance():
    for total in (1, 7, 16, 128, 129):
        for W in (1, 2, 3, 8):
            spans = [xdist.shard_bounds(total, W, r) for r in range(W)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        xdist.shard_bounds(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fake_local_op(q, kv, scale):
    # stands in for the CUDA op: any row-wise independent function of the batch shard
    return (q * scale + kv.sum(dim=1, keepdim=True)).contiguous()


def _worker(rank, world, port, total, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        q = torch.randn(total, 4, 8, generator=g)
        kv = torch.randn(total, 5, 8, generator=g)
        full = _fake_local_op(q, kv, 0.5)
        out = xdist.sharded_decode(_fake_local_op, [q, kv], 0.5)
        ok = torch.equal(out, full)
        # pre-sharded layout (each rank owns its rows), only for equal shards
        if total % world == 0:
            lo, hi = xdist.shard_bounds(total, world, rank)
            out2 = xdist.sharded_decode(_fake_local_op, [q[lo:hi], kv[lo:hi]], 0.5, presharded=True)
            ok = ok and torch.equal(out2, full)
        # head sharding: cut dim 1 of q, replicate kv, gather along heads
        def head_op(qh, kv_, s):
            return (qh * s + kv_.sum(dim=1, keepdim=True)[:, :, :]).contiguous()
        out3 = xdist.head_sharded_decode(head_op, [q], [1], kv, 0.5)
        ok = ok and torch.equal(out3, full)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [6, 7])
def test_sharded_decode_gloo_world2(total):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), total, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
