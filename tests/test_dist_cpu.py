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


def test_peer_gather_plan_layout_and_epochs():
    """Host side of the peer-store all-gather: buffer layout, the alternation of the two halves, argument checks
    (the kernel side needs GPUs that can map each other's memory)."""
    from kernel_collections_b200.dist import PeerGatherPlan
    p = PeerGatherPlan((16, 32, 1, 128), 2, 8)
    assert p.shard_bytes == 16 * 32 * 128 * 2
    assert p.flags_offset == 2 * 8 * p.shard_bytes and p.total_bytes >= p.flags_offset + 8 * 4
    calls = [p.next_call() for _ in range(5)]
    assert [e for e, _ in calls] == [1, 2, 3, 4, 5]
    assert [off for _, off in calls] == [8 * p.shard_bytes, 0, 8 * p.shard_bytes, 0, 8 * p.shard_bytes]
    with pytest.raises(ValueError):
        PeerGatherPlan((3, 1), 2, 4)          # 6 bytes: not a multiple of 16
    with pytest.raises(ValueError):
        PeerGatherPlan((8,), 2, 17)
    # the C entry point rejects what the kernel could not handle, without a GPU
    import ctypes as C
    from kernel_collections_b200 import _C
    lib = _C.load()
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    assert lib.xkv_peer_allgather(None, 1024, ptrs, 4096, 0, 2, 1, None, None) == -1
    assert lib.xkv_peer_allgather(0x4000, 1000, ptrs, 4096, 0, 2, 1, None, None) == -3      # shard not a multiple of 16
    assert lib.xkv_peer_allgather(0x4000, 1024, ptrs, 1024, 0, 2, 1, None, None) == -1      # flags inside the data
    assert lib.xkv_peer_allgather(0x4000, 1024, ptrs, 4096, 0, 2, 0, None, None) == -1      # epoch 0 is the empty state
    assert lib.xkv_peer_allgather(0x4000, 1024, ptrs, 4096, 2, 2, 1, None, None) == -1      # rank out of range
