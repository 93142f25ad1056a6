"""The peer-store all-gather (xkv_peer_allgather) on two GPUs of one box: one rank per GPU (child processes,
NCCL group for the rendezvous and for the comparison), shards written straight into every rank's symmetric
buffer, against torch.distributed.all_gather_into_tensor on the same shards, over several steps (both halves
of the buffer, epochs).  Skipped where fewer than two GPUs are visible or symmetric memory cannot be set up."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from kernel_collections_b200.dist import PeerAllGather
        shape = (4, 32, 1, 128)
        try:
            pg = PeerAllGather(shape, torch.bfloat16, dev)
        except Exception as e:  # no symmetric memory on this system: nothing to test
            q.put((rank, "skip", repr(e)))
            return
        ok = True
        for step in range(6):
            g = torch.Generator(device=dev).manual_seed(100 * step + rank)
            local = torch.randn(shape, generator=g, device=dev).bfloat16()
            got = pg(local)
            want = local.new_empty((world * shape[0],) + shape[1:])
            dist.all_gather_into_tensor(want, local)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want) and pg.status()[0] == 0
        q.put((rank, "ok" if ok else "mismatch", ""))
    finally:
        dist.destroy_process_group()


def test_peer_gather_matches_nccl_all_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, "a rank did not finish"
    results = [q.get(timeout=5) for _ in range(world)]
    if any(r[1] == "skip" for r in results):
        pytest.skip(f"symmetric memory unavailable: {results[0][2]}")
    assert all(r[1] == "ok" for r in results), results
