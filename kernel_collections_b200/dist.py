"""Batch (or head) sharding across the GPUs of one box.

Every batch row of a decode step is independent, so the batch is cut into contiguous shards,
each rank runs the single-GPU op on its shard, and one all-gather puts the outputs together.
Nothing else crosses NVLink.  The functions take the local op as a callable, so the shard /
gather logic is testable on CPU ranks (gloo) without a GPU.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def shard_bounds(total: int, world_size: int, rank: int):
    """Contiguous, balanced [begin, end) of `total` items for `rank` (first ranks get the extras)."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world size")
    base, extra = divmod(total, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch(tensors: Sequence[torch.Tensor], world_size: int, rank: int, dim: int = 0):
    """Slice every tensor to this rank's shard along `dim` (views, no copy)."""
    out = []
    for t in tensors:
        lo, hi = shard_bounds(t.shape[dim], world_size, rank)
        out.append(t.narrow(dim, lo, hi - lo))
    return out


def all_gather_outputs(local: torch.Tensor, total: int, group=None, dim: int = 0) -> torch.Tensor:
    """All-gather per-rank outputs whose `dim` sizes follow shard_bounds(total, W, r).

    Equal shards along dim 0 use one all_gather_into_tensor (a single NCCL kernel on
    NVLink); ragged shards or another dim fall back to all_gather on padded buffers."""
    W = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if W == 1:
        return local
    sizes = [shard_bounds(total, W, r)[1] - shard_bounds(total, W, r)[0] for r in range(W)]
    if local.shape[dim] != sizes[rank]:
        raise ValueError("local output does not match this rank's shard")
    if dim == 0 and len(set(sizes)) == 1 and local.is_contiguous():
        out = local.new_empty((total,) + tuple(local.shape[1:]))
        dist.all_gather_into_tensor(out, local, group=group)
        return out
    mx = max(sizes)
    moved = local.movedim(dim, 0).contiguous()
    pad = moved.new_zeros((mx,) + tuple(moved.shape[1:]))
    pad[: sizes[rank]] = moved
    bufs = [torch.empty_like(pad) for _ in range(W)]
    dist.all_gather(bufs, pad, group=group)
    out = torch.cat([bufs[r][: sizes[r]] for r in range(W)], dim=0)
    return out.movedim(0, dim)


def sharded_decode(local_op: Callable[..., torch.Tensor], batch_tensors: Sequence[torch.Tensor],
                   *args, group=None, presharded: bool = False, **kwargs) -> torch.Tensor:
    """Run `local_op(*batch_shards, *args, **kwargs)` on this rank's batch shard and all-gather
    the outputs along the batch.  With presharded=True the tensors already hold only this
    rank's rows (the layout a real deployment keeps: each GPU owns its sequences' caches)."""
    W = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = list(batch_tensors) if presharded else shard_batch(batch_tensors, W, rank)
    local = local_op(*shards, *args, **kwargs)
    total = local.shape[0] * W if presharded else batch_tensors[0].shape[0]
    return all_gather_outputs(local, total, group=group)


def head_sharded_decode(local_op: Callable[..., torch.Tensor], head_tensors: Sequence[torch.Tensor],
                        head_dims: Sequence[int], *args, group=None, out_head_dim: int = 1, **kwargs):
    """MLA-style head sharding: tensors in `head_tensors` are cut along their `head_dims`, the
    latent is replicated (passed in *args), and outputs are gathered along the head axis."""
    W = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = []
    for t, d in zip(head_tensors, head_dims):
        lo, hi = shard_bounds(t.shape[d], W, rank)
        shards.append(t.narrow(d, lo, hi - lo))
    local = local_op(*shards, *args, **kwargs)
    total = head_tensors[0].shape[head_dims[0]]
    return all_gather_outputs(local, total, group=group, dim=out_head_dim)


class PeerAllGather:
    """All-gather of equal per-rank output shards along dim 0 with the library's peer-store kernel
    (xkv_peer_allgather) instead of a collective: one small launch per step, for decode steps short enough
    that a collective's 30-60 us show.  The gather buffer lives in symmetric memory (every rank's copy is
    mapped into all ranks of the box); two halves alternate between calls, so the tensor returned by call n
    stays valid until call n + 2.

    Construction is collective over `group` and raises if symmetric memory cannot be set up on this system
    (callers then keep `all_gather_outputs`).  The host-side bookkeeping (layout, epochs, halves) is in
    `PeerGatherPlan`, which needs no GPU."""

    def __init__(self, local_shape, dtype, device, group=None):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from . import _C
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.plan = PeerGatherPlan(local_shape, torch.empty((), dtype=dtype).element_size(), self.world)
        self.local_shape, self.dtype, self.device = tuple(local_shape), dtype, device
        self.buf = symm_mem.empty(self.plan.total_bytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe this group's buffers")
        self._ptrs = (C.c_void_p * self.world)(*ptrs)
        self._status = torch.zeros(8, dtype=torch.int32, device=device)
        self._lib = _C.load()
        self._check = _C.check
        dist.barrier(group)                  # every rank's flags are zero before anyone publishes into them

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        if tuple(local.shape) != self.local_shape or local.dtype != self.dtype or not local.is_contiguous():
            raise ValueError("local shard does not match the shape / dtype this gather was built for")
        epoch, half_off = self.plan.next_call()
        with torch.cuda.device(self.device):
            rc = self._lib.xkv_peer_allgather(local.data_ptr(), self.plan.shard_bytes, self._ptrs, self.plan.flags_offset,
                                              self.rank, self.world, epoch, self._status.data_ptr(),
                                              torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "xkv_peer_allgather")
        out = self.buf[half_off: half_off + self.world * self.plan.shard_bytes].view(self.dtype)
        return out.view((self.world * self.local_shape[0],) + self.local_shape[1:])

    def status(self):
        """(code, role, peer, epoch) left by a wait that gave up; (0, ...) when all peers showed up."""
        return tuple(self._status[:4].tolist())


class PeerGatherPlan:
    """Layout and call bookkeeping of PeerAllGather: [2 halves][world][shard] then `world` flag words."""

    def __init__(self, local_shape, elem_size: int, world: int):
        n = 1
        for d in local_shape:
            n *= int(d)
        self.shard_bytes = n * elem_size
        if self.shard_bytes == 0 or self.shard_bytes % 16 != 0:
            raise ValueError("a shard must be a non-empty multiple of 16 bytes")
        if not (1 <= world <= 16):
            raise ValueError("1 to 16 ranks")
        self.world = world
        self.flags_offset = 2 * world * self.shard_bytes
        self.total_bytes = self.flags_offset + 256
        self.epoch = 0

    def next_call(self):
        """(epoch, byte offset of the half this call fills); epochs start at 1 and alternate the halves."""
        self.epoch += 1
        if self.epoch >= 2 ** 32:
            raise OverflowError("epoch counter exhausted")
        return self.epoch, (self.epoch & 1) * self.world * self.shard_bytes
