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
