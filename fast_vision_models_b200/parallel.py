"""Multi-GPU plumbing: batch-sharded replicas, one process per GPU, no collective on the forward path.

The reference is single-process / single-GPU. Inference shards by images, so the only exchanges are optional and sit
outside the forward: a final gather of logits or class maps, and the reduction of timings for reporting.
All functions work on any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests) and degrade to no-ops when
no process group is initialised.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def world() -> Tuple[int, int]:
    """(rank, world_size); (0, 1) without a process group."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_range(n_items: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous [start, end) of `n_items` owned by `rank`; earlier ranks take the remainder (sizes differ by <= 1)."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world size")
    base, rem = divmod(n_items, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_batch(x: torch.Tensor) -> torch.Tensor:
    """This rank's slice of a global batch (dimension 0)."""
    rank, ws = world()
    a, b = shard_range(x.shape[0], rank, ws)
    return x[a:b]


def gather_batch(local: torch.Tensor, global_items: int) -> torch.Tensor:
    """All ranks' per-image results (logits [n_local, ...] or class maps) concatenated in rank order on every rank.
    Shards may differ by one item: they are padded to the largest shard for the all_gather and trimmed after."""
    rank, ws = world()
    if ws == 1:
        return local
    sizes = [shard_range(global_items, r, ws) for r in range(ws)]
    most = max(b - a for a, b in sizes)
    buf = local
    if local.shape[0] < most:
        pad = torch.zeros((most - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        buf = torch.cat([local, pad], 0)
    outs: List[torch.Tensor] = [torch.empty_like(buf) for _ in range(ws)]
    dist.all_gather(outs, buf.contiguous())
    return torch.cat([o[: b - a] for o, (a, b) in zip(outs, sizes)], 0)


def max_over_ranks(values: List[float], device=None) -> List[float]:
    """Element-wise maximum of a list of floats over all ranks (timings are reported as the slowest rank's)."""
    rank, ws = world()
    if ws == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]
