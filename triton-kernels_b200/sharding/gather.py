"""Optional collection of output shards on every rank.

The attention path needs no collective to compute; when a caller wants the whole
output on each rank this is one ``all_gather`` over the process group (NCCL over
NVLink on GPUs, gloo on CPU for the tests)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def all_gather_outputs(shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """Gather equally shaped shards; returns the list ordered by rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return [shard]
    flat = shard.contiguous()
    out = torch.empty((world * flat.shape[0],) + tuple(flat.shape[1:]), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return list(out.chunk(world, dim=0))


def all_gather_ragged(shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """Gather shards whose leading dimension differs per rank (ragged prefill partitions)."""
    world = dist.get_world_size(group)
    if world == 1:
        return [shard]
    n = torch.tensor([shard.shape[0]], dtype=torch.int64, device=shard.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(s.item()) for s in sizes]
    cap = max(sizes)
    padded = torch.zeros((cap,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    padded[: shard.shape[0]] = shard
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded, group=group)
    return [b[:s] for b, s in zip(bufs, sizes)]
