"""Partitioning of the attention work across the GPUs of one box.

Every (sequence, KV-head group) is independent in all three entry points
(reference: ``batch = pid1 // Q_HEADS; kv_head = q_head * KV_HEADS // Q_HEADS``,
kernels/attention.py:461-463, kernels/decode.py:46-48), so the path shards with no
data-path collective.  These helpers are pure Python and are tested on CPU.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def contiguous_shard(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the units rank owns when n_units are dealt out in contiguous, near-equal runs."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n_units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def batch_head_units(batch: int, kv_heads: int, world: int, rank: int) -> List[Tuple[int, int]]:
    """Dense prefill: the (batch, kv_head) units of this rank, contiguous in batch-major order."""
    begin, end = contiguous_shard(batch * kv_heads, world, rank)
    return [(u // kv_heads, u % kv_heads) for u in range(begin, end)]


def balance_sequences(lengths: Sequence[int], world: int, *, causal_prefill: bool = True) -> List[List[int]]:
    """Longest-processing-time greedy assignment of sequences to ranks.

    The cost of a causal prefill sequence grows with L^2 (L(L+1)/2 score entries), of a decode
    sequence with L; ties keep the lower sequence index first so the plan is deterministic."""
    if world <= 0:
        raise ValueError("world must be positive")
    cost = [(n * (n + 1) // 2) if causal_prefill else n for n in (int(x) for x in lengths)]
    order = sorted(range(len(cost)), key=lambda i: (-cost[i], i))
    loads = [0] * world
    bins: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        bins[r].append(i)
        loads[r] += cost[i]
    for b in bins:
        b.sort()
    return bins


def kv_head_shard(kv_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """Speculative decode at scale: each rank owns a contiguous run of KV heads (one head per GPU at 8 GPUs
    with 8 KV heads).  When there are more ranks than heads the surplus ranks replicate heads round-robin."""
    if world <= kv_heads:
        return contiguous_shard(kv_heads, world, rank)
    h = rank % kv_heads
    return h, h + 1
