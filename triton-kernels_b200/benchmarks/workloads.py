"""Seeded synthetic workloads of the five benchmark configurations.

Lengths are drawn on the CPU with ``torch.Generator().manual_seed(seed)`` so that they are the
same on every machine; tensor values are N(0,1) cast to the dtype.  Every builder takes the
target device and an optional (rank, world) shard and returns a ``Workload`` whose ``run()``
calls the public entry point and whose ``flops`` / ``kv_bytes`` are the algorithmic figures
the roofline is computed from:

  prefill FLOPs  = sum over sequences of 4 * D * QH * (visible (q, k) pairs)
  decode bytes   = sum of lengths * KVH * D * 2 (K and V) * element size   (each KV byte once per KV head)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from sharding.planner import balance_sequences, contiguous_shard, kv_head_shard


@dataclass
class Workload:
    name: str
    kind: str                      # "prefill" | "decode" | "spec"
    run: Callable[[], torch.Tensor]
    tensors: Dict[str, torch.Tensor]
    meta: Dict[str, object]
    flops: float
    kv_bytes: float
    host_inputs: List[str] = field(default_factory=list)   # tensor names copied H2D per step end to end


def _lengths(seed: int, n: int, lo: int, hi: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def _randn(shape, dtype, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)


def c1_cpu_case(seed: int = 0):
    """fp32, batch 1, 8 q heads / 2 kv heads, seq 512, head_dim 64, causal; CPU tensors."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((512, 8, 64), generator=g)
    k = torch.randn((512, 2, 64), generator=g)
    v = torch.randn((512, 2, 64), generator=g)
    return q, k, v


def c2_dense_prefill(device, seed: int = 0, *, batch: int = 2, q_heads: int = 32, kv_heads: int = 8,
                     seq: int = 2048, head_dim: int = 128, dtype=torch.bfloat16,
                     shard: Tuple[int, int] = (0, 1), units: Optional[Sequence[Tuple[int, int]]] = None) -> Workload:
    """Dense causal GQA prefill.  ``units`` (list of (batch, kv_head)) restricts the call to a shard:
    the rank then holds q heads of those kv heads only, stacked along the batch axis."""
    from kernels.attention import flash_attention_v2

    group = q_heads // kv_heads
    if units is None:
        q = _randn((batch, q_heads, seq, head_dim), dtype, device, seed * 1000 + 1 + shard[0])
        k = _randn((batch, kv_heads, seq, head_dim), dtype, device, seed * 1000 + 2 + shard[0])
        v = _randn((batch, kv_heads, seq, head_dim), dtype, device, seed * 1000 + 3 + shard[0])
        n_units = batch * kv_heads
    else:
        n_units = len(units)
        q = _randn((n_units, group, seq, head_dim), dtype, device, seed * 1000 + 1 + shard[0])
        k = _randn((n_units, 1, seq, head_dim), dtype, device, seed * 1000 + 2 + shard[0])
        v = _randn((n_units, 1, seq, head_dim), dtype, device, seed * 1000 + 3 + shard[0])
    flops = 4.0 * head_dim * n_units * group * seq * (seq + 1) / 2
    t = dict(q=q, k=k, v=v)
    return Workload(
        "c2_dense_causal_prefill", "prefill",
        lambda: flash_attention_v2(t["q"], t["k"], t["v"], is_causal=True),
        t, dict(batch=batch, q_heads=q_heads, kv_heads=kv_heads, seq=seq, head_dim=head_dim, units=n_units),
        flops, float((q.numel() * 2 + k.numel() + v.numel()) * q.element_size()), ["q", "k", "v"],
    )


def c3_lengths(seed: int = 0, n: int = 16, lo: int = 128, hi: int = 4096) -> List[int]:
    return _lengths(seed, n, lo, hi)


def c3_ragged_prefill(device, seed: int = 0, *, n_seqs: int = 16, lo: int = 128, hi: int = 4096,
                      q_heads: int = 32, kv_heads: int = 8, head_dim: int = 128, dtype=torch.bfloat16,
                      shard: Tuple[int, int] = (0, 1), index_dtype=torch.int32, weak: bool = False) -> Workload:
    """Ragged varlen causal prefill.  Strong scaling: the n_seqs sequences are split over ranks by
    balanced causal cost.  Weak scaling: every rank holds n_seqs sequences of the configuration's lengths with its
    own values."""
    from kernels.attention import flash_attention_v2

    rank, world = shard
    if weak or world == 1:
        lens = c3_lengths(seed, n_seqs, lo, hi)      # weak scaling: every rank draws the same lengths, other values
    else:
        all_lens = c3_lengths(seed, n_seqs, lo, hi)
        lens = [all_lens[i] for i in balance_sequences(all_lens, world, causal_prefill=True)[rank]]
    total = sum(lens)
    q = _randn((max(total, 1), q_heads, head_dim), dtype, device, seed * 1000 + 11 + rank)[:total]
    k = _randn((max(total, 1), kv_heads, head_dim), dtype, device, seed * 1000 + 12 + rank)[:total]
    v = _randn((max(total, 1), kv_heads, head_dim), dtype, device, seed * 1000 + 13 + rank)[:total]
    indptr = torch.zeros(len(lens) + 1, dtype=torch.int64)
    if lens:
        indptr[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0)
    indptr = indptr.to(index_dtype).to(device)
    flops = sum(4.0 * head_dim * q_heads * n * (n + 1) / 2 for n in lens)
    t = dict(q=q, k=k, v=v, indptr=indptr)
    return Workload(
        "c3_ragged_causal_prefill", "prefill",
        lambda: flash_attention_v2(t["q"], t["k"], t["v"], is_causal=True, q_indptr=t["indptr"], kv_indptr=t["indptr"]),
        t, dict(lengths=lens, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, total_tokens=total),
        flops, float((q.numel() * 2 + k.numel() + v.numel()) * q.element_size()), ["q", "k", "v", "indptr"],
    )


def _paged_pool(device, lens: Sequence[int], kv_heads: int, head_dim: int, page_size: int, dtype, seed: int):
    """Shared pools with seeded random page permutations; K and V use independent permutations.
    Unused table entries are -1."""
    blocks = [(n + page_size - 1) // page_size for n in lens]
    n_pages = sum(blocks)
    width = max(blocks) if blocks else 1
    g = torch.Generator().manual_seed(seed * 7919 + 17)
    tables = []
    for _ in range(2):
        perm = torch.randperm(n_pages, generator=g).to(torch.int32)
        table = torch.full((len(lens), width), -1, dtype=torch.int32)
        cur = 0
        for i, nb in enumerate(blocks):
            table[i, :nb] = perm[cur: cur + nb]
            cur += nb
        tables.append(table.to(device))
    k_cache = _randn((n_pages * page_size, kv_heads, head_dim), dtype, device, seed * 1000 + 21)
    v_cache = _randn((n_pages * page_size, kv_heads, head_dim), dtype, device, seed * 1000 + 22)
    return k_cache, v_cache, tables[0], tables[1], n_pages


def gather_paged(cache: torch.Tensor, table: torch.Tensor, length: int, page_size: int) -> torch.Tensor:
    """Rows of one sequence, in logical order, out of a paged cache (used by checkers)."""
    nb = (length + page_size - 1) // page_size
    pages = table[:nb].to(torch.int64)
    rows = (pages[:, None] * page_size + torch.arange(page_size, device=cache.device)[None, :]).reshape(-1)[:length]
    return cache[rows]


def c4_paged_decode(device, seed: int = 0, *, batch: int = 64, lo: int = 512, hi: int = 8192, page_size: int = 16,
                    q_heads: int = 32, kv_heads: int = 8, head_dim: int = 128, dtype=torch.bfloat16,
                    shard: Tuple[int, int] = (0, 1), weak: bool = False) -> Workload:
    """Paged-KV decode, sharded by batch."""
    from kernels.decode import decode_attention

    rank, world = shard
    if weak or world == 1:
        lens = _lengths(seed, batch, lo, hi)         # weak scaling: every rank draws the same lengths, other values
    else:
        all_lens = _lengths(seed, batch, lo, hi)
        b0, b1 = contiguous_shard(batch, world, rank)
        lens = all_lens[b0:b1]
    k_cache, v_cache, kt, vt, n_pages = _paged_pool(device, lens, kv_heads, head_dim, page_size, dtype, seed + rank)
    q = _randn((len(lens), q_heads, head_dim), dtype, device, seed * 1000 + 23 + rank)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=device)
    kv_bytes = float(sum(lens)) * kv_heads * head_dim * 2 * q.element_size()
    flops = 4.0 * q_heads * head_dim * sum(lens)
    t = dict(q=q, k_cache=k_cache, v_cache=v_cache, lens=lens_t, k_table=kt, v_table=vt)
    return Workload(
        "c4_paged_decode", "decode",
        lambda: decode_attention(t["q"], t["k_cache"], t["v_cache"], kv_indptr=t["lens"], k_block_table=t["k_table"],
                                 v_block_table=t["v_table"], kv_page_size=page_size),
        t, dict(lengths=lens, page_size=page_size, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                pages=n_pages, tokens=sum(lens)),
        flops, kv_bytes, ["q", "lens", "k_table", "v_table"],
    )


def c5_paged_spec_decode(device, seed: int = 0, *, batch: int = 32, drafts: int = 5, lo: int = 1024, hi: int = 32768,
                         page_size: int = 16, q_heads: int = 64, kv_heads: int = 8, head_dim: int = 128,
                         dtype=torch.bfloat16, shard: Tuple[int, int] = (0, 1), weak: bool = False) -> Workload:
    """Paged speculative decode, causal among the drafts; sharded by KV head (one head per GPU at 8 GPUs)."""
    from kernels.speculative_decode import speculative_decode_attention

    rank, world = shard
    group = q_heads // kv_heads
    ctx = _lengths(seed, batch, lo, hi)
    lens = [c + drafts for c in ctx]
    if weak or world == 1:
        my_heads = kv_heads
    else:
        h0, h1 = kv_head_shard(kv_heads, world, rank)
        my_heads = h1 - h0
    k_cache, v_cache, kt, vt, n_pages = _paged_pool(device, lens, my_heads, head_dim, page_size, dtype, seed + rank)
    q = _randn((batch, my_heads * group, drafts, head_dim), dtype, device, seed * 1000 + 31 + rank)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=device)
    kv_bytes = float(sum(lens)) * my_heads * head_dim * 2 * q.element_size()
    flops = 4.0 * my_heads * group * drafts * head_dim * sum(lens)
    t = dict(q=q, k_cache=k_cache, v_cache=v_cache, lens=lens_t, k_table=kt, v_table=vt)
    return Workload(
        "c5_paged_spec_decode", "spec",
        lambda: speculative_decode_attention(t["q"], t["k_cache"], t["v_cache"], causal=True, kv_indptr=t["lens"],
                                             k_block_table=t["k_table"], v_block_table=t["v_table"],
                                             kv_page_size=page_size),
        t, dict(lengths=lens, drafts=drafts, page_size=page_size, q_heads=my_heads * group, kv_heads=my_heads,
                head_dim=head_dim, pages=n_pages, tokens=sum(lens)),
        flops, kv_bytes, ["q", "lens", "k_table", "v_table"],
    )


# ---------------------------------------------------------------------------
# Strong scaling: ONE problem (the configuration as named, generated from the seed alone, the same on every rank)
# cut into the shards the configuration names.  Every builder returns
#   (shard workload of this rank, the whole problem as a workload, assemble(list of per-rank outputs) -> whole output)
# so that a caller can compare the gathered shards with the same problem computed on one GPU.
# ---------------------------------------------------------------------------
def _clone_workload(full: Workload, run, tensors, flops, kv_bytes, meta_extra) -> Workload:
    return Workload(full.name, full.kind, run, tensors, dict(full.meta, **meta_extra), flops, kv_bytes,
                    list(full.host_inputs))


def c2_strong(device, seed: int, rank: int, world: int, **cfg):
    """Dense prefill cut into (batch, KV head) units; a rank owns a contiguous run of them in batch-major order and
    holds the q heads of its KV heads only, stacked along the batch axis."""
    from kernels.attention import flash_attention_v2
    from sharding.planner import batch_head_units

    full = c2_dense_prefill(device, seed, **cfg)
    m = full.meta
    group = m["q_heads"] // m["kv_heads"]
    units = batch_head_units(m["batch"], m["kv_heads"], world, rank)
    q, k, v = full.tensors["q"], full.tensors["k"], full.tensors["v"]
    t = dict(q=torch.stack([q[b, h * group:(h + 1) * group] for b, h in units]),
             k=torch.stack([k[b, h:h + 1] for b, h in units]), v=torch.stack([v[b, h:h + 1] for b, h in units]))
    frac = len(units) / (m["batch"] * m["kv_heads"])
    shard = _clone_workload(full, lambda: flash_attention_v2(t["q"], t["k"], t["v"], is_causal=True), t,
                            full.flops * frac, full.kv_bytes * frac, dict(units=len(units)))

    def assemble(parts):
        return torch.cat(parts).reshape(m["batch"], m["q_heads"], m["seq"], m["head_dim"])

    return shard, full, assemble


def c3_strong(device, seed: int, rank: int, world: int, **cfg):
    """Ragged prefill: whole sequences dealt to ranks by balanced causal cost (longest first, greedy)."""
    from kernels.attention import flash_attention_v2

    full = c3_ragged_prefill(device, seed, **cfg)
    lens = full.meta["lengths"]
    bins = balance_sequences(lens, world, causal_prefill=True)
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    mine = bins[rank]
    d, qh = full.meta["head_dim"], full.meta["q_heads"]

    def pick(x):
        if not mine:
            return x[:0].clone()
        return torch.cat([x[starts[i]:starts[i + 1]] for i in mine])

    my_lens = [lens[i] for i in mine]
    indptr = torch.zeros(len(my_lens) + 1, dtype=torch.int64)
    if my_lens:
        indptr[1:] = torch.tensor(my_lens, dtype=torch.int64).cumsum(0)
    t = dict(q=pick(full.tensors["q"]), k=pick(full.tensors["k"]), v=pick(full.tensors["v"]),
             indptr=indptr.to(full.tensors["indptr"].dtype).to(device))
    flops = sum(4.0 * d * qh * n * (n + 1) / 2 for n in my_lens)
    shard = _clone_workload(
        full, lambda: flash_attention_v2(t["q"], t["k"], t["v"], is_causal=True, q_indptr=t["indptr"], kv_indptr=t["indptr"]),
        t, flops, float((t["q"].numel() * 2 + 2 * t["k"].numel()) * 2), dict(lengths=my_lens, total_tokens=sum(my_lens)))

    def assemble(parts):
        out = torch.empty_like(full.tensors["q"])
        for r, part in enumerate(parts):
            cur = 0
            for i in bins[r]:
                out[starts[i]:starts[i + 1]] = part[cur:cur + lens[i]]
                cur += lens[i]
        return out

    return shard, full, assemble


def c4_strong(device, seed: int, rank: int, world: int, **cfg):
    """Paged decode cut by batch: a rank owns a contiguous run of sequences (their q rows, lengths and block-table
    rows); the page pool is the whole problem's, of which it touches only its sequences' pages."""
    from kernels.decode import decode_attention

    full = c4_paged_decode(device, seed, **cfg)
    lens = full.meta["lengths"]
    b0, b1 = contiguous_shard(len(lens), world, rank)
    ft = full.tensors
    t = dict(q=ft["q"][b0:b1].contiguous(), k_cache=ft["k_cache"], v_cache=ft["v_cache"], lens=ft["lens"][b0:b1].contiguous(),
             k_table=ft["k_table"][b0:b1].contiguous(), v_table=ft["v_table"][b0:b1].contiguous())
    ps = full.meta["page_size"]
    frac = sum(lens[b0:b1]) / max(sum(lens), 1)
    shard = _clone_workload(
        full, lambda: decode_attention(t["q"], t["k_cache"], t["v_cache"], kv_indptr=t["lens"], k_block_table=t["k_table"],
                                       v_block_table=t["v_table"], kv_page_size=ps),
        t, full.flops * frac, full.kv_bytes * frac, dict(lengths=lens[b0:b1], tokens=sum(lens[b0:b1])))
    return shard, full, lambda parts: torch.cat(parts)


def c5_strong(device, seed: int, rank: int, world: int, **cfg):
    """Paged speculative decode cut by KV head: a rank holds the pages of its KV heads (one head per GPU at 8 GPUs
    with 8 KV heads) and the q heads that share them."""
    from kernels.speculative_decode import speculative_decode_attention

    full = c5_paged_spec_decode(device, seed, **cfg)
    m = full.meta
    group = m["q_heads"] // m["kv_heads"]
    h0, h1 = kv_head_shard(m["kv_heads"], world, rank)
    ft = full.tensors
    t = dict(q=ft["q"][:, h0 * group:h1 * group].contiguous(), k_cache=ft["k_cache"][:, h0:h1].contiguous(),
             v_cache=ft["v_cache"][:, h0:h1].contiguous(), lens=ft["lens"], k_table=ft["k_table"], v_table=ft["v_table"])
    ps = m["page_size"]
    frac = (h1 - h0) / m["kv_heads"]
    shard = _clone_workload(
        full, lambda: speculative_decode_attention(t["q"], t["k_cache"], t["v_cache"], causal=True, kv_indptr=t["lens"],
                                                   k_block_table=t["k_table"], v_block_table=t["v_table"], kv_page_size=ps),
        t, full.flops * frac, full.kv_bytes * frac, dict(q_heads=(h1 - h0) * group, kv_heads=h1 - h0))
    return shard, full, lambda parts: torch.cat(parts, dim=1)


STRONG = {"c2": c2_strong, "c3": c3_strong, "c4": c4_strong, "c5": c5_strong}
