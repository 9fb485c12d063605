"""Launch planning for the attention path, restated in Python.

These are mirrors of the planning rules compiled into ``libb200attn.so`` (csrc/decode.cu ``decode_pass_group`` /
``decode_ws_layout`` / ``decode_plan_kernel`` and the prefill grid in csrc/prefill.cu), which replace the
reference's split heuristics (kernels/attention.py:836-841, kernels/decode.py:271-278,
kernels/speculative_decode.py:301-309).  Nothing on the product path calls them: the library plans for itself.
They exist so that the rules can be unit-tested without a GPU, and ``decode_workspace_bytes`` is compared with the
library's own ``b200attn_decode_workspace_bytes`` in the GPU tests so that the two cannot drift apart unnoticed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

DECODE_TILE_TOKENS = 64       # keys per cp.async stage
PREFILL_BLOCK_M = 128         # query rows per tensor-core tile
PREFILL_SLOTS = 2             # query tiles per CTA
PREFILL_BLOCK_N = 128         # keys per tile


@dataclass
class DecodePlan:
    target_items: int
    min_chunk: int
    max_items: int
    mma_tiles: int     # 16-row MMA tiles that hold group x q_len rows
    key_slices: int    # warps that split the keys of one stage
    threads: int
    wave_items: int = 0      # items of one KV head resident at once (one wave); 0: a single wave is never planned
    item_overhead: int = 0   # start-up + merge of an item in keys of streaming time (the planner's cost estimate)
    equal_split: bool = True


def decode_pass_group(group: int, q_len: int) -> int:
    """q heads of one KV head that one launch serves: at most 128 q rows (group x draft tokens) per CTA; a larger
    group is cut into the largest equal sub-groups that fit."""
    q_len = max(1, q_len)
    g = group
    while g > 1 and (g * q_len > 128 or group % g != 0):
        g -= 1
    return max(g, 1)


def decode_workspace_bytes(plan: "DecodePlan", batch: int, kv_heads: int, head_dim: int, rows: int,
                           cast_q_elems: int = 0, cast_kv_elems: int = 0) -> int:
    """Bytes of scratch a decode call needs: header, item prefix, merge tickets, item records, (m, l) and O partials,
    each rounded up to 256 bytes (csrc/decode.cu decode_ws_layout) - and, for fp32 inputs of a speculative-decode
    call, the fp16 copies of q, k and v (``cast_*_elems`` elements each)."""
    up = lambda x: (x + 255) & ~255
    off = 256
    off = up(off + 4 * (batch + 1))
    off = up(off + 4 * batch * kv_heads)
    off = up(off + 32 * plan.max_items)
    slots = plan.max_items * kv_heads
    off = up(off + 4 * slots * rows * 2)
    off = up(off + 4 * slots * rows * head_dim)
    if cast_kv_elems:
        off = up(off + 2 * cast_q_elems)
        off = up(off + 2 * cast_kv_elems)
        off = up(off + 2 * cast_kv_elems)
    return off


def decode_plan(sm_count: int, batch: int, q_heads: int, kv_heads: int, q_len: int, fp32: bool = False) -> DecodePlan:
    group = decode_pass_group(q_heads // kv_heads, q_len)
    rows = group * q_len
    # fp32 inputs of a speculative-decode call (several q rows per head) run the tensor-core kernels on fp16 copies
    # and are planned like 16-bit inputs (unless k and v would need more than 8 GiB of copies: csrc/decode.cu)
    fp32 = fp32 and rows <= 16 and q_len <= 1
    # six (item, kv head) CTAs per SM for the tensor-core kernels (a whole number of waves at 2 or 3 resident CTAs
    # per SM), eight for the fp32 kernel
    target = max(1, (sm_count * (8 if fp32 else 6)) // max(1, kv_heads))
    by_rows = -(-(rows * 8) // DECODE_TILE_TOKENS) * DECODE_TILE_TOKENS
    min_chunk = max(128, by_rows)
    tiles = -(-rows // 16)
    slices = 4 if tiles <= 2 else (2 if tiles <= 4 else 1)
    wide = rows > 16           # more than one 16-row tile: the tcgen05 kernel, two resident CTAs per SM (else three)
    wave = 0 if fp32 else max(1, (sm_count * (2 if wide else 3)) // max(1, kv_heads))
    overhead = 0 if fp32 else (448 if wide else 128)
    return DecodePlan(target, min_chunk, target + batch, tiles, slices, 32 * (tiles * slices + 1), wave, overhead,
                      not fp32)


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


def _item_tokens(plan: DecodePlan, length: int, n: int, chunk: int) -> int:
    """Keys per item of a sequence cut into ``n`` items (csrc/decode.cu seq_chunk)."""
    if not plan.equal_split:
        return chunk
    return max(DECODE_TILE_TOKENS, _round_up(-(-length // n), DECODE_TILE_TOKENS))


def _pick_chunk(plan: DecodePlan, lens: Sequence[int], target: int):
    """First of 32 candidates between total / target and twice that with at most ``target`` items:
    (chunk, items, largest item, found)."""
    total = sum(lens)
    base = max(_round_up(-(-total // target), DECODE_TILE_TOKENS), plan.min_chunk)
    last = None
    for k in range(32):
        chunk = _round_up(base + (base * k) // 32, DECODE_TILE_TOKENS)
        counts = [max(1, -(-n // chunk)) for n in lens]
        biggest = max([min(n, _item_tokens(plan, n, c, chunk)) for n, c in zip(lens, counts)], default=0)
        last = (chunk, sum(counts), biggest)
        if last[1] <= target:
            return last + (True,)
    return last + (False,)


def decode_chunk_tokens(plan: DecodePlan, lengths: Sequence[int]) -> int:
    """Chunk size the device planner picks for these lengths: the smallest of 32 candidates between
    total / target_items and twice that which splits the batch into at most target_items items - or, when the
    batch also fits a single wave of resident CTAs and the estimate favours it (largest item + per-item overhead
    against the average load of a resident CTA + half an item), the single-wave chunk."""
    lens = [max(0, int(n)) for n in lengths]
    total = sum(lens)
    chunk, items, _, _ = _pick_chunk(plan, lens, plan.target_items)
    if 0 < plan.wave_items < plan.target_items and items > plan.wave_items:
        w_chunk, _, w_biggest, found = _pick_chunk(plan, lens, plan.wave_items)
        if found:
            several = (total + items * plan.item_overhead) / plan.wave_items + 0.5 * (total / items + plan.item_overhead)
            if w_biggest + plan.item_overhead < several:
                chunk = w_chunk
    return chunk


def decode_items(plan: DecodePlan, lengths: Sequence[int]) -> List[int]:
    """Work items (KV chunks) per sequence; their sum never exceeds plan.max_items."""
    chunk = decode_chunk_tokens(plan, lengths)
    return [max(1, -(-max(0, int(n)) // chunk)) for n in lengths]


def prefill_items(layout: str, batch: int, q_heads: int, kv_heads: int, max_q: int = 0, total_q: int = 0) -> int:
    """Work items of the persistent prefill kernel.  An item is two 128-row query tiles that share a KV head: two
    neighbouring q heads over the same rows when the GQA group is even, else two consecutive row tiles of one head."""
    head_pair = (q_heads // kv_heads) % 2 == 0
    rows = PREFILL_BLOCK_M if head_pair else PREFILL_BLOCK_M * PREFILL_SLOTS
    units = q_heads // 2 if head_pair else q_heads
    if layout == "ragged":
        return (total_q // rows + batch) * units
    return -(-max_q // rows) * units * batch


def paged_box_rows(page_size: int) -> int:
    """Tokens per TMA box for a paged cache: the largest power of two dividing the page size, at most one tile."""
    box = 1
    while box < PREFILL_BLOCK_N and page_size % (box * 2) == 0:
        box *= 2
    return box
