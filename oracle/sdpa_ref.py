"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, device-agnostically, the correctness oracle that the
reference's own tests use for prefill, decode and speculative decode:
per-sequence ``torch.nn.functional.scaled_dot_product_attention`` on inputs
up-cast to fp32, with K/V heads repeated for GQA/MQA.  The arithmetic lives in
a third-party dependency of the reference (``torch``, pinned 2.12.1 in its
``uv.lock``; 2.11.0 here); ``softmax_ref.py`` restates the published formula
softmax(QK^T/sqrt(D))V in fp64 numpy so the oracle does not hinge on a torch
version, and ``tests/test_oracle.py`` pins one against the other and against
the committed golden vectors.

Parity status: pinned to the reference's own oracle functions.  The reference holds no
stored vectors, seeds or known-answer literals for this path and its kernels cannot run
without a GPU, but its tests' ``get_reference_outputs`` / ``allocate_paged_cache`` /
tolerance functions are pure torch and run on CPU.  ``tests/golden/make_golden.py`` imports
them from a reference checkout and records their outputs on seeded inputs;
``tests/test_oracle.py`` checks this restatement against those fixtures, against the fp64
restatement and against analytic known answers.  On a GPU the reference's three test
modules themselves run unmodified against the package (``oracle/stage_reference_tests.py``,
``tests/test_zr_reference_suite.py``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
arm of ``bench.py`` may import this module.  The product path never does.

Reference call sites followed:
  prefill  : tests/test_attention.py:80-98
  decode   : tests/test_decode.py:69-90
  spec     : tests/test_speculative_decode.py:76-126 (mask rule :103-114)
  tolerance: tests/test_attention.py:20-30
  paged scatter: tests/test_attention.py:101-134
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

# tests/test_attention.py:20-24 (identical tables in the decode / spec tests)
BASE_TOL = {
    torch.float16: dict(base_atol=1e-2, rtol=1e-2, eps=2e-3),
    torch.bfloat16: dict(base_atol=2e-2, rtol=2e-2, eps=4e-3),
    torch.float32: dict(base_atol=1e-3, rtol=1e-2, eps=2e-3),
}


def attn_tolerances(dtype: torch.dtype, n: int) -> dict:
    """atol = base_atol * sqrt(max(N,1)) + eps, rtol per dtype
    (tests/test_attention.py:27-30)."""
    cfg = BASE_TOL[dtype]
    return dict(atol=cfg["base_atol"] * math.sqrt(max(n, 1)) + cfg["eps"], rtol=cfg["rtol"])


def strict_max_abs(dtype: torch.dtype) -> float:
    """The un-scaled bar: max-abs error <= base_atol (bf16 2e-2, fp16 1e-2, fp32 1e-3)."""
    return BASE_TOL[dtype]["base_atol"]


def _expand_kv(k_ref: torch.Tensor, v_ref: torch.Tensor, qh: int, kvh: int):
    if qh != kvh:
        groups = qh // kvh
        k_ref = k_ref.repeat_interleave(groups, dim=1)
        v_ref = v_ref.repeat_interleave(groups, dim=1)
    return k_ref, v_ref


def prefill_reference(qs, ks, vs, qh: int, kvh: int, is_causal: bool) -> List[torch.Tensor]:
    """Per sequence: q (L_q, QH, D), k/v (L_kv, KVH, D) -> (L_q, QH, D) fp32.
    Follows tests/test_attention.py:80-98."""
    refs = []
    for q, k, v in zip(qs, ks, vs):
        q_ref = q.transpose(0, 1).unsqueeze(0).float()
        k_ref = k.transpose(0, 1).unsqueeze(0).float()
        v_ref = v.transpose(0, 1).unsqueeze(0).float()
        k_ref, v_ref = _expand_kv(k_ref, v_ref, qh, kvh)
        out = F.scaled_dot_product_attention(q_ref, k_ref, v_ref, is_causal=is_causal)
        refs.append(out.squeeze(0).transpose(0, 1))
    return refs


def decode_reference(qs, ks, vs, qh: int, kvh: int) -> List[torch.Tensor]:
    """Per sequence: q (QH, D), k/v (L, KVH, D) -> (QH, D) fp32.
    Follows tests/test_decode.py:69-90."""
    refs = []
    for q, k, v in zip(qs, ks, vs):
        q_ref = q.unsqueeze(0).unsqueeze(2).float()
        k_ref = k.transpose(0, 1).unsqueeze(0).float()
        v_ref = v.transpose(0, 1).unsqueeze(0).float()
        k_ref, v_ref = _expand_kv(k_ref, v_ref, qh, kvh)
        out = F.scaled_dot_product_attention(q_ref, k_ref, v_ref)
        refs.append(out.squeeze(0).squeeze(1))
    return refs


def draft_mask(m: int, n_total: int, device=None) -> torch.Tensor:
    """Boolean (M, N_total) mask: draft row i sees every context key and draft
    keys 0..i; the M draft keys are the LAST M keys
    (tests/test_speculative_decode.py:103-114)."""
    n_ctx = n_total - m
    mask = torch.ones((m, n_total), dtype=torch.bool, device=device)
    for i in range(m):
        mask[i, n_ctx + i + 1:] = False
    return mask


def spec_decode_reference(qs, ks, vs, qh: int, kvh: int, causal: bool) -> List[torch.Tensor]:
    """Per sequence: q (QH, M, D), k/v (L, KVH, D) where, when ``causal``, the
    last M rows of k/v are the draft tokens' own K/V -> (QH, M, D) fp32.
    Follows tests/test_speculative_decode.py:76-126 (there the draft rows are
    appended inside the oracle; here the caller passes the already-appended
    K/V, which is what the kernel sees)."""
    refs = []
    for q, k, v in zip(qs, ks, vs):
        q_ref = q.unsqueeze(0).float()
        k_ref = k.transpose(0, 1).unsqueeze(0).float()
        v_ref = v.transpose(0, 1).unsqueeze(0).float()
        k_ref, v_ref = _expand_kv(k_ref, v_ref, qh, kvh)
        mask = None
        if causal:
            mask = draft_mask(q_ref.shape[2], k_ref.shape[2], q_ref.device)
        out = F.scaled_dot_product_attention(q_ref, k_ref, v_ref, attn_mask=mask, is_causal=False)
        refs.append(out.squeeze(0))
    return refs


# --------------------------------------------------------------------------
# Layout packers (what the reference tests do inline before calling a kernel)
# --------------------------------------------------------------------------

def pack_dense_prefill(qs, ks, vs):
    """tests/test_attention.py:159-170: zero-padded (B,H,L,D) tensors."""
    b = len(qs)
    qh, d = qs[0].shape[1], qs[0].shape[2]
    kvh = ks[0].shape[1]
    max_q = max(x.shape[0] for x in qs)
    max_kv = max(x.shape[0] for x in ks)
    q = torch.zeros((b, qh, max_q, d), dtype=qs[0].dtype, device=qs[0].device)
    k = torch.zeros((b, kvh, max_kv, d), dtype=qs[0].dtype, device=qs[0].device)
    v = torch.zeros_like(k)
    for i in range(b):
        q[i, :, : qs[i].shape[0]] = qs[i].transpose(0, 1)
        k[i, :, : ks[i].shape[0]] = ks[i].transpose(0, 1)
        v[i, :, : vs[i].shape[0]] = vs[i].transpose(0, 1)
    return q, k, v


def pack_ragged(seqs, index_dtype=torch.int32):
    """tests/test_attention.py:177-183: concatenation + prefix sums.  The
    reference builds the prefix with ``tensor(int32).cumsum`` which promotes to
    int64; ``index_dtype`` lets tests cover both widths."""
    lens = [int(s.shape[0]) for s in seqs]
    packed = torch.cat(list(seqs), dim=0)
    indptr = torch.zeros(len(lens) + 1, dtype=torch.int64)
    indptr[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0)
    return packed, indptr.to(index_dtype).to(packed.device)


def pack_paged(
    seqs: Sequence[torch.Tensor],
    page_size: int,
    *,
    permute_seed: Optional[int] = None,
    extra_pages: int = 0,
    pad_value: int = 0,
    poison: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Scatter per-sequence (L, H, D) tensors into a paged cache
    ``[pages*page_size, H, D]`` with an int32 block table ``[B, max_blocks]``.

    With the defaults this is the reference fixture (pages handed out
    sequentially, zero cache, zero-padded table: tests/test_attention.py:101-134).
    ``permute_seed`` hands pages out in a seeded random order over a pool with
    ``extra_pages`` spare pages, ``pad_value`` fills unused table entries
    (benchmarks/attention.py:415-420 uses -1) and ``poison`` pre-fills the cache
    (NaN/Inf) so that page tails and unused pages must never reach the output.
    Returns (cache, table, lengths[int32])."""
    lens = [int(s.shape[0]) for s in seqs]
    b = len(lens)
    heads, dim = seqs[0].shape[1], seqs[0].shape[2]
    blocks = [(n + page_size - 1) // page_size for n in lens]
    max_blocks = max(max(blocks), 1)
    total_blocks = sum(blocks) + extra_pages
    dev = seqs[0].device
    cache = torch.zeros((max(total_blocks, 1) * page_size, heads, dim), dtype=seqs[0].dtype, device=dev)
    if poison is not None:
        cache.fill_(poison)
    table = torch.full((b, max_blocks), pad_value, dtype=torch.int32)
    if permute_seed is None:
        order = torch.arange(total_blocks)
    else:
        g = torch.Generator().manual_seed(permute_seed)
        order = torch.randperm(total_blocks, generator=g)
    cur = 0
    for i in range(b):
        for logical in range(blocks[i]):
            phys = int(order[cur])
            cur += 1
            table[i, logical] = phys
            start = logical * page_size
            end = min(start + page_size, lens[i])
            cache[phys * page_size: phys * page_size + (end - start)] = seqs[i][start:end]
    return cache, table.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)
