"""Speculative (multi-token) decode attention entry point (drop-in for the reference's
``kernels/speculative_decode.py:228-366``)."""
from __future__ import annotations

import torch

from utils.validation import validate_decode

from .decode import _launch_decode


def speculative_decode_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = False,
    kv_indptr: torch.Tensor | None = None,
    k_block_table: torch.Tensor | None = None,
    v_block_table: torch.Tensor | None = None,
    kv_page_size: int | None = None,
) -> torch.Tensor:
    """Attention for M <= 16 draft tokens per sequence.

    Dense  : q (B, QH, M, D), k/v (B, KVH, N, D)
    Ragged : q (B, QH, M, D), k/v (total_kv, KVH, D), kv_indptr (B + 1,)
    Paged  : q (B, QH, M, D), k/v (total_kv_tokens, KVH, D), kv_indptr (B,) lengths, block tables, page size

    With ``causal=True`` the last M keys of every sequence are the draft tokens' own
    keys (the passed length includes them) and draft row i does not see draft keys
    i+1..M-1; every draft row sees the whole context.
    """
    prob = validate_decode(q, k, v, kv_indptr, k_block_table, v_block_table, kv_page_size, spec=True)
    return _launch_decode(q, k, v, prob, causal=bool(causal))
