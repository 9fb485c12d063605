"""Argument validation and layout dispatch for the attention entry points.

The reference validates inline with ``assert`` (kernels/attention.py:762-834,
kernels/decode.py:236-269, kernels/speculative_decode.py:262-297); the same
checks, raising the same exception types, live here so that they run before any
native call.  Nothing in this module touches the GPU or imports Triton.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

DENSE, RAGGED, PAGED = 0, 1, 2
SUPPORTED_HEAD_DIMS = (64, 128)
SUPPORTED_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
MAX_DRAFT_TOKENS = 16  # kernels/speculative_decode.py:297


@dataclass
class AttentionProblem:
    """Everything the native call needs, derived from the tensors."""

    layout: int
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    q_len: int = 1          # decode / spec: M; prefill dense & paged: M
    max_kv: int = 0         # dense: N; paged: table width * page size
    total_q: int = 0        # ragged prefill
    total_kv: int = 0       # ragged rows, or rows of the paged cache
    table_stride: int = 0
    page_size: int = 0
    indptr_is_i64: bool = False
    q_indptr: Optional[torch.Tensor] = None
    kv_indptr: Optional[torch.Tensor] = None
    k_table: Optional[torch.Tensor] = None
    v_table: Optional[torch.Tensor] = None


def detect_layout(q_indptr, kv_indptr, k_block_table, *, prefill: bool) -> int:
    """Mode is selected purely by which optional tensors are present
    (kernels/attention.py:766-767, kernels/decode.py:240-241)."""
    if k_block_table is not None:
        return PAGED
    if prefill:
        return RAGGED if q_indptr is not None else DENSE
    return RAGGED if kv_indptr is not None else DENSE


def _check_common(q, k, v) -> None:
    assert q.dtype == k.dtype == v.dtype, "Tensors must have the same dtype"
    assert q.device == k.device == v.device, "Tensors must be on the same device"
    assert q.is_cuda, "Tensors must be on a CUDA device"
    assert q.dtype in SUPPORTED_DTYPES, f"unsupported dtype {q.dtype}"
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous(), "q, k and v must be contiguous"


def _check_head_dim(d: int) -> None:
    assert d in SUPPORTED_HEAD_DIMS, f"head_dim {d} is not built; supported: {SUPPORTED_HEAD_DIMS}"


def _index_tensor(t: torch.Tensor, device, name: str) -> torch.Tensor:
    assert t.dtype in (torch.int32, torch.int64), f"{name} must be int32 or int64"
    assert t.device == device, f"{name} must be on the same device as q"
    return t.contiguous()


def _table(t: torch.Tensor, device, name: str) -> torch.Tensor:
    assert t.ndim == 2, f"{name} must be (B, max_blocks_per_seq)"
    assert t.device == device, f"{name} must be on the same device as q"
    assert t.dtype in (torch.int32, torch.int64), f"{name} must be an integer tensor"
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    return t.contiguous()


def validate_prefill(q, k, v, q_indptr, kv_indptr, k_block_table, v_block_table, kv_page_size) -> AttentionProblem:
    """Checks of kernels/attention.py:762-834."""
    _check_common(q, k, v)
    layout = detect_layout(q_indptr, kv_indptr, k_block_table, prefill=True)
    if layout == DENSE:
        assert q.ndim == 4 and k.ndim == 4 and v.ndim == 4
        batch, q_heads, m, head_dim = q.shape
        batch_k, kv_heads, n, head_dim_k = k.shape
        batch_v, kv_heads_v, n_v, head_dim_v = v.shape
        assert batch == batch_k == batch_v
        assert kv_heads == kv_heads_v
        assert n == n_v
        assert head_dim == head_dim_k == head_dim_v
        assert q_heads % kv_heads == 0
        _check_head_dim(head_dim)
        return AttentionProblem(DENSE, batch, q_heads, kv_heads, head_dim, q_len=m, max_kv=n)
    if layout == RAGGED:
        assert q.ndim == 3 and k.ndim == 3 and v.ndim == 3
        total_q, q_heads, head_dim = q.shape
        total_kv, kv_heads, head_dim_k = k.shape
        total_v, kv_heads_v, head_dim_v = v.shape
        assert total_kv == total_v
        assert kv_heads == kv_heads_v
        assert head_dim == head_dim_k == head_dim_v
        assert q_heads % kv_heads == 0
        assert q_indptr is not None
        assert kv_indptr is not None
        _check_head_dim(head_dim)
        q_indptr = _index_tensor(q_indptr, q.device, "q_indptr")
        kv_indptr = _index_tensor(kv_indptr, q.device, "kv_indptr")
        assert q_indptr.ndim == 1 and kv_indptr.ndim == 1 and q_indptr.numel() == kv_indptr.numel()
        assert q_indptr.numel() >= 1
        if kv_indptr.dtype != q_indptr.dtype:
            kv_indptr = kv_indptr.to(q_indptr.dtype)
        return AttentionProblem(
            RAGGED, q_indptr.numel() - 1, q_heads, kv_heads, head_dim,
            total_q=total_q, total_kv=total_kv, indptr_is_i64=q_indptr.dtype == torch.int64,
            q_indptr=q_indptr, kv_indptr=kv_indptr,
        )
    assert q.ndim == 4 and k.ndim == 3 and v.ndim == 3
    batch, q_heads, m, head_dim = q.shape
    total_cache, kv_heads, head_dim_k = k.shape
    total_cache_v, kv_heads_v, head_dim_v = v.shape
    assert total_cache == total_cache_v
    assert kv_heads == kv_heads_v
    assert head_dim == head_dim_k == head_dim_v
    assert q_heads % kv_heads == 0
    assert kv_page_size is not None
    assert kv_indptr is not None
    assert k_block_table is not None
    assert v_block_table is not None
    _check_head_dim(head_dim)
    return _paged_problem(q, batch, q_heads, kv_heads, head_dim, m, total_cache, kv_indptr, k_block_table,
                          v_block_table, kv_page_size)


def _paged_problem(q, batch, q_heads, kv_heads, head_dim, m, total_cache, kv_indptr, k_table, v_table, page_size):
    page_size = int(page_size)
    assert page_size > 0, "kv_page_size must be positive"
    kv_indptr = _index_tensor(kv_indptr, q.device, "kv_indptr")
    assert kv_indptr.ndim == 1 and kv_indptr.numel() == batch, "paged kv_indptr holds one length per sequence"
    k_table = _table(k_table, q.device, "k_block_table")
    v_table = _table(v_table, q.device, "v_block_table")
    assert k_table.shape == v_table.shape and k_table.shape[0] == batch
    return AttentionProblem(
        PAGED, batch, q_heads, kv_heads, head_dim, q_len=m,
        max_kv=k_table.shape[1] * page_size, total_kv=total_cache, table_stride=k_table.shape[1],
        page_size=page_size, indptr_is_i64=kv_indptr.dtype == torch.int64, kv_indptr=kv_indptr,
        k_table=k_table, v_table=v_table,
    )


def validate_decode(q, k, v, kv_indptr, k_block_table, v_block_table, kv_page_size, *, spec: bool) -> AttentionProblem:
    """Checks of kernels/decode.py:236-269 (q is (B, QH, D)) and
    kernels/speculative_decode.py:262-297 (q is (B, QH, M, D), M <= 16)."""
    _check_common(q, k, v)
    layout = detect_layout(None, kv_indptr, k_block_table, prefill=False)
    if spec:
        assert q.ndim == 4, "q must be (B, QH, M, D)"
        batch, q_heads, m, head_dim = q.shape
    else:
        assert q.ndim == 3, "q must be (B, QH, D)"
        batch, q_heads, head_dim = q.shape
        m = 1
    _check_head_dim(head_dim)
    if layout == PAGED:
        assert k_block_table is not None and v_block_table is not None
        assert kv_page_size is not None
        assert kv_indptr is not None, "kv_indptr (sequence context lengths) must be provided for paged mode."
        assert k.ndim in (3, 4) and v.ndim == k.ndim
        kv_heads = k.shape[2] if k.ndim == 4 else k.shape[1]  # kernels/decode.py:251
        assert k.shape == v.shape and k.shape[-1] == head_dim
        total_cache = k.shape[0] * k.shape[1] if k.ndim == 4 else k.shape[0]
        prob = _paged_problem(q, batch, q_heads, kv_heads, head_dim, m, total_cache, kv_indptr, k_block_table,
                              v_block_table, kv_page_size)
    elif layout == RAGGED:
        if kv_indptr is None:
            raise ValueError("kv_indptr must be provided for ragged mode.")
        assert k.ndim == 3 and v.ndim == 3
        total_kv, kv_heads, d_k = k.shape
        assert k.shape == v.shape and d_k == head_dim
        kv_indptr = _index_tensor(kv_indptr, q.device, "kv_indptr")
        assert kv_indptr.ndim == 1 and kv_indptr.numel() == batch + 1
        prob = AttentionProblem(RAGGED, batch, q_heads, kv_heads, head_dim, q_len=m, total_kv=total_kv,
                                indptr_is_i64=kv_indptr.dtype == torch.int64, kv_indptr=kv_indptr)
    else:
        assert k.ndim == 4 and v.ndim == 4
        batch_k, kv_heads, n, d_k = k.shape
        assert k.shape == v.shape and batch_k == batch and d_k == head_dim
        prob = AttentionProblem(DENSE, batch, q_heads, kv_heads, head_dim, q_len=m, max_kv=n)
    assert q_heads % prob.kv_heads == 0
    if spec:
        assert m <= MAX_DRAFT_TOKENS, "Speculative decode is intended for small draft lengths (M <= 16)."
        assert m >= 1
    return prob
