"""Prefill attention entry points (drop-ins for the reference's
``kernels/attention.py``: ``flash_attention_v2`` :749-927 and ``flash_attention_v1`` :249-364).

Host code only validates, allocates the output and calls the sm_100a kernel
through the C ABI (``b200attn_prefill``).  No Triton, no CPU path.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from utils.validation import RAGGED, validate_prefill

from . import _native


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def flash_attention_v2(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    is_causal: bool = False,
    q_indptr: torch.Tensor | None = None,
    kv_indptr: torch.Tensor | None = None,
    k_block_table: torch.Tensor | None = None,
    v_block_table: torch.Tensor | None = None,
    kv_page_size: int | None = None,
) -> torch.Tensor:
    """Scaled-dot-product attention forward, scale 1/sqrt(D), optional top-left causal mask.

    Dense  : q (B, QH, M, D), k/v (B, KVH, N, D)
    Ragged : q (total_q, QH, D), k/v (total_kv, KVH, D), q_indptr / kv_indptr (B + 1,) prefix sums
    Paged  : q (B, QH, M, D), k/v cache (cache_tokens, KVH, D), kv_indptr (B,) lengths,
             k_block_table / v_block_table (B, max_blocks) int32, kv_page_size

    Returns a tensor shaped and typed like ``q``.
    """
    prob = validate_prefill(q, k, v, q_indptr, kv_indptr, k_block_table, v_block_table, kv_page_size)
    out = torch.empty_like(q)
    if q.numel() == 0:
        return out
    stream = torch.cuda.current_stream(q.device).cuda_stream
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()

    args = _native.PrefillArgs()
    args.q, args.k, args.v, args.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    args.q_indptr = prob.q_indptr.data_ptr() if prob.q_indptr is not None else None
    args.kv_indptr = prob.kv_indptr.data_ptr() if prob.kv_indptr is not None else None
    args.k_table = prob.k_table.data_ptr() if prob.k_table is not None else None
    args.v_table = prob.v_table.data_ptr() if prob.v_table is not None else None
    args.total_q = prob.total_q
    args.total_kv = prob.total_kv
    args.table_stride = prob.table_stride
    args.dtype = _native.DTYPE_CODE[q.dtype]
    args.layout = prob.layout
    args.indptr_is_i64 = int(prob.indptr_is_i64)
    args.batch = prob.batch
    args.q_heads = prob.q_heads
    args.kv_heads = prob.kv_heads
    args.max_q = 0 if prob.layout == RAGGED else prob.q_len
    args.max_kv = prob.max_kv
    args.head_dim = prob.head_dim
    args.page_size = prob.page_size
    args.is_causal = int(bool(is_causal))
    args.device = dev
    args.sm_scale = 1.0 / math.sqrt(prob.head_dim)

    lib = _native.lib()
    need = lib.b200attn_prefill_workspace_bytes(C.byref(args))
    ws = _native.workspace(q.device, stream, need)
    args.workspace = ws.data_ptr()
    args.workspace_bytes = ws.numel()
    _native.check(lib.b200attn_prefill(C.byref(args), C.c_void_p(stream)), "b200attn_prefill")
    return out


def flash_attention_v1(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    is_causal: bool = False,
    q_indptr: torch.Tensor | None = None,
    kv_indptr: torch.Tensor | None = None,
    k_block_table: torch.Tensor | None = None,
    v_block_table: torch.Tensor | None = None,
    kv_page_size: int | None = None,
) -> torch.Tensor:
    """Same signature and semantics as the reference's single-pass variant
    (kernels/attention.py:249-260); served by the same kernel as ``flash_attention_v2``.

    One difference for fp32 inputs: the reference's v1 kernel keeps q, k and v in fp32 and multiplies in TF32
    (kernels/attention.py:177-240), its v2 kernel rounds them to fp16 (:547-633).  This build follows v2 for both
    names, so fp32 inputs are rounded to fp16 before the tensor cores: values beyond +-65504 become infinite here
    where the reference's v1 would keep them finite, and the result is accurate to the 16-bit class (4e-3), not to
    TF32."""
    return flash_attention_v2(
        q, k, v, is_causal=is_causal, q_indptr=q_indptr, kv_indptr=kv_indptr,
        k_block_table=k_block_table, v_block_table=v_block_table, kv_page_size=kv_page_size,
    )
