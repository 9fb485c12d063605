"""Decode attention entry point (drop-in for the reference's ``kernels/decode.py:203-331``)
and the launcher shared with speculative decode."""
from __future__ import annotations

import ctypes as C
import math

import torch

from utils.validation import AttentionProblem, validate_decode

from . import _native


def _launch_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, prob: AttentionProblem, causal: bool) -> torch.Tensor:
    out = torch.empty_like(q)
    if q.numel() == 0:
        return out
    stream = torch.cuda.current_stream(q.device).cuda_stream
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()

    args = _native.DecodeArgs()
    args.q, args.k, args.v, args.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    args.kv_indptr = prob.kv_indptr.data_ptr() if prob.kv_indptr is not None else None
    args.k_table = prob.k_table.data_ptr() if prob.k_table is not None else None
    args.v_table = prob.v_table.data_ptr() if prob.v_table is not None else None
    args.total_kv = prob.total_kv
    args.table_stride = prob.table_stride
    args.dtype = _native.DTYPE_CODE[q.dtype]
    args.layout = prob.layout
    args.indptr_is_i64 = int(prob.indptr_is_i64)
    args.batch = prob.batch
    args.q_heads = prob.q_heads
    args.kv_heads = prob.kv_heads
    args.q_len = prob.q_len
    args.max_kv = prob.max_kv
    args.head_dim = prob.head_dim
    args.page_size = prob.page_size
    args.causal_drafts = int(bool(causal))
    args.device = dev
    args.sm_scale = 1.0 / math.sqrt(prob.head_dim)

    lib = _native.lib()
    need = lib.b200attn_decode_workspace_bytes(C.byref(args))
    if need == 0:
        raise RuntimeError(f"b200attn_decode_workspace_bytes failed: {_native.last_error()}")
    ws = _native.workspace(q.device, stream, need)
    args.workspace = ws.data_ptr()
    args.workspace_bytes = ws.numel()
    _native.check(lib.b200attn_decode(C.byref(args), C.c_void_p(stream)), "b200attn_decode")
    return out


def decode_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    kv_indptr: torch.Tensor | None = None,
    k_block_table: torch.Tensor | None = None,
    v_block_table: torch.Tensor | None = None,
    kv_page_size: int | None = None,
) -> torch.Tensor:
    """Decode attention (one query token per sequence) with dense, ragged and paged KV.

    Dense  : q (B, QH, D), k/v (B, KVH, N, D)
    Ragged : q (B, QH, D), k/v (total_kv, KVH, D), kv_indptr (B + 1,)
    Paged  : q (B, QH, D), k/v (total_kv_tokens, KVH, D), kv_indptr (B,) context lengths,
             k_block_table / v_block_table (B, max_blocks_per_seq), kv_page_size
    """
    prob = validate_decode(q, k, v, kv_indptr, k_block_table, v_block_table, kv_page_size, spec=False)
    return _launch_decode(q, k, v, prob, causal=False)
