"""Write side of the paged KV cache: scatter new K or V rows into the pages named by a block table.

The reference has no such entry point; its tests and benchmarks fill paged caches with a Python double loop
(tests/test_attention.py:101-134, benchmarks/attention.py:351-431).  This is the step that precedes paged decode
in any real caller, done on the GPU through ``b200attn_paged_append``."""
from __future__ import annotations

import ctypes as C

import torch

from . import _native


def append_paged_kv(
    cache: torch.Tensor,
    block_table: torch.Tensor,
    src: torch.Tensor,
    src_indptr: torch.Tensor,
    kv_page_size: int,
    *,
    dst_pos: torch.Tensor | None = None,
) -> torch.Tensor:
    """Copy ``src`` rows into ``cache`` in place and return ``cache``.

    cache       (pages * page_size, H, D) or (pages, page_size, H, D)
    block_table (B, max_blocks_per_seq) int32
    src         (total_new, H, D): the new rows of all sequences, packed in sequence order
    src_indptr  (B + 1,) prefix sums over ``src`` rows (int32 or int64)
    dst_pos     (B,) position inside each sequence of its first new row; None = 0 (fill from scratch)
    """
    assert cache.is_cuda and src.is_cuda and block_table.is_cuda and src_indptr.is_cuda, "tensors must be on a CUDA device"
    assert cache.device == src.device == block_table.device == src_indptr.device
    assert cache.dtype == src.dtype, "cache and src must have the same dtype"
    assert cache.is_contiguous() and src.is_contiguous(), "cache and src must be contiguous"
    assert src.ndim == 3 and cache.ndim in (3, 4) and tuple(cache.shape[-2:]) == tuple(src.shape[-2:])
    page = int(kv_page_size)
    assert page > 0
    cache_rows = cache.shape[0] * cache.shape[1] if cache.ndim == 4 else cache.shape[0]
    assert block_table.ndim == 2 and block_table.dtype in (torch.int32, torch.int64)
    table = block_table if block_table.dtype == torch.int32 else block_table.to(torch.int32)
    table = table.contiguous()
    batch = table.shape[0]
    assert src_indptr.dtype in (torch.int32, torch.int64) and src_indptr.numel() == batch + 1
    src_indptr = src_indptr.contiguous()
    if dst_pos is not None:
        assert dst_pos.numel() == batch and dst_pos.device == src.device
        dst_pos = dst_pos.to(src_indptr.dtype).contiguous()
    row_bytes = src.shape[1] * src.shape[2] * src.element_size()
    assert row_bytes % 16 == 0, "heads * head_dim * element size must be a multiple of 16 bytes"
    if src.shape[0] == 0 or batch == 0:
        return cache
    stream = torch.cuda.current_stream(src.device).cuda_stream
    ws = _native.workspace(src.device, stream, 256)
    a = _native.PagedAppendArgs()
    a.src, a.cache = src.data_ptr(), cache.data_ptr()
    a.src_indptr = src_indptr.data_ptr()
    a.dst_pos = dst_pos.data_ptr() if dst_pos is not None else None
    a.table = table.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.total_rows, a.cache_rows, a.table_stride = src.shape[0], cache_rows, table.shape[1]
    a.row_bytes, a.indptr_is_i64 = row_bytes, int(src_indptr.dtype == torch.int64)
    a.batch, a.page_size = batch, page
    a.device = src.device.index if src.device.index is not None else torch.cuda.current_device()
    _native.check(_native.lib().b200attn_paged_append(C.byref(a), C.c_void_p(stream)), "b200attn_paged_append")
    return cache
