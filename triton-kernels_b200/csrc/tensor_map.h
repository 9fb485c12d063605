// Host helper: TMA tensor maps over token-major 16-bit tensors.
#pragma once

#include <cuda.h>

namespace b200attn {

// 3-D map over a [tokens][heads][D] 16-bit tensor (heads == 1 for tensors whose rows of one head are
// contiguous): box = 64 elements x 1 head x box_rows tokens, 128-byte swizzle, zero fill out of bounds.
// `dtype` is B200ATTN_F16 or B200ATTN_BF16.  Returns 0 or a B200ATTN_E_* code.
int make_token_map(CUtensorMap* m, int dtype, const void* base, long long tokens, int heads, int D, int box_rows);

// 4-D map used by the decode kernels: dims (64 elements, token rows, D/64 column blocks, heads) with strides
// (row_stride_bytes, 128, head_stride_bytes); box = 64 x box_rows x D/64 x 1, 128-byte swizzle.  One copy
// brings box_rows keys of one head as [column block][row][128 B] into shared memory.
int make_kv_rows_map(CUtensorMap* m, int dtype, const void* base, long long rows, int heads, int D, int box_rows,
                     long long row_stride_bytes, long long head_stride_bytes);

}  // namespace b200attn
