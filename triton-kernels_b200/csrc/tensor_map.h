// Host helper: TMA tensor maps over token-major 16-bit tensors.
#pragma once

#include <cuda.h>

namespace b200attn {

// 3-D map over a [tokens][heads][D] 16-bit tensor (heads == 1 for tensors whose rows of one head are
// contiguous): box = 64 elements x 1 head x box_rows tokens, 128-byte swizzle, zero fill out of bounds.
// `dtype` is B200ATTN_F16 or B200ATTN_BF16.  Returns 0 or a B200ATTN_E_* code.
int make_token_map(CUtensorMap* m, int dtype, const void* base, long long tokens, int heads, int D, int box_rows);

}  // namespace b200attn
