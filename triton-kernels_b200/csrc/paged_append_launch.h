// Host/device shared declarations for the paged-cache append kernel.
#pragma once

#include <cuda_runtime.h>

#include "../../include/b200attn.h"

namespace b200attn {

struct PagedAppendParams {
  const void* src;
  void* cache;
  const void* src_indptr;
  const void* dst_pos;
  const int* table;
  int* header;            // workspace header, word 0 = device error code
  long long total_rows;
  long long table_stride;
  int row_bytes;          // bytes of one token row (heads * head_dim * element size), a multiple of 16
  int indptr_is_i64;
  int batch;
  int page_size;
  int num_pages;
};

int launch_paged_append(const b200attn_paged_append_args_t& a, int sm_count, cudaStream_t stream);

}  // namespace b200attn
