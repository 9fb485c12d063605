// Host/device shared declarations for the prefill path.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/b200attn.h"

namespace b200attn {

struct PrefillParams {
  void* out;
  const void* q_indptr;
  const void* kv_indptr;
  const int* k_table;
  const int* v_table;
  int* header;          // workspace header, word 0 = device error code
  int* work_counter;    // workspace header words 8, 9: items drawn beyond the first of each CTA; CTAs finished
  int total_items;
  long long table_stride;
  int layout;
  int indptr_is_i64;
  int batch;
  int q_heads;
  int kv_heads;
  int group;
  int max_q;
  int max_kv;
  int page_size;
  int box_rows;         // tokens per TMA box of a paged cache
  int num_pages;
  int is_causal;
  int out_align32;      // the output pointer is 32-byte aligned: the epilogue may use 32-byte stores
  int head_pair;        // 1: the two slots of a work item are two q heads of one KV head over the same 128 rows
  int kv_split;         // parts every sequence's KV range is cut into (1: not split)
  int kv_split_len;     // keys per part (a multiple of 128)
  float* lse;           // split only: log-sum-exp per (virtual sequence, q head, row), log2 domain
  float scale_log2;
};

size_t prefill_workspace_bytes(const b200attn_prefill_args_t& a, int sm_count);
int launch_prefill(const b200attn_prefill_args_t& a, int sm_count, cudaStream_t stream);

}  // namespace b200attn
