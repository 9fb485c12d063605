// Host/device shared declarations for the decode path.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/b200attn.h"

namespace b200attn {

// Kernel parameter block (passed by value).
struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const void* kv_indptr;
  const int* k_table;
  const int* v_table;
  int* header;       // [0] error code, [1] chunk tokens, [2] number of work items
  int* item_start;   // [batch + 1] prefix of per-sequence chunk counts
  int* counters;     // [batch * kv_heads] merge tickets
  int4* item_info;   // [max_items][2]: {sequence, chunk, chunks of the sequence, first item of the sequence}, {len, -, start lo, start hi}
  float* part_ml;    // [slot][rows][2]  (running max in log2 units, running sum)
  float* part_o;     // [slot][rows][D]  un-normalised accumulators
  long long total_kv;
  long long table_stride;
  int layout;
  int indptr_is_i64;
  int batch;
  int q_heads;
  int kv_heads;
  int group;         // q heads per kv head served by this launch
  int head_stride;   // q heads per kv head in the tensors
  int head0;         // first q head (inside each kv head's group) this launch serves
  int q_len;         // M
  int rows;          // group * M: q rows that share one kv head
  int n_mtiles;      // ceil(rows / 16)
  int max_kv;
  int page_size;
  int page_shift;    // log2(page_size) or -1
  int num_pages;
  int box_shift;     // log2 of the keys per TMA box (paged: the largest power of two that divides the page size, <= 64)
  int causal;
  int target_items;
  int wave_items;    // items of one KV head that are resident at once (one wave of CTAs); 0: never plan a single wave
  int item_overhead; // start-up and merge of a work item, in keys of streaming time (planner's cost estimate)
  int min_chunk;
  int equal_split;   // 1: a sequence's items are of equal size; 0: full chunks and one remainder
  int max_items;
  float scale_log2;  // sm_scale * log2(e)
};

struct DecodeWsLayout {
  size_t item_start_off;
  size_t counters_off;
  size_t info_off;
  size_t ml_off;
  size_t o_off;
  size_t total;
  int target_items;
  int wave_items;    // items of one KV head that are resident at once (one wave of CTAs); 0: never plan a single wave
  int item_overhead; // start-up and merge of a work item, in keys of streaming time (planner's cost estimate)
  int min_chunk;
  int max_items;
  // fp32 inputs of a speculative-decode call: fp16 copies of q, k, v that the tensor-core kernels read
  // (0 elements: no copies, the launch reads the caller's tensors)
  size_t cast_q_off, cast_k_off, cast_v_off;
  size_t cast_q_elems, cast_kv_elems;
};

int decode_pass_group(int group, int q_len);
// `allow_cast` false: plan fp32 inputs for the fp32 FMA kernel whatever the row count (no room for copies)
DecodeWsLayout decode_ws_layout(const b200attn_decode_args_t& a, int sm_count, bool allow_cast = true);
int launch_decode(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream, bool allow_cast = true);
int launch_decode_static(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream);
int check_decode_static(int device, cudaStream_t stream, int32_t* code);

}  // namespace b200attn
