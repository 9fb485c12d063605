// Paged KV-cache write side: scatters new K or V rows of every sequence into the pages its block table names.
// It is the inverse of the gather the attention kernels perform and replaces the Python double loop of the
// reference's fixtures (tests/test_attention.py:101-134, benchmarks/attention.py:351-431).  Pure byte movement:
// one warp per token row, 16-byte pieces, every source and destination byte touched once.
#include "common.cuh"
#include "paged_append_launch.h"

namespace b200attn {

namespace {

__global__ void __launch_bounds__(256) paged_append_kernel(const PagedAppendParams p) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int pieces = p.row_bytes >> 4;
  for (long long row = warp; row < p.total_rows; row += nwarps) {
    // sequence that owns this source row: last b with indptr[b] <= row
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (load_index(p.src_indptr, p.indptr_is_i64, mid) <= row) lo = mid; else hi = mid;
    }
    const int b = lo;
    const long long first = load_index(p.src_indptr, p.indptr_is_i64, b);
    const long long end = load_index(p.src_indptr, p.indptr_is_i64, b + 1);
    if (row < first || row >= end) continue;  // malformed prefix sums: nothing is written
    long long pos = row - first;
    if (p.dst_pos) pos += load_index(p.dst_pos, p.indptr_is_i64, b);
    const long long lp = pos / p.page_size;
    if (pos < 0 || lp >= p.table_stride) {
      if (lane == 0) p.header[0] = DEV_ERR_PAGE_RANGE;
      continue;
    }
    const int page = __ldg(p.table + static_cast<long long>(b) * p.table_stride + lp);
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) p.header[0] = DEV_ERR_PAGE_RANGE;   // reported, never dereferenced
      continue;
    }
    const long long dst_row = static_cast<long long>(page) * p.page_size + (pos - lp * p.page_size);
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.src) + row * p.row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.cache) + dst_row * p.row_bytes);
    for (int i = lane; i < pieces; i += 32) dst[i] = __ldg(src + i);
  }
}

}  // namespace

int launch_paged_append(const b200attn_paged_append_args_t& a, int sm_count, cudaStream_t stream) {
  PagedAppendParams p;
  p.src = a.src; p.cache = a.cache; p.src_indptr = a.src_indptr; p.dst_pos = a.dst_pos; p.table = a.table;
  p.header = static_cast<int*>(a.workspace);
  p.total_rows = a.total_rows; p.table_stride = a.table_stride;
  p.row_bytes = a.row_bytes; p.indptr_is_i64 = a.indptr_is_i64; p.batch = a.batch; p.page_size = a.page_size;
  const long long pages = a.cache_rows / a.page_size;
  p.num_pages = static_cast<int>(pages > 0x7fffffff ? 0x7fffffff : pages);
  if (a.total_rows == 0) return B200ATTN_OK;
  const long long warps_needed = a.total_rows;
  long long blocks = (warps_needed + 7) / 8;              // 8 warps per block
  const long long cap = static_cast<long long>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  paged_append_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "paged_append_kernel launch");
  return B200ATTN_OK;
}

}  // namespace b200attn
