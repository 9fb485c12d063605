#include "tensor_map.h"

#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"

namespace b200attn {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link-time dependency on libcuda
EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Encoding a map costs a driver call of a microsecond or two, three of them per prefill launch.  Serving loops call
// with the same buffers and shapes over and over, so the last few maps are kept, keyed on everything that went into
// them (the map holds nothing but those values: a buffer that was freed and reallocated at the same address with the
// same shape yields the same map).
struct MapKey {
  const void* base;
  long long a, b, c;
  int kind, dtype, heads, D, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && a == o.a && b == o.b && c == o.c && kind == o.kind && dtype == o.dtype && heads == o.heads &&
           D == o.D && box_rows == o.box_rows;
  }
};
constexpr int kMapCache = 32;
struct MapCache {
  std::mutex mu;
  MapKey keys[kMapCache];
  CUtensorMap maps[kMapCache];
  bool used[kMapCache] = {};
  int next = 0;
  bool find(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < kMapCache; ++i)
      if (used[i] && keys[i] == k) { *out = maps[i]; return true; }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> lock(mu);
    keys[next] = k; maps[next] = m; used[next] = true;
    next = (next + 1) % kMapCache;
  }
};
MapCache g_map_cache;
}  // namespace

int make_token_map(CUtensorMap* m, int dtype, const void* base, long long tokens, int heads, int D, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return B200ATTN_E_CUDA; }
  if (tokens < 1) tokens = 1;  // an empty tensor still needs a well-formed map; it is never dereferenced
  const MapKey key{base, tokens, 0, 0, 3, dtype, heads, D, box_rows};
  if (g_map_cache.find(key, m)) return 0;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(D) * 2 * heads};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == B200ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (tokens=%lld heads=%d D=%d box_rows=%d)", static_cast<int>(r),
              tokens, heads, D, box_rows);
    return B200ATTN_E_CUDA;
  }
  g_map_cache.put(key, *m);
  return 0;
}

int make_kv_rows_map(CUtensorMap* m, int dtype, const void* base, long long rows, int heads, int D, int box_rows,
                     long long row_stride_bytes, long long head_stride_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return B200ATTN_E_CUDA; }
  if (rows < 1) rows = 1;
  const MapKey key{base, rows, row_stride_bytes, head_stride_bytes, 4, dtype, heads, D, box_rows};
  if (g_map_cache.find(key, m)) return 0;
  const int chunks = D / 64;
  const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(chunks), static_cast<cuuint64_t>(heads)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride_bytes), 128, static_cast<cuuint64_t>(head_stride_bytes)};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(chunks), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == B200ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (4-D) failed with CUresult %d (rows=%lld heads=%d D=%d box_rows=%d)", static_cast<int>(r),
              rows, heads, D, box_rows);
    return B200ATTN_E_CUDA;
  }
  g_map_cache.put(key, *m);
  return 0;
}

}  // namespace b200attn
