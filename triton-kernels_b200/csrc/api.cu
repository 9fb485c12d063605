// C ABI of the attention hot path: argument checks, device bookkeeping, dispatch.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "decode_launch.h"
#include "paged_append_launch.h"
#include "softmax_launch.h"
#include "prefill_launch.h"
#include "sm100_ptx.cuh"

namespace b200attn {

namespace {
thread_local char g_error[512] = "";

struct DeviceCache {
  bool valid = false;
  b200attn_device_info_t info{};
};
constexpr int kMaxDevices = 64;
DeviceCache g_devices[kMaxDevices];
std::mutex g_device_mutex;
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return B200ATTN_E_CUDA;
}

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  struct Entry { const void* kernel; int device; size_t bytes; };
  static Entry table[256];
  static int count = 0;
  static std::mutex mu;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(mu);
  Entry* hit = nullptr;
  for (int i = 0; i < count; ++i)
    if (table[i].kernel == kernel && table[i].device == device) { hit = &table[i]; break; }
  if (hit && hit->bytes >= bytes) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
  if (hit) hit->bytes = bytes;
  else if (count < 256) table[count++] = Entry{kernel, device, bytes};
  return 0;
}

static int query_device(int device, b200attn_device_info_t* out) {
  if (device < 0 || device >= kMaxDevices) { set_error("device ordinal %d out of range", device); return B200ATTN_E_INVALID; }
  std::lock_guard<std::mutex> lock(g_device_mutex);
  DeviceCache& c = g_devices[device];
  if (!c.valid) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
    c.info.sm_count = prop.multiProcessorCount;
    c.info.cc_major = prop.major;
    c.info.cc_minor = prop.minor;
    c.info.max_smem_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
    c.valid = true;
  }
  *out = c.info;
  return B200ATTN_OK;
}

// makes `device` current for the duration of a call
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  int enter(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != device) {
      e = cudaSetDevice(device);
      if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
      changed = true;
    }
    return 0;
  }
  ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_common(int dtype, int layout, int batch, int q_heads, int kv_heads, int head_dim) {
  if (dtype != B200ATTN_F16 && dtype != B200ATTN_BF16 && dtype != B200ATTN_F32) { set_error("unknown dtype %d", dtype); return B200ATTN_E_INVALID; }
  if (layout != B200ATTN_DENSE && layout != B200ATTN_RAGGED && layout != B200ATTN_PAGED) { set_error("unknown layout %d", layout); return B200ATTN_E_INVALID; }
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) { set_error("bad batch/head counts (B=%d QH=%d KVH=%d)", batch, q_heads, kv_heads); return B200ATTN_E_INVALID; }
  if (head_dim != 64 && head_dim != 128) { set_error("head_dim %d is not built (64 or 128)", head_dim); return B200ATTN_E_UNSUPPORTED; }
  return 0;
}

static int check_arch(int device, b200attn_device_info_t* info) {
  int rc = query_device(device, info);
  if (rc) return rc;
  if (info->cc_major != 10) {
    set_error("device %d is sm_%d%d; this library contains sm_100a code only", device, info->cc_major, info->cc_minor);
    return B200ATTN_E_ARCH;
  }
  return 0;
}

// One warp waits on an mbarrier that nothing will ever complete, with the same bounded wait the attention kernels
// use (only the try limit differs), records the expiry the way they do and returns.
__global__ void wait_expiry_selftest_kernel(int* header, uint32_t tries) {
  __shared__ uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) { ptx::mbar_init(b, 1); ptx::mbar_fence_init(); }
  __syncwarp();
  const bool ok = ptx::mbar_wait_limit(b, 0, tries);
  if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) header[0] = DEV_ERR_WAIT_EXPIRED;
}

}  // namespace b200attn

using namespace b200attn;

extern "C" {

int b200attn_abi_version(void) { return B200ATTN_ABI_VERSION; }

const char* b200attn_last_error(void) { return g_error; }

int b200attn_device_info(int device, b200attn_device_info_t* info) {
  if (!info) { set_error("info is null"); return B200ATTN_E_INVALID; }
  return query_device(device, info);
}

size_t b200attn_prefill_workspace_bytes(const b200attn_prefill_args_t* a) {
  if (!a || a->kv_heads <= 0 || a->q_heads <= 0) return 0;
  b200attn_device_info_t info = {};
  if (query_device(a->device, &info)) return 0;
  return prefill_workspace_bytes(*a, info.sm_count);
}

size_t b200attn_decode_workspace_bytes(const b200attn_decode_args_t* a) {
  if (!a || a->kv_heads <= 0 || a->batch < 0) return 0;
  b200attn_device_info_t info = {};
  if (query_device(a->device, &info)) return 0;
  return decode_ws_layout(*a, info.sm_count).total;
}

int b200attn_prefill(const b200attn_prefill_args_t* a, void* cuda_stream) {
  if (!a) { set_error("args is null"); return B200ATTN_E_INVALID; }
  int rc = check_common(a->dtype, a->layout, a->batch, a->q_heads, a->kv_heads, a->head_dim);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->out) { set_error("prefill: null tensor pointer"); return B200ATTN_E_INVALID; }
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) { set_error("prefill: tensors must be 16-byte aligned"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_RAGGED && (!a->q_indptr || !a->kv_indptr || a->total_q < 0 || a->total_kv < 0)) { set_error("prefill: ragged layout needs q_indptr, kv_indptr and totals"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_PAGED && (!a->kv_indptr || !a->k_table || !a->v_table || a->page_size <= 0 || a->table_stride < 0)) { set_error("prefill: paged layout needs lengths, both block tables and a page size"); return B200ATTN_E_INVALID; }
  if (a->layout != B200ATTN_RAGGED && (a->max_q < 0 || (a->layout == B200ATTN_DENSE && a->max_kv < 0))) { set_error("prefill: negative extent"); return B200ATTN_E_INVALID; }
  b200attn_device_info_t info = {};
  if ((rc = check_arch(a->device, &info))) return rc;
  if (a->batch == 0) return B200ATTN_OK;
  DeviceGuard guard;
  if ((rc = guard.enter(a->device))) return rc;
  return launch_prefill(*a, info.sm_count, static_cast<cudaStream_t>(cuda_stream));
}

int b200attn_decode(const b200attn_decode_args_t* a, void* cuda_stream) {
  if (!a) { set_error("args is null"); return B200ATTN_E_INVALID; }
  int rc = check_common(a->dtype, a->layout, a->batch, a->q_heads, a->kv_heads, a->head_dim);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->out) { set_error("decode: null tensor pointer"); return B200ATTN_E_INVALID; }
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) { set_error("decode: tensors must be 16-byte aligned"); return B200ATTN_E_INVALID; }
  if (a->q_len < 1 || a->q_len > 16) { set_error("decode: q_len %d outside 1..16", a->q_len); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_RAGGED && (!a->kv_indptr || a->total_kv < 0)) { set_error("decode: ragged layout needs kv_indptr and total_kv"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_PAGED && (!a->kv_indptr || !a->k_table || !a->v_table || a->page_size <= 0 || a->table_stride < 0)) { set_error("decode: paged layout needs lengths, both block tables and a page size"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_DENSE && a->max_kv < 0) { set_error("decode: negative extent"); return B200ATTN_E_INVALID; }
  b200attn_device_info_t info = {};
  if ((rc = check_arch(a->device, &info))) return rc;
  if (a->batch == 0) return B200ATTN_OK;
  DeviceGuard guard;
  if ((rc = guard.enter(a->device))) return rc;
  return launch_decode(*a, info.sm_count, static_cast<cudaStream_t>(cuda_stream));
}

int b200attn_decode_static(const b200attn_decode_args_t* a, void* cuda_stream) {
  if (!a) { set_error("args is null"); return B200ATTN_E_INVALID; }
  int rc = check_common(a->dtype, a->layout, a->batch, a->q_heads, a->kv_heads, a->head_dim);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->out) { set_error("decode_static: null tensor pointer"); return B200ATTN_E_INVALID; }
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) { set_error("decode_static: tensors must be 16-byte aligned"); return B200ATTN_E_INVALID; }
  if (a->q_len < 1 || a->q_len > 16) { set_error("decode_static: q_len %d outside 1..16", a->q_len); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_RAGGED && (!a->kv_indptr || a->total_kv < 0)) { set_error("decode_static: ragged layout needs kv_indptr and total_kv"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_PAGED && (!a->kv_indptr || !a->k_table || !a->v_table || a->page_size <= 0 || a->table_stride < 0)) { set_error("decode_static: paged layout needs lengths, both block tables and a page size"); return B200ATTN_E_INVALID; }
  if (a->layout == B200ATTN_DENSE && a->max_kv < 0) { set_error("decode_static: negative extent"); return B200ATTN_E_INVALID; }
  b200attn_device_info_t info = {};
  if ((rc = check_arch(a->device, &info))) return rc;
  if (a->batch == 0) return B200ATTN_OK;
  DeviceGuard guard;
  if ((rc = guard.enter(a->device))) return rc;
  return launch_decode_static(*a, info.sm_count, static_cast<cudaStream_t>(cuda_stream));
}

int b200attn_decode_static_check(int device, void* cuda_stream, int32_t* code) {
  b200attn_device_info_t info = {};
  int rc;
  if ((rc = check_arch(device, &info))) return rc;
  DeviceGuard guard;
  if ((rc = guard.enter(device))) return rc;
  return check_decode_static(device, static_cast<cudaStream_t>(cuda_stream), code);
}

int b200attn_selftest_wait_expiry(int device, void* workspace, uint32_t tries, void* cuda_stream) {
  if (!workspace) { set_error("workspace is null"); return B200ATTN_E_INVALID; }
  if (tries == 0 || tries > (1u << 20)) { set_error("selftest: tries %u outside 1..2^20", tries); return B200ATTN_E_INVALID; }
  b200attn_device_info_t info = {};
  int rc;
  if ((rc = check_arch(device, &info))) return rc;
  DeviceGuard guard;
  if ((rc = guard.enter(device))) return rc;
  wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(static_cast<int*>(workspace), tries);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "selftest kernel launch");
  return B200ATTN_OK;
}

int b200attn_paged_append(const b200attn_paged_append_args_t* a, void* cuda_stream) {
  if (!a) { set_error("args is null"); return B200ATTN_E_INVALID; }
  if (a->batch < 0 || a->total_rows < 0 || a->cache_rows < 0 || a->table_stride < 0 || a->page_size <= 0) { set_error("paged_append: negative extent or bad page size"); return B200ATTN_E_INVALID; }
  if (a->row_bytes <= 0 || (a->row_bytes & 15)) { set_error("paged_append: row_bytes %d is not a positive multiple of 16", a->row_bytes); return B200ATTN_E_UNSUPPORTED; }
  if (a->batch == 0 || a->total_rows == 0) return B200ATTN_OK;
  if (!a->src || !a->cache || !a->src_indptr || !a->table) { set_error("paged_append: null pointer"); return B200ATTN_E_INVALID; }
  if (!aligned16(a->src) || !aligned16(a->cache)) { set_error("paged_append: src and cache must be 16-byte aligned"); return B200ATTN_E_INVALID; }
  if (!a->workspace || a->workspace_bytes < static_cast<size_t>(kHeaderBytes)) { set_error("paged_append: workspace needs %d bytes", kHeaderBytes); return B200ATTN_E_WORKSPACE; }
  b200attn_device_info_t info = {};
  int rc;
  if ((rc = check_arch(a->device, &info))) return rc;
  DeviceGuard guard;
  if ((rc = guard.enter(a->device))) return rc;
  return launch_paged_append(*a, info.sm_count, static_cast<cudaStream_t>(cuda_stream));
}

int b200attn_softmax(const b200attn_softmax_args_t* a, void* cuda_stream) {
  if (!a) { set_error("args is null"); return B200ATTN_E_INVALID; }
  if (a->rows < 0 || a->cols < 0) { set_error("softmax: negative extent"); return B200ATTN_E_INVALID; }
  if (a->rows == 0 || a->cols == 0) return B200ATTN_OK;
  if (!a->x || !a->out) { set_error("softmax: null pointer"); return B200ATTN_E_INVALID; }
  if (a->dtype != B200ATTN_F16 && a->dtype != B200ATTN_BF16 && a->dtype != B200ATTN_F32) { set_error("softmax: unknown dtype %d", a->dtype); return B200ATTN_E_UNSUPPORTED; }
  b200attn_device_info_t info = {};
  int rc;
  if ((rc = check_arch(a->device, &info))) return rc;
  DeviceGuard guard;
  if ((rc = guard.enter(a->device))) return rc;
  return launch_softmax(*a, info.sm_count, static_cast<cudaStream_t>(cuda_stream));
}

int b200attn_check_workspace(void* workspace, void* cuda_stream, int32_t* code) {
  if (!workspace) { set_error("workspace is null"); return B200ATTN_E_INVALID; }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  int32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e, "reading the workspace error word");
  if (code) *code = word;
  if (word != 0) {
    // the whole header: a kernel that gave up may also have left its scheduling counters behind
    e = cudaMemsetAsync(workspace, 0, kHeaderBytes, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "clearing the workspace error word");
    set_error("a kernel reported device error code %d (1 = bounded wait expired, 2 = block-table entry out of range, 3 = planner overflow)", word);
    return B200ATTN_E_DEVICE;
  }
  return B200ATTN_OK;
}

}  // extern "C"
