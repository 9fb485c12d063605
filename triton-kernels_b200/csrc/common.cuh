// Shared device/host helpers for the sm_100a attention kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200attn.h"

namespace b200attn {

// ---------------------------------------------------------------------------
// host-side error text (thread local; returned by b200attn_last_error)
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
// Raises a kernel's dynamic shared-memory limit to `bytes` on the current device, once per (kernel, device): later
// calls with the same or a smaller size return without a runtime call.  Returns 0 or a B200ATTN_E_* code.
int ensure_dynamic_smem(const void* kernel, size_t bytes);

// Device error codes written to the workspace header word 0.
enum DeviceErr : int {
  DEV_OK = 0,
  DEV_ERR_WAIT_EXPIRED = 1,   // a bounded mbarrier wait ran out
  DEV_ERR_PAGE_RANGE = 2,     // a block-table entry pointed outside the cache
  DEV_ERR_PLAN = 3            // planner produced more work items than the workspace holds
};

constexpr int kHeaderBytes = 256;  // workspace header: int32 words, word 0 = error code

// ---------------------------------------------------------------------------
// small device utilities
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ long long load_index(const void* p, int is_i64, long long i) {
  return is_i64 ? static_cast<const long long*>(p)[i]
                : static_cast<long long>(static_cast<const int*>(p)[i]);
}

template <typename T> struct ElemTraits;
template <> struct ElemTraits<__half> {
  static constexpr int kDtype = B200ATTN_F16;
  __device__ static __forceinline__ uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ float to_float(__half x) { return __half2float(x); }
  __device__ static __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kDtype = B200ATTN_BF16;
  __device__ static __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};
template <> struct ElemTraits<float> {
  static constexpr int kDtype = B200ATTN_F32;
  __device__ static __forceinline__ float to_float(float x) { return x; }
  __device__ static __forceinline__ float from_float(float x) { return x; }
};

// ---------------------------------------------------------------------------
// cp.async (16-byte, zero-fill when src_bytes == 0)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---------------------------------------------------------------------------
// warp-level MMA (m16n8k16, fp32 accumulate) and ldmatrix
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_m16n8k16<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                      uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_m16n8k16<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace b200attn
