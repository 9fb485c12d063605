// Inline-PTX wrappers for the Blackwell (sm_100a) features the kernels use: mbarrier, TMA tiled loads and untiled bulk
// loads, tensor memory (TMEM) allocation / load / store, tcgen05.mma with shared-memory descriptors.  Every copy lands
// in the issuing CTA's own shared memory; the only cluster traffic is st_async_pair (8-byte remote stores between the
// CTAs of a softmax cluster).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace b200attn {
namespace ptx {

// ------------------------------ mbarrier -----------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait: returns false when the phase has not completed after `limit` tries.  The loop lives in one asm
// block - a completed phase costs the caller two instructions, which matters for a warp that has to share its issue
// slots with busy neighbours - and every failed try suspends the thread in hardware for up to a microsecond or so,
// so the try count bounds the wait in time.
constexpr uint32_t kWaitTries = 4194304;   // 2^22 tries: between a tenth of a second and a few seconds
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, uint32_t limit) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\t"
      "mov.u32 n, 0;\n\t"
      "B200ATTN_WAIT_LOOP:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra B200ATTN_WAIT_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 p, n, %3;\n\t"
      "@p bra B200ATTN_WAIT_LOOP;\n\t"
      "mov.u32 %0, 0;\n\t"
      "bra B200ATTN_WAIT_END;\n\t"
      "B200ATTN_WAIT_DONE:\n\t"
      "mov.u32 %0, 1;\n\t"
      "B200ATTN_WAIT_END:\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(limit)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) { return mbar_wait_limit(bar, parity, kWaitTries); }

// Asynchronous 8-byte store of (a, b) to the shared-memory address `slot` of CTA `cta_rank` of this cluster; the
// receiver's mbarrier at `bar` (same offsets in every CTA) is credited with the 8 bytes when they have landed.
__device__ __forceinline__ void st_async_pair(uint32_t slot, uint32_t bar, uint32_t cta_rank, float a, float b) {
  asm volatile(
      "{\n\t.reg .u32 rs, rb;\n\t"
      "mapa.shared::cluster.u32 rs, %0, %2;\n\t"
      "mapa.shared::cluster.u32 rb, %1, %2;\n\t"
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [rs], {%3, %4}, [rb];\n\t}\n"
      ::"r"(slot), "r"(bar), "r"(cta_rank), "f"(a), "f"(b)
      : "memory");
}

// Untiled bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

// ------------------------------ programmatic dependent launch ----------------
// A grid launched with programmatic stream serialisation may start while the grid before it in the stream is still
// running; grid_dep_wait blocks until that grid has completed and its writes are visible (a no-op in a grid launched
// the ordinary way).  grid_dep_launch_dependents, in the earlier grid, lets the later one be scheduled from then on.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// ------------------------------ named barriers --------------------------------
// `count` threads in all; an arriving thread does not wait.
__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(ptr)); }
__device__ __forceinline__ void named_bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;\n" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory"); }

// ------------------------------ proxies / fences ----------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// ------------------------------ TMA ------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load global -> this CTA's shared memory, completion on an mbarrier.
// c0 is the innermost (contiguous) coordinate and must keep c0 * elem_size 16-byte aligned.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

// brings the box into L2 only (no shared-memory destination, no completion to wait for)
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];\n"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// ------------------------------ TMEM -----------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp reads lane (base_lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 64 consecutive 32-bit columns in the 16x256b register layout: thread t of the warp receives, for
// every group i of 8 columns, r[4i], r[4i+1] = lane (base_lane + t / 4), columns 8i + 2 (t % 4) + {0, 1} and
// r[4i+2], r[4i+3] = the same columns of lane (base_lane + t / 4 + 8).  Four neighbouring threads thus hold 8
// consecutive columns of a row, which is what a coalesced row-major store needs.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// More accesses in the 16-lane layouts.  16x256b (see tmem_ld_16x256b_x8): thread t holds, per group i of 8 columns,
// lane t / 4, columns 8i + 2 (t % 4) + {0, 1} in r[4i], r[4i+1] and lane t / 4 + 8 in r[4i+2], r[4i+3].
// 16x128b: thread t holds, per group i of 4 columns, lane t / 4, column 4i + t % 4 in r[2i] and lane t / 4 + 8 in
// r[2i+1] - which is where the packed pair of the 16x256b columns 8i + 2 (t % 4) + {0, 1} belongs.
// 16 columns at a time in the same layout: for code that runs rarely and must not hold many registers
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ------------------------------ packed fp32 pairs ------------------------------
__device__ __forceinline__ uint64_t pack_f2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_f2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// ------------------------------ tcgen05.mma ----------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, rows of 128 bytes packed
// back to back (8-row groups every 1024 bytes).  `lbo_bytes` is the distance
// between 128-byte-wide column blocks of an MN-major operand (ignored for
// K-major operands, where one MMA never leaves the 128-byte row).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);              // start address, bits [0,14)
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;          // leading byte offset, bits [16,30)
  d |= static_cast<uint64_t>((1024u >> 4) & 0x3FFFu) << 32;              // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                                   // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                                   // layout: SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 (fp16/bf16 inputs, fp32 accumulate).
//   ab_format: 0 = fp16, 1 = bf16;  b_mn_major: B operand is MN-major (N contiguous)
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, int ab_format, int b_mn_major) {
  return (1u << 4)                                     // accumulator format: fp32
         | (static_cast<uint32_t>(ab_format) << 7)     // A format
         | (static_cast<uint32_t>(ab_format) << 10)    // B format
         | (0u << 15)                                  // A K-major (or TMEM)
         | (static_cast<uint32_t>(b_mn_major) << 16)   // B major
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (static_cast<uint32_t>(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same two MMAs with the descriptors passed as (low, high) 32-bit halves: the issuing thread keeps the
// constant high words in registers and only adds byte offsets (>> 4) to the low words between MMAs.
__device__ __forceinline__ void mma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32-byte global store (address 32-byte aligned)
__device__ __forceinline__ void st_global_v8(void* ptr, uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3, uint32_t v4,
                                             uint32_t v5, uint32_t v6, uint32_t v7) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"l"(ptr), "r"(v0), "r"(v1), "r"(v2), "r"(v3),
               "r"(v4), "r"(v5), "r"(v6), "r"(v7)
               : "memory");
}

// ---------------------------------------------------------------------------
// Batched issue.  The whole (converged) warp executes these; only the lane whose `lead` is non-zero issues the
// tensor-core instructions.  Keeping the warp converged lets the descriptor arithmetic run once per warp instead
// of on a divergent single-lane path, which matters when the other warps of the SM sub-partition are busy: a
// divergent issuer was measured to fall to a sixth of the tensor-core rate under an FMA-bound neighbour, the
// converged form to about two thirds.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t r;
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\tselp.b32 %0, 1, 0, q;\n\t}\n" : "=r"(r));
  return r;
}

#define B200ATTN_SS_STEP(OFF)                                                                   \
  "add.s64 a1, %1, " #OFF ";\n\tadd.s64 b1, %2, " #OFF ";\n\t"                                  \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, t;\n\t"

// D/16 k-steps of a K-major x K-major product whose operands are 128-row, 128-byte-swizzled tiles stored as
// 64-element column blocks of 16 KiB: k-step kk starts (kk / 4) * 16 KiB + (kk % 4) * 32 bytes into both tiles.
template <int KSTEPS>
__device__ __forceinline__ void mma_ss_batch(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate_first, uint32_t lead) {
  static_assert(KSTEPS == 4 || KSTEPS == 8, "head dimension 64 or 128");
  if constexpr (KSTEPS == 8) {
    asm volatile(
        "{\n\t.reg .pred p, t, e;\n\t.reg .b64 a1, b1;\n\t"
        "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        B200ATTN_SS_STEP(2) B200ATTN_SS_STEP(4) B200ATTN_SS_STEP(6)
        B200ATTN_SS_STEP(1024) B200ATTN_SS_STEP(1026) B200ATTN_SS_STEP(1028) B200ATTN_SS_STEP(1030)
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, t, e;\n\t.reg .b64 a1, b1;\n\t"
        "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        B200ATTN_SS_STEP(2) B200ATTN_SS_STEP(4) B200ATTN_SS_STEP(6)
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead) : "memory");
  }
}
#undef B200ATTN_SS_STEP

#define B200ATTN_TS_STEP(AOFF, BOFF)                                                            \
  "add.u32 a1, %1, " #AOFF ";\n\tadd.s64 b1, %2, " #BOFF ";\n\t"                                \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n\t"

// Eight k-steps (128 keys) of O += P V: A is packed 16-bit P, keys 0..63 in the 32 tensor-memory columns at `a_tmem`
// and keys 64..127 in the 32 columns at `a_tmem + kPHalfStride`; B is an MN-major 128-row V tile, 16 rows (2 KiB)
// per k-step.
constexpr uint32_t kPHalfStride = 64;
__device__ __forceinline__ void mma_ts_batch8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate_first, uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1;\n\t.reg .b64 b1;\n\t"
      "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      B200ATTN_TS_STEP(8, 128) B200ATTN_TS_STEP(16, 256) B200ATTN_TS_STEP(24, 384)
      B200ATTN_TS_STEP(64, 512) B200ATTN_TS_STEP(72, 640) B200ATTN_TS_STEP(80, 768) B200ATTN_TS_STEP(88, 896)
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead) : "memory");
  static_assert(kPHalfStride == 64, "the offsets in the instruction list above");
}
#undef B200ATTN_TS_STEP

#define B200ATTN_TSK_STEP(AOFF, BOPND)                                                          \
  "add.u32 a1, %1, " #AOFF ";\n\tadd.s64 b1, %2, " BOPND ";\n\t"                                \
  "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n\t"

// KSTEPS k-steps of S = Q K^T with Q as packed 16-bit in tensor memory (8 columns per k-step) and K a K-major,
// 128-byte-swizzled tile stored as 64-element column blocks of CHUNK16 * 16 bytes.
template <int KSTEPS, int CHUNK16>
__device__ __forceinline__ void mma_ts_kmajor_batch(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate_first, uint32_t lead) {
  static_assert(KSTEPS == 4 || KSTEPS == 8, "head dimension 64 or 128");
  if constexpr (KSTEPS == 8) {
    asm volatile(
        "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1;\n\t.reg .b64 b1;\n\t"
        "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        B200ATTN_TSK_STEP(8, "2") B200ATTN_TSK_STEP(16, "4") B200ATTN_TSK_STEP(24, "6")
        B200ATTN_TSK_STEP(32, "%6") B200ATTN_TSK_STEP(40, "%7") B200ATTN_TSK_STEP(48, "%8") B200ATTN_TSK_STEP(56, "%9")
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead),
        "n"(CHUNK16), "n"(CHUNK16 + 2), "n"(CHUNK16 + 4), "n"(CHUNK16 + 6) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1;\n\t.reg .b64 b1;\n\t"
        "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        B200ATTN_TSK_STEP(8, "2") B200ATTN_TSK_STEP(16, "4") B200ATTN_TSK_STEP(24, "6")
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead) : "memory");
  }
}

// Four k-steps (64 keys) of O += P V: A is packed 16-bit P in 32 tensor-memory columns at `a_tmem`; B is 64 rows
// of an MN-major V tile, 16 rows (2 KiB) per k-step.
__device__ __forceinline__ void mma_ts_batch4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate_first, uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred p, t, e;\n\t.reg .b32 a1;\n\t.reg .b64 b1;\n\t"
      "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, 0, 0;\n\tsetp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      B200ATTN_TSK_STEP(8, "128") B200ATTN_TSK_STEP(16, "256") B200ATTN_TSK_STEP(24, "384")
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(lead) : "memory");
}
#undef B200ATTN_TSK_STEP

// tcgen05.commit issued by the lane whose `lead` is non-zero (warp converged)
__device__ __forceinline__ void mma_commit_lead(uint32_t bar, uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred e;\n\tsetp.ne.b32 e, %1, 0;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar), "r"(lead)
      : "memory");
}

// mbarrier arrives once every tcgen05 operation this thread issued so far has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

}  // namespace ptx
}  // namespace b200attn
