// Row softmax / log-softmax over the last dimension for sm_100a (HBM-bound: one read, one write).
//
// Replaces the reference's small / medium / partial + merge + finalize kernels (kernels/softmax.py:18-150 and
// :239-375): there a row longer than one block is read twice (three launches when it is split over programs).
// Here a row is read once, kept on the SM and normalised from there.  Rows whose bytes are a multiple of 16:
//   softmax_reg_kernel     up to 16 384 fp32 / 16-bit elements: one CTA per row, the row in registers
//   softmax_pipe_kernel    up to 864 KiB: a CTA, or a cluster of 2, 4 or 8 CTAs, per row; slices of up to 108 KiB arrive
//                          by bulk copies into a ring of 2 to 8 shared-memory stages, so the next rows load while
//                          this one is reduced and written
//   softmax_regc_kernel    up to 1 MiB: the row in the registers of a cluster of eight CTAs
//   softmax_cluster_kernel up to 1.6 MB: 200 KiB per CTA in shared memory, cluster of eight
// Any other row:
//   softmax_row_kernel     up to 200 KiB: one CTA per row, the row in shared memory
//   softmax_cluster_kernel up to 1.6 MB (as above)
//   softmax_stream_kernel  beyond: one CTA per row, online (max, sum) pass, then a second read
// Clusters exchange their (max, sum) pairs through distributed shared memory; the pipelined and register kernels do it
// with asynchronous remote stores that count on the receiver's mbarrier, because a cluster-wide barrier also waits
// for the previous row's global stores.
// All arithmetic is fp32, like the reference's `.to(tl.float32)`: expf for fp32 rows in registers, ex2.approx of
// (x - max) * log2(e) for 16-bit types and for fp32 rows in the pipelined kernel (tl.exp compiles to the same).  `out` may alias `x`: a row is written only after all of it has been staged (the streaming kernel
// reads element i right before it writes element i), and rows staged ahead of time are other rows.
#include <cooperative_groups.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "softmax_launch.h"

namespace cg = cooperative_groups;

namespace b200attn {

namespace {

constexpr int kRowSmemBytes = 200 * 1024;   // row bytes one CTA stages
constexpr int kMaxCluster = 8;              // portable cluster size
constexpr int kPipeSliceBytes = 108 * 1024; // longest slice of a row per CTA of the pipelined kernel (two are staged)
constexpr int kPipeStages = 8;              // shorter slices: as many stages as fit 216 KiB, up to this many

__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide reductions through a 32-float scratch array; every thread gets the result
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();                 // scratch may still be read from a previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : -INFINITY;
  return warp_max(r);
}
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : 0.f;
  return warp_sum(r);
}

// the same without the leading barrier: the caller guarantees a barrier between the last read of `scratch` and this call
__device__ __forceinline__ float block_max_nolead(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  return warp_max(lane < nw ? scratch[lane] : -INFINITY);
}
__device__ __forceinline__ float block_sum_nolead(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  return warp_sum(lane < nw ? scratch[lane] : 0.f);
}

template <typename T> struct Vec16 { static constexpr int kElems = 16 / sizeof(T); };

template <typename T> __device__ __forceinline__ float fast_or_exact_exp(float x) {
  // 16-bit outputs round away far more than the approximate exponential loses; fp32 outputs need expf
  if constexpr (sizeof(T) == 2) return __expf(x);
  else return expf(x);
}


// (max, sum of exp(x - max)) of two parts
__device__ __forceinline__ void merge_ml(float& m, float& l, float m2, float l2) {
  const float g = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : expf(m - g);
  const float b = (m2 == -INFINITY) ? 0.f : expf(m2 - g);
  l = l * a + l2 * b;
  m = g;
}

// Stage `n` elements of a row in shared memory (16-byte copies when VEC) and return this thread's running max.
template <typename T, bool VEC>
__device__ __forceinline__ float stage_row(const T* src, T* row, long long n) {
  float mx = -INFINITY;
  if constexpr (VEC) {
    constexpr int E = Vec16<T>::kElems;
    const long long nv = n / E;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(row);
    for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 u = s4[i];       // (plain load: `out` may alias `x`)
      d4[i] = u;
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int k = 0; k < E; ++k) mx = fmaxf(mx, ElemTraits<T>::to_float(e[k]));
    }
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
      const T v = src[i];
      row[i] = v;
      mx = fmaxf(mx, ElemTraits<T>::to_float(v));
    }
  }
  return mx;
}

template <typename T, bool VEC>
__device__ __forceinline__ float row_exp_sum(const T* row, long long n, float m) {
  float s = 0.f;
  if (m == -INFINITY) return 0.f;
  if constexpr (VEC) {
    constexpr int E = Vec16<T>::kElems;
    const long long nv = n / E;
    const uint4* r4 = reinterpret_cast<const uint4*>(row);
    for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 u = r4[i];
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int k = 0; k < E; ++k) s += fast_or_exact_exp<T>(ElemTraits<T>::to_float(e[k]) - m);
    }
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) s += fast_or_exact_exp<T>(ElemTraits<T>::to_float(row[i]) - m);
  }
  return s;
}

// softmax: exp(x - m) / l;  log-softmax: (x - m) - log l  (in this order: m + log l would lose log l next to a
// large m)
template <typename T, bool LOG>
__device__ __forceinline__ T finish(float x, float m, float k) {
  if constexpr (LOG) return ElemTraits<T>::from_float((x - m) - k);
  else return ElemTraits<T>::from_float(fast_or_exact_exp<T>(x - m) * k);
}

template <typename T, bool LOG, bool VEC>
__device__ __forceinline__ void write_row(const T* row, T* dst, long long n, float m, float k) {
  if constexpr (VEC) {
    constexpr int E = Vec16<T>::kElems;
    const long long nv = n / E;
    const uint4* r4 = reinterpret_cast<const uint4*>(row);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
      uint4 u = r4[i];
      T* e = reinterpret_cast<T*>(&u);
#pragma unroll
      for (int q = 0; q < E; ++q) e[q] = finish<T, LOG>(ElemTraits<T>::to_float(e[q]), m, k);
      d4[i] = u;
    }
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = finish<T, LOG>(ElemTraits<T>::to_float(row[i]), m, k);
  }
}

// the constant the write pass needs: 1 / l for softmax, log l for log-softmax
template <bool LOG>
__device__ __forceinline__ float final_constant(float m, float l) {
  (void)m;
  if constexpr (LOG) return logf(l);
  else return 1.f / l;
}

// ---------------------------------------------------------------------------
// one CTA per row, the row in registers: thread t holds the 16-byte pieces t, t + blockDim, ... (VPT of them)
// ---------------------------------------------------------------------------

// the elements of one 32-bit word of a 16-byte piece (two 16-bit values, or one float) <-> fp32
template <typename T> __device__ __forceinline__ void word_to_floats(uint32_t w, float* f) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    f[0] = __uint_as_float(w << 16);                 // a bf16 is the upper half of the fp32 with the same value
    f[1] = __uint_as_float(w & 0xffff0000u);
  } else if constexpr (std::is_same<T, __half>::value) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w));
    f[0] = t.x;
    f[1] = t.y;
  } else {
    f[0] = __uint_as_float(w);
  }
}
template <typename T> __device__ __forceinline__ uint32_t floats_to_word(const float* f) {
  if constexpr (sizeof(T) == 2) return ElemTraits<T>::pack2(f[0], f[1]);
  else return __float_as_uint(f[0]);
}

// CL: the row is spread over the CTAs of a thread-block cluster (CTA `rank` holds the pieces rank * slice ...); each
// CTA normalises against its own maximum first, the (max, sum) pairs meet in distributed shared memory, and the
// correction exp(own max - row max) / row sum goes into the constant of the store loop.  The pairs are double
// buffered by row parity, so one cluster barrier per row is enough.
template <typename T, bool LOG, int VPT, bool CL>
__device__ __forceinline__ void softmax_reg_body(const T* x, T* out, long long rows, long long cols) {
  constexpr int E = Vec16<T>::kElems;
  constexpr int W = E / 4;                           // elements per 32-bit word
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ float scratch[32];
  __shared__ __align__(8) float2 pairs[2][kMaxCluster];   // CL: every CTA's (max, sum) of the even / odd row in work
  __shared__ __align__(8) uint64_t pair_bar[2];           // CL: completes when all pairs of that row have landed
  int nv = static_cast<int>(cols / E);
  unsigned csize = 1;
  int rank = 0;
  if constexpr (CL) {
    cg::cluster_group cluster = cg::this_cluster();
    rank = static_cast<int>(cluster.block_rank());
    csize = cluster.num_blocks();
    if (threadIdx.x == 0) {
      ptx::mbar_init(smem_u32(&pair_bar[0]), 1);
      ptx::mbar_init(smem_u32(&pair_bar[1]), 1);
      ptx::mbar_fence_init();
    }
    cluster.sync();                                  // once: every peer's barriers exist before anyone sends
    const int slice = (nv + static_cast<int>(csize) - 1) / static_cast<int>(csize);
    x += static_cast<long long>(slice) * rank * E;   // this CTA's pieces start here within every row
    out += static_cast<long long>(slice) * rank * E;
    nv = max(0, min(slice, nv - slice * rank));
  }
  const unsigned row_step = gridDim.x / csize;
  unsigned iter = 0;                                 // rows this CTA has worked on
  for (long long r = blockIdx.x / csize; r < rows; r += row_step, ++iter) {
    const unsigned parity = iter & 1u;
    const uint4* s4 = reinterpret_cast<const uint4*>(x + r * cols);
    uint4* d4 = reinterpret_cast<uint4*>(out + r * cols);
    float f[VPT * E];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nv) {
        const uint4 u = s4[i];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) word_to_floats<T>(w[q], &f[k * E + q * W]);
#pragma unroll
        for (int q = 0; q < E; ++q) mx = fmaxf(mx, f[k * E + q]);
      } else {
#pragma unroll
        for (int q = 0; q < E; ++q) f[k * E + q] = -INFINITY;
      }
    }
    const float m = block_max(mx, scratch);
    float sum = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int j = 0; j < VPT * E; ++j) {
        // 16-bit outputs round away far more than the approximate exponential loses: exp2((x - m) log2e), the
        // difference first (it is exact for x near m, whatever the magnitude of m); fp32 outputs need expf.
        // exp(-inf) = 0 for the padding.
        float ev;
        if constexpr (sizeof(T) == 2) ev = fast_exp2((f[j] - m) * kLog2e);
        else ev = expf(f[j] - m);
        sum += ev;
        if constexpr (!LOG) f[j] = ev;
      }
    } else if constexpr (CL && !LOG) {
      // this CTA's part is all -inf but the row may not be: its outputs are zeros
#pragma unroll
      for (int j = 0; j < VPT * E; ++j) f[j] = 0.f;
    }
    float l = block_sum(sum, scratch);
    float own = 1.f;                                 // CL: exp(own max - row max)
    float m_row = m;
    if constexpr (CL) {
      // Thread 0 posts this CTA's pair into every CTA's `pairs` (its own included) with asynchronous remote stores
      // that count bytes on the receiver's barrier: no cluster-wide barrier, no fence that would wait for the
      // previous row's global stores.  Slot reuse is safe: a peer can send row r + 2 only after it has seen this
      // CTA's pair of row r + 1, which thread 0 sends after all threads here have read the pairs of row r.
      const uint32_t bar = smem_u32(&pair_bar[parity]);
      if (threadIdx.x == 0) {
        ptx::mbar_arrive_expect_tx(bar, csize * 8u);
        const uint32_t slot = smem_u32(&pairs[parity][rank]);
        for (unsigned p = 0; p < csize; ++p) ptx::st_async_pair(slot, bar, p, m, l);
      }
      const bool landed = ptx::mbar_wait(bar, (iter >> 1) & 1u);
      float gm = -INFINITY, gl = 0.f;
      for (unsigned p = 0; p < csize; ++p) merge_ml(gm, gl, pairs[parity][p].x, pairs[parity][p].y);
      if (!landed) gl = __int_as_float(0x7fc00000);  // bounded wait ran out: the row comes out as NaN, never a hang
      own = (m == -INFINITY) ? 0.f : expf(m - gm);
      m_row = gm;
      l = gl;
    }
    float kk = final_constant<LOG>(m_row, l);
    if constexpr (CL && !LOG) kk *= own;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nv) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float t[W];
#pragma unroll
          for (int e = 0; e < W; ++e) {
            const float v = f[k * E + q * W + e];
            if constexpr (LOG) t[e] = (v - m_row) - kk;
            else t[e] = m_row == -INFINITY ? __int_as_float(0x7fc00000) : v * kk;
          }
          w[q] = floats_to_word<T>(t);
        }
        d4[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  // (a CTA may leave right away: it has received every pair sent to it, and its own last pairs have been received
  // by peers that are still waiting for them or already past that wait)
}

template <typename T, bool LOG, int VPT>
__global__ void __launch_bounds__(1024) softmax_reg_kernel(const T* x, T* out, long long rows, long long cols) {
  softmax_reg_body<T, LOG, VPT, false>(x, out, rows, cols);
}
// two CTAs per SM while a thread holds 16 elements
template <typename T, bool LOG, int VPT>
__global__ void __launch_bounds__(1024, VPT * (16 / sizeof(T)) <= 16 ? 2 : 1)
softmax_regc_kernel(const T* x, T* out, long long rows, long long cols) {
  softmax_reg_body<T, LOG, VPT, true>(x, out, rows, cols);
}

// ---------------------------------------------------------------------------
// one CTA per row, the row in shared memory
// ---------------------------------------------------------------------------
template <typename T, bool LOG, bool VEC>
__global__ void softmax_row_kernel(const T* x, T* out, long long rows, long long cols) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float scratch[32];
  T* row = reinterpret_cast<T*>(smem_raw);
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* src = x + r * cols;
    __syncthreads();               // the previous row has been written out of `row`
    float m = stage_row<T, VEC>(src, row, cols);
    m = block_max(m, scratch);     // (its barriers also publish the staged row)
    const float l = block_sum(row_exp_sum<T, VEC>(row, cols, m), scratch);
    write_row<T, LOG, VEC>(row, out + r * cols, cols, m, final_constant<LOG>(m, l));
  }
}

// ---------------------------------------------------------------------------
// one cluster per row: every CTA stages a slice, (max, sum) pairs meet in distributed shared memory
// ---------------------------------------------------------------------------
template <typename T, bool LOG, bool VEC>
__global__ void softmax_cluster_kernel(const T* x, T* out, long long rows, long long cols,
                                       long long slice) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float scratch[32];
  __shared__ float ml[2];          // this CTA's (max, sum), read by its peers
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), csize = cluster.num_blocks();
  T* row = reinterpret_cast<T*>(smem_raw);
  const long long c0 = std::min<long long>(cols, slice * rank);
  const long long n = std::min<long long>(cols - c0, slice);
  const long long nclusters = gridDim.x / csize;
  for (long long r = blockIdx.x / csize; r < rows; r += nclusters) {
    const T* src = x + r * cols + c0;
    float m = stage_row<T, VEC>(src, row, n);
    m = block_max(m, scratch);
    const float l = block_sum(row_exp_sum<T, VEC>(row, n, m), scratch);
    if (threadIdx.x == 0) { ml[0] = m; ml[1] = l; }
    cluster.sync();                // every CTA's pair is in place
    float gm = -INFINITY, gl = 0.f;
    for (unsigned p = 0; p < csize; ++p) {
      const float* peer = cluster.map_shared_rank(ml, p);
      merge_ml(gm, gl, peer[0], peer[1]);
    }
    cluster.sync();                // all pairs have been read: they may be overwritten for the next row
    write_row<T, LOG, VEC>(row, out + r * cols + c0, n, gm, final_constant<LOG>(gm, gl));
    __syncthreads();               // `row` is free again
  }
}

// ---------------------------------------------------------------------------
// long rows, pipelined: a CTA (alone, or as one of a cluster of 2, 4 or 8 that share a row) keeps two slices in shared
// memory; the bulk copy of the next row's slice runs while the current one is reduced and written out, so loads are
// in flight all the time.  Clusters exchange (max, sum) pairs like softmax_regc_kernel does.
// ---------------------------------------------------------------------------
template <typename T, bool LOG>
__global__ void __launch_bounds__(1024, 1)
softmax_pipe_kernel(const T* x, T* out, long long rows, long long cols, int slice /* 16-byte pieces per CTA */,
                    int csize, int stages /* slices staged, 2..kPipeStages */) {
  constexpr int E = Vec16<T>::kElems;
  constexpr int W = E / 4;
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float scratch[2][32];                   // [0] for the maxima, [1] for the sums: each is rewritten only
                                                     // after the barrier that ends the row
  __shared__ __align__(8) float2 pairs[2][kMaxCluster];
  __shared__ __align__(8) uint64_t pair_bar[2];
  __shared__ __align__(8) uint64_t full_bar[kPipeStages];
  const int rank = csize > 1 ? static_cast<int>(cg::this_cluster().block_rank()) : 0;
  const int nv_row = static_cast<int>(cols / E);
  const int nv = max(0, min(slice, nv_row - slice * rank));
  const uint32_t bytes = static_cast<uint32_t>(nv) * 16u;
  x += static_cast<long long>(slice) * rank * E;
  out += static_cast<long long>(slice) * rank * E;
  uint4* const base = reinterpret_cast<uint4*>(smem_raw);   // stage s at base + s * slice
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) ptx::mbar_init(smem_u32(&pair_bar[i]), 1);
    for (int i = 0; i < kPipeStages; ++i) ptx::mbar_init(smem_u32(&full_bar[i]), 1);
    ptx::mbar_fence_init();
  }
  if (csize > 1) cg::this_cluster().sync(); else __syncthreads();
  const unsigned row_step = gridDim.x / csize;
  const long long r0 = blockIdx.x / csize;
  if (threadIdx.x == 0 && nv > 0) {
    for (int s = 0; s < stages - 1; ++s) {
      const long long r = r0 + static_cast<long long>(s) * row_step;
      if (r >= rows) break;
      ptx::mbar_arrive_expect_tx(smem_u32(&full_bar[s]), bytes);
      ptx::bulk_load(smem_u32(base + static_cast<size_t>(s) * slice), x + r * cols, bytes, smem_u32(&full_bar[s]));
    }
  }
  unsigned iter = 0;
  int b = 0;                                         // stage of this iteration
  unsigned phase = 0;                                // and the parity its barrier completes with
  bool ok = true;
  for (long long r = r0; r < rows; r += row_step, ++iter) {
    if (threadIdx.x == 0 && nv > 0) {
      // refill the stage the previous iteration used: it was read for the last time before the barrier that ended
      // that iteration
      const long long rn = r + static_cast<long long>(stages - 1) * row_step;
      if (rn < rows) {
        const int bn = b == 0 ? stages - 1 : b - 1;
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive_expect_tx(smem_u32(&full_bar[bn]), bytes);
        ptx::bulk_load(smem_u32(base + static_cast<size_t>(bn) * slice), x + rn * cols, bytes, smem_u32(&full_bar[bn]));
      }
    }
    if (nv > 0) ok = ptx::mbar_wait(smem_u32(&full_bar[b]), phase) && ok;
    uint4* row = base + static_cast<size_t>(b) * slice;
    float mx = -INFINITY;
    if constexpr (sizeof(T) == 2) {
      // the maximum of 16-bit values is exact in 16 bits: one packed instruction per two elements, unpacked once
      using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
      const uint32_t ninf2 = std::is_same<T, __half>::value ? 0xfc00fc00u : 0xff80ff80u;
      uint32_t acc = ninf2;
#pragma unroll 2
      for (int i = threadIdx.x; i < nv; i += 1024) {
        const uint4 u = row[i];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const T2 t = __hmax2(*reinterpret_cast<const T2*>(&acc), *reinterpret_cast<const T2*>(&w[q]));
          acc = *reinterpret_cast<const uint32_t*>(&t);
        }
      }
      float f[2];
      word_to_floats<T>(acc, f);
      mx = fmaxf(f[0], f[1]);
    } else {
#pragma unroll 2
      for (int i = threadIdx.x; i < nv; i += 1024) {
        const uint4 u = row[i];
        mx = fmaxf(mx, fmaxf(fmaxf(__uint_as_float(u.x), __uint_as_float(u.y)),
                             fmaxf(__uint_as_float(u.z), __uint_as_float(u.w))));
      }
    }
    const float m = block_max_nolead(mx, scratch[0]);
    float sum = 0.f;
    if (m != -INFINITY) {
#pragma unroll 2
      for (int i = threadIdx.x; i < nv; i += 1024) {
        const uint4 u = row[i];
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float f[W];
          word_to_floats<T>(w[q], f);
#pragma unroll
          for (int e = 0; e < W; ++e) {
            if constexpr (sizeof(T) == 2) {
              sum += fast_exp2((f[e] - m) * kLog2e);
            } else {
              // ex2.approx is within 2^-22 relative, the scaled difference within 2^-24 of its own magnitude: inside
              // the fp32 tolerance, and what the reference's tl.exp compiles to
              const float ev = fast_exp2((f[e] - m) * kLog2e);
              sum += ev;
              if constexpr (!LOG) w[q] = __float_as_uint(ev);   // fp32 softmax keeps exp(x - m) in place
            }
          }
        }
        if constexpr (sizeof(T) == 4 && !LOG) row[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    float l = block_sum_nolead(sum, scratch[1]);
    float m_row = m, own = 1.f;
    if (csize > 1) {
      const unsigned parity = iter & 1u;
      const uint32_t bar = smem_u32(&pair_bar[parity]);
      if (threadIdx.x == 0) {
        ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(csize) * 8u);
        const uint32_t slot = smem_u32(&pairs[parity][rank]);
        for (int p = 0; p < csize; ++p) ptx::st_async_pair(slot, bar, p, m, l);
      }
      ok = ptx::mbar_wait(bar, (iter >> 1) & 1u) && ok;
      float gm = -INFINITY, gl = 0.f;
      for (int p = 0; p < csize; ++p) merge_ml(gm, gl, pairs[parity][p].x, pairs[parity][p].y);
      own = (m == -INFINITY) ? 0.f : expf(m - gm);
      m_row = gm;
      l = gl;
    }
    if (!ok) l = __int_as_float(0x7fc00000);         // a bounded wait ran out: NaN rows, never a hang
    float kk = final_constant<LOG>(m_row, l);
    if constexpr (!LOG && sizeof(T) == 4) kk *= own;
    // 16-bit softmax: exp(x - m) / l = exp2((x - m) log2e - log2 l), the division folded into the exponent (l >= 1
    // whenever the row has a finite maximum)
    const float neg_log2_l = LOG ? 0.f : -__log2f(l);
    const bool nan_row = m_row == -INFINITY;
    uint4* d4 = reinterpret_cast<uint4*>(out + r * cols);
#pragma unroll 2
    for (int i = threadIdx.x; i < nv; i += 1024) {
      const uint4 u = row[i];
      uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[W];
        word_to_floats<T>(w[q], f);
#pragma unroll
        for (int e = 0; e < W; ++e) {
          if constexpr (LOG) {
            f[e] = (f[e] - m_row) - kk;
          } else if constexpr (sizeof(T) == 2) {
            f[e] = nan_row ? __int_as_float(0x7fc00000) : fast_exp2(fmaf(f[e] - m_row, kLog2e, neg_log2_l));
          } else {
            // (a slice of -inf only still holds -inf, not exp: its outputs are zeros unless the whole row is -inf)
            f[e] = nan_row ? __int_as_float(0x7fc00000) : (m == -INFINITY ? 0.f : f[e] * kk);
          }
        }
        w[q] = floats_to_word<T>(f);
      }
      d4[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();                                 // `row` may be refilled
    if (++b == stages) { b = 0; phase ^= 1u; }
  }
}

// ---------------------------------------------------------------------------
// rows that do not fit a cluster: online (max, sum), then a second read
// ---------------------------------------------------------------------------
template <typename T, bool LOG>
__global__ void softmax_stream_kernel(const T* x, T* out, long long rows, long long cols) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* src = x + r * cols;
    T* dst = out + r * cols;
    float m = -INFINITY, l = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) {
      const float v = ElemTraits<T>::to_float(src[i]);
      if (v > m) { l = (m == -INFINITY) ? 0.f : l * expf(m - v); m = v; }
      if (v != -INFINITY) l += expf(v - m);
    }
    const float gm = block_max(m, scratch);
    const float part = (m == -INFINITY) ? 0.f : l * expf(m - gm);
    const float gl = block_sum(part, scratch);
    const float k = final_constant<LOG>(gm, gl);
    for (long long i = threadIdx.x; i < cols; i += blockDim.x)
      dst[i] = finish<T, LOG>(ElemTraits<T>::to_float(src[i]), gm, k);
  }
}

template <typename K>
int set_smem_limit(K kernel, size_t bytes) {
  return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

template <typename T, bool LOG, bool VEC>
int launch_typed(const b200attn_softmax_args_t& a, int sm_count, cudaStream_t stream) {
  const T* x = static_cast<const T*>(a.x);
  T* out = static_cast<T*>(a.out);
  const long long rows = a.rows, cols = a.cols;
  const size_t row_bytes = static_cast<size_t>(cols) * sizeof(T);
  constexpr int E = 16 / static_cast<int>(sizeof(T));
  constexpr int kMaxVpt = 32 / E;                      // 32 elements per thread
  constexpr int kPrefVpt = 16 / E;                     // 16 elements per thread: 32 registers, two 1024-thread CTAs per SM
  if (VEC && cols / E <= 1024LL * kPrefVpt) {
    const int nv = static_cast<int>(cols / E);
    int threads = 64;
    while (threads < 1024 && threads * 4 < nv) threads *= 2;
    int vpt = 1;
    while (threads * vpt < nv) vpt *= 2;
    const long long max_grid = static_cast<long long>(sm_count) * (2048 / threads) * 4;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(rows, max_grid));
    switch (vpt) {
      case 1: softmax_reg_kernel<T, LOG, 1><<<grid, threads, 0, stream>>>(x, out, rows, cols); break;
      case 2: softmax_reg_kernel<T, LOG, 2><<<grid, threads, 0, stream>>>(x, out, rows, cols); break;
      case 4: softmax_reg_kernel<T, LOG, 4><<<grid, threads, 0, stream>>>(x, out, rows, cols); break;
      default: break;                                 // (not reached: vpt <= kPrefVpt <= 4)
    }
  } else if (VEC && row_bytes <= static_cast<size_t>(kPipeSliceBytes) * kMaxCluster) {
    // measured against the alternatives below on every length from 24 576 elements up: the pipelined kernel wins
    const long long nv = cols / E;
    int csize = 1;
    while ((nv + csize - 1) / csize * 16 > kPipeSliceBytes) csize *= 2;
    const int slice = static_cast<int>((nv + csize - 1) / csize);
    const int stages = std::max(2, std::min<int>(kPipeStages, 2 * kPipeSliceBytes / (slice * 16)));
    const size_t smem = static_cast<size_t>(slice) * 16 * stages;
    auto kernel = softmax_pipe_kernel<T, LOG>;
    int rc = set_smem_limit(kernel, smem);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = csize > 1 ? 1 : 0;
    // the grid is exactly what the GPU holds at once (each CTA or cluster loops over rows)
    thread_local int key_csize = 0, resident = 0;
    thread_local size_t key_smem = 0;
    if (key_csize != csize || key_smem != smem) {
      int n = 0;
      if (csize > 1) {
        cfg.gridDim = dim3(static_cast<unsigned>(sm_count / csize * csize), 1, 1);
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters(softmax)");
      } else {
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 1024, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor(softmax)");
        n *= sm_count;
      }
      resident = std::max(1, n);
      key_csize = csize;
      key_smem = smem;
    }
    const long long clusters = std::min<long long>(rows, resident);
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * csize), 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, x, out, rows, cols, slice, csize, stages);
    if (e != cudaSuccess) return cuda_fail(e, "softmax pipelined kernel launch");
  } else if (VEC && cols / E <= 1024LL * kMaxVpt * kMaxCluster) {
    // up to 1 MiB: the row in the registers of eight CTAs, 32 elements per thread
    const int csize = kMaxCluster;
    auto kernel = softmax_regc_kernel<T, LOG, kMaxVpt>;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // the grid is exactly the clusters the GPU holds at once (each loops over rows); asked of the driver once.  The
    // answer depends on the device model only, and only B200 is accepted.
    static int cached = 0;
    if (cached == 0) {
      cfg.gridDim = dim3(static_cast<unsigned>(sm_count / csize * csize), 1, 1);
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
      if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters(softmax)");
      cached = std::max(1, n);
    }
    const long long clusters = std::min<long long>(rows, cached);
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * csize), 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, x, out, rows, cols);
    if (e != cudaSuccess) return cuda_fail(e, "softmax register cluster kernel launch");
  } else if (row_bytes <= static_cast<size_t>(kRowSmemBytes)) {
    // threads: enough for 16-byte pieces to keep every lane busy on short rows, 1024 on long ones
    int threads = 64;
    while (threads < 1024 && static_cast<long long>(threads) * 8 < cols) threads *= 2;
    const size_t smem = (row_bytes + 15) & ~static_cast<size_t>(15);
    int rc = set_smem_limit(softmax_row_kernel<T, LOG, VEC>, smem);
    if (rc) return rc;
    const long long max_grid = static_cast<long long>(sm_count) * 32;
    const unsigned grid = static_cast<unsigned>(std::min<long long>(rows, max_grid));
    softmax_row_kernel<T, LOG, VEC><<<grid, threads, smem, stream>>>(x, out, rows, cols);
  } else if (row_bytes <= static_cast<size_t>(kRowSmemBytes) * kMaxCluster) {
    // more CTAs per row while a slice stays above 64 KiB (fp32) / 128 KiB (16-bit), measured: smaller CTAs share an SM
    // and one's loads overlap another's stores
    int csize = 2;
    while (csize < kMaxCluster && (static_cast<size_t>(kRowSmemBytes) * csize < row_bytes || row_bytes / csize > (sizeof(T) == 4 ? 64 : 128) * 1024)) csize *= 2;
    long long slice = (cols + csize - 1) / csize;
    slice = ((slice + E - 1) / E) * E;                 // slices start on 16-byte boundaries of the row
    const size_t smem = static_cast<size_t>(slice) * sizeof(T);
    int rc = set_smem_limit(softmax_cluster_kernel<T, LOG, VEC>, smem);
    if (rc) return rc;
    const int per_sm = std::max<int>(1, std::min<int>(2, static_cast<int>((220 * 1024) / (smem + 1024))));
    const long long clusters = std::min<long long>(rows, std::max(1, sm_count * per_sm / csize));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * csize), 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, softmax_cluster_kernel<T, LOG, VEC>, x, out, rows, cols, slice);
    if (e != cudaSuccess) return cuda_fail(e, "softmax cluster kernel launch");
  } else {
    const unsigned grid = static_cast<unsigned>(std::min<long long>(rows, static_cast<long long>(sm_count) * 2));
    softmax_stream_kernel<T, LOG><<<grid, 1024, 0, stream>>>(x, out, rows, cols);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "softmax kernel launch");
  return B200ATTN_OK;
}

template <typename T>
int launch_dtype(const b200attn_softmax_args_t& a, int sm_count, cudaStream_t stream) {
  // 16-byte copies need every row to start on a 16-byte boundary
  const bool vec = (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 &&
                   (static_cast<size_t>(a.cols) * sizeof(T)) % 16 == 0;
  if (a.log_softmax) {
    return vec ? launch_typed<T, true, true>(a, sm_count, stream) : launch_typed<T, true, false>(a, sm_count, stream);
  }
  return vec ? launch_typed<T, false, true>(a, sm_count, stream) : launch_typed<T, false, false>(a, sm_count, stream);
}

}  // namespace

int launch_softmax(const b200attn_softmax_args_t& a, int sm_count, cudaStream_t stream) {
  switch (a.dtype) {
    case B200ATTN_F16: return launch_dtype<__half>(a, sm_count, stream);
    case B200ATTN_BF16: return launch_dtype<__nv_bfloat16>(a, sm_count, stream);
    case B200ATTN_F32: return launch_dtype<float>(a, sm_count, stream);
    default: set_error("softmax: unknown dtype %d", a.dtype); return B200ATTN_E_UNSUPPORTED;
  }
}

}  // namespace b200attn
