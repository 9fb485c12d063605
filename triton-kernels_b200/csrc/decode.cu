// Decode and speculative-decode attention for sm_100a (HBM-bound path).
//
// One launch family replaces the reference's split kernel + merge kernel pairs
// (kernels/decode.py:22-200, kernels/speculative_decode.py:22-226):
//
//   decode_plan_kernel : 1 CTA.  Reads the sequence lengths on the device (no host sync), picks the KV chunk size
//       (the smallest of 32 candidates that keeps the batch at or below `target_items` work items, a whole number of
//       waves of resident CTAs - or of a single wave, when the batch cuts into that few near-equal items and an
//       estimate of the run time favours it), splits every sequence into equal items and writes one record per item
//       in execution order, longest first.  A work item is (sequence, KV chunk); a unit is (item, kv head), heads
//       fastest.
//   decode_mma_kernel  : up to 16 q rows per KV head.  All q rows that share the KV head (group size G x draft
//       tokens M) are packed into 16-row MMA tiles, so every K/V byte is read from HBM once per KV head (the
//       reference re-reads it once per q head).  A producer warp stages K/V tiles of 64 keys by TMA (one 4-D box per
//       page and operand) through a 2- or 3-stage mbarrier ring; block-table entries outside the cache are reported
//       and never dereferenced, V rows past the sequence end are zeroed in shared memory.  QK^T and PV run on
//       bf16/fp16 mma.sync with fp32 accumulation and an online softmax in the exp2 domain.
//   decode_umma_kernel : more than 16 q rows per KV head (speculative decode).  One 128-row tcgen05 tile: Q is
//       written to tensor memory once per unit, P once per 64-key tile, so both MMAs take their A operand from TMEM
//       and shared memory is read once per K/V byte.  Persistent: one wave of CTAs walks the unit list, the producer
//       runs ahead across units.  Same planner and partial format; merges are claimed in the CTAs' teardown.
//   decode_simt_kernel : the fp32-input variant, fp32 FMA arithmetic like the reference's decode kernel.
//   A unit whose sequence has a single chunk writes the output directly; otherwise it writes an (m, l, acc) partial
//       and takes a ticket.  In the one-CTA-per-unit kernels (emit_and_merge) the CTA that draws the last ticket of
//       its (sequence, kv head) performs the log-sum-exp merge; in the persistent kernel a CTA that has run out of
//       units claims complete pairs and merges them.  No CTA ever waits for another.
#include <algorithm>
#include <mutex>
#include <type_traits>
#include <utility>

#include "common.cuh"
#include "decode_launch.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace b200attn {

namespace {

constexpr int kTileN = 64;
constexpr int kMaxStages = 4;
constexpr int kPlanThreads = 1024;
constexpr int kPlanBuckets = 32;    // size classes of the execution order (longest items first)
constexpr int kPlanLenCache = 4096; // sequences whose lengths the planner keeps in shared memory

struct SeqInfo {
  long long start;  // ragged: first row of the sequence
  int len;
};

__device__ __forceinline__ SeqInfo seq_info(const DecodeParams& p, int b) {
  SeqInfo s;
  s.start = 0;
  if (p.layout == B200ATTN_DENSE) {
    s.len = p.max_kv;
  } else if (p.layout == B200ATTN_RAGGED) {
    long long a = load_index(p.kv_indptr, p.indptr_is_i64, b);
    long long e = load_index(p.kv_indptr, p.indptr_is_i64, b + 1);
    a = a < 0 ? 0 : (a > p.total_kv ? p.total_kv : a);
    e = e < a ? a : (e > p.total_kv ? p.total_kv : e);
    s.start = a;
    s.len = static_cast<int>(e - a);
  } else {
    long long n = load_index(p.kv_indptr, p.indptr_is_i64, b);
    long long cap = p.table_stride * static_cast<long long>(p.page_size);
    n = n < 0 ? 0 : (n > cap ? cap : n);
    s.len = static_cast<int>(n);
  }
  return s;
}

// element offset of row `t` of sequence `b`, head `h`; -1 when the block table entry is out of range
__device__ __forceinline__ long long row_offset(const DecodeParams& p, const int* table, int b, int h,
                                                long long seq_start, int t, int D) {
  if (p.layout == B200ATTN_DENSE) {
    return ((static_cast<long long>(b) * p.kv_heads + h) * p.max_kv + t) * D;
  } else if (p.layout == B200ATTN_RAGGED) {
    return ((seq_start + t) * p.kv_heads + h) * D;
  } else {
    int lp, off;
    if (p.page_shift >= 0) {
      lp = t >> p.page_shift;
      off = t & (p.page_size - 1);
    } else {
      lp = t / p.page_size;
      off = t - lp * p.page_size;
    }
    const int page = __ldg(table + static_cast<long long>(b) * p.table_stride + lp);
    if (page < 0 || page >= p.num_pages) return -1;
    return ((static_cast<long long>(page) * p.page_size + off) * p.kv_heads + h) * D;
  }
}

__device__ __forceinline__ int find_sequence(const int* item_start, int batch, int item) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (item_start[mid] <= item) lo = mid; else hi = mid;
  }
  return lo;
}

// Fills `rows` combined rows with NaN accumulators and (m, l) = (0, 1); every thread of the CTA takes part.
__device__ __forceinline__ void poison_rows(float* comb_o, float* comb_ml, int rows, int d) {
  const float nan = __int_as_float(0x7fc00000);
  for (int i = threadIdx.x; i < rows * d; i += blockDim.x) comb_o[i] = nan;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) { comb_ml[2 * i] = 0.f; comb_ml[2 * i + 1] = 1.f; }
}

// ---------------------------------------------------------------------------
// Merge of the n_chunks published partials of one (sequence, kv head) into its output rows, by the `nt` threads
// t = 0 .. nt-1 of the CTA that drew the last ticket: g = max m; O = sum 2^(m-g) acc / sum 2^(m-g) l
// (kernels/decode.py:186-197).  Leaves the ticket counter at zero for the next call.
// ---------------------------------------------------------------------------
template <typename T, int D>
__device__ __forceinline__ void merge_chunks(const DecodeParams& p, int b, int h, int n_chunks, int item0, T* out,
                                             int t, int nt) {
  constexpr int D4 = D / 4;
  const int R = p.rows;
  __threadfence();
  // One pass with a running maximum, two output elements and four chunks per step: the 24 loads of a step do not
  // depend on each other or on the running state, so they are in flight together (the merge is a chain of L2 round
  // trips otherwise).
  constexpr int E = 2;
  const long long slot0 = static_cast<long long>(item0) * p.kv_heads + h;   // chunk k lives in slot0 + k * kv_heads
  const int total = R * D4;
  for (int idx0 = t; idx0 < total; idx0 += nt * E) {
    int r[E], d4[E];
    bool live[E];
    float mg[E], l[E];
    float4 acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int idx = idx0 + e * nt;
      live[e] = idx < total;
      const int id = live[e] ? idx : idx0;
      r[e] = id / D4;
      d4[e] = id - r[e] * D4;
      mg[e] = -INFINITY;
      l[e] = 0.f;
      acc[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int k0 = 0; k0 < n_chunks; k0 += 4) {
      float mk[E][4], lk[E][4];
      float4 o[E][4];
#pragma unroll
      for (int e = 0; e < E; ++e) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool on = k0 + j < n_chunks;
          const long long s = slot0 + static_cast<long long>(on ? k0 + j : k0) * p.kv_heads;
          const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (s * R + r[e]) * 2));
          o[e][j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (s * R + r[e]) * D + d4[e] * 4));
          mk[e][j] = on ? ml.x : -INFINITY;
          lk[e][j] = ml.y;
        }
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float mn = fmaxf(fmaxf(mg[e], fmaxf(mk[e][0], mk[e][1])), fmaxf(mk[e][2], mk[e][3]));
        const float keep = (mg[e] == -INFINITY) ? 0.f : fast_exp2(mg[e] - mn);
        acc[e].x *= keep; acc[e].y *= keep; acc[e].z *= keep; acc[e].w *= keep;
        l[e] *= keep;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w = (mk[e][j] == -INFINITY) ? 0.f : fast_exp2(mk[e][j] - mn);
          acc[e].x += w * o[e][j].x; acc[e].y += w * o[e][j].y; acc[e].z += w * o[e][j].z; acc[e].w += w * o[e][j].w;
          l[e] += w * lk[e][j];
        }
        mg[e] = mn;
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if (!live[e]) continue;
      const float inv = l[e] > 0.f ? 1.f / l[e] : 0.f;
      T* dst = out + static_cast<long long>(r[e]) * D + d4[e] * 4;
      if constexpr (sizeof(T) == 2) {
        uint2 u;
        u.x = ElemTraits<T>::pack2(acc[e].x * inv, acc[e].y * inv);
        u.y = ElemTraits<T>::pack2(acc[e].z * inv, acc[e].w * inv);
        *reinterpret_cast<uint2*>(dst) = u;
      } else {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[e].x * inv, acc[e].y * inv, acc[e].z * inv, acc[e].w * inv);
      }
    }
  }
  if (t == 0) p.counters[b * p.kv_heads + h] = 0;  // leave the counter ready for the next call
}

// ---------------------------------------------------------------------------
// Emit the CTA's combined (m, l, acc) rows, then merge if this CTA is the last
// of its (sequence, kv head).  `comb_o` is smem [KS][rows_pad][D] fp32,
// `comb_ml` is smem [KS][rows_pad][2] = (m in log2 units, l).
// ---------------------------------------------------------------------------
template <typename T, int D>
__device__ __forceinline__ void emit_and_merge(const DecodeParams& p, int b, int h, int c, int n_chunks,
                                               int item0, const float* comb_o, const float* comb_ml,
                                               int KS, int rows_pad, int* s_ticket) {
  constexpr int D4 = D / 4;
  const int R = p.rows;
  T* out = static_cast<T*>(p.out) +
           ((static_cast<long long>(b) * p.q_heads + static_cast<long long>(h) * p.head_stride + p.head0) * p.q_len) * D;
  const long long slot = (static_cast<long long>(item0) + c) * p.kv_heads + h;
  for (int idx = threadIdx.x; idx < R * D4; idx += blockDim.x) {
    const int r = idx / D4, d4 = idx - r * D4;
    float mg = -INFINITY;
    for (int k = 0; k < KS; ++k) mg = fmaxf(mg, comb_ml[(k * rows_pad + r) * 2]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
    for (int k = 0; k < KS; ++k) {
      const float mk = comb_ml[(k * rows_pad + r) * 2];
      const float w = (mk == -INFINITY) ? 0.f : fast_exp2(mk - mg);
      const float4 o = *reinterpret_cast<const float4*>(comb_o + (static_cast<size_t>(k) * rows_pad + r) * D + d4 * 4);
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
      l += w * comb_ml[(k * rows_pad + r) * 2 + 1];
    }
    if (n_chunks == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* dst = out + static_cast<long long>(r) * D + d4 * 4;
      if constexpr (sizeof(T) == 2) {
        uint2 u;
        u.x = ElemTraits<T>::pack2(acc.x * inv, acc.y * inv);
        u.y = ElemTraits<T>::pack2(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(dst) = u;
      } else {
        *reinterpret_cast<float4*>(dst) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
      }
    } else {
      *reinterpret_cast<float4*>(p.part_o + (slot * R + r) * D + d4 * 4) = acc;
      if (d4 == 0) {
        p.part_ml[(slot * R + r) * 2] = mg;
        p.part_ml[(slot * R + r) * 2 + 1] = l;
      }
    }
  }
  if (n_chunks == 1) return;

  // publish the partial, draw a ticket; the last arrival merges (nobody waits)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) *s_ticket = atomicAdd(p.counters + b * p.kv_heads + h, 1);
  __syncthreads();
  if (*s_ticket != n_chunks - 1) return;
  merge_chunks<T, D>(p, b, h, n_chunks, item0, out, threadIdx.x, blockDim.x);
}

// ---------------------------------------------------------------------------
// Planner
// ---------------------------------------------------------------------------
// Keys per work item of a sequence of `len` keys that is split into `n` items.  Equal split: every item covers the
// same number of keys (a multiple of the 64-key tile), the last takes what is left.  Otherwise: the planner's chunk
// size, i.e. full chunks and one remainder.
__device__ __forceinline__ int seq_chunk(int len, int n, int global_chunk, int equal_split) {
  if (!equal_split) return global_chunk;
  const int per = (len + n - 1) / n;
  const int c = ((per + kTileN - 1) / kTileN) * kTileN;
  return c < kTileN ? kTileN : c;
}

// ceil(a / b) for a >= 0, b > 0 with `inv_b` = 1 / b in float: exact (the float quotient is at most one off for
// a < 2^22, and is corrected; larger a take the integer division).
__device__ __forceinline__ int ceil_div_fast(int a, int b, float inv_b) {
  if (a >= (1 << 22)) return static_cast<int>((static_cast<long long>(a) + b - 1) / b);
  int q = __float2int_ru(static_cast<float>(a) * inv_b);
  if (q * b < a) ++q;
  else if (q > 0 && (q - 1) * b >= a) --q;
  return q;
}

__global__ void __launch_bounds__(kPlanThreads) decode_plan_kernel(const DecodeParams p) {
  __shared__ long long s_tot[32];
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  __shared__ int s_chunk;
  __shared__ int s_cand_chunk[kPlanThreads / 32], s_cand_items[kPlanThreads / 32], s_cand_max[kPlanThreads / 32];
  __shared__ int s_pick_items;
  __shared__ int s_hist[kPlanBuckets];     // items per size class, then the class's first execution slot
  __shared__ int s_cursor[kPlanBuckets];
  __shared__ int s_len[kPlanLenCache];      // sequence lengths, read from global memory once
  __shared__ int s_first[kPlanLenCache + 1]; // item prefix per sequence (a copy of item_start that needs no round trip)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // The attention kernel behind this one is launched with programmatic stream serialisation: its CTAs may be
  // scheduled now and wait (griddepcontrol.wait) until this grid has completed, which takes its launch latency off
  // the critical path.
  ptx::grid_dep_launch_dependents();
  if (tid < kPlanBuckets) { s_hist[tid] = 0; s_cursor[tid] = 0; }
  const bool cached = p.batch <= kPlanLenCache;
  auto len_of = [&](int b) -> int { return cached ? s_len[b] : seq_info(p, b).len; };

  long long tot = 0;
  for (int b = tid; b < p.batch; b += kPlanThreads) {
    const int len = seq_info(p, b).len;
    if (cached) s_len[b] = len;
    tot += len;
  }
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  if (lane == 0) s_tot[warp] = tot;
  __syncthreads();
  // Chunk size: the smallest of 32 candidates between total / target_items and twice that for which the batch
  // splits into at most target_items items.  target_items is a whole number of waves of resident CTAs, so the grid
  // never spills a few CTAs into one more wave (measured: 2.9 waves run 8 % faster than 3.4).  One warp per candidate.
  // Then the same for a single wave (wave_items): when every sequence can be cut into near-equal items that are all
  // resident at once, nothing is started or merged a second or third time on an SM, which is worth more than the
  // finer grain of several waves if the lengths allow it (measured, 32 x 8 192 keys, 40 rows per KV head: 212 us
  // against 245 us; one KV head of that batch: 91 us against 159 us).  The two plans are compared by an estimate
  // of their run time in keys: the largest item plus the per-item overhead for one wave, the average load of a
  // resident CTA plus half an item for several.
  long long t = 0;
  for (int w = 0; w < kPlanThreads / 32; ++w) t += s_tot[w];
  // (the two divisions per sequence go through a float reciprocal, corrected to the exact quotient: a pass over 256
  // lengths with integer divisions cost 2 us, and the pass runs once or twice per call)
  auto evaluate = [&](int target, bool with_largest) {
    long long base = (t + target - 1) / target;
    base = ((base + kTileN - 1) / kTileN) * kTileN;
    if (base < p.min_chunk) base = p.min_chunk;
    if (base > (1 << 29)) base = 1 << 29;
    long long cand = base + (base * warp) / 32;
    cand = ((cand + kTileN - 1) / kTileN) * kTileN;
    const int ck = static_cast<int>(cand);
    const float inv_ck = 1.f / static_cast<float>(ck);
    long long n = 0;
    int biggest = 0;
    for (int b = lane; b < p.batch; b += 32) {
      const int len = len_of(b);
      int v = ceil_div_fast(len, ck, inv_ck);
      if (v < 1) v = 1;
      n += v;
      if (with_largest) {
        int per = ck;
        if (p.equal_split) {
          per = ((ceil_div_fast(len, v, __frcp_rn(static_cast<float>(v))) + kTileN - 1) / kTileN) * kTileN;
          if (per < kTileN) per = kTileN;
        }
        biggest = max(biggest, min(len, per));
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      n += __shfl_xor_sync(0xffffffffu, n, o);
      biggest = max(biggest, __shfl_xor_sync(0xffffffffu, biggest, o));
    }
    if (lane == 0) {
      s_cand_chunk[warp] = ck;
      s_cand_items[warp] = n > 0x7fffffff ? 0x7fffffff : static_cast<int>(n);
      s_cand_max[warp] = biggest;
    }
  };
  evaluate(p.target_items, false);
  __syncthreads();
  if (tid == 0) {
    int pick = kPlanThreads / 32 - 1;
    for (int k = 0; k < kPlanThreads / 32; ++k) {
      if (s_cand_items[k] <= p.target_items) { pick = k; break; }
    }
    s_chunk = s_cand_chunk[pick];
    s_pick_items = s_cand_items[pick];
    s_carry = 0;
  }
  __syncthreads();
  // (a batch of more sequences than a wave has CTAs cannot fit one: every sequence is at least one item)
  if (p.wave_items > 0 && p.wave_items < p.target_items && s_pick_items > p.wave_items && p.batch <= p.wave_items) {
    evaluate(p.wave_items, true);
    __syncthreads();
    if (tid == 0) {
      int pick = -1;
      for (int k = 0; k < kPlanThreads / 32; ++k) {
        if (s_cand_items[k] <= p.wave_items) { pick = k; break; }
      }
      if (pick >= 0) {
        const float ovh = static_cast<float>(p.item_overhead);
        const float n_several = static_cast<float>(s_pick_items);
        const float several = (static_cast<float>(t) + n_several * ovh) / static_cast<float>(p.wave_items) +
                              0.5f * (static_cast<float>(t) / n_several + ovh);
        const float one = static_cast<float>(s_cand_max[pick]) + ovh;
        if (one < several) s_chunk = s_cand_chunk[pick];
      }
    }
  }
  for (int i = tid; i < p.batch * p.kv_heads; i += kPlanThreads) p.counters[i] = 0;
  __syncthreads();
  const int chunk = s_chunk;

  for (int base = 0; base < p.batch; base += kPlanThreads) {
    const int b = base + tid;
    int v = 0;
    if (b < p.batch) {
      const int len = len_of(b);
      v = (len + chunk - 1) / chunk;
      if (v < 1) v = 1;
    }
    int incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += n;
      }
      s_warp[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int carry = s_carry;
    const int before = warp > 0 ? s_warp[warp - 1] : 0;
    if (b < p.batch) {
      p.item_start[b + 1] = carry + before + incl;
      if (cached) s_first[b + 1] = carry + before + incl;
    }
    __syncthreads();
    if (tid == 0) s_carry = carry + s_warp[31];
    __syncthreads();
  }
  __syncthreads();
  // Per-item records, so that a CTA learns everything about its work item from one 32-byte read.  Records are laid
  // out in execution order: longest items first (by size class), so that the CTAs still running when the grid
  // drains are the short ones.  item_start keeps the per-sequence (logical) numbering, which is what the partial
  // results and the merge use.
  auto size_class = [&](int item_len) -> int {
    int q = kPlanBuckets - 1 - static_cast<int>((static_cast<long long>(item_len) * kPlanBuckets) / (chunk + 1));
    return q < 0 ? 0 : (q > kPlanBuckets - 1 ? kPlanBuckets - 1 : q);
  };
  // (a sequence's first n - 1 items have the same size, its last one takes the remainder: two size classes)
  for (int b = tid; b < p.batch; b += kPlanThreads) {
    const int len = len_of(b);
    const int first = b == 0 ? 0 : (cached ? s_first[b] : p.item_start[b]);
    const int n = (cached ? s_first[b + 1] : p.item_start[b + 1]) - first;
    const int per = seq_chunk(len, n, chunk, p.equal_split);
    const int rem = max(0, len - (n - 1) * per);
    if (n > 1) atomicAdd(&s_hist[size_class(per)], n - 1);
    atomicAdd(&s_hist[size_class(rem)], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int q = 0; q < kPlanBuckets; ++q) { const int c = s_hist[q]; s_hist[q] = run; run += c; }
  }
  __syncthreads();
  for (int b = tid; b < p.batch; b += kPlanThreads) {
    const SeqInfo si = seq_info(p, b);
    const int first = b == 0 ? 0 : (cached ? s_first[b] : p.item_start[b]);
    const int n = (cached ? s_first[b + 1] : p.item_start[b + 1]) - first;
    const int per = seq_chunk(si.len, n, chunk, p.equal_split);
    const int rem = max(0, si.len - (n - 1) * per);
    const int4 rec1 = make_int4(si.len, per, static_cast<int>(si.start & 0xffffffffll), static_cast<int>(si.start >> 32));
    if (n > 1) {
      const int q = size_class(per);
      const int pos = s_hist[q] + atomicAdd(&s_cursor[q], n - 1);
      for (int c = 0; c < n - 1 && pos + c < p.max_items; ++c) {
        p.item_info[2 * (pos + c)] = make_int4(b, c, n, first);
        p.item_info[2 * (pos + c) + 1] = rec1;
      }
    }
    const int q = size_class(rem);
    const int pos = s_hist[q] + atomicAdd(&s_cursor[q], 1);
    if (pos < p.max_items) {
      p.item_info[2 * pos] = make_int4(b, n - 1, n, first);
      p.item_info[2 * pos + 1] = rec1;
    }
  }
  if (tid == 0) {
    p.item_start[0] = 0;
    int n_items = s_carry;
    if (n_items > p.max_items) {
      p.header[0] = DEV_ERR_PLAN;
      n_items = 0;
    }
    p.header[1] = chunk;
    p.header[2] = n_items;
    p.header[3] = 0;          // tickets drawn and not merged yet (tcgen05 kernel)
    p.header[4] = 0;          // units drawn beyond the CTAs' first ones (tcgen05 kernel)
  }
}

// ---------------------------------------------------------------------------
// bf16 / fp16 tensor-core kernel.
// Warps 0 .. n_mtiles*key_slices-1 consume; the last warp is the TMA producer.
// A stage holds 64 keys: K as D/64 column blocks of [64 rows][128 B] (128-byte swizzle, as
// written by the TMA), then V in the same form.
// ---------------------------------------------------------------------------
struct __align__(8) DecodeCtrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int ticket;
  int abort_flag;
};

// Byte offset of the 128-byte row (key t of the tile, column block cb) inside a K or V tile.  A tile is a
// sequence of TMA boxes of `1 << box_shift` keys, each stored as [column block][key][128 B].
template <int CHUNKS>
__device__ __forceinline__ uint32_t tile_row_offset(int t, int cb, int box_shift) {
  const int box = t >> box_shift, r = t & ((1 << box_shift) - 1);
  return static_cast<uint32_t>((((box * CHUNKS + cb) << box_shift) + r) << 7);
}
// address of 16-byte piece `pc` (0..7) of that row under the 128-byte swizzle (tile base 1024-byte aligned)
__device__ __forceinline__ uint32_t swz_piece(uint32_t row_off, int pc) {
  return row_off + (((pc ^ (row_off >> 7)) & 7) << 4);
}

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  const bool ok = ptx::mbar_wait(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

// Block-table read-ahead of a producer warp for paged caches: lane i owns box i of a 64-key tile (`on` only when a
// tile has at most 32 boxes).  fetch() issues the two table reads of the tile that starts at key t0 and leaves the
// raw entries in the caller's registers; row() turns an entry into the cache row of the lane's box, once the entry is
// needed (checking it then, so that nothing waits for the read before).
constexpr int kNoPage = static_cast<int>(0x80000000u);
struct PageAhead {
  const int* ktab;
  const int* vtab;
  int lane, boxes, box_rows;
  bool on;
  __device__ __forceinline__ PageAhead(const DecodeParams& p, int b, int lane_) : lane(lane_) {
    boxes = kTileN >> p.box_shift;
    box_rows = 1 << p.box_shift;
    on = p.layout == B200ATTN_PAGED && boxes <= 32;
    page_shift = p.page_shift;
    page_size = p.page_size;
    ktab = on ? p.k_table + static_cast<long long>(b) * p.table_stride : nullptr;
    vtab = on ? p.v_table + static_cast<long long>(b) * p.table_stride : nullptr;
  }
  __device__ __forceinline__ void retarget(const DecodeParams& p, int b) {
    if (on) {
      ktab = p.k_table + static_cast<long long>(b) * p.table_stride;
      vtab = p.v_table + static_cast<long long>(b) * p.table_stride;
    }
  }
  __device__ __forceinline__ void fetch(int t0, int t_end, int& kp, int& vp) const {
    const int t = t0 + lane * box_rows;
    kp = vp = kNoPage;
    if (lane < boxes && t < t_end) {
      // (page size known only at run time; a shift when it is a power of two)
      kp = __ldg(ktab + page_of(t));
      vp = __ldg(vtab + page_of(t));
    }
  }
  int page_shift, page_size;
  __device__ __forceinline__ int page_of(int t) const { return page_shift >= 0 ? (t >> page_shift) : t / page_size; }
  __device__ __forceinline__ int row(const DecodeParams& p, int page, int t0) const {
    if (page == kNoPage) return -1;
    const int t = t0 + lane * box_rows;
    const int off = page_shift >= 0 ? (t & (page_size - 1)) : t % page_size;
    // an entry outside the cache is reported and replaced by page 0: never dereferenced, output stays finite
    const bool bad = page < 0 || page >= p.num_pages;
    if (bad) p.header[0] = DEV_ERR_PAGE_RANGE;
    return p.num_pages > 0 ? (bad ? 0 : page) * p.page_size + off : -1;
  }
};

// The Q fragments are re-read from shared memory at every k-step instead of living in 4*D/16 registers per thread:
// that keeps the kernel at 128 registers, so two or three CTAs share an SM.
// NB: 16-key blocks a consumer warp handles per step (2 when a warp owns 32 or more keys of a stage).
// T: element type of q, k, v as the kernel reads them; OutT: element type of the output rows (T, or float when the
// inputs are fp16 copies of fp32 tensors).
template <typename T, int D, int kStages, int NB, int kMaxThreads, int kMinBlocks, typename OutT = T>
__global__ void __launch_bounds__(kMaxThreads, kMinBlocks) decode_mma_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                         const __grid_constant__ CUtensorMap tm_v,
                                                         const DecodeParams p) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int CPR = D * 2 / 16;            // 16-byte pieces per row
  constexpr int ROW_BYTES = D * 2;
  constexpr int CHUNKS = D / 64;             // 128-byte column blocks
  constexpr int CHUNK_BYTES = kTileN * 128;  // one column block of a 64-key tile
  constexpr int TILE_BYTES = CHUNKS * CHUNK_BYTES;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int KSTEPS = D / 16;

  ptx::grid_dep_wait();      // the planner's records are complete and visible from here on
  const int n_items = p.header[2];
  // heads vary fastest across CTAs: the CTAs that run side by side walk the same pages and read
  // neighbouring head slices of each token row, which keeps DRAM rows open
  const int item = blockIdx.x / p.kv_heads;
  if (item >= n_items) return;
  const int h = blockIdx.x - item * p.kv_heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int NMT = p.n_mtiles;
  const int n_cwarps = (blockDim.x >> 5) - 1;   // consumer warps
  const int KS = n_cwarps / NMT;
  const int mt = warp % NMT, ks = warp / NMT;   // meaningful for consumer warps only
  const int rows_pad = NMT * 16;
  const bool is_producer = warp == n_cwarps;

  const int4 rec0 = __ldg(p.item_info + 2 * item);
  const int4 rec1 = __ldg(p.item_info + 2 * item + 1);
  const int b = rec0.x, c = rec0.y, n_chunks = rec0.z, item0 = rec0.w;
  const int chunk = rec1.y;              // keys per item of this sequence
  SeqInfo si;
  si.len = rec1.x;
  si.start = (static_cast<long long>(rec1.w) << 32) | static_cast<unsigned int>(rec1.z);
  const int len = si.len;
  const int t_begin = c * chunk;
  const int t_end = min(len, t_begin + chunk);
  const int ntiles = t_end > t_begin ? (t_end - t_begin + kTileN - 1) / kTileN : 0;

  // smem: [stages (1024-byte aligned)] [Q rows] [control]
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_base = smem;
  unsigned char* q_smem = smem + kStages * STAGE_BYTES;
  DecodeCtrl* ctrl = reinterpret_cast<DecodeCtrl*>(q_smem + rows_pad * ROW_BYTES);
  const uint32_t stage_s = smem_u32(stage_base);
  const uint32_t q_s = smem_u32(q_smem);

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(smem_u32(&ctrl->full[i]), 1);
      ptx::mbar_init(smem_u32(&ctrl->empty[i]), n_cwarps);
    }
    ctrl->abort_flag = 0;
    ptx::mbar_fence_init();
  }
  // Q rows (group x drafts, contiguous in memory) -> smem, zero padded to 16-row tiles
  {
    const T* qg = static_cast<const T*>(p.q) +
                  ((static_cast<long long>(b) * p.q_heads + static_cast<long long>(h) * p.head_stride + p.head0) * p.q_len) * D;
    for (int idx = tid; idx < rows_pad * CPR; idx += blockDim.x) {
      const int row = idx / CPR, ch = idx % CPR;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (row < p.rows) val = __ldg(reinterpret_cast<const uint4*>(qg + static_cast<long long>(row) * D + ch * 8));
      *reinterpret_cast<uint4*>(q_smem + row * ROW_BYTES + ((ch ^ (row & 7)) << 4)) = val;
    }
  }
  __syncthreads();

  float m_used[2] = {-INFINITY, -INFINITY};  // exponent reference baked into o[] and l_run[]
  float l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
  const int r0 = mt * 16 + (lane >> 2);
  const int r1 = r0 + 8;

  if (is_producer) {
    // =========================== TMA producer ===========================
    if (lane == 0) { ptx::prefetch_tensormap(&tm_k); ptx::prefetch_tensormap(&tm_v); }
    int h_coord = h;
    long long row0 = si.start;               // ragged
    if (p.layout == B200ATTN_DENSE) { h_coord = 0; row0 = (static_cast<long long>(b) * p.kv_heads + h) * p.max_kv; }
    bool ok = true;
    int issued = 0;
    // Paged caches with at most one box per lane and tile: the block-table entries of a tile are read one tile ahead,
    // into two plain registers (an array indexed by a loop counter would live in local memory and the read would be
    // waited for at once), so that the table read is over by the time the tile's stage comes free.
    const PageAhead ahead(p, b, lane);
    int kp_next = kNoPage, vp_next = kNoPage;
    if (ahead.on && ntiles > 0) ahead.fetch(t_begin, t_end, kp_next, vp_next);
    for (int tile = 0; tile < ntiles; ++tile) {
      const int stage = tile % kStages, use = tile / kStages;
      if (use > 0) {
        ok = warp_wait(smem_u32(&ctrl->empty[stage]), (use - 1) & 1);
        if (!ok) break;
      }
      const int t0 = t_begin + tile * kTileN;
      const uint32_t kdst = stage_s + stage * STAGE_BYTES;
      const uint32_t vdst = kdst + TILE_BYTES;
      const uint32_t bar = smem_u32(&ctrl->full[stage]);
      if (p.layout != B200ATTN_PAGED) {
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(bar, STAGE_BYTES);
          const int row = static_cast<int>(row0 + t0);
          ptx::tma_load_4d(kdst, &tm_k, bar, 0, row, 0, h_coord);
          ptx::tma_load_4d(vdst, &tm_v, bar, 0, row, 0, h_coord);
        }
      } else if (ahead.on) {
        const int kr = ahead.row(p, kp_next, t0), vr = ahead.row(p, vp_next, t0);
        int count = (kr >= 0) + (vr >= 0);
        for (int off = 16; off > 0; off >>= 1) count += __shfl_xor_sync(0xffffffffu, count, off);
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * ahead.box_rows * 128 * CHUNKS);
        __syncwarp();
        const uint32_t boff = static_cast<uint32_t>(lane) * ahead.box_rows * 128 * CHUNKS;
        if (kr >= 0) ptx::tma_load_4d(kdst + boff, &tm_k, bar, 0, kr, 0, h_coord);
        if (vr >= 0) ptx::tma_load_4d(vdst + boff, &tm_v, bar, 0, vr, 0, h_coord);
        if (tile + 1 < ntiles) ahead.fetch(t0 + kTileN, t_end, kp_next, vp_next);
      } else {
        // one box of box_rows keys per (lane, round); only pages that hold keys of this chunk are fetched
        const int boxes = kTileN >> p.box_shift;
        const int box_rows = 1 << p.box_shift;
        const int* ktab = p.k_table + static_cast<long long>(b) * p.table_stride;
        const int* vtab = p.v_table + static_cast<long long>(b) * p.table_stride;
        int krow[2], vrow[2];
        int count = 0, n = 0;
        for (int i = lane; i < boxes; i += 32, ++n) {
          const int t = t0 + i * box_rows;
          int kr = -1, vr = -1;
          if (t < t_end) {
            int lp, off;
            if (p.page_shift >= 0) { lp = t >> p.page_shift; off = t & (p.page_size - 1); }
            else { lp = t / p.page_size; off = t - lp * p.page_size; }
            const int kp = __ldg(ktab + lp), vp = __ldg(vtab + lp);
            // an entry outside the cache is reported and replaced by page 0: never dereferenced, output stays finite
            const bool kbad = kp < 0 || kp >= p.num_pages, vbad = vp < 0 || vp >= p.num_pages;
            if (kbad || vbad) p.header[0] = DEV_ERR_PAGE_RANGE;
            if (p.num_pages > 0) {
              kr = (kbad ? 0 : kp) * p.page_size + off;
              vr = (vbad ? 0 : vp) * p.page_size + off;
            }
          }
          krow[n] = kr; vrow[n] = vr;
          count += (kr >= 0) + (vr >= 0);
        }
        for (int off = 16; off > 0; off >>= 1) count += __shfl_xor_sync(0xffffffffu, count, off);
        if (lane == 0) ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * box_rows * 128 * CHUNKS);
        __syncwarp();
        n = 0;
        for (int i = lane; i < boxes; i += 32, ++n) {
          const uint32_t boff = static_cast<uint32_t>(i) * box_rows * 128 * CHUNKS;
          if (krow[n] >= 0) ptx::tma_load_4d(kdst + boff, &tm_k, bar, 0, krow[n], 0, h_coord);
          if (vrow[n] >= 0) ptx::tma_load_4d(vdst + boff, &tm_v, bar, 0, vrow[n], 0, h_coord);
        }
      }
      issued = tile + 1;
    }
    if (!ok) {
      if (lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; ctrl->abort_flag = 1; }
      // bounded drain of the copies still in flight before the CTA may exit
      for (int t = max(0, issued - kStages); t < issued; ++t)
        ptx::mbar_wait(smem_u32(&ctrl->full[t % kStages]), (t / kStages) & 1);
    }
  } else {
    // =========================== consumers ===========================
    uint32_t qf[4];
    const int q_row = mt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const uint32_t q_rbase = q_s + q_row * ROW_BYTES;
    int lim0 = len - 1, lim1 = len - 1;  // last visible key index for each of this lane's two rows
    if (p.causal) {
      lim0 = len - p.q_len + (r0 % p.q_len);
      lim1 = len - p.q_len + (r1 % p.q_len);
    }
    const int lim_min = min(lim0, lim1);
    const float sl2 = p.scale_log2;
    bool ok = true;

    for (int tile = 0; tile < ntiles; ++tile) {
      const int stage = tile % kStages, use = tile / kStages;
      ok = warp_wait(smem_u32(&ctrl->full[stage]), use & 1);
      if (!ok) break;
      const uint32_t ks_base = stage_s + stage * STAGE_BYTES;
      const uint32_t vs_base = ks_base + TILE_BYTES;
      const int tile_t0 = t_begin + tile * kTileN;
      const int valid = len - tile_t0;  // keys of this tile that belong to the sequence

      // one step = NB consecutive 16-key blocks: the softmax bookkeeping (max, shuffles, rescale test) and the
      // Q fragment reads are shared by the NB blocks
      for (int sb = ks * NB; sb < kTileN / 16; sb += KS * NB) {
        const int tok0 = sb * 16;             // within tile
        const int abs0 = tile_t0 + tok0;      // within sequence
        if (abs0 >= t_end) break;
        if (valid < tok0 + 16 * NB) {
          // keys past the sequence end get P == 0, but their V rows may hold anything (page tails,
          // the next sequence, stale shared memory): zero them so that 0 * x stays 0
          unsigned char* vtile = stage_base + stage * STAGE_BYTES + TILE_BYTES;
          const int first = max(valid, tok0);
          const int npieces = (tok0 + 16 * NB - first) * CHUNKS * 8;
          for (int i = lane; i < npieces; i += 32) {
            const int t = first + i / (CHUNKS * 8), cb = (i >> 3) % CHUNKS;
            *reinterpret_cast<uint4*>(vtile + tile_row_offset<CHUNKS>(t, cb, p.box_shift) + ((i & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
          }
          __syncwarp();
        }
        float s[2 * NB][4];
#pragma unroll
        for (int i = 0; i < 2 * NB; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
        {
          const int mat = lane >> 3;
          uint32_t roff[NB][CHUNKS];
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const int trow = tok0 + nb * 16 + (mat >> 1) * 8 + (lane & 7);
#pragma unroll
            for (int cb = 0; cb < CHUNKS; ++cb) roff[nb][cb] = tile_row_offset<CHUNKS>(trow, cb, p.box_shift);
          }
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const int ch = kk * 2 + (mat & 1);   // 16-byte piece index along D
            const int qch = kk * 2 + (lane >> 4);
            ldmatrix_x4(qf, q_rbase + ((qch ^ (q_row & 7)) << 4));
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              uint32_t kb[4];
              ldmatrix_x4(kb, ks_base + swz_piece(roff[nb][ch >> 3], ch & 7));
              mma_m16n8k16<T>(s[2 * nb], qf, kb[0], kb[1]);
              mma_m16n8k16<T>(s[2 * nb + 1], qf, kb[2], kb[3]);
            }
          }
        }
        // scale, mask (only where the step reaches a row's last visible key), online softmax in the exp2 domain
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const bool all_visible = __all_sync(0xffffffffu, abs0 + 16 * NB - 1 <= lim_min);
        if (all_visible) {
#pragma unroll
          for (int nt = 0; nt < 2 * NB; ++nt) {
            s[nt][0] *= sl2; s[nt][1] *= sl2; s[nt][2] *= sl2; s[nt][3] *= sl2;
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < 2 * NB; ++nt) {
            const int col = abs0 + nt * 8 + 2 * (lane & 3);
            s[nt][0] = (col <= lim0) ? s[nt][0] * sl2 : -INFINITY;
            s[nt][1] = (col + 1 <= lim0) ? s[nt][1] * sl2 : -INFINITY;
            s[nt][2] = (col <= lim1) ? s[nt][2] * sl2 : -INFINITY;
            s[nt][3] = (col + 1 <= lim1) ? s[nt][3] * sl2 : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // the accumulators are rescaled only when a row's max grew by more than 2^8; until then the
        // older reference keeps being used (exact: the same reference normalises the row at the end)
        const bool need0 = (mx0 - m_used[0]) > 8.f, need1 = (mx1 - m_used[1]) > 8.f;
        if (__any_sync(0xffffffffu, need0 || need1)) {
          float a0 = 1.f, a1 = 1.f;
          if (need0) { a0 = fast_exp2(m_used[0] - mx0); m_used[0] = mx0; }
          if (need1) { a1 = fast_exp2(m_used[1] - mx1); m_used[1] = mx1; }
          l_run[0] *= a0; l_run[1] *= a1;
#pragma unroll
          for (int i = 0; i < D / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        }
        const float ms0 = (m_used[0] == -INFINITY) ? 0.f : m_used[0];
        const float ms1 = (m_used[1] == -INFINITY) ? 0.f : m_used[1];
        uint32_t pa[NB][4];
#pragma unroll
        for (int nt = 0; nt < 2 * NB; ++nt) {
          const float p0 = fast_exp2(s[nt][0] - ms0), p1 = fast_exp2(s[nt][1] - ms0);
          const float p2 = fast_exp2(s[nt][2] - ms1), p3 = fast_exp2(s[nt][3] - ms1);
          l_run[0] += p0 + p1;   // per-lane partial row sums; reduced over the quad at the end
          l_run[1] += p2 + p3;
          pa[nt >> 1][(nt & 1) * 2 + 0] = ElemTraits<T>::pack2(p0, p1);
          pa[nt >> 1][(nt & 1) * 2 + 1] = ElemTraits<T>::pack2(p2, p3);
        }
        {
          const int mat = lane >> 3;
          uint32_t roff[NB][CHUNKS];
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const int trow = tok0 + nb * 16 + (mat & 1) * 8 + (lane & 7);
#pragma unroll
            for (int cb = 0; cb < CHUNKS; ++cb) roff[nb][cb] = tile_row_offset<CHUNKS>(trow, cb, p.box_shift);
          }
#pragma unroll
          for (int n0 = 0; n0 < D / 16; ++n0) {
            const int ch = n0 * 2 + (mat >> 1);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              uint32_t vb[4];
              ldmatrix_x4_trans(vb, vs_base + swz_piece(roff[nb][ch >> 3], ch & 7));
              mma_m16n8k16<T>(o[2 * n0], pa[nb], vb[0], vb[1]);
              mma_m16n8k16<T>(o[2 * n0 + 1], pa[nb], vb[2], vb[3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(smem_u32(&ctrl->empty[stage]));
    }
    if (!ok && lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; ctrl->abort_flag = 1; }
  }
  __syncthreads();  // every tile consumed (or the CTA gave up): the stage ring is free for the cross-warp combine

  float* comb_o = reinterpret_cast<float*>(stage_base);
  float* comb_ml = comb_o + static_cast<size_t>(KS) * rows_pad * D;
  if (!is_producer) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    float* o0 = comb_o + (static_cast<size_t>(ks) * rows_pad + r0) * D;
    float* o1 = comb_o + (static_cast<size_t>(ks) * rows_pad + r1) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + 2 * (lane & 3);
      *reinterpret_cast<float2*>(o0 + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(o1 + col) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
      comb_ml[(ks * rows_pad + r0) * 2] = m_used[0];
      comb_ml[(ks * rows_pad + r0) * 2 + 1] = l_run[0];
      comb_ml[(ks * rows_pad + r1) * 2] = m_used[1];
      comb_ml[(ks * rows_pad + r1) * 2 + 1] = l_run[1];
    }
  }
  __syncthreads();
  if (ctrl->abort_flag) {
    // A bounded wait ran out: the CTA's rows are unknown.  It still emits and draws its ticket, so that the
    // (sequence, kv head) is merged and its counter returns to zero, but with NaN rows: the failure shows in the
    // output as well as in the error word.
    poison_rows(comb_o, comb_ml, KS * rows_pad, D);
    __syncthreads();
  }
  emit_and_merge<OutT, D>(p, b, h, c, n_chunks, item0, comb_o, comb_ml, KS, rows_pad, &ctrl->ticket);
}

// ---------------------------------------------------------------------------
// tcgen05 kernel for many q rows per KV head (speculative decode: group x drafts > 16 rows).
//
// With 17..128 rows the warp-level MMA kernel above is bound by shared-memory bandwidth: every K/V fragment is
// re-read by ldmatrix once per 16-row tile.  Here the rows are padded to one 128-row tcgen05 tile whose A operands
// live in tensor memory (Q is written there once per work unit, P once per key tile), so shared memory is read
// exactly once per K/V byte, by the tensor core.  Per 64-key tile: S = Q K^T (TS MMA, 128 x 64 x D) -> the softmax
// warps (thread = q row, only the warps that hold real rows work) read S from TMEM, mask, keep the running max / sum
// in the exp2 domain with the lazy 2^8 rescale, write P as packed 16-bit over S -> O += P V (TS MMA, V is the
// MN-major B operand).  Two CTAs share an SM (256 TMEM columns, 3 stages of 64 keys each), which overlaps one CTA's
// softmax with the other's MMAs.
//
// The kernel is persistent: the grid is one wave (two CTAs per SM); a CTA starts with unit (item, kv head) number
// blockIdx.x of the planner's longest-first list and its producer warp draws further units from a counter in the
// workspace header, publishing them to the MMA and softmax warps through a four-deep ring in shared memory.  The
// producer runs ahead into the next unit while the last tiles of the current one are still being consumed: the stage
// ring - the bytes the SM keeps in flight, which is what bounds this kernel - never drains between units, and tensor
// memory, barriers and tensor maps are set up once per CTA.  For that the epilogue leaves shared memory alone: each
// softmax thread writes its O row from registers to the output (single-chunk sequences) or to the partials; merges
// are claimed by CTAs in their teardown.  Planner and partial / ticket formats are shared with the kernels above.
// ---------------------------------------------------------------------------
constexpr int kUmmaStages = 3;
constexpr int kUmmaTmemCols = 256;
constexpr int kUmmaUnitRing = 4;      // units the producer may be ahead of the slowest consumer
constexpr int kUmmaMaxClaims = 1;     // merges a CTA takes per sweep of the ticket counters in its teardown
constexpr int kMergeClaimed = 1 << 30; // added to a pair's ticket counter by the CTA that merges it

struct __align__(8) UmmaCtrl {
  uint64_t full[kUmmaStages];
  uint64_t empty[kUmmaStages];
  uint64_t q_ready;   // softmax warps -> MMA warp: the unit's Q rows are in tensor memory
  uint64_t s_full;    // MMA warp -> softmax warps (commit): S of a tile
  uint64_t p_ready;   // softmax warps -> MMA warp: P of a tile
  uint64_t o_done;    // MMA warp -> softmax warps (commit): PV of a tile
  uint64_t o_free;    // softmax warps -> MMA warp: the finished unit's O has been read out of tensor memory
  uint64_t rows_out;  // softmax threads: my partial rows of the unit are written and fenced
  uint64_t unit_full[kUmmaUnitRing];    // producer -> MMA and softmax warps: slot r % ring holds the CTA's r-th unit
  uint64_t unit_empty[kUmmaUnitRing];   // MMA warp + softmax warps -> producer: done with that slot
  int unit_ring[kUmmaUnitRing];         // unit indices (n_units or more: the CTA has no r-th unit)
  int published;                        // units published so far, the end mark included
  uint32_t tmem_base;
  int abort_flag;
  int abort_round;    // first round (unit of this CTA) whose output may be incomplete after a wait ran out
  int ready;          // teardown: (sequence, kv head) pairs whose chunks are all published and that nobody merges yet
  int n_reserved;     // teardown: claim attempts of this sweep
  int n_claimed;      // teardown: pairs this CTA claimed in this sweep
  int claimed[kUmmaMaxClaims];
};

// One (work item, kv head) unit as every role of the CTA reads it from the planner's records.
struct UmmaUnit {
  long long seq_start;
  int b, h, c, n_chunks, item0, len, t_begin, t_end, ntiles;
};

__device__ __forceinline__ UmmaUnit umma_unit(const DecodeParams& p, int u) {
  UmmaUnit w;
  const int item = u / p.kv_heads;
  w.h = u - item * p.kv_heads;
  const int4 rec0 = __ldg(p.item_info + 2 * item);
  const int4 rec1 = __ldg(p.item_info + 2 * item + 1);
  w.b = rec0.x; w.c = rec0.y; w.n_chunks = rec0.z; w.item0 = rec0.w;
  w.len = rec1.x;
  w.seq_start = (static_cast<long long>(rec1.w) << 32) | static_cast<unsigned int>(rec1.z);
  w.t_begin = w.c * rec1.y;                       // rec1.y: keys per item of this sequence
  w.t_end = min(w.len, w.t_begin + rec1.y);
  w.ntiles = w.t_end > w.t_begin ? (w.t_end - w.t_begin + kTileN - 1) / kTileN : 0;
  return w;
}

// T: element type of q, k, v as the kernel reads them; OutT: element type of the output rows (T, or float when the
// inputs are fp16 copies of fp32 tensors).
template <typename T, int D, typename OutT = T>
__global__ void __launch_bounds__(192, 2) decode_umma_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                             const __grid_constant__ CUtensorMap tm_v,
                                                             const DecodeParams p) {
  using namespace ptx;
  extern __shared__ unsigned char smem_raw[];
  constexpr int CHUNKS = D / 64;
  constexpr int CHUNK_BYTES = kTileN * 128;
  constexpr int TILE_BYTES = CHUNKS * CHUNK_BYTES;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int kQCols = D / 2;               // TMEM columns of the packed 16-bit Q tile
  constexpr int kSCol = kQCols;               // S (64 fp32 columns); P overwrites its first 32
  constexpr int kOCol = kQCols + kTileN;      // O (D fp32 columns)
  static_assert(kOCol + D <= kUmmaTmemCols, "TMEM budget");
  constexpr int kProducer = 4, kMma = 5;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.rows;
  const int active_warps = (R + 31) >> 5;      // softmax warps that own real rows
  const int n_softmax = active_warps * 32;

  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  UmmaCtrl* ctrl = reinterpret_cast<UmmaCtrl*>(smem + kUmmaStages * STAGE_BYTES);
  const uint32_t smem_base = smem_u32(smem);

  if (tid == 0) {
    for (int i = 0; i < kUmmaStages; ++i) { mbar_init(smem_u32(&ctrl->full[i]), 1); mbar_init(smem_u32(&ctrl->empty[i]), 1); }
    mbar_init(smem_u32(&ctrl->q_ready), n_softmax);
    mbar_init(smem_u32(&ctrl->s_full), 1);
    mbar_init(smem_u32(&ctrl->p_ready), n_softmax);
    mbar_init(smem_u32(&ctrl->o_done), 1);
    mbar_init(smem_u32(&ctrl->o_free), n_softmax);
    mbar_init(smem_u32(&ctrl->rows_out), n_softmax);
    for (int i = 0; i < kUmmaUnitRing; ++i) {
      mbar_init(smem_u32(&ctrl->unit_full[i]), 1);
      mbar_init(smem_u32(&ctrl->unit_empty[i]), 1 + active_warps);
    }
    ctrl->published = 0;
    ctrl->abort_flag = 0;
    ctrl->abort_round = 0x7fffffff;
    mbar_fence_init();
  }
  if (warp == kMma) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kUmmaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort_flag;

  ptx::grid_dep_wait();      // the planner's records are complete and visible from here on
  const int n_units = p.header[2] * p.kv_heads;
  const int G = static_cast<int>(gridDim.x), me = static_cast<int>(blockIdx.x);
  // Units are handed out dynamically, longest first: a CTA's first unit is its own index, later ones are drawn from a
  // counter in the workspace header by the producer warp, which publishes them to the other warps through a small
  // ring in shared memory (a static deal cannot follow a batch of a few long and many short sequences: the CTAs that
  // were dealt one more long unit finish last).  unit_at(r): the CTA's r-th unit, n_units or more when there is
  // none, -1 when the (bounded) wait for the producer ran out.
  auto unit_at = [&](int r) -> int {
    if (!warp_wait(smem_u32(&ctrl->unit_full[r % kUmmaUnitRing]), (r / kUmmaUnitRing) & 1)) return -1;
    return *reinterpret_cast<volatile int*>(&ctrl->unit_ring[r % kUmmaUnitRing]);
  };
  auto unit_done = [&](int r) {   // this warp will not read slot r again
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctrl->unit_empty[r % kUmmaUnitRing]));
  };

  if (warp == kProducer) {
    // =========================== TMA producer ===========================
    if (lane == 0) { prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v); }
    bool ok = true;
    int g = 0;                                   // tiles issued so far, over all units
    const int box_rows = 1 << p.box_shift;
    // block-table entries are read one tile ahead, across units too (see PageAhead)
    PageAhead ahead(p, 0, lane);
    int kp_next = kNoPage, vp_next = kNoPage;
    int ahead_g = -1;                            // running tile index the entries in kp_next / vp_next belong to
    auto publish = [&](int r, int u) {            // lane 0
      ctrl->unit_ring[r % kUmmaUnitRing] = u;
      ctrl->published = r + 1;
      mbar_arrive(smem_u32(&ctrl->unit_full[r % kUmmaUnitRing]));
    };
    int u = me < n_units ? me : n_units;
    if (lane == 0) publish(0, u);
    for (int r = 0; ok && u < n_units; ++r) {
      const UmmaUnit w = umma_unit(p, u);
      ahead.retarget(p, w.b);
      int h_coord = w.h;
      long long row0 = w.seq_start;
      if (p.layout == B200ATTN_DENSE) { h_coord = 0; row0 = (static_cast<long long>(w.b) * p.kv_heads + w.h) * p.max_kv; }
      for (int tile = 0; tile < w.ntiles; ++tile) {
        const int stage = g % kUmmaStages, use = g / kUmmaStages;
        if (use > 0) {
          ok = warp_wait(smem_u32(&ctrl->empty[stage]), (use - 1) & 1);
          if (!ok || *abort_flag) { ok = false; break; }
        }
        const int t0 = w.t_begin + tile * kTileN;
        const uint32_t kdst = smem_base + stage * STAGE_BYTES;
        const uint32_t vdst = kdst + TILE_BYTES;
        const uint32_t bar = smem_u32(&ctrl->full[stage]);
        if (p.layout != B200ATTN_PAGED) {
          if (lane == 0) {
            mbar_arrive_expect_tx(bar, STAGE_BYTES);
            const int row = static_cast<int>(row0 + t0);
#pragma unroll
            for (int cc = 0; cc < CHUNKS; ++cc) {
              tma_load_3d(kdst + cc * CHUNK_BYTES, &tm_k, bar, cc * 64, h_coord, row);
              tma_load_3d(vdst + cc * CHUNK_BYTES, &tm_v, bar, cc * 64, h_coord, row);
            }
          }
        } else if (ahead.on) {
          if (ahead_g != g) ahead.fetch(t0, w.t_end, kp_next, vp_next);   // first tile of the CTA, or after an empty unit
          const int kr = ahead.row(p, kp_next, t0), vr = ahead.row(p, vp_next, t0);
          int count = (kr >= 0) + (vr >= 0);
          for (int off = 16; off > 0; off >>= 1) count += __shfl_xor_sync(0xffffffffu, count, off);
          if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * box_rows * 128 * CHUNKS);
          __syncwarp();
          const uint32_t roff = static_cast<uint32_t>(lane) * box_rows * 128;
#pragma unroll
          for (int cc = 0; cc < CHUNKS; ++cc) {
            if (kr >= 0) tma_load_3d(kdst + cc * CHUNK_BYTES + roff, &tm_k, bar, cc * 64, h_coord, kr);
            if (vr >= 0) tma_load_3d(vdst + cc * CHUNK_BYTES + roff, &tm_v, bar, cc * 64, h_coord, vr);
          }
          // read ahead: the next tile of this unit (the first tile of the next unit: after the draw below)
          if (tile + 1 < w.ntiles) {
            ahead.fetch(t0 + kTileN, w.t_end, kp_next, vp_next);
            ahead_g = g + 1;
          }
        } else {
          const int boxes = kTileN >> p.box_shift;
          const int* ktab = p.k_table + static_cast<long long>(w.b) * p.table_stride;
          const int* vtab = p.v_table + static_cast<long long>(w.b) * p.table_stride;
          int krow[2], vrow[2];
          int count = 0, n = 0;
          for (int i = lane; i < boxes; i += 32, ++n) {
            const int t = t0 + i * box_rows;
            int kr = -1, vr = -1;
            if (t < w.t_end) {
              int lp, off;
              if (p.page_shift >= 0) { lp = t >> p.page_shift; off = t & (p.page_size - 1); }
              else { lp = t / p.page_size; off = t - lp * p.page_size; }
              const int kp = __ldg(ktab + lp), vp = __ldg(vtab + lp);
              // an entry outside the cache is reported and replaced by page 0: never dereferenced, output stays finite
              const bool kbad = kp < 0 || kp >= p.num_pages, vbad = vp < 0 || vp >= p.num_pages;
              if (kbad || vbad) p.header[0] = DEV_ERR_PAGE_RANGE;
              if (p.num_pages > 0) {
                kr = (kbad ? 0 : kp) * p.page_size + off;
                vr = (vbad ? 0 : vp) * p.page_size + off;
              }
            }
            krow[n] = kr; vrow[n] = vr;
            count += (kr >= 0) + (vr >= 0);
          }
          for (int off = 16; off > 0; off >>= 1) count += __shfl_xor_sync(0xffffffffu, count, off);
          if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * box_rows * 128 * CHUNKS);
          __syncwarp();
          n = 0;
          for (int i = lane; i < boxes; i += 32, ++n) {
            const uint32_t roff = static_cast<uint32_t>(i) * box_rows * 128;
#pragma unroll
            for (int cc = 0; cc < CHUNKS; ++cc) {
              if (krow[n] >= 0) tma_load_3d(kdst + cc * CHUNK_BYTES + roff, &tm_k, bar, cc * 64, h_coord, krow[n]);
              if (vrow[n] >= 0) tma_load_3d(vdst + cc * CHUNK_BYTES + roff, &tm_v, bar, cc * 64, h_coord, vrow[n]);
            }
          }
        }
        ++g;
      }
      if (!ok) break;
      // The unit's last copy is on its way: only now draw the next unit (as late as the ring allows, so that the
      // longest-first list is dealt to whoever runs dry first), publish it, and pull what its first steps need -
      // the block-table entries of its first tile, its Q rows (into L2) - ahead of the warps that will ask for them.
      int u_next = n_units;
      if (r + 1 >= kUmmaUnitRing) {
        ok = warp_wait(smem_u32(&ctrl->unit_empty[(r + 1) % kUmmaUnitRing]), ((r + 1) / kUmmaUnitRing - 1) & 1);
        if (!ok || *abort_flag) { ok = false; break; }
      }
      if (lane == 0) {
        u_next = min(G + atomicAdd(p.header + 4, 1), n_units);
        publish(r + 1, u_next);
      }
      u_next = __shfl_sync(0xffffffffu, u_next, 0);
      if (u_next < n_units) {
        const UmmaUnit w2 = umma_unit(p, u_next);
        if (ahead.on && w2.ntiles > 0) {
          ahead.retarget(p, w2.b);
          ahead.fetch(w2.t_begin, w2.t_end, kp_next, vp_next);
          ahead_g = g;
        }
        const T* q2 = static_cast<const T*>(p.q) +
                      ((static_cast<long long>(w2.b) * p.q_heads + static_cast<long long>(w2.h) * p.head_stride + p.head0) * p.q_len) * D;
        for (int i = lane; i < (R * D * static_cast<int>(sizeof(T))) / 128; i += 32) prefetch_l2(reinterpret_cast<const char*>(q2) + i * 128);
      }
      u = u_next;
    }
    if (!ok) {
      if (lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
      // bounded drain of the copies still in flight before the CTA may exit
      for (int t = max(0, g - kUmmaStages); t < g; ++t)
        mbar_wait(smem_u32(&ctrl->full[t % kUmmaStages]), (t / kUmmaStages) & 1);
    }
  } else if (warp == kMma) {
    // =========================== MMA issuer ===========================
    constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr uint32_t idesc_s = make_idesc_f16(128, kTileN, kFmt, 0);
    constexpr uint32_t idesc_o = make_idesc_f16(128, D, kFmt, 1);
    const uint64_t kdesc = make_smem_desc_sw128(smem_base, 16);
    const uint64_t vdesc = make_smem_desc_sw128(smem_base, CHUNK_BYTES);
    // The warp stays converged while it issues (every lane runs the descriptor arithmetic, one elected lane issues
    // the tensor-core instructions and their commits): a divergent single-lane issuer loses most of its issue slots
    // to busy neighbouring warps.
    const uint32_t lead = elect_one();
    auto issue_s = [&](int gi) {
      const uint64_t kb = kdesc + static_cast<uint64_t>(((gi % kUmmaStages) * STAGE_BYTES) >> 4);
      mma_ts_kmajor_batch<D / 16, (CHUNK_BYTES >> 4)>(tmem + kSCol, tmem, kb, idesc_s, 0u, lead);
      mma_commit_lead(smem_u32(&ctrl->s_full), lead);
    };
    bool ok = true;
    int g = 0;                                   // tiles consumed so far, over all units
    // (the record of the next unit is read while the current one runs: two L2 round trips less at every hand-over)
    for (int r = 0; ok; ++r) {
      const int u = unit_at(r);
      if (u < 0) { ok = false; break; }
      if (u >= n_units) break;
      const UmmaUnit w = umma_unit(p, u);
      ok = warp_wait(smem_u32(&ctrl->q_ready), r & 1);
      if (!ok || *abort_flag) { ok = false; break; }
      if (w.ntiles == 0) {
        // nothing to multiply; keep the o_free phase in step (the softmax warps arrive once per unit)
        if (r > 0) ok = warp_wait(smem_u32(&ctrl->o_free), (r - 1) & 1);
        unit_done(r);
        continue;
      }
      ok = warp_wait(smem_u32(&ctrl->full[g % kUmmaStages]), (g / kUmmaStages) & 1);
      if (!ok) break;
      tc_fence_after();
      issue_s(g);
      for (int tile = 0; tile < w.ntiles && ok; ++tile, ++g) {
        const int stage = g % kUmmaStages;
        // what does not depend on the softmax warps comes before the wait for their P: the next K tile (loaded long
        // ago in steady state), the zero fill of V rows past the end, the operand descriptor
        if (tile + 1 < w.ntiles) {
          ok = warp_wait(smem_u32(&ctrl->full[(g + 1) % kUmmaStages]), ((g + 1) / kUmmaStages) & 1);
          if (!ok) break;
        }
        const int valid = w.len - (w.t_begin + tile * kTileN);
        if (valid < kTileN) {
          // keys past the sequence end carry P == 0 but their V rows may hold anything: zero them so 0 * x stays 0
          // (the stage is complete: its K half was consumed by S(tile))
          unsigned char* vbuf = smem + stage * STAGE_BYTES + TILE_BYTES;
          const int first = valid > 0 ? valid : 0;
          const int n16 = (kTileN - first) * 8;
          for (int cc = 0; cc < CHUNKS; ++cc) {
            uint4* dst = reinterpret_cast<uint4*>(vbuf + cc * CHUNK_BYTES + first * 128);
            for (int i = lane; i < n16; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        const uint64_t vb = vdesc + static_cast<uint64_t>((stage * STAGE_BYTES + TILE_BYTES) >> 4);
        ok = warp_wait(smem_u32(&ctrl->p_ready), g & 1);
        if (!ok) break;
        if (tile == 0 && r > 0) {
          // this PV starts a new accumulator: the previous unit's O must have left tensor memory
          ok = warp_wait(smem_u32(&ctrl->o_free), (r - 1) & 1);
          if (!ok) break;
        }
        tc_fence_after();
        mma_ts_batch4(tmem + kOCol, tmem + kSCol, vb, idesc_o, tile > 0 ? 1u : 0u, lead);
        mma_commit_lead(smem_u32(&ctrl->o_done), lead);
        if (tile + 1 < w.ntiles) issue_s(g + 1);
        // K_tile was read by S(tile) (complete: its P has come back) and V_tile by the PV just issued
        mma_commit_lead(smem_u32(&ctrl->empty[stage]), lead);
      }
      if (ok) unit_done(r);
    }
    if (!ok && lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
  } else if (warp < active_warps) {
    // =========================== softmax warps: thread = q row ===========================
    const int row = tid;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = p.scale_log2;
    const uint32_t tS = tmem + lane_off + kSCol;
    const uint32_t tO = tmem + lane_off + kOCol;
    bool ok = true;
    int g = 0;                                   // tiles consumed so far, over all units
    int merges = 0;                              // units of this CTA that went through the ticket (barrier phases)
    int r = 0;
    auto rows_of = [&](const UmmaUnit& w) {
      return (static_cast<long long>(w.b) * p.q_heads + static_cast<long long>(w.h) * p.head_stride + p.head0) * p.q_len;
    };
    // Q row -> TMEM as the packed 16-bit A operand (rows past R are zero).  Called when the S MMAs of the unit before
    // have all completed (this warp has consumed their last score tile), i.e. before that unit's epilogue, so that
    // the MMA warp can start on the next unit while the rows of the finished one are written out.
    auto write_q = [&](int unit, const UmmaUnit& w) {
      if (unit >= n_units) return;
      const T* qg = static_cast<const T*>(p.q) + rows_of(w) * D;
#pragma unroll
      for (int cc = 0; cc < kQCols / 32; ++cc) {
        uint32_t qv[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 x = make_uint4(0u, 0u, 0u, 0u);
          if (row < R) x = __ldg(reinterpret_cast<const uint4*>(qg + static_cast<long long>(row) * D) + cc * 8 + i);
          qv[i * 4 + 0] = x.x; qv[i * 4 + 1] = x.y; qv[i * 4 + 2] = x.z; qv[i * 4 + 3] = x.w;
        }
        tmem_st32(tmem + lane_off + cc * 32, qv);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&ctrl->q_ready));
    };
    // The ticket of a unit's pair is drawn by thread 0 one unit later (or in the teardown): by then the barrier that
    // says "all rows are written" completed long ago and the fence before the ticket has nothing left to wait for.
    int owed_pair = -1, owed_round = 0;          // thread 0: pair whose ticket is still to be drawn, and its unit's round
    auto draw_owed_ticket = [&]() {
      if (tid != 0 || owed_pair < 0) return;
      if (mbar_wait(smem_u32(&ctrl->rows_out), (merges - 1) & 1)) {
        __threadfence();                         // the rows the other softmax threads wrote before they arrived, too
        atomicAdd(p.counters + owed_pair, 1);
        atomicAdd(p.header + 3, 1);              // tickets drawn and not merged yet (a hint for the teardown)
      } else {
        p.header[0] = DEV_ERR_WAIT_EXPIRED;
        *abort_flag = 1;
      }
      owed_pair = -1;
    };
    int u = unit_at(0);
    if (u < 0) ok = false;
    UmmaUnit w = umma_unit(p, min(max(u, 0), max(n_units - 1, 0)));
    if (ok) write_q(u, w);
    for (; ok; ++r) {
      if (u >= n_units) break;
      const long long row_base = rows_of(w);
      float m_used = -INFINITY, l_run = 0.f;               // per-row softmax state
      int lim = w.len - 1;                                 // last visible key of this row
      if (p.causal) lim = w.len - p.q_len + (row % p.q_len);
      for (int tile = 0; tile < w.ntiles; ++tile, ++g) {
        ok = warp_wait(smem_u32(&ctrl->s_full), g & 1);
        if (!ok || *abort_flag) { ok = false; break; }
        tc_fence_after();
        const int limit = lim - (w.t_begin + tile * kTileN);   // columns 0..limit of this tile are visible
        uint32_t ca[32], cb[32];
        tmem_ld32(tS, ca);
        tmem_ld32(tS + 32, cb);
        tmem_wait_ld();
        if (limit < kTileN - 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i > limit) ca[i] = 0xff800000u;          // -inf
            if (32 + i > limit) cb[i] = 0xff800000u;
          }
        }
        float ma = max3(__uint_as_float(ca[0]), __uint_as_float(ca[1]), __uint_as_float(ca[2]));
        float mb = max3(__uint_as_float(cb[0]), __uint_as_float(cb[1]), __uint_as_float(cb[2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2) {
          ma = max3(ma, __uint_as_float(ca[i]), __uint_as_float(ca[i + 1]));
          mb = max3(mb, __uint_as_float(cb[i]), __uint_as_float(cb[i + 1]));
        }
        const float mx = max3(ma, mb, fmaxf(__uint_as_float(ca[31]), __uint_as_float(cb[31]))) * sl2;
        const bool need = (mx - m_used) > 8.f;
        float alpha = 1.f;
        if (need) { alpha = fast_exp2(m_used - mx); m_used = mx; l_run *= alpha; }
        if (tile > 0 && __any_sync(0xffffffffu, need)) {
          // PV(tile-1) has completed once S(tile) is visible (MMAs complete in issue order); the wait is immediate
          ok = warp_wait(smem_u32(&ctrl->o_done), (g - 1) & 1);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t ov[32];
            tmem_ld32(tO + cc * 32, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tO + cc * 32, ov);
          }
        }
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        float rs = 0.f;
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(ca[2 * i]), sl2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(ca[2 * i + 1]), sl2, neg_m));
          const float p2 = fast_exp2(fmaf(__uint_as_float(cb[2 * i]), sl2, neg_m));
          const float p3 = fast_exp2(fmaf(__uint_as_float(cb[2 * i + 1]), sl2, neg_m));
          rs += (p0 + p1) + (p2 + p3);
          pk[i] = ElemTraits<T>::pack2(p0, p1);
          pk[16 + i] = ElemTraits<T>::pack2(p2, p3);
        }
        l_run += rs;
        tmem_st32(tS, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->p_ready));
      }
      if (!ok) break;
      // the next unit (published by the producer when it issued this unit's last copy, its Q rows already on their
      // way into L2): its Q goes to tensor memory before this unit's rows are written out
      const int u_next = unit_at(r + 1);
      if (u_next < 0) { ok = false; break; }
      const UmmaUnit w_next = u_next < n_units ? umma_unit(p, u_next) : w;
      write_q(u_next, w_next);
      // ---------------- the unit's rows leave tensor memory ----------------
      if (w.ntiles > 0) {
        ok = warp_wait(smem_u32(&ctrl->o_done), (g - 1) & 1);
        if (!ok) break;
        tc_fence_after();
      }
      const bool single = w.n_chunks == 1;
      const long long slot = (static_cast<long long>(w.item0) + w.c) * p.kv_heads + w.h;
      OutT* out = static_cast<OutT*>(p.out) + row_base * D;
      const float inv = single ? (l_run > 0.f ? 1.f / l_run : 0.f) : 1.f;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t ov[32];
        if (w.ntiles > 0) {
          tmem_ld32(tO + cc * 32, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (cc == D / 32 - 1) {
          // O is in registers: the MMA warp may start the next unit's accumulator
          tc_fence_before();
          mbar_arrive(smem_u32(&ctrl->o_free));
        }
        if (row < R) {
          if (single) {
            if constexpr (sizeof(OutT) == 2) {
              uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * D + cc * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 x;
                x.x = ElemTraits<OutT>::pack2(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
                x.y = ElemTraits<OutT>::pack2(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
                x.z = ElemTraits<OutT>::pack2(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
                x.w = ElemTraits<OutT>::pack2(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
                dst[i] = x;
              }
            } else {
              float4* dst = reinterpret_cast<float4*>(out + static_cast<long long>(row) * D + cc * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                dst[i] = make_float4(__uint_as_float(ov[4 * i]) * inv, __uint_as_float(ov[4 * i + 1]) * inv,
                                     __uint_as_float(ov[4 * i + 2]) * inv, __uint_as_float(ov[4 * i + 3]) * inv);
            }
          } else {
            float4* dst = reinterpret_cast<float4*>(p.part_o + (slot * R + row) * D + cc * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(ov[4 * i]), __uint_as_float(ov[4 * i + 1]),
                                   __uint_as_float(ov[4 * i + 2]), __uint_as_float(ov[4 * i + 3]));
          }
        }
      }
      if (!single) {
        if (row < R) {
          p.part_ml[(slot * R + row) * 2] = m_used;
          p.part_ml[(slot * R + row) * 2 + 1] = l_run;
        }
        // Publish the partial.  Nobody merges here: the merge is left to the teardown of whichever CTA gets to it first
        // (see there), so the softmax warps go straight on to their next unit.  The softmax threads meet on an
        // mbarrier with a bounded wait, never on bar.sync: a warp that gave up must not hang the rest.
        draw_owed_ticket();
        mbar_arrive(smem_u32(&ctrl->rows_out));
        owed_pair = w.b * p.kv_heads + w.h;
        owed_round = r;
        ++merges;
      }
      unit_done(r);
      w = w_next;
      u = u_next;
    }
    if (ok) draw_owed_ticket();
    if (!ok) {
      // (a unit whose ticket was still owed counts as unfinished: its pair will never be merged)
      atomicMin(&ctrl->abort_round, (tid == 0 && owed_pair >= 0) ? owed_round : r);
      if (lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
    }
  }
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMma) { tc_fence_after(); tmem_dealloc(tmem, kUmmaTmemCols); }
  // Merges.  A (sequence, kv head) pair whose chunks have all drawn their tickets is merged by whichever CTA claims
  // it while sweeping the ticket counters here, with all of its threads: CTAs that finish early take the pairs that
  // are complete, the CTA that draws a pair's last ticket sweeps after it did, so every pair is merged by the time
  // the last CTA leaves, and no CTA waits for another.  A CTA takes one pair per sweep and sweeps again as long as it
  // saw a complete pair; header[3] (tickets drawn and not merged) lets a CTA skip the sweep when there is nothing.
  if (!ctrl->abort_flag) {
    const int n_pairs = p.batch * p.kv_heads;
    for (int sweep = 0; sweep < n_pairs + 64; ++sweep) {
      if (tid == 0) {
        ctrl->ready = *reinterpret_cast<volatile int*>(p.header + 3);
        ctrl->n_reserved = 0;
        ctrl->n_claimed = 0;
      }
      __syncthreads();
      if (ctrl->ready <= 0) break;
      for (int e = tid; e < n_pairs; e += static_cast<int>(blockDim.x)) {
        const int pair = (e + me * 61) % n_pairs;            // CTAs start their sweeps at different pairs
        const int b = pair / p.kv_heads;
        const int n = p.item_start[b + 1] - p.item_start[b];
        if (n > 1 && *reinterpret_cast<volatile int*>(p.counters + pair) == n &&
            atomicAdd(&ctrl->n_reserved, 1) < kUmmaMaxClaims &&
            atomicCAS(p.counters + pair, n, n + kMergeClaimed) == n) {
          atomicSub(p.header + 3, n);
          ctrl->claimed[atomicAdd(&ctrl->n_claimed, 1)] = pair;
        }
      }
      __syncthreads();
      if (ctrl->n_reserved == 0) break;                      // no complete pair in sight: whoever completes one sweeps
      const int n_claimed = ctrl->n_claimed;
      for (int i = 0; i < n_claimed; ++i) {
        const int pair = ctrl->claimed[i];
        const int b = pair / p.kv_heads, h = pair - b * p.kv_heads;
        const int item0 = p.item_start[b];
        OutT* out = static_cast<OutT*>(p.out) +
                    ((static_cast<long long>(b) * p.q_heads + static_cast<long long>(h) * p.head_stride + p.head0) * p.q_len) * D;
        merge_chunks<OutT, D>(p, b, h, p.item_start[b + 1] - item0, item0, out, tid, static_cast<int>(blockDim.x));
      }
      __syncthreads();
    }
  }
  if (ctrl->abort_flag) {
    // A bounded wait ran out: the rows of the unit the softmax warps were in, and of the units this CTA had not
    // reached, are unknown.  They are filled with NaN (and their tickets are not drawn, so nobody merges over them):
    // the failure shows in the output as well as in the error word.
    const OutT nan_t = ElemTraits<OutT>::from_float(__int_as_float(0x7fc00000));
    // (the slots of units the softmax warps have not finished cannot have been reused by the producer)
    for (int r = ctrl->abort_round; r < ctrl->published; ++r) {
      const int u = ctrl->unit_ring[r % kUmmaUnitRing];
      if (u >= n_units) break;
      const UmmaUnit w = umma_unit(p, u);
      OutT* out = static_cast<OutT*>(p.out) +
                  ((static_cast<long long>(w.b) * p.q_heads + static_cast<long long>(w.h) * p.head_stride + p.head0) * p.q_len) * D;
      for (int i = tid; i < R * D; i += blockDim.x) out[i] = nan_t;
    }
  }
}

// ---------------------------------------------------------------------------
// fp32 kernel: fp32 FMA dot products, one warp per q row, lanes split head_dim
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) decode_simt_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ticket;
  constexpr int VEC = D / 32;  // floats per lane
  ptx::grid_dep_wait();      // the planner's records are complete and visible from here on
  const int n_items = p.header[2];
  // heads vary fastest across CTAs: the CTAs that run side by side walk the same pages and read
  // neighbouring head slices of each token row, which keeps DRAM rows open
  const int item = blockIdx.x / p.kv_heads;
  if (item >= n_items) return;
  const int h = blockIdx.x - item * p.kv_heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int R = p.rows;

  const int b = find_sequence(p.item_start, p.batch, item);
  const int item0 = p.item_start[b];
  const int c = item - item0;
  const int n_chunks = p.item_start[b + 1] - item0;
  const SeqInfo si = seq_info(p, b);
  const int len = si.len;
  const int chunk = seq_chunk(len, n_chunks, p.header[1], p.equal_split);
  const int t_begin = c * chunk;
  const int t_end = min(len, t_begin + chunk);

  float* comb_o = reinterpret_cast<float*>(smem);                            // [KS][R][D], KS * R <= max(R, warps)
  float* comb_ml = comb_o + static_cast<size_t>(max(R, nwarps)) * D;         // [KS][R][2]
  const float* kg = static_cast<const float*>(p.k);
  const float* vg = static_cast<const float*>(p.v);
  const float* qg = static_cast<const float*>(p.q) +
                    ((static_cast<long long>(b) * p.q_heads + static_cast<long long>(h) * p.head_stride + p.head0) * p.q_len) * D;
  const float sl2 = p.scale_log2;

  // A warp owns one q row (lanes split head_dim) and takes four keys per step: four independent dot products and
  // shuffle reductions in flight, one online-softmax update for the four.  With fewer rows than warps (plain decode
  // with a small GQA group) the warps of a row split its keys in groups of four and leave one partial each, which
  // emit_and_merge combines like the key slices of the tensor-core kernel.
  constexpr int TB = 4;
  const int KS = (R <= nwarps && nwarps % R == 0) ? nwarps / R : 1;
  for (int rr = warp; rr < R * KS; rr += nwarps) {
    const int r = rr % R, ks = rr / R;
    float qv[VEC], acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) { qv[i] = qg[static_cast<long long>(r) * D + lane * VEC + i]; acc[i] = 0.f; }
    const int lim = p.causal ? (len - p.q_len + (r % p.q_len)) : (len - 1);
    const int stop = min(t_end, lim + 1);
    float m = -INFINITY, l = 0.f;
    for (int t = t_begin + ks * TB; t < stop; t += KS * TB) {
      float dot[TB], vv[TB][VEC];
#pragma unroll
      for (int j = 0; j < TB; ++j) {
        dot[j] = -INFINITY;                       // a key past the end, or on a page outside the cache, weighs nothing
#pragma unroll
        for (int i = 0; i < VEC; ++i) vv[j][i] = 0.f;
        if (t + j >= stop) continue;
        const long long ko = row_offset(p, p.k_table, b, h, si.start, t + j, D);
        const long long vo = (p.layout == B200ATTN_PAGED) ? row_offset(p, p.v_table, b, h, si.start, t + j, D) : ko;
        if (ko < 0 || vo < 0) {
          if (lane == 0) p.header[0] = DEV_ERR_PAGE_RANGE;
          continue;
        }
        float kv[VEC];
        if constexpr (VEC == 4) {
          const float4 k4 = __ldg(reinterpret_cast<const float4*>(kg + ko) + lane);
          const float4 v4 = __ldg(reinterpret_cast<const float4*>(vg + vo) + lane);
          kv[0] = k4.x; kv[1] = k4.y; kv[2] = k4.z; kv[3] = k4.w;
          vv[j][0] = v4.x; vv[j][1] = v4.y; vv[j][2] = v4.z; vv[j][3] = v4.w;
        } else {
          const float2 k2 = __ldg(reinterpret_cast<const float2*>(kg + ko) + lane);
          const float2 v2 = __ldg(reinterpret_cast<const float2*>(vg + vo) + lane);
          kv[0] = k2.x; kv[1] = k2.y;
          vv[j][0] = v2.x; vv[j][1] = v2.y;
        }
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) d = fmaf(qv[i], kv[i], d);
        dot[j] = d;
      }
      // (-inf + -inf stays -inf through the reduction: every lane of the warp took the same branch for key j)
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int j = 0; j < TB; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], off);
      }
      float mn = m;
#pragma unroll
      for (int j = 0; j < TB; ++j) { dot[j] *= sl2; mn = fmaxf(mn, dot[j]); }
      if (mn == -INFINITY) continue;              // nothing visible yet
      const float a = fast_exp2(m - mn);          // m == -inf: exp2(-inf) = 0
      l *= a;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] *= a;
#pragma unroll
      for (int j = 0; j < TB; ++j) {
        const float pw = fast_exp2(dot[j] - mn);
        l += pw;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(pw, vv[j][i], acc[i]);
      }
      m = mn;
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) comb_o[(static_cast<size_t>(ks) * R + r) * D + lane * VEC + i] = acc[i];
    if (lane == 0) { comb_ml[(ks * R + r) * 2] = m; comb_ml[(ks * R + r) * 2 + 1] = l; }
  }
  __syncthreads();
  emit_and_merge<float, D>(p, b, h, c, n_chunks, item0, comb_o, comb_ml, KS, R, &s_ticket);
}

// Launches `kernel` so that it may be scheduled while the planner before it in the stream is still running; the
// kernel itself waits (grid_dep_wait) before it reads what the planner wrote.
template <typename... Params, typename... Args>
cudaError_t launch_after_planner(void (*kernel)(Params...), dim3 grid, int threads, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

}  // namespace

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// q heads of one KV head that one launch serves.  A CTA holds at most 128 q rows (group x draft tokens) per KV head;
// a larger group is cut into the largest equal sub-groups that fit, one launch each over the same K/V (the reference
// takes any head ratio: kernels/speculative_decode.py:262-299).
int decode_pass_group(int group, int q_len) {
  if (q_len < 1) q_len = 1;
  int g = group;
  while (g > 1 && (g * q_len > 128 || group % g != 0)) --g;
  return g < 1 ? 1 : g;
}

DecodeWsLayout decode_ws_layout(const b200attn_decode_args_t& a, int sm_count, bool allow_cast) {
  DecodeWsLayout w;
  const int group = decode_pass_group(a.kv_heads > 0 ? a.q_heads / a.kv_heads : 1, a.q_len);
  const int rows = group * a.q_len;
  // fp32 inputs of a speculative-decode call (more than one q row per head, or more than 16 rows per KV head) are
  // rounded to fp16 in the workspace and run on the tensor-core kernels with fp32 accumulation and fp32 output: the
  // reference multiplies them with tl.dot on fp32 operands, i.e. in TF32, which keeps the same ten mantissa bits
  // (kernels/speculative_decode.py:153,175); one fp32 FMA warp per q row re-reads K/V once per row and is one to two
  // orders of magnitude slower there.  Plain decode (one q row per head), which the reference computes in fp32 FMAs
  // (kernels/decode.py:146-160), stays on the fp32 kernel.
  // (not when the copies would be huge - a paged cache is copied whole - : beyond kCastLimitBytes the call stays on
  // the fp32 kernel rather than ask the caller for that much scratch)
  constexpr size_t kCastLimitBytes = size_t(8) << 30;
  const size_t kv_rows_all = a.layout == B200ATTN_DENSE ? static_cast<size_t>(a.batch) * a.kv_heads * a.max_kv
                                                        : static_cast<size_t>(a.total_kv > 0 ? a.total_kv : 0) * a.kv_heads;
  const bool cast16 = allow_cast && a.dtype == B200ATTN_F32 && (rows > 16 || a.q_len > 1) &&
                      kv_rows_all * a.head_dim * 4 <= kCastLimitBytes;
  const bool f32_kernel = a.dtype == B200ATTN_F32 && !cast16;
  // Six (item, kv head) CTAs per SM: two or three waves of the tensor-core kernels (3 or 2 resident CTAs per SM).
  // Fewer, longer CTAs amortise start-up and merge; the planner keeps the item count at or below this, so the grid
  // is a whole number of waves.  (Measured on B200, paged decode and speculative decode: 4 / 6 / 8 / 12 / 16 per SM
  // give 0.84 / 0.83 / 0.81 / 0.80 / 0.78 and 0.71 / 0.70 / 0.73 / 0.67 / 0.64 of the copy bandwidth without the
  // whole-wave rule, 0.76 for speculative decode with it.)  The fp32 kernel keeps eight.
  const int per_sm = f32_kernel ? 8 : 6;
  long long target = (static_cast<long long>(sm_count) * per_sm) / std::max(1, a.kv_heads);
  if (target < 1) target = 1;
  w.target_items = static_cast<int>(target);
  // one wave of the tensor-core kernels: 2 (tcgen05 kernel, more than 16 rows) or 3 resident CTAs per SM; their
  // per-item start-up + merge cost in keys of streaming time (from the sweeps quoted in the planner)
  w.wave_items = 0;
  w.item_overhead = 0;
  if (!f32_kernel) {
    const bool wide = rows > 16;
    w.wave_items = static_cast<int>(std::max<long long>(1, (static_cast<long long>(sm_count) * (wide ? 2 : 3)) / std::max(1, a.kv_heads)));
    w.item_overhead = wide ? 448 : 128;
  }
  // keep the partial write (rows x D fp32) small next to the chunk's K/V bytes
  int min_chunk = 128;
  const int by_rows = ((rows * 8 + kTileN - 1) / kTileN) * kTileN;
  if (by_rows > min_chunk) min_chunk = by_rows;
  w.min_chunk = min_chunk;
  w.max_items = w.target_items + a.batch;
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  size_t off = kHeaderBytes;
  w.item_start_off = off; off = up(off + sizeof(int) * (static_cast<size_t>(a.batch) + 1));
  w.counters_off = off;   off = up(off + sizeof(int) * static_cast<size_t>(a.batch) * a.kv_heads);
  w.info_off = off;       off = up(off + 32 * static_cast<size_t>(w.max_items));
  const size_t slots = static_cast<size_t>(w.max_items) * a.kv_heads;
  w.ml_off = off;         off = up(off + sizeof(float) * slots * rows * 2);
  w.o_off = off;          off = up(off + sizeof(float) * slots * rows * a.head_dim);
  w.cast_q_off = w.cast_k_off = w.cast_v_off = 0;
  w.cast_q_elems = w.cast_kv_elems = 0;
  if (cast16) {
    w.cast_q_elems = static_cast<size_t>(a.batch) * a.q_heads * a.q_len * a.head_dim;
    const size_t kv_rows = a.layout == B200ATTN_DENSE ? static_cast<size_t>(a.batch) * a.kv_heads * a.max_kv
                                                      : static_cast<size_t>(a.total_kv) * a.kv_heads;
    w.cast_kv_elems = kv_rows * a.head_dim;
    w.cast_q_off = off; off = up(off + 2 * w.cast_q_elems);
    w.cast_k_off = off; off = up(off + 2 * w.cast_kv_elems);
    w.cast_v_off = off; off = up(off + 2 * w.cast_kv_elems);
  }
  w.total = off;
  return w;
}

namespace {
int launch_decode_pass(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream, const DecodeWsLayout& w,
                       int pass_group, int head0, bool f32_out);

// fp32 -> fp16, four elements per thread (every tensor here is a whole number of head_dim rows)
__global__ void __launch_bounds__(256) decode_cast_f16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst,
                                                              size_t n4) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 x = __ldg(src + i);
    dst[i] = make_uint2(ElemTraits<__half>::pack2(x.x, x.y), ElemTraits<__half>::pack2(x.z, x.w));
  }
}
}  // namespace

int launch_decode(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream, bool allow_cast) {
  const DecodeWsLayout w = decode_ws_layout(a, sm_count, allow_cast);
  if (a.workspace == nullptr || a.workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(a.workspace) & 255)) {
    set_error("decode: workspace needs %zu bytes, 256-byte aligned (got %zu)", w.total, a.workspace_bytes);
    return B200ATTN_E_WORKSPACE;
  }
  const int group = a.q_heads / a.kv_heads;
  const int pass_group = decode_pass_group(group, a.q_len);
  b200attn_decode_args_t b = a;
  if (w.cast_kv_elems > 0) {
    // fp16 copies of q, k, v (see decode_ws_layout); the launches below read them and write fp32 rows
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    const void* src[3] = {a.q, a.k, a.v};
    void* dst[3] = {ws + w.cast_q_off, ws + w.cast_k_off, ws + w.cast_v_off};
    const size_t elems[3] = {w.cast_q_elems, w.cast_kv_elems, w.cast_kv_elems};
    for (int i = 0; i < 3; ++i) {
      const size_t n4 = elems[i] / 4;
      if (n4 == 0) continue;
      const unsigned blocks = static_cast<unsigned>(std::min<size_t>((n4 + 255) / 256, static_cast<size_t>(sm_count) * 16));
      decode_cast_f16_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float4*>(src[i]), static_cast<uint2*>(dst[i]), n4);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "decode_cast_f16_kernel launch");
    }
    b.q = dst[0]; b.k = dst[1]; b.v = dst[2];
    b.dtype = B200ATTN_F16;
  }
  // one launch per sub-group of q heads; they run back to back on the stream and share the workspace
  for (int head0 = 0; head0 < group; head0 += pass_group) {
    const int rc = launch_decode_pass(b, sm_count, stream, w, pass_group, head0, w.cast_kv_elems > 0);
    if (rc) return rc;
  }
  return B200ATTN_OK;
}

namespace {
// `f32_out`: the inputs are the fp16 copies of fp32 tensors and the output rows are fp32
int launch_decode_pass(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream, const DecodeWsLayout& w,
                       int pass_group, int head0, bool f32_out) {
  DecodeParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out;
  p.kv_indptr = a.kv_indptr; p.k_table = a.k_table; p.v_table = a.v_table;
  unsigned char* ws = static_cast<unsigned char*>(a.workspace);
  p.header = reinterpret_cast<int*>(ws);
  p.item_start = reinterpret_cast<int*>(ws + w.item_start_off);
  p.counters = reinterpret_cast<int*>(ws + w.counters_off);
  p.item_info = reinterpret_cast<int4*>(ws + w.info_off);
  p.part_ml = reinterpret_cast<float*>(ws + w.ml_off);
  p.part_o = reinterpret_cast<float*>(ws + w.o_off);
  p.total_kv = a.total_kv; p.table_stride = a.table_stride;
  p.layout = a.layout; p.indptr_is_i64 = a.indptr_is_i64;
  p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads;
  p.head_stride = a.q_heads / a.kv_heads; p.head0 = head0;
  p.group = pass_group; p.q_len = a.q_len; p.rows = p.group * a.q_len;
  p.n_mtiles = (p.rows + 15) / 16;
  p.max_kv = a.max_kv; p.page_size = a.layout == B200ATTN_PAGED ? a.page_size : 1;
  p.page_shift = -1;
  if (p.page_size > 0 && (p.page_size & (p.page_size - 1)) == 0) {
    int s = 0; while ((1 << s) < p.page_size) ++s;
    p.page_shift = s;
  }
  p.num_pages = a.layout == B200ATTN_PAGED ? static_cast<int>(std::min<long long>(a.total_kv / p.page_size, 0x7fffffff)) : 0;
  p.causal = a.causal_drafts ? 1 : 0;
  p.box_shift = 6;
  p.target_items = w.target_items; p.min_chunk = w.min_chunk; p.max_items = w.max_items;
  p.wave_items = w.wave_items; p.item_overhead = w.item_overhead;
  // Equal items per sequence and longest-first order let the greedy CTA dispatch pair long and short items: with two
  // or three whole waves the grid drains almost level (measured on B200, 16-token pages: 0.80 -> 0.84 of the copy
  // bandwidth for paged decode, 0.68 -> 0.76 for speculative decode).
  p.equal_split = a.dtype != B200ATTN_F32 ? 1 : 0;
  p.scale_log2 = a.sm_scale * 1.4426950408889634f;

  decode_plan_kernel<<<1, kPlanThreads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "decode_plan_kernel launch");

  const dim3 grid(static_cast<unsigned>(w.max_items) * a.kv_heads, 1);
  const int D = a.head_dim;
  if (a.dtype == B200ATTN_F32) {
    const size_t smem = sizeof(float) * static_cast<size_t>(std::max(p.rows, 4)) * (D + 2);   // 4 warps: see the kernel
    int rc = 0;
    if (D == 128) { rc = set_smem(decode_simt_kernel<128>, smem); if (rc) return rc; launch_after_planner(decode_simt_kernel<128>, grid, 128, smem, stream, p); }
    else          { rc = set_smem(decode_simt_kernel<64>, smem);  if (rc) return rc; launch_after_planner(decode_simt_kernel<64>, grid, 128, smem, stream, p); }
  } else if (p.rows > 16) {
    // many q rows per KV head: one 128-row tcgen05 tile with Q and P in tensor memory
    CUtensorMap tk, tv;
    int rc = 0;
    int box = kTileN;
    if (a.layout == B200ATTN_PAGED) {
      box = 1;
      while (box < kTileN && (a.page_size % (box * 2)) == 0) box *= 2;
    }
    p.box_shift = 0;
    while ((1 << p.box_shift) < box) ++p.box_shift;
    long long tokens;
    int heads;
    if (a.layout == B200ATTN_DENSE) { tokens = static_cast<long long>(a.batch) * a.kv_heads * a.max_kv; heads = 1; }
    else { tokens = a.total_kv; heads = a.kv_heads; }
    if ((rc = make_token_map(&tk, a.dtype, a.k, tokens, heads, D, box))) return rc;
    if ((rc = make_token_map(&tv, a.dtype, a.v, tokens, heads, D, box))) return rc;
    const size_t stage_bytes = static_cast<size_t>(kUmmaStages) * 2 * kTileN * D * 2;
    const size_t smem = 1024 + stage_bytes + sizeof(UmmaCtrl);
    // persistent: one wave of two CTAs per SM walks the unit list (fewer CTAs when the list cannot be longer)
    const unsigned wave = 2u * static_cast<unsigned>(sm_count);
    const dim3 grid(std::min(static_cast<unsigned>(w.max_items) * a.kv_heads, wave), 1);
#define B200ATTN_LAUNCH_UMMA(TYPE, DIM, OUT)                             \
    do {                                                                 \
      rc = set_smem(decode_umma_kernel<TYPE, DIM, OUT>, smem);           \
      if (rc) return rc;                                                 \
      launch_after_planner(decode_umma_kernel<TYPE, DIM, OUT>, grid, 192, smem, stream, tk, tv, p); \
    } while (0)
    if (f32_out) {
      if (D == 128) B200ATTN_LAUNCH_UMMA(__half, 128, float); else B200ATTN_LAUNCH_UMMA(__half, 64, float);
    } else if (a.dtype == B200ATTN_BF16) {
      if (D == 128) B200ATTN_LAUNCH_UMMA(__nv_bfloat16, 128, __nv_bfloat16); else B200ATTN_LAUNCH_UMMA(__nv_bfloat16, 64, __nv_bfloat16);
    } else {
      if (D == 128) B200ATTN_LAUNCH_UMMA(__half, 128, __half); else B200ATTN_LAUNCH_UMMA(__half, 64, __half);
    }
#undef B200ATTN_LAUNCH_UMMA
  } else {
    // at most 16 q rows per KV head reach this kernel (more go to the tcgen05 kernel above): one 16-row tile, four
    // consumer warps that split every K/V tile by key slice, and the producer warp
    const int nmt = p.n_mtiles;
    if (nmt != 1) { set_error("decode: %d row tiles per KV head in the warp-level kernel", nmt); return B200ATTN_E_UNSUPPORTED; }
    const int ksl = 4;
    const int threads = 32 * (nmt * ksl + 1);
    // measured on B200 (paged decode, 32/8 heads): 2 stages with Q re-read from shared memory lets three CTAs share an
    // SM and hides each CTA's start-up and merge behind its neighbours
    const int stages = 2;
    const size_t stage_bytes = static_cast<size_t>(stages) * 2 * kTileN * D * 2;
    const size_t comb_bytes = sizeof(float) * static_cast<size_t>(ksl) * nmt * 16 * (D + 2);
    const size_t smem = 1024 + std::max(stage_bytes, comb_bytes) + static_cast<size_t>(nmt) * 16 * D * 2 + sizeof(DecodeCtrl);
    // tensor maps over K and V: (D, heads, tokens), one box = 64 elements x 1 head x box_rows keys
    CUtensorMap tk, tv;
    int rc = 0;
    int box = kTileN;
    if (a.layout == B200ATTN_PAGED) {
      box = 1;
      while (box < kTileN && (a.page_size % (box * 2)) == 0) box *= 2;
    }
    p.box_shift = 0;
    while ((1 << p.box_shift) < box) ++p.box_shift;
    if (a.layout == B200ATTN_DENSE) {
      const long long rows = static_cast<long long>(a.batch) * a.kv_heads * a.max_kv;
      if ((rc = make_kv_rows_map(&tk, a.dtype, a.k, rows, 1, D, box, D * 2ll, D * 2ll))) return rc;
      if ((rc = make_kv_rows_map(&tv, a.dtype, a.v, rows, 1, D, box, D * 2ll, D * 2ll))) return rc;
    } else {
      const long long rstride = static_cast<long long>(a.kv_heads) * D * 2;
      if ((rc = make_kv_rows_map(&tk, a.dtype, a.k, a.total_kv, a.kv_heads, D, box, rstride, D * 2ll))) return rc;
      if ((rc = make_kv_rows_map(&tv, a.dtype, a.v, a.total_kv, a.kv_heads, D, box, rstride, D * 2ll))) return rc;
    }
#define B200ATTN_LAUNCH_DECODE_V(TYPE, DIM, STAGES, NBLK, MAXT, MINB, OUT)                               \
    do {                                                                                                  \
      rc = set_smem(decode_mma_kernel<TYPE, DIM, STAGES, NBLK, MAXT, MINB, OUT>, smem);                  \
      if (rc) return rc;                                                                                  \
      launch_after_planner(decode_mma_kernel<TYPE, DIM, STAGES, NBLK, MAXT, MINB, OUT>, grid, threads, smem, stream, tk, tv, p);\
    } while (0)
#define B200ATTN_LAUNCH_DECODE(TYPE, DIM, OUT) B200ATTN_LAUNCH_DECODE_V(TYPE, DIM, 2, 1, 160, 3, OUT)
    if (f32_out) {
      if (D == 128) B200ATTN_LAUNCH_DECODE(__half, 128, float); else B200ATTN_LAUNCH_DECODE(__half, 64, float);
    } else if (a.dtype == B200ATTN_BF16) {
      if (D == 128) B200ATTN_LAUNCH_DECODE(__nv_bfloat16, 128, __nv_bfloat16); else B200ATTN_LAUNCH_DECODE(__nv_bfloat16, 64, __nv_bfloat16);
    } else {
      if (D == 128) B200ATTN_LAUNCH_DECODE(__half, 128, __half); else B200ATTN_LAUNCH_DECODE(__half, 64, __half);
    }
#undef B200ATTN_LAUNCH_DECODE_V
#undef B200ATTN_LAUNCH_DECODE
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "decode kernel launch");
  return B200ATTN_OK;
}
}  // namespace

// ---------------------------------------------------------------------------
// Decode without any caller-provided or allocated scratch memory.
//
// Some hosts of this library are not allowed to allocate device memory at the moment they need
// attention: an inference server that hands its whole HBM budget to the KV cache at start-up and
// forbids allocations afterwards, a plug-in running inside another framework's memory pool, or
// code running while that framework is recording its work and must not disturb its allocator.
// For them the planner tables, merge tickets and split-KV partials live in this fixed array,
// which is part of the loaded module: every GPU that loads the library holds kStaticScratchBytes
// of it until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
constexpr int kScratchMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kScratchMaxDevices] = {};
}  // namespace

// `a.device` must be the current device.  The first call on a device resolves the device address of
// the array (in host code `g_decode_scratch` itself is only a handle, not something a kernel may be
// given); later calls reuse the cached address.
int launch_decode_static(const b200attn_decode_args_t& a, int sm_count, cudaStream_t stream) {
  if (a.device < 0 || a.device >= kScratchMaxDevices) {
    set_error("decode_static: device ordinal %d out of range", a.device);
    return B200ATTN_E_INVALID;
  }
  const DecodeWsLayout w = decode_ws_layout(a, sm_count, /*allow_cast=*/false);
  if (w.total > kStaticScratchBytes) {
    set_error("decode_static: this problem needs %zu bytes of scratch but the built-in array holds %zu; "
              "use b200attn_decode with a caller-provided workspace", w.total, kStaticScratchBytes);
    return B200ATTN_E_WORKSPACE;
  }
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[a.device] == nullptr) {
      void* resolved = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&resolved, g_decode_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(decode scratch)");
      g_scratch_ptr[a.device] = resolved;
    }
    ptr = g_scratch_ptr[a.device];
  }
  b200attn_decode_args_t b = a;
  b.workspace = ptr;
  b.workspace_bytes = kStaticScratchBytes;
  // The planner kernel rewrites the item prefix and zeroes the merge tickets at the start of every
  // call, and partial slots are always written before they are read, so stale contents are harmless.
  return launch_decode(b, sm_count, stream, /*allow_cast=*/false);
}


// Reads and clears the device error word of the built-in array (word 0, where the kernels of
// launch_decode_static report an expired wait, an out-of-range block-table entry or a planner overflow).
// One small copy on `stream`, which it synchronises; allocates nothing.  `device` must be current.
int check_decode_static(int device, cudaStream_t stream, int32_t* code) {
  if (device < 0 || device >= kScratchMaxDevices) {
    set_error("decode_static_check: device ordinal %d out of range", device);
    return B200ATTN_E_INVALID;
  }
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[device] == nullptr) {
      void* resolved = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&resolved, g_decode_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(decode scratch)");
      g_scratch_ptr[device] = resolved;
    }
    ptr = g_scratch_ptr[device];
  }
  int32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, ptr, sizeof(word), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "reading the built-in array's error word");
  if (code) *code = word;
  if (word == 0) return B200ATTN_OK;
  e = cudaMemsetAsync(ptr, 0, sizeof(word), stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "clearing the built-in array's error word");
  set_error("a decode_static kernel reported device error code %d (1 = bounded wait expired, 2 = block-table entry "
            "out of range, 3 = planner overflow)", word);
  return B200ATTN_E_DEVICE;
}

}  // namespace b200attn
