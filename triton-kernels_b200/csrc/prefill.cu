// Prefill attention forward for sm_100a: tcgen05 tensor cores, TMEM accumulators,
// TMA-staged K/V ring, online softmax in registers.
//
// Replaces the reference's partial + merge launch pair (kernels/attention.py:430-746).
//
// Persistent kernel, one CTA per SM.  A work item is two 128-row query tiles ("slots") that share a KV head.
// Warp roles (576 threads):
//   warps 0-15 : softmax; warp w serves slot w / 8, TMEM lane quadrant w % 4 and 16 of its 32 query rows.  Tensor
//                memory is read in the 16x256b layout, which puts the 128 scores of a row into the four threads of
//                a quad: row maxima and sums are two shuffles away, nothing is exchanged through shared memory
//   warp  16   : scheduler + TMA producer (draws work items, loads Q, then the K_j / V_j tiles of 128 keys in pairs
//                {V_j, K_j+1} through two stages of two buffers; paged caches are fetched one page-sized box at a
//                time from the block table)
//   warp  17   : tcgen05.mma issuer and TMEM owner; the warp stays converged, one elected lane issues
// TMEM (512 columns): S0 | S1 | O0 | O1.  Per KV tile j and slot s:
//   S_s = Q_s K_j^T   (SS MMA, 128x128xD)            -> commit s_full[s]
//   the slot's warps read S_s, mask, keep a running max / sum per row in the exp2 domain, rescale O_s in TMEM only
//   when the max moved by more than 2^8, and write P_s as packed 16-bit (16x128b layout) over the first 32 columns
//   of each 64-column half of S_s                                     -> arrive p_ready[s]
//   O_s += P_s V_j    (TS MMA, A from TMEM, V is the MN-major B operand) -> commit o_done[s]
// The two slots are interleaved so that one slot's softmax overlaps the other's MMAs.  At the end of an item the
// MMA warp issues the first score tile of the next item behind the last PVs, and the softmax warps finish the old
// item's epilogue lazily: O is normalised and read out at the end of the next item's first tile and stored while
// the tensor cores work on that tile.
//
// Every mbarrier wait is bounded; on expiry the role records DEV_ERR_WAIT_EXPIRED
// in the workspace header and falls through to the common teardown (TMEM is freed).
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "prefill_launch.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace b200attn {

namespace {

using namespace ptx;

constexpr int kBM = 128;           // query rows per slot
constexpr int kBN = 128;           // keys per K/V tile
constexpr int kSlots = 2;
constexpr int kRing = 4;           // K/V tile buffers: two stages of one V buffer and one K buffer
constexpr int kStages = 2;         // a stage holds the pair {V_j, K_j+1}: one barrier to wait for, one to release
constexpr int kSoftmaxWarps = 16;  // 4 warpgroups: (slot 0 | slot 1) x (columns 0-63 | 64-127)
constexpr int kThreads = 576;
constexpr int kProducerWarp = 16;
constexpr int kMmaWarp = 17;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// Of every 4 pairs of scores, this many are exponentiated on the FMA pipes (range reduction + cubic
// polynomial, relative error 7.5e-5, far below the 16-bit rounding of P) instead of the MUFU unit,
// which at 16 results per clock per SM is as scarce as the tensor pipe at head_dim 128.
#ifndef B200ATTN_EXP_EMU_OF4
#define B200ATTN_EXP_EMU_OF4 1
#endif
constexpr int kExpEmuOf4 = B200ATTN_EXP_EMU_OF4;



// Everything one work item needs; decoded once by the scheduler warp.  An item is two 128-row query tiles
// ("slots") that share one KV head: with an even GQA group the same 128 rows of two neighbouring q heads (equal
// causal extents, so both slots always have work), otherwise two consecutive row tiles of one q head.
struct ItemWork {
  bool valid;
  int len_q, len_k;
  long long kv_row0;   // first kv row this item reads (dense / ragged)
  int kv_tok0;         // first key of the sequence this item reads (non-zero only when the KV range is split)
  long long out_row0[kSlots];   // first output row (the partial buffer's rows when the KV range is split)
  int kv_head_coord;
  int b;
  int q_head[kSlots];
  long long q_row0[kSlots];   // first q row of the sequence on the token axis of the q tensor map
  int q_head_coord[kSlots];
  int m0[kSlots];      // first query row of each slot inside the sequence
  int nkv[kSlots];     // 128-key tiles each slot visits
  int nkv_max;
};

// shared-memory control block placed after the tiles
struct __align__(8) Control {
  uint64_t q_full;
  uint64_t q_empty;
  uint64_t kv_full[kStages];     // pair {V_j, K_j+1} (or K_0 alone / V_last alone) has landed
  uint64_t kv_empty[kStages];    // ... has been consumed by the MMAs
  uint64_t s_full[kSlots];
  uint64_t p_ready[kSlots];
  uint64_t o_done[kSlots];
  uint64_t o_free[kSlots];
  uint64_t sched_full[2];
  uint64_t sched_empty[2];
  int sched_item[2];
  ItemWork sched_work[2];   // decoded by the scheduler, read by every other warp
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
struct SmemPlan {
  static constexpr int kChunks = D / 64;                   // 128-byte column blocks per row
  static constexpr int kChunkBytes = kBN * 128;            // one column block of a 128-row tile
  static constexpr int kTileBytes = kChunks * kChunkBytes; // 128 x D 16-bit tile
  static constexpr int kQOff = 0;
  static constexpr int kRingOff = kSlots * kTileBytes;
  static constexpr int kCtrlOff = kRingOff + kRing * kTileBytes;
  static constexpr int kTotal = kCtrlOff + static_cast<int>(sizeof(Control));
};

// bounded mbarrier wait whose verdict is uniform over the (converged) warp
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  const bool ok = mbar_wait(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ int blocks_of(int len_q, int rows) { return (len_q + rows - 1) / rows; }

// Ragged layout: warp-cooperative search of the (sequence, row block) that owns flat block index x.
__device__ __forceinline__ bool find_ragged_work(const PrefillParams& p, int x, int rows, int lane, int* out_b, int* out_pair) {
  int base = 0;
  for (int b0 = 0; b0 < p.batch; b0 += 32) {
    const int b = b0 + lane;
    int cnt = 0;
    if (b < p.batch) {
      const long long a = load_index(p.q_indptr, p.indptr_is_i64, b);
      const long long e = load_index(p.q_indptr, p.indptr_is_i64, b + 1);
      const long long n = e > a ? e - a : 0;
      cnt = blocks_of(static_cast<int>(n), rows);
    }
    int incl = cnt;
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    const int excl = incl - cnt;
    const bool hit = (x >= base + excl) && (x < base + incl);
    const unsigned mask = __ballot_sync(0xffffffffu, hit);
    if (mask) {
      const int src = __ffs(mask) - 1;
      *out_b = b0 + src;
      *out_pair = x - (base + __shfl_sync(0xffffffffu, excl, src));
      return true;
    }
    base += __shfl_sync(0xffffffffu, incl, 31);
  }
  return false;
}

// fp32 inputs: q, k and v are first rounded to fp16 into the workspace (the reference's kernel does the
// same cast in registers, kernels/attention.py:547,572,594,614) and the result is written back as fp32.
__global__ void __launch_bounds__(256) cast_f32_to_f16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst,
                                                              long long n4) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 f = __ldg(src + i);
    uint2 u;
    u.x = ElemTraits<__half>::pack2(f.x, f.y);
    u.y = ElemTraits<__half>::pack2(f.z, f.w);
    dst[i] = u;
  }
}

__device__ __forceinline__ ItemWork decode_item(const PrefillParams& p, int item, int lane) {
  ItemWork w;
  const int heads_per_item = p.head_pair ? 2 : 1;
  const int head_units = p.q_heads / heads_per_item;
  const int rows = p.head_pair ? kBM : 2 * kBM;      // query rows an item covers
  int wb = -1, wblock = 0, wunit = 0;
  if (p.layout == B200ATTN_RAGGED) {
    wunit = item % head_units;
    // Under a causal mask the row blocks are handed out from the end of the packed tensor backwards: the later
    // blocks of a sequence are the heavier ones, and the blocks left for the drain of the grid are then the first,
    // light ones of the first sequences (the sizes are not known on the host, so there is no global order by weight).
    const int nflat = p.total_items / head_units;
    const int flat = item / head_units;
    if (!find_ragged_work(p, p.is_causal ? nflat - 1 - flat : flat, rows, lane, &wb, &wblock)) wb = -1;
  } else {
    // row blocks are the slowest-varying index and, under a causal mask, are handed out heaviest first;
    // the q heads of one KV head are neighbours and share its K/V in L2
    // with a split KV range every (sequence, KV part) pair is a sequence of its own here ("virtual" batch index)
    const int per_block = head_units * p.batch * p.kv_split;
    const int nblocks = blocks_of(p.max_q, rows);
    const int blk = item / per_block, rest = item - blk * per_block;
    wblock = p.is_causal ? (nblocks - 1 - blk) : blk;
    wunit = rest % head_units;
    wb = rest / head_units;
  }
  w.valid = wb >= 0;
  const int vb = wb;                                   // virtual batch index: rows of the partial buffer
  int part = 0;
  if (p.kv_split > 1 && wb >= 0) { part = wb % p.kv_split; wb /= p.kv_split; }
  w.b = wb;
  w.kv_tok0 = part * p.kv_split_len;
  w.len_q = w.len_k = 0;
  w.kv_row0 = 0;
  w.kv_head_coord = 0;
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    w.q_head[s] = p.head_pair ? wunit * 2 + s : wunit;
    w.m0[s] = p.head_pair ? wblock * kBM : (wblock * kSlots + s) * kBM;
    w.q_row0[s] = 0;
    w.out_row0[s] = 0;
    w.q_head_coord[s] = 0;
  }
  if (w.valid) {
    const int kv_head = w.q_head[0] / p.group;
    if (p.layout == B200ATTN_RAGGED) {
      const long long qa = load_index(p.q_indptr, p.indptr_is_i64, wb);
      const long long qe = load_index(p.q_indptr, p.indptr_is_i64, wb + 1);
      const long long ka = load_index(p.kv_indptr, p.indptr_is_i64, wb);
      const long long ke = load_index(p.kv_indptr, p.indptr_is_i64, wb + 1);
      w.len_q = static_cast<int>(qe > qa ? qe - qa : 0);
      w.len_k = static_cast<int>(ke > ka ? ke - ka : 0);
      w.kv_row0 = ka;
      w.kv_head_coord = kv_head;
#pragma unroll
      for (int s = 0; s < kSlots; ++s) { w.q_row0[s] = qa; w.out_row0[s] = qa; w.q_head_coord[s] = w.q_head[s]; }
    } else {
      w.len_q = p.max_q;
#pragma unroll
      for (int s = 0; s < kSlots; ++s) {
        w.q_row0[s] = (static_cast<long long>(wb) * p.q_heads + w.q_head[s]) * p.max_q;
        w.out_row0[s] = (static_cast<long long>(vb) * p.q_heads + w.q_head[s]) * p.max_q;
      }
      if (p.layout == B200ATTN_DENSE) {
        w.len_k = p.max_kv;
        w.kv_row0 = (static_cast<long long>(wb) * p.kv_heads + kv_head) * p.max_kv + w.kv_tok0;
      } else {
        long long n = load_index(p.kv_indptr, p.indptr_is_i64, wb);
        const long long cap = p.table_stride * static_cast<long long>(p.page_size);
        n = n < 0 ? 0 : (n > cap ? cap : n);
        w.len_k = static_cast<int>(n);
        w.kv_head_coord = kv_head;
      }
      if (p.kv_split > 1) {
        // this item sees the keys [kv_tok0, kv_tok0 + kv_split_len) of the sequence only
        int local = w.len_k - w.kv_tok0;
        local = local < 0 ? 0 : (local > p.kv_split_len ? p.kv_split_len : local);
        w.len_k = local;
      }
    }
  }
  w.nkv_max = 0;
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    int n = 0;
    if (w.valid && w.m0[s] < w.len_q) {
      int kv_hi = w.len_k;
      if (p.is_causal) kv_hi = min(kv_hi, min(w.m0[s] + kBM, w.len_q) - w.kv_tok0);
      n = kv_hi > 0 ? (kv_hi + kBN - 1) / kBN : 0;
    }
    w.nkv[s] = n;
    w.nkv_max = max(w.nkv_max, n);
  }
  return w;
}

// Persistent kernel: one CTA per SM; work items are drawn from a global counter (heaviest first).
// The producer warp is also the scheduler: it publishes item indices through a 2-deep ring, so it can fetch Q
// and the first K/V tiles of the next item while the other roles finish the current one.
// kPaged: the instantiation launched for paged K/V; only it carries the block-table read-ahead of the producer (in
// the dense / ragged kernel that code, though never run, cost 1 % on the dense benchmark configuration).  The other
// layout checks stay run-time checks.
template <typename T, int D, typename OutT, bool kPaged>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
  using Plan = SmemPlan<D>;
  extern __shared__ unsigned char smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctrl = reinterpret_cast<Control*>(smem + Plan::kCtrlOff);
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // The scheduler / producer warp sets the barriers up itself and goes straight on to draw and decode its first item
  // and to issue the first copies: it only arrives at the start-up barrier, it does not wait there for the TMEM
  // allocation of the MMA warp (it never touches tensor memory).  Everybody else waits until both are done.
  if (warp == kProducerWarp) {
    if (lane == 0) {
      mbar_init(smem_u32(&ctrl->q_full), 1);
      mbar_init(smem_u32(&ctrl->q_empty), 1);
      for (int i = 0; i < kStages; ++i) { mbar_init(smem_u32(&ctrl->kv_full[i]), 1); mbar_init(smem_u32(&ctrl->kv_empty[i]), 1); }
      for (int s = 0; s < kSlots; ++s) {
        mbar_init(smem_u32(&ctrl->s_full[s]), 1);
        mbar_init(smem_u32(&ctrl->p_ready[s]), 2 * kBM);
        mbar_init(smem_u32(&ctrl->o_done[s]), 1);
        mbar_init(smem_u32(&ctrl->o_free[s]), 8);          // one arrival per softmax warp of the slot
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&ctrl->sched_full[i]), 1);
        mbar_init(smem_u32(&ctrl->sched_empty[i]), kSoftmaxWarps + 1);
      }
      ctrl->abort_flag = 0;
      mbar_fence_init();
    }
    __syncwarp();
    named_bar_arrive(1, kThreads);
  } else {
    // ---------------- TMEM allocation (MMA warp owns it) ----------------
    if (warp == kMmaWarp) {
      tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
      tmem_relinquish();
    }
    tc_fence_before();
    named_bar_sync(1, kThreads);
    tc_fence_after();
  }
  const uint32_t tmem = warp == kProducerWarp ? 0u : ctrl->tmem_base;   // (the producer never uses it)
  volatile int* abort_flag = &ctrl->abort_flag;

  if (warp == kProducerWarp) {
    // =========================== scheduler + TMA producer ===========================
    if (lane == 0) { prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v); }
    bool ok = true;
    int pair_e = 0;       // K/V pairs issued so far, across items
    int pair_lo = 0;      // first pair of the current item
    for (int k = 0; ok; ++k) {
      if (k >= 2) {
        ok = warp_wait(smem_u32(&ctrl->sched_empty[k & 1]), ((k >> 1) - 1) & 1);
        if (!ok || *abort_flag) { ok = false; break; }
      }
      int item = -1;
      if (lane == 0) {
        // the first item of a CTA is its own index (the grid never exceeds the item count); later ones are drawn
        item = k == 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
        if (item >= p.total_items) item = -1;
      }
      item = __shfl_sync(0xffffffffu, item, 0);
      ItemWork w;
      if (item >= 0) w = decode_item(p, item, lane);
      if (lane == 0) {
        if (item >= 0) ctrl->sched_work[k & 1] = w;
        ctrl->sched_item[k & 1] = item;
        mbar_arrive(smem_u32(&ctrl->sched_full[k & 1]));
      }
      if (item < 0) break;
      if (k >= 1 && lane == 0) {
        // the previous item is still running: pull this item's Q tiles and first K/V tiles into L2 now, so the
        // copies issued once the Q buffer is free only pay an L2 round trip
        for (int s = 0; s < kSlots; ++s) {
          if (w.nkv[s] == 0) continue;
          for (int c = 0; c < Plan::kChunks; ++c)
            tma_prefetch_3d(&tm_q, c * 64, w.q_head_coord[s], static_cast<int>(w.q_row0[s] + w.m0[s]));
        }
        if (p.layout != B200ATTN_PAGED && w.nkv_max > 0) {
          for (int c = 0; c < Plan::kChunks; ++c) {
            tma_prefetch_3d(&tm_k, c * 64, w.kv_head_coord, static_cast<int>(w.kv_row0));
            tma_prefetch_3d(&tm_v, c * 64, w.kv_head_coord, static_cast<int>(w.kv_row0));
          }
        }
      }
      // Q may be overwritten once every S MMA of the previous item has completed
      if (k >= 1) {
        ok = warp_wait(smem_u32(&ctrl->q_empty), (k - 1) & 1);
        if (!ok || *abort_flag) { ok = false; break; }
      }
      if (lane == 0) {
        uint32_t bytes = 0;
        for (int s = 0; s < kSlots; ++s) if (w.nkv[s] > 0) bytes += Plan::kTileBytes;
        if (bytes > 0) {
          mbar_arrive_expect_tx(smem_u32(&ctrl->q_full), bytes);
          for (int s = 0; s < kSlots; ++s) {
            if (w.nkv[s] == 0) continue;
            for (int c = 0; c < Plan::kChunks; ++c)
              tma_load_3d(smem_base + Plan::kQOff + s * Plan::kTileBytes + c * Plan::kChunkBytes, &tm_q,
                          smem_u32(&ctrl->q_full), c * 64, w.q_head_coord[s], static_cast<int>(w.q_row0[s] + w.m0[s]));
          }
        } else {
          mbar_arrive(smem_u32(&ctrl->q_full));   // keeps one q_full phase per item
        }
      }
      // K/V tiles travel in pairs that share one barrier: pair 0 of an item is K_0 alone, pair j + 1 is {V_j, K_j+1}
      // (the last one V alone).  Stage = pair % 2; its V buffer is ring buffer 2 * stage, its K buffer 2 * stage + 1.
      pair_lo = pair_e;
      const int npairs = w.nkv_max > 0 ? w.nkv_max + 1 : 0;
      // Paged K/V with at most 32 boxes per tile (one per lane): the raw block-table entries of a pair's boxes (V of
      // tile pi - 1, K of tile pi) are read one pair ahead, into two plain registers, so that the table read is not
      // between "stage free" and "copies issued" (the ring is only two pairs deep).
      constexpr int kNoPage = static_cast<int>(0x80000000u);
      const int pf_boxes = kPaged ? kBN / p.box_rows : 0;
      const bool pf = kPaged && pf_boxes <= 32;
      int pg_v = kNoPage, pg_k = kNoPage;
      auto fetch_pages = [&](int pi) {
        const int tv = (pi - 1) * kBN + lane * p.box_rows, tk = pi * kBN + lane * p.box_rows;
        pg_v = (lane < pf_boxes && pi >= 1 && tv < w.len_k)
                   ? __ldg(p.v_table + static_cast<long long>(w.b) * p.table_stride + (tv + w.kv_tok0) / p.page_size) : kNoPage;
        pg_k = (lane < pf_boxes && pi < w.nkv_max && tk < w.len_k)
                   ? __ldg(p.k_table + static_cast<long long>(w.b) * p.table_stride + (tk + w.kv_tok0) / p.page_size) : kNoPage;
      };
      if (pf && npairs > 0) fetch_pages(0);
      for (int pi = 0; pi < npairs && ok; ++pi, ++pair_e) {
        const int stage = pair_e % kStages;
        const int use = pair_e / kStages;
        if (use > 0) {
          ok = warp_wait(smem_u32(&ctrl->kv_empty[stage]), (use - 1) & 1);
          if (!ok || *abort_flag) { ok = false; break; }
        }
        const uint32_t bar = smem_u32(&ctrl->kv_full[stage]);
        const bool has_v = pi >= 1, has_k = pi < w.nkv_max;
        const int jv = pi - 1, jk = pi;               // tile indices of the V and the K of this pair
        const uint32_t vdst = smem_base + Plan::kRingOff + (2 * stage) * Plan::kTileBytes;
        const uint32_t kdst = vdst + Plan::kTileBytes;
        if (p.layout != B200ATTN_PAGED) {
          if (lane == 0) {
            mbar_arrive_expect_tx(bar, (has_v ? Plan::kTileBytes : 0) + (has_k ? Plan::kTileBytes : 0));
            for (int c = 0; c < Plan::kChunks; ++c) {
              if (has_v)
                tma_load_3d(vdst + c * Plan::kChunkBytes, &tm_v, bar, c * 64, w.kv_head_coord,
                            static_cast<int>(w.kv_row0 + static_cast<long long>(jv) * kBN));
              if (has_k)
                tma_load_3d(kdst + c * Plan::kChunkBytes, &tm_k, bar, c * 64, w.kv_head_coord,
                            static_cast<int>(w.kv_row0 + static_cast<long long>(jk) * kBN));
            }
          }
        } else if (pf) {
          // one box per lane and operand from the prefetched table entries
          auto row_of = [&](int page, int t) -> int {
            if (page == kNoPage) return -1;
            // an entry outside the cache is reported and replaced by page 0: never dereferenced, output stays finite
            const bool bad = page < 0 || page >= p.num_pages;
            if (bad) p.header[0] = DEV_ERR_PAGE_RANGE;
            return p.num_pages > 0 ? (bad ? 0 : page) * p.page_size + (t + w.kv_tok0) % p.page_size : -1;
          };
          const int rv = row_of(pg_v, jv * kBN + lane * p.box_rows);
          const int rk = row_of(pg_k, jk * kBN + lane * p.box_rows);
          int count = (rv >= 0) + (rk >= 0);
          for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
          if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * p.box_rows * 128 * Plan::kChunks);
          __syncwarp();
          for (int c = 0; c < Plan::kChunks; ++c) {
            if (rv >= 0)
              tma_load_3d(vdst + c * Plan::kChunkBytes + lane * p.box_rows * 128, &tm_v, bar, c * 64, w.kv_head_coord, rv);
            if (rk >= 0)
              tma_load_3d(kdst + c * Plan::kChunkBytes + lane * p.box_rows * 128, &tm_k, bar, c * 64, w.kv_head_coord, rk);
          }
          if (pi + 1 < npairs) fetch_pages(pi + 1);
        } else {
          // one box of `box_rows` tokens per lane per round and operand; only pages that exist are fetched
          const int boxes = kBN / p.box_rows;
          int rows_v[4], rows_k[4];
          int nmine = 0;
          int count = 0;
          auto page_row = [&](const int* table, int t) -> int {
            if (t >= w.len_k) return -1;
            const int tg = t + w.kv_tok0;          // position in the whole sequence
            const int lp = tg / p.page_size;
            const int page = __ldg(table + lp);
            // an entry outside the cache is reported and replaced by page 0: never dereferenced, output stays finite
            const bool bad = page < 0 || page >= p.num_pages;
            if (bad) p.header[0] = DEV_ERR_PAGE_RANGE;
            return p.num_pages > 0 ? (bad ? 0 : page) * p.page_size + (tg - lp * p.page_size) : -1;
          };
          const int* vtab = p.v_table + static_cast<long long>(w.b) * p.table_stride;
          const int* ktab = p.k_table + static_cast<long long>(w.b) * p.table_stride;
          for (int i = lane; i < boxes; i += 32) {
            const int rv = has_v ? page_row(vtab, jv * kBN + i * p.box_rows) : -1;
            const int rk = has_k ? page_row(ktab, jk * kBN + i * p.box_rows) : -1;
            rows_v[nmine] = rv;
            rows_k[nmine] = rk;
            ++nmine;
            count += (rv >= 0) + (rk >= 0);
          }
          for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
          if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(count) * p.box_rows * 128 * Plan::kChunks);
          __syncwarp();
          int kk = 0;
          for (int i = lane; i < boxes; i += 32, ++kk) {
            for (int c = 0; c < Plan::kChunks; ++c) {
              if (rows_v[kk] >= 0)
                tma_load_3d(vdst + c * Plan::kChunkBytes + i * p.box_rows * 128, &tm_v, bar, c * 64, w.kv_head_coord, rows_v[kk]);
              if (rows_k[kk] >= 0)
                tma_load_3d(kdst + c * Plan::kChunkBytes + i * p.box_rows * 128, &tm_k, bar, c * 64, w.kv_head_coord, rows_k[kk]);
            }
          }
        }
      }
    }
    if (!ok) {
      if (lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
      // drain: wait (bounded) for the copies still in flight before the CTA may exit
      for (int e = max(pair_lo, pair_e - kStages); e < pair_e; ++e) mbar_wait(smem_u32(&ctrl->kv_full[e % kStages]), (e / kStages) & 1);
    }
    if (lane == 0) {
      // This CTA draws no more items.  The last CTA to get here puts both counters back to zero for the next
      // launch on this workspace (every other CTA's draws are ordered before its own increment by the fence).
      __threadfence();
      if (atomicAdd(p.work_counter + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        atomicExch(p.work_counter, 0);
        atomicExch(p.work_counter + 1, 0);
      }
    }
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr uint32_t idesc_s = make_idesc_f16(kBM, kBN, kFmt, 0);
    constexpr uint32_t idesc_o = make_idesc_f16(kBM, D, kFmt, 1);
    const uint32_t tmem_S[kSlots] = {tmem, tmem + kBN};
    const uint32_t tmem_O[kSlots] = {tmem + 2 * kBN, tmem + 2 * kBN + D};
    bool ok = true;
    // Descriptor words are prepared once: the high words never change, the low words are a base
    // (start address >> 4) plus small constants, so issuing one MMA costs the single thread a few adds.
    const uint64_t kdesc = make_smem_desc_sw128(smem_base, 16);                    // K-major operands (Q, K)
    const uint64_t vdesc = make_smem_desc_sw128(smem_base, Plan::kChunkBytes);     // MN-major operand (V)
    int pair_base = 0;            // pair that holds K_0 of the current item (pair j + 1 holds V_j and K_j+1)
    // per-slot state as scalars (an array indexed by the slot would live in local memory)
    int tiles_done0 = 0, tiles_done1 = 0;       // score tiles issued per slot so far (barrier phases run across items)
    bool pre_issued0 = false, pre_issued1 = false;   // first score tile of the coming item already issued
    auto pair_full_wait = [&](int pr) -> bool {
      return warp_wait(smem_u32(&ctrl->kv_full[pr % kStages]), (pr / kStages) & 1);
    };
    // The warp stays converged while it issues: every lane runs the descriptor arithmetic, one elected lane
    // issues the tensor-core instructions and their commits.
    const uint32_t lead = elect_one();
    // operand descriptors of the K and the V buffer of a pair's stage
    auto k_desc_of = [&](int pr) -> uint64_t {
      return kdesc + static_cast<uint64_t>((Plan::kRingOff + (2 * (pr % kStages) + 1) * Plan::kTileBytes) >> 4);
    };
    auto v_desc_of = [&](int pr) -> uint64_t {
      return vdesc + static_cast<uint64_t>((Plan::kRingOff + (2 * (pr % kStages)) * Plan::kTileBytes) >> 4);
    };
    auto issue_s = [&](int s, uint64_t kb) {
      // S_s = Q_s K^T : K-major A and B, D/16 k-steps
      const uint64_t qa = kdesc + static_cast<uint64_t>((Plan::kQOff + s * Plan::kTileBytes) >> 4);
      mma_ss_batch<D / 16>(tmem_S[s], qa, kb, idesc_s, 0u, lead);
      mma_commit_lead(smem_u32(&ctrl->s_full[s]), lead);
    };
    auto issue_pv = [&](int s, uint64_t vb, bool first) {
      // O_s (+)= P_s V : A = packed 16-bit P, 32 TMEM columns at the start of each 64-column half of the S tile;
      // B = V, MN-major
      mma_ts_batch8(tmem_O[s], tmem_S[s], vb, idesc_o, first ? 0u : 1u, lead);
      mma_commit_lead(smem_u32(&ctrl->o_done[s]), lead);
    };

    for (int k = 0; ok; ++k) {
      ok = warp_wait(smem_u32(&ctrl->sched_full[k & 1]), (k >> 1) & 1);
      if (!ok || *abort_flag) { ok = false; break; }
      const int item = ctrl->sched_item[k & 1];
      if (item < 0) break;
      const ItemWork& wr = ctrl->sched_work[k & 1];
      const int nkv0 = wr.nkv[0], nkv1 = wr.nkv[1], nkv_max = wr.nkv_max, len_k = wr.len_k;
      ok = warp_wait(smem_u32(&ctrl->q_full), k & 1);
      if (!ok) break;
      if (nkv_max > 0) {
        ok = pair_full_wait(pair_base);
        if (!ok) break;
        tc_fence_after();
        // (slots whose first score tile was already issued while the previous item finished are skipped)
        if (nkv0 > 0 && !pre_issued0) issue_s(0, k_desc_of(pair_base));
        if (nkv1 > 0 && !pre_issued1) issue_s(1, k_desc_of(pair_base));
        mma_commit_lead(smem_u32(&ctrl->kv_empty[pair_base % kStages]), lead);
        if (nkv_max == 1) mma_commit_lead(smem_u32(&ctrl->q_empty), lead);
      } else {
        mma_commit_lead(smem_u32(&ctrl->q_empty), lead);
      }
      pre_issued0 = pre_issued1 = false;
      for (int j = 0; j < nkv_max && ok; ++j) {
        const int pr = pair_base + 1 + j;     // the pair {V_j, K_j+1}
        const bool last_iter = j + 1 == nkv_max;
        // On the last tile of the item the first score tile of the next item is issued right behind each slot's
        // final PV, so the softmax warps can carry straight on.  Everything waited
        // for here (next item published, its Q and first K tile loaded) depends only on work this warp has
        // already issued: Q may be replaced once the last score MMAs of this item, issued one tile ago, complete.
        int next_state = 0;            // 0 = not looked at yet, 1 = ready, -1 = nothing to issue ahead
        int next_nkv0 = 0, next_nkv1 = 0;   // tiles per slot of the next item
        auto prepare_next = [&]() -> bool {
          if (next_state != 0) return true;
          next_state = -1;
          if (!warp_wait(smem_u32(&ctrl->sched_full[(k + 1) & 1]), ((k + 1) >> 1) & 1)) return false;
          if (ctrl->sched_item[(k + 1) & 1] < 0) return true;
          const ItemWork& wn = ctrl->sched_work[(k + 1) & 1];
          if (wn.nkv_max == 0) return true;
          next_nkv0 = wn.nkv[0];
          next_nkv1 = wn.nkv[1];
          if (!warp_wait(smem_u32(&ctrl->q_full), (k + 1) & 1)) return false;
          if (!pair_full_wait(pair_base + nkv_max + 1)) return false;
          next_state = 1;
          return true;
        };
        // Everything that does not depend on the softmax warps is waited for and computed before their P is: the
        // pair {V_j, K_j+1} (one barrier; in steady state loaded long ago), the operand descriptors, and on the last
        // tile the next item.  Between a slot's P and its two batches of MMAs the warp then only runs the issue.
        ok = pair_full_wait(pr);
        if (!ok) break;
        {
          const int valid = len_k - j * kBN;
          if (valid < kBN) {
            // keys past the sequence end carry P == 0 but their V rows may hold anything (stale
            // shared memory, the next sequence, poisoned page tails): zero them so 0 * x stays 0
            unsigned char* vbuf = smem + Plan::kRingOff + (2 * (pr % kStages)) * Plan::kTileBytes;
            const int first = valid > 0 ? valid : 0;
            const int n16 = (kBN - first) * 8;  // 16-byte pieces per column block
            for (int c = 0; c < Plan::kChunks; ++c) {
              uint4* dst = reinterpret_cast<uint4*>(vbuf + c * Plan::kChunkBytes + first * 128);
              for (int i = lane; i < n16; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
        }
        int pr_k = pr;                // pair whose K buffer the score MMAs issued in this iteration read
        if (last_iter) {
          ok = prepare_next();
          if (!ok) break;
          pr_k = pair_base + nkv_max + 1;       // K_0 of the next item (read only when next_state == 1)
        }
        const uint64_t vb = v_desc_of(pr);
        const uint64_t kb = k_desc_of(pr_k);
        auto slot_step = [&](const int s, const int nkv_s, const int next_nkv_s, int& tiles_done, bool& pre_issued) -> bool {
          if (j >= nkv_s) return true;
          const bool s_next = last_iter ? (next_state == 1 && next_nkv_s > 0) : (j + 1 < nkv_s);
          if (j == 0 && k > 0) {
            // the first PV of an item overwrites O: the epilogue of the previous item must have read it out
            // (the softmax warps do that just before they hand over this tile's P)
            if (!warp_wait(smem_u32(&ctrl->o_free[s]), (k - 1) & 1)) return false;
          }
          if (!warp_wait(smem_u32(&ctrl->p_ready[s]), tiles_done & 1)) return false;
          tc_fence_after();
          issue_pv(s, vb, j == 0);
          if (s_next) {
            issue_s(s, kb);
            if (last_iter) pre_issued = true;
          }
          ++tiles_done;
          return true;
        };
        ok = slot_step(0, nkv0, next_nkv0, tiles_done0, pre_issued0);
        if (ok) ok = slot_step(1, nkv1, next_nkv1, tiles_done1, pre_issued1);
        if (!ok) break;
        if (last_iter) {
          // a slot that ran out of tiles earlier in this item gets its head start here
          ok = prepare_next();
          if (!ok) break;
          if (next_state == 1) {
            if (!pre_issued0 && next_nkv0 > 0) { tc_fence_after(); issue_s(0, kb); pre_issued0 = true; }
            if (!pre_issued1 && next_nkv1 > 0) { tc_fence_after(); issue_s(1, kb); pre_issued1 = true; }
          }
        }
        // V_j and K_j+1 have been read by everything that will read them: one commit releases the stage
        mma_commit_lead(smem_u32(&ctrl->kv_empty[pr % kStages]), lead);
        // the last score MMAs of the item have been issued: Q may be replaced once they complete
        if (j + 2 == nkv_max) mma_commit_lead(smem_u32(&ctrl->q_empty), lead);
      }
      if (nkv_max > 0) pair_base += nkv_max + 1;
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[k & 1]));
      __syncwarp();
    }
    if (!ok && lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
  } else if (warp < kSoftmaxWarps) {
    // =========================== softmax warps ===========================
    // Warp w serves slot w / 8, the TMEM lane quadrant w % 4 (the only lanes it may touch) and, inside the quadrant,
    // the sixteen query rows 16 h .. 16 h + 15 with h = (w / 4) % 2.  Tensor memory is read in the 16x256b layout:
    // thread t holds the columns 8 i + 2 (t % 4) + {0, 1} (i = 0 .. 15) of row A = t / 4 and of row B = A + 8, so the
    // 128 scores of a row live in the four threads of a quad and row maxima and sums are two shuffles away: no
    // exchange through shared memory, no barrier inside a tile.
    const int s = warp >> 3;
    const int qd = warp & 3;
    const int h = (warp >> 2) & 1;
    const int q = lane & 3;
    const int rowA = qd * 32 + h * 16 + (lane >> 2);    // 0..127 inside the slot; row B = row A + 8
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32 + h * 16) << 16;
    const uint32_t tS = tmem + s * kBN + lane_off;
    const uint32_t tO = tmem + 2 * kBN + s * D + lane_off;
    const float sl2 = p.scale_log2;
    int tile_cnt = 0;     // score tiles of this slot consumed so far (barrier phases run across items)
    bool ok = true;
    // The epilogue of an item is finished lazily: O is read out of tensor memory at the end of the first score
    // tile of the slot's next item (its PV is the first thing that overwrites O) and the global stores are issued
    // after that tile's P has been handed over, so they drain while the tensor cores work on it.
    bool pend = false;        // an item's output is still in tensor memory
    bool pend_acc = false;    // ... and it has an accumulator (false: the slot had no keys, the output is zero)
    int pend_phase = 0;       // o_done phase of its last PV
    int pend_rows = 0;        // rows of the tile that exist in the sequence
    float pend_la = 0.f, pend_lb = 0.f;   // row sums of rows A and B
    long long pend_off = 0;   // element offset of row A's first output column
    long long pend_stride = 0;   // elements between consecutive rows of the output
    constexpr bool k16 = !std::is_same<OutT, float>::value;
    auto quad_max = [](float v) {
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
      return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    };
    auto quad_sum = [](float v) {
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      return v + __shfl_xor_sync(0xffffffffu, v, 2);
    };
    // 4 x 4 transpose of two-word items across the four threads of a quad (lane bits 0-1): on return item m of
    // thread q is what item q of thread m was.  x[2m], x[2m+1] are the words of item m.
    auto quad_transpose = [&](uint32_t (&x)[8]) {
      const bool b1 = (lane & 2) != 0, b0 = (lane & 1) != 0;
#pragma unroll
      for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int wd = 0; wd < 2; ++wd) {
          uint32_t& lo = x[2 * m + wd];
          uint32_t& hi = x[2 * (m + 2) + wd];
          const uint32_t recv = __shfl_xor_sync(0xffffffffu, b1 ? lo : hi, 2);
          if (b1) lo = recv; else hi = recv;
        }
      }
#pragma unroll
      for (int m = 0; m < 4; m += 2) {
#pragma unroll
        for (int wd = 0; wd < 2; ++wd) {
          uint32_t& lo = x[2 * m + wd];
          uint32_t& hi = x[2 * (m + 1) + wd];
          const uint32_t recv = __shfl_xor_sync(0xffffffffu, b0 ? lo : hi, 1);
          if (b0) lo = recv; else hi = recv;
        }
      }
    };
    auto flush = [&](bool hand_over) -> bool {
      if (pend_acc) {
        if (!warp_wait(smem_u32(&ctrl->o_done[s]), pend_phase)) return false;
      }
      tc_fence_after();
      const float inv_a = pend_la > 0.f ? 1.f / pend_la : 0.f;
      const float inv_b = pend_lb > 0.f ? 1.f / pend_lb : 0.f;
      auto o_is_free = [&]() {
        // O has been read out: the MMA warp may start the next item's PV into it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->o_free[s]));
      };
      auto hand = [&]() {
        if (hand_over) {
          // this tile's P goes to the MMA warp before the stores are issued
          tc_fence_before();
          mbar_arrive(smem_u32(&ctrl->p_ready[s]));
        }
      };
      constexpr int kChunksO = D / 64;
      if constexpr (k16) {
        // 16-bit output: 64 columns of a row are one 128-byte line.  A quad holds 8 consecutive columns per group;
        // transposed inside the quad, every thread owns 32 contiguous bytes and a store instruction writes 8 full
        // lines instead of one piece of 32 different lines.
        uint32_t line[kChunksO][2][8];     // [64-column chunk][row A / row B][32 bytes of the row's line]
#pragma unroll
        for (int c = 0; c < kChunksO; ++c) {
          uint32_t v[32];
          if (pend_acc) {
            tmem_ld_16x256b_x8(tO + c * 64, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (c == kChunksO - 1) o_is_free();
          uint32_t a[8], b[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a[i] = ElemTraits<T>::pack2(__uint_as_float(v[4 * i]) * inv_a, __uint_as_float(v[4 * i + 1]) * inv_a);
            b[i] = ElemTraits<T>::pack2(__uint_as_float(v[4 * i + 2]) * inv_b, __uint_as_float(v[4 * i + 3]) * inv_b);
          }
          // thread q of the quad holds word q of each 16-byte block i; it ends up with blocks 2q and 2q+1 whole
          quad_transpose(a);
          quad_transpose(b);
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            line[c][0][m] = a[2 * m];  line[c][0][4 + m] = a[2 * m + 1];
            line[c][1][m] = b[2 * m];  line[c][1][4 + m] = b[2 * m + 1];
          }
        }
        hand();
#pragma unroll
        for (int ab = 0; ab < 2; ++ab) {
          if (rowA + 8 * ab < pend_rows) {
#pragma unroll
            for (int c = 0; c < kChunksO; ++c) {
              T* out = static_cast<T*>(p.out) + pend_off + ab * 8 * pend_stride + c * 64 + q * 16;
              const uint32_t (&u)[8] = line[c][ab];
              if (p.out_align32) {
                st_global_v8(out, u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7]);
              } else {
                *reinterpret_cast<uint4*>(out) = make_uint4(u[0], u[1], u[2], u[3]);
                *reinterpret_cast<uint4*>(out + 8) = make_uint4(u[4], u[5], u[6], u[7]);
              }
            }
          }
        }
      } else {
        // fp32 output: a thread holds two consecutive columns per group, a quad 32 contiguous bytes of a row
#pragma unroll
        for (int c = 0; c < kChunksO; ++c) {
          uint32_t v[32];
          if (pend_acc) {
            tmem_ld_16x256b_x8(tO + c * 64, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (c == kChunksO - 1) { o_is_free(); hand(); }
          float* out = static_cast<float*>(p.out) + pend_off + c * 64 + q * 2;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (rowA < pend_rows)
              *reinterpret_cast<float2*>(out + i * 8) = make_float2(__uint_as_float(v[4 * i]) * inv_a, __uint_as_float(v[4 * i + 1]) * inv_a);
            if (rowA + 8 < pend_rows)
              *reinterpret_cast<float2*>(out + 8 * pend_stride + i * 8) =
                  make_float2(__uint_as_float(v[4 * i + 2]) * inv_b, __uint_as_float(v[4 * i + 3]) * inv_b);
          }
        }
      }
      pend = false;
      return true;
    };
    for (int k = 0; ok; ++k) {
      ok = warp_wait(smem_u32(&ctrl->sched_full[k & 1]), (k >> 1) & 1);
      if (!ok || *abort_flag) { ok = false; break; }
      const int item = ctrl->sched_item[k & 1];
      if (item < 0) break;
      // (the few fields needed are read from shared memory where they are used, not held across the tile loop)
      const ItemWork& w = ctrl->sched_work[k & 1];
      const int n = w.nkv[s];
      const int m0s = w.m0[s];
      const int len_k = w.len_k;
      const int row_abs = m0s + rowA - w.kv_tok0;       // query index of row A relative to the item's first key (row B: + 8)
      if (pend && n == 0) {
        // no score tile in this item to hang the previous item's epilogue on
        ok = flush(false);
        if (!ok) break;
      }
      float m_a = -INFINITY, m_b = -INFINITY;   // exponent references currently baked into O and l
      float l_a = 0.f, l_b = 0.f;               // partial row sums over this thread's columns
      for (int j = 0; j < n; ++j, ++tile_cnt) {
        ok = warp_wait(smem_u32(&ctrl->s_full[s]), tile_cnt & 1);
        if (!ok || *abort_flag) { ok = false; break; }
        tc_fence_after();
        // masking is needed only on the tile that holds the sequence end or the causal diagonal; `lim` is the last
        // visible column of the tile for the row
        int lim_a = len_k - 1 - j * kBN, lim_b = lim_a;
        if (p.is_causal) { lim_a = min(lim_a, row_abs - j * kBN); lim_b = min(lim_b, row_abs + 8 - j * kBN); }
        const bool masked = min(lim_a, lim_b) < kBN - 1;
        if (masked) {
          // The mask is written into the score tile itself (-inf over the hidden columns) before the two passes
          // below, which then have one form for every tile: a masked copy of their bodies, run once per item from a
          // cold instruction cache, cost more than this extra round trip through tensor memory.
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tmem_ld_16x256b_x8(tS + c * 64, v);
            tmem_wait_ld();
            const int ta = lim_a - c * 64 - 2 * q, tb = lim_b - c * 64 - 2 * q;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                v[4 * i + e] = (8 * i + e > ta) ? 0xff800000u : v[4 * i + e];           // -inf
                v[4 * i + 2 + e] = (8 * i + e > tb) ? 0xff800000u : v[4 * i + 2 + e];
              }
            }
            tmem_st_16x256b_x8(tS + c * 64, v);
          }
          tmem_wait_st();
        }
        float mx_a, mx_b;
        uint32_t v_hi[32];     // columns 64..127 of the tile stay in registers from pass 1 to pass 2
        {
          // pass 1: row maxima.  Columns 0..63 are read again in pass 2 (all 128 scores cannot be held across it).
          uint32_t v[32];
          tmem_ld_16x256b_x8(tS, v);
          tmem_ld_16x256b_x8(tS + 64, v_hi);
          tmem_wait_ld();
          float a0 = fmaxf(__uint_as_float(v[0]), __uint_as_float(v[1]));
          float b0 = fmaxf(__uint_as_float(v[2]), __uint_as_float(v[3]));
#pragma unroll
          for (int i = 1; i < 8; ++i) {
            a0 = max3(a0, __uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]));
            b0 = max3(b0, __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a0 = max3(a0, __uint_as_float(v_hi[4 * i]), __uint_as_float(v_hi[4 * i + 1]));
            b0 = max3(b0, __uint_as_float(v_hi[4 * i + 2]), __uint_as_float(v_hi[4 * i + 3]));
          }
          mx_a = quad_max(a0);
          mx_b = quad_max(b0);
        }
        const float mn_a = fmaxf(m_a, mx_a * sl2), mn_b = fmaxf(m_b, mx_b * sl2);
        const bool need_a = (mn_a - m_a) > kRescaleThreshold;   // false for NaN / (-inf)-(-inf)
        const bool need_b = (mn_b - m_b) > kRescaleThreshold;
        float alpha_a = 1.f, alpha_b = 1.f;
        if (need_a) { alpha_a = fast_exp2(m_a - mn_a); m_a = mn_a; l_a *= alpha_a; }
        if (need_b) { alpha_b = fast_exp2(m_b - mn_b); m_b = mn_b; l_b *= alpha_b; }
        if (j > 0 && __any_sync(0xffffffffu, need_a || need_b)) {
          // PV(j-1) has landed in O once S(j) is visible (the MMAs complete in issue order); waiting on its
          // barrier phase is then immediate, and skipping the wait on other tiles is harmless because the
          // barrier can never run two phases ahead of this warp
          ok = warp_wait(smem_u32(&ctrl->o_done[s]), (tile_cnt - 1) & 1);
          if (!ok) break;
          tc_fence_after();
          // (rare: 16 columns at a time and not unrolled, so that the scores held in registers stay there)
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t ov[8];
            tmem_ld_16x256b_x2(tO + c * 16, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              ov[4 * i] = __float_as_uint(__uint_as_float(ov[4 * i]) * alpha_a);
              ov[4 * i + 1] = __float_as_uint(__uint_as_float(ov[4 * i + 1]) * alpha_a);
              ov[4 * i + 2] = __float_as_uint(__uint_as_float(ov[4 * i + 2]) * alpha_b);
              ov[4 * i + 3] = __float_as_uint(__uint_as_float(ov[4 * i + 3]) * alpha_b);
            }
            tmem_st_16x256b_x2(tO + c * 16, ov);
          }
        }
        const float neg_a = (m_a == -INFINITY) ? 0.f : -m_a, neg_b = (m_b == -INFINITY) ? 0.f : -m_b;
        uint64_t rs_a = pack_f2(0.f, 0.f), rs_b = pack_f2(0.f, 0.f);
        const uint64_t sl2_2 = pack_f2(sl2, sl2), nega_2 = pack_f2(neg_a, neg_a), negb_2 = pack_f2(neg_b, neg_b);
        auto exp_pair = [&](uint32_t x0, uint32_t x1, uint64_t neg2, uint64_t& rs, bool emulate) -> uint32_t {
          const uint64_t t2 = fma_f2(pack_f2(__uint_as_float(x0), __uint_as_float(x1)), sl2_2, neg2);
          float p0, p1;
          if (emulate) {
            // 2^t = 2^n * 2^r with n = round(t), r in [-0.5, 0.5]; n is read off the magic-number sum
            float a, b;
            unpack_f2(t2, a, b);
            const uint64_t tc = pack_f2(fmaxf(a, -126.f), fmaxf(b, -126.f));
            const uint64_t tm = add_f2(tc, pack_f2(12582912.f, 12582912.f));
            const uint64_t nf = add_f2(tm, pack_f2(-12582912.f, -12582912.f));
            const uint64_t r = fma_f2(nf, pack_f2(-1.f, -1.f), tc);
            uint64_t pq = fma_f2(r, pack_f2(0.055171482f, 0.055171482f), pack_f2(0.2426109f, 0.2426109f));
            pq = fma_f2(pq, r, pack_f2(0.69326097f, 0.69326097f));
            pq = fma_f2(pq, r, pack_f2(0.99992812f, 0.99992812f));
            float q0, q1, m0f, m1f;
            unpack_f2(pq, q0, q1);
            unpack_f2(tm, m0f, m1f);
            p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(m0f) << 23));
            p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(m1f) << 23));
          } else {
            float a, b;
            unpack_f2(t2, a, b);
            p0 = fast_exp2(a);
            p1 = fast_exp2(b);
          }
          rs = add_f2(rs, pack_f2(p0, p1));
          return ElemTraits<T>::pack2(p0, p1);
        };
        // pass 2, 64 columns at a time: exponentials, row sums, P as packed 16-bit in the 16x128b layout (the pair of
        // columns 8 i + 2 q + {0, 1} of a half is packed column 4 i + q).  Each half of P goes over the first 32
        // columns of its own half of S (kPHalfStride apart), so the upper half, still in registers, is done first
        // and only the lower half is read from tensor memory a second time.
        auto exp_half = [&](const uint32_t (&v)[32], uint32_t dst) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool emu = (i & 3) < kExpEmuOf4;
            pk[2 * i] = exp_pair(v[4 * i], v[4 * i + 1], nega_2, rs_a, emu);
            pk[2 * i + 1] = exp_pair(v[4 * i + 2], v[4 * i + 3], negb_2, rs_b, emu);
          }
          tmem_st_16x128b_x8(dst, pk);
        };
        exp_half(v_hi, tS + ptx::kPHalfStride);
        {
          uint32_t v[32];
          tmem_ld_16x256b_x8(tS, v);
          tmem_wait_ld();
          exp_half(v, tS);
        }
        {
          float r0, r1;
          unpack_f2(rs_a, r0, r1);
          l_a += r0 + r1;
          unpack_f2(rs_b, r0, r1);
          l_b += r0 + r1;
        }
        tmem_wait_st();
        if (pend) {
          // first tile of an item: the previous item's O must leave tensor memory before this tile's PV
          ok = flush(true);
          if (!ok) break;
        } else {
          tc_fence_before();
          mbar_arrive(smem_u32(&ctrl->p_ready[s]));
        }
      }
      if (!ok) break;
      // ---------------- the item's epilogue becomes pending ----------------
      const int len_q = w.len_q;
      const bool slot_live = w.valid && m0s < len_q;
      const long long qrow0 = w.out_row0[s];
      const int qhead = w.q_head[s];
      pend = true;
      pend_acc = n > 0;
      pend_phase = (tile_cnt - 1) & 1;
      pend_rows = slot_live ? min(kBM, len_q - m0s) : 0;
      pend_la = quad_sum(l_a);
      pend_lb = quad_sum(l_b);
      if (p.lse != nullptr && q == 0) {
        // split KV range: the merge needs every row's log-sum-exp (log2 domain; -inf for a row that saw no key)
        float* lse = p.lse + qrow0 + m0s + rowA;
        if (rowA < (slot_live ? min(kBM, len_q - m0s) : 0)) lse[0] = pend_la > 0.f ? m_a + log2f(pend_la) : -INFINITY;
        if (rowA + 8 < (slot_live ? min(kBM, len_q - m0s) : 0)) lse[8] = pend_lb > 0.f ? m_b + log2f(pend_lb) : -INFINITY;
      }
      if (p.layout == B200ATTN_RAGGED) {
        pend_stride = static_cast<long long>(p.q_heads) * D;
        pend_off = ((qrow0 + m0s + rowA) * p.q_heads + qhead) * D;
      } else {
        pend_stride = D;
        pend_off = (qrow0 + m0s + rowA) * D;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[k & 1]));
    }
    if (ok && pend) ok = flush(false);
    if (!ok && lane == 0) { p.header[0] = DEV_ERR_WAIT_EXPIRED; *abort_flag = 1; }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

namespace {

// Merge of the parts of a split KV range.  part[(b * parts + s)][h][r][:] holds the normalised output of part s and
// lse[...] its log-sum-exp (log2 domain): out = sum_s 2^(lse_s - max) part_s / sum_s 2^(lse_s - max)
// (the reference's merge kernel, kernels/attention.py:659-746, on normalised instead of raw accumulators).
template <typename OutT, int D>
__global__ void __launch_bounds__(256) prefill_merge_kernel(const OutT* __restrict__ part, const float* __restrict__ lse,
                                                            OutT* __restrict__ out, long long rows_per_batch, int batch,
                                                            int parts) {
  constexpr int VEC = 16 / sizeof(OutT);          // elements per 16-byte piece
  constexpr int PIECES = D / VEC;
  const long long total = static_cast<long long>(batch) * rows_per_batch * PIECES;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int piece = static_cast<int>(idx % PIECES);
    const long long row = idx / PIECES;                    // (b, h, r) flattened
    const long long b = row / rows_per_batch, hr = row - b * rows_per_batch;
    float mx = -INFINITY;
    for (int sp = 0; sp < parts; ++sp) mx = fmaxf(mx, __ldg(lse + (b * parts + sp) * rows_per_batch + hr));
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    float wsum = 0.f;
    for (int sp = 0; sp < parts; ++sp) {
      const long long prow = (b * parts + sp) * rows_per_batch + hr;
      const float l = __ldg(lse + prow);
      const float w = (l == -INFINITY) ? 0.f : fast_exp2(l - mx);
      wsum += w;
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(part + prow * D) + piece);
      const OutT* e = reinterpret_cast<const OutT*>(&u);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += w * ElemTraits<OutT>::to_float(e[i]);
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    uint4 o;
    OutT* oe = reinterpret_cast<OutT*>(&o);
#pragma unroll
    for (int i = 0; i < VEC; ++i) oe[i] = ElemTraits<OutT>::from_float(acc[i] * inv);
    reinterpret_cast<uint4*>(out + row * D)[piece] = o;
  }
}

// How a launch with few work items cuts every sequence's KV range, so that more SMs than there are (query tile, head
// pair, sequence) items have work: the reference splits KV when B x QH < SMs (kernels/attention.py:836-841).  Dense and
// paged layouts only: a ragged problem's lengths are not known on the host.
struct SplitPlan {
  int parts;        // 1: no split
  int part_len;     // keys per part, a multiple of 128
};
SplitPlan split_plan(const b200attn_prefill_args_t& a, int sm_count) {
  SplitPlan sp{1, 0};
  if (a.layout == B200ATTN_RAGGED || a.batch <= 0 || a.max_q <= 0 || sm_count <= 0) return sp;
  const int group = a.q_heads / a.kv_heads;
  const bool head_pair = group % 2 == 0;
  const int item_rows = head_pair ? kBM : 2 * kBM;
  const long long head_units = head_pair ? a.q_heads / 2 : a.q_heads;
  const long long nblocks = (a.max_q + item_rows - 1) / item_rows;
  const long long items = nblocks * head_units * a.batch;
  const long long kv_cap = a.layout == B200ATTN_DENSE ? a.max_kv : a.table_stride * static_cast<long long>(a.page_size);
  const long long tiles = (kv_cap + kBN - 1) / kBN;            // longest item, in 128-key steps
  if (items <= 0 || tiles < 8) return sp;
  // steps of all items: under a causal mask row block r stops at its diagonal
  long long total = 0;
  for (long long r = 0; r < nblocks; ++r) {
    const long long reach = a.is_causal ? std::min<long long>(tiles, ((r + 1) * item_rows + kBN - 1) / kBN) : tiles;
    total += reach;
  }
  total *= head_units * a.batch;
  // Estimated duration in units of one 128-key step of both slots: the longest item or the average load of an SM,
  // whichever is larger, with about two steps of fixed cost per item (pipeline fill, masked tile, epilogue) and two
  // more for the merge launch.  Measured anchors on B200: B = 16, 8/2 heads, 128 x 2 048 cross attention (64 items)
  // 45 -> 36 us in two parts; a 512-key range in two parts is slower than unsplit (hence four tiles per part at least).
  auto cost = [&](long long parts) -> double {
    const double longest = static_cast<double>((tiles + parts - 1) / parts) + 2.0;
    const double load = (static_cast<double>(total) + 2.0 * static_cast<double>(items * parts)) / sm_count;
    return std::max(longest, load) + (parts > 1 ? 2.0 : 0.0);
  };
  long long best = 1;
  double best_cost = cost(1);
  for (long long parts = 2; parts <= 8 && tiles / parts >= 4; parts *= 2) {
    const double c = cost(parts);
    if (c < 0.85 * cost(1) && c < best_cost) { best = parts; best_cost = c; }
  }
  if (best < 2) return sp;
  const long long per = (tiles + best - 1) / best;
  sp.part_len = static_cast<int>(per * kBN);
  sp.parts = static_cast<int>((tiles + per - 1) / per);
  if (sp.parts < 2) sp.parts = 1;
  return sp;
}

struct CastPlan {
  size_t q_elems, kv_elems, q_off, k_off, v_off, total;
};
CastPlan cast_plan(const b200attn_prefill_args_t& a) {
  CastPlan c{};
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  const size_t D = static_cast<size_t>(a.head_dim);
  if (a.layout == B200ATTN_RAGGED) {
    c.q_elems = static_cast<size_t>(a.total_q) * a.q_heads * D;
    c.kv_elems = static_cast<size_t>(a.total_kv) * a.kv_heads * D;
  } else {
    c.q_elems = static_cast<size_t>(a.batch) * a.q_heads * a.max_q * D;
    c.kv_elems = a.layout == B200ATTN_DENSE ? static_cast<size_t>(a.batch) * a.kv_heads * a.max_kv * D
                                            : static_cast<size_t>(a.total_kv) * a.kv_heads * D;
  }
  c.q_off = kHeaderBytes;
  c.k_off = up(c.q_off + c.q_elems * 2);
  c.v_off = up(c.k_off + c.kv_elems * 2);
  c.total = up(c.v_off + c.kv_elems * 2);
  return c;
}
}  // namespace

namespace {
// workspace: header | fp32 inputs rounded to fp16 (fp32 calls) | parts of a split KV range and their log-sum-exps
struct WsPlan {
  size_t part_off, lse_off, total;
  SplitPlan split;
};
WsPlan ws_plan(const b200attn_prefill_args_t& a, int sm_count) {
  WsPlan w{};
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  size_t off = a.dtype == B200ATTN_F32 ? cast_plan(a).total : static_cast<size_t>(kHeaderBytes);
  w.split = split_plan(a, sm_count);
  if (w.split.parts > 1) {
    const size_t rows = static_cast<size_t>(a.batch) * w.split.parts * a.q_heads * a.max_q;
    const size_t esz = a.dtype == B200ATTN_F32 ? 4 : 2;
    w.part_off = off; off = up(off + rows * a.head_dim * esz);
    w.lse_off = off;  off = up(off + rows * sizeof(float));
  }
  w.total = off;
  return w;
}
}  // namespace

size_t prefill_workspace_bytes(const b200attn_prefill_args_t& a, int sm_count) { return ws_plan(a, sm_count).total; }

int launch_prefill(const b200attn_prefill_args_t& a_in, int sm_count, cudaStream_t stream) {
  const WsPlan wsp = ws_plan(a_in, sm_count);
  const size_t need = wsp.total;
  if (a_in.workspace == nullptr || a_in.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a_in.workspace) & 255)) {
    set_error("prefill: workspace needs %zu bytes, 256-byte aligned (got %zu)", need, a_in.workspace_bytes);
    return B200ATTN_E_WORKSPACE;
  }
  b200attn_prefill_args_t a = a_in;
  const bool f32 = a_in.dtype == B200ATTN_F32;
  if (f32) {
    const CastPlan c = cast_plan(a_in);
    unsigned char* ws = static_cast<unsigned char*>(a_in.workspace);
    const void* src[3] = {a_in.q, a_in.k, a_in.v};
    const size_t off[3] = {c.q_off, c.k_off, c.v_off};
    const size_t cnt[3] = {c.q_elems, c.kv_elems, c.kv_elems};
    for (int i = 0; i < 3; ++i) {
      const long long n4 = static_cast<long long>(cnt[i] / 4);  // head_dim is a multiple of 4
      if (n4 == 0) continue;
      const int blocks = static_cast<int>(std::min<long long>((n4 + 255) / 256, static_cast<long long>(sm_count) * 16));
      cast_f32_to_f16_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float4*>(src[i]),
                                                         reinterpret_cast<uint2*>(ws + off[i]), n4);
    }
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) return cuda_fail(ce, "cast kernel launch");
    a.q = ws + c.q_off; a.k = ws + c.k_off; a.v = ws + c.v_off;
    a.dtype = B200ATTN_F16;
  }
  const int D = a.head_dim;
  PrefillParams p;
  p.out = a.out; p.q_indptr = a.q_indptr; p.kv_indptr = a.kv_indptr;
  p.k_table = a.k_table; p.v_table = a.v_table;
  p.header = static_cast<int*>(a.workspace);
  p.work_counter = p.header + 8;
  p.table_stride = a.table_stride;
  p.layout = a.layout; p.indptr_is_i64 = a.indptr_is_i64;
  p.batch = a.batch; p.q_heads = a.q_heads; p.kv_heads = a.kv_heads; p.group = a.q_heads / a.kv_heads;
  p.max_q = a.max_q; p.max_kv = a.max_kv;
  p.page_size = a.layout == B200ATTN_PAGED ? a.page_size : 1;
  p.box_rows = kBN;
  p.num_pages = 0;
  p.is_causal = a.is_causal ? 1 : 0;
  p.head_pair = (p.group % 2 == 0) ? 1 : 0;
  p.out_align32 = (reinterpret_cast<uintptr_t>(a.out) & 31) == 0 ? 1 : 0;
  const int item_rows = p.head_pair ? kBM : 2 * kBM;
  const int head_units = p.head_pair ? a.q_heads / 2 : a.q_heads;
  p.scale_log2 = a.sm_scale * 1.4426950408889634f;
  p.kv_split = wsp.split.parts;
  p.kv_split_len = wsp.split.part_len;
  p.lse = nullptr;
  if (p.kv_split > 1) {
    // the kernel writes every part's normalised output and log-sum-exp into the workspace; a merge kernel follows
    unsigned char* ws = static_cast<unsigned char*>(a_in.workspace);
    p.out = ws + wsp.part_off;
    p.lse = reinterpret_cast<float*>(ws + wsp.lse_off);
    p.out_align32 = 1;
  }

  CUtensorMap tq, tk, tv;
  int rc;
  dim3 grid;
  long long total_items = 0;
  if (a.layout == B200ATTN_RAGGED) {
    if ((rc = make_token_map(&tq, a.dtype, a.q, a.total_q, a.q_heads, D, kBM))) return rc;
    if ((rc = make_token_map(&tk, a.dtype, a.k, a.total_kv, a.kv_heads, D, kBN))) return rc;
    if ((rc = make_token_map(&tv, a.dtype, a.v, a.total_kv, a.kv_heads, D, kBN))) return rc;
    const long long pairs = a.total_q / item_rows + a.batch;
    total_items = pairs * head_units;
  } else {
    const long long q_rows = static_cast<long long>(a.batch) * a.q_heads * a.max_q;
    if ((rc = make_token_map(&tq, a.dtype, a.q, q_rows, 1, D, kBM))) return rc;
    if (a.layout == B200ATTN_DENSE) {
      const long long kv_rows = static_cast<long long>(a.batch) * a.kv_heads * a.max_kv;
      if ((rc = make_token_map(&tk, a.dtype, a.k, kv_rows, 1, D, kBN))) return rc;
      if ((rc = make_token_map(&tv, a.dtype, a.v, kv_rows, 1, D, kBN))) return rc;
    } else {
      // largest power of two that divides the page size, capped at the tile: every box stays inside one page
      int box = 1;
      while (box < kBN && (a.page_size % (box * 2)) == 0) box *= 2;
      p.box_rows = box;
      p.num_pages = static_cast<int>(std::min<long long>(a.total_kv / a.page_size, 0x7fffffff));
      if ((rc = make_token_map(&tk, a.dtype, a.k, a.total_kv, a.kv_heads, D, box))) return rc;
      if ((rc = make_token_map(&tv, a.dtype, a.v, a.total_kv, a.kv_heads, D, box))) return rc;
    }
    total_items = static_cast<long long>((a.max_q + item_rows - 1) / item_rows) * head_units * a.batch * p.kv_split;
  }
  if (total_items <= 0) return B200ATTN_OK;
  if (total_items > 0x7fffffff) { set_error("prefill: too many work items"); return B200ATTN_E_UNSUPPORTED; }
  p.total_items = static_cast<int>(total_items);
  grid = dim3(static_cast<unsigned>(std::min<long long>(total_items, sm_count)), 1, 1);
  // The two counters in the header (next item, CTAs finished) are zero here: the workspace starts zeroed and
  // the last CTA of every launch puts them back.

  cudaError_t e;
#define B200ATTN_LAUNCH_PREFILL(TYPE, DIM, OUT)                                                          \
  do {                                                                                                   \
    const size_t smem = std::max<size_t>(SmemPlan<DIM>::kTotal + 1024, 120 * 1024);                      \
    if (a.layout == B200ATTN_PAGED) {                                                                    \
      if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(prefill_kernel<TYPE, DIM, OUT, true>), smem))) return rc; \
      prefill_kernel<TYPE, DIM, OUT, true><<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);             \
    } else {                                                                                             \
      if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(prefill_kernel<TYPE, DIM, OUT, false>), smem))) return rc; \
      prefill_kernel<TYPE, DIM, OUT, false><<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);            \
    }                                                                                                    \
  } while (0)
  if (f32) {
    if (D == 128) B200ATTN_LAUNCH_PREFILL(__half, 128, float); else B200ATTN_LAUNCH_PREFILL(__half, 64, float);
  } else if (a.dtype == B200ATTN_BF16) {
    if (D == 128) B200ATTN_LAUNCH_PREFILL(__nv_bfloat16, 128, __nv_bfloat16); else B200ATTN_LAUNCH_PREFILL(__nv_bfloat16, 64, __nv_bfloat16);
  } else {
    if (D == 128) B200ATTN_LAUNCH_PREFILL(__half, 128, __half); else B200ATTN_LAUNCH_PREFILL(__half, 64, __half);
  }
#undef B200ATTN_LAUNCH_PREFILL
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "prefill kernel launch");
  if (p.kv_split > 1) {
    const long long rows_per_batch = static_cast<long long>(a.q_heads) * a.max_q;
    const long long pieces = static_cast<long long>(a.batch) * rows_per_batch * (D / (f32 ? 4 : 8));
    const int blocks = static_cast<int>(std::min<long long>((pieces + 255) / 256, static_cast<long long>(sm_count) * 8));
#define B200ATTN_LAUNCH_MERGE(OUT, DIM)                                                                              \
    prefill_merge_kernel<OUT, DIM><<<blocks, 256, 0, stream>>>(static_cast<const OUT*>(p.out), p.lse,                 \
                                                               static_cast<OUT*>(a_in.out), rows_per_batch, a.batch, p.kv_split)
    if (f32) { if (D == 128) B200ATTN_LAUNCH_MERGE(float, 128); else B200ATTN_LAUNCH_MERGE(float, 64); }
    else if (a.dtype == B200ATTN_BF16) { if (D == 128) B200ATTN_LAUNCH_MERGE(__nv_bfloat16, 128); else B200ATTN_LAUNCH_MERGE(__nv_bfloat16, 64); }
    else { if (D == 128) B200ATTN_LAUNCH_MERGE(__half, 128); else B200ATTN_LAUNCH_MERGE(__half, 64); }
#undef B200ATTN_LAUNCH_MERGE
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "prefill merge kernel launch");
  }
  return B200ATTN_OK;
}

}  // namespace b200attn
