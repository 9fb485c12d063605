/*
 * b200attn — C ABI of the B200 (sm_100a) attention hot path.
 *
 * Plain pointers and sizes only; no torch types.  Every entry point is
 * asynchronous on the stream it is given, never synchronises the device,
 * never allocates or frees device memory, and returns 0 on success or a
 * negative B200ATTN_E_* code (text via b200attn_last_error()).
 *
 * The functions replace the Triton launches behind these reference entry
 * points (paths are relative to the reference project):
 *
 *   b200attn_prefill  <- kernels/attention.py:749-927  flash_attention_v2
 *                        (partial kernel :430-656 + merge kernel :659-746),
 *                        and flash_attention_v1 :249-364 (same semantics)
 *   b200attn_decode   <- kernels/decode.py:203-331  decode_attention
 *                        (split kernel :22-168 + merge :171-200) and
 *                        kernels/speculative_decode.py:228-366
 *                        speculative_decode_attention (split :22-186 +
 *                        merge :189-226); decode is the M == 1 case
 *   b200attn_*_workspace_bytes <- the torch.empty fp32 workspaces at
 *                        kernels/attention.py:852-864, kernels/decode.py:280-292,
 *                        kernels/speculative_decode.py:311-323
 *   b200attn_softmax  <- kernels/softmax.py:152-236 softmax, :378-462 log_softmax
 *   b200attn_device_info <- torch.cuda.get_device_properties(...).multi_processor_count
 *                        at kernels/attention.py:836, kernels/decode.py:273
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_ABI_VERSION 1

/* element type of q/k/v/out */
enum { B200ATTN_F16 = 0, B200ATTN_BF16 = 1, B200ATTN_F32 = 2 };
/* K/V layout (reference "TYPE" 0/1/2: kernels/attention.py:785,810,832) */
enum { B200ATTN_DENSE = 0, B200ATTN_RAGGED = 1, B200ATTN_PAGED = 2 };

/* status codes */
enum {
  B200ATTN_OK = 0,
  B200ATTN_E_INVALID = -1,      /* bad argument (null pointer, bad shape, misalignment) */
  B200ATTN_E_UNSUPPORTED = -2,  /* head_dim / dtype / page size outside the built kernels */
  B200ATTN_E_ARCH = -3,         /* device is not compute capability 10.x */
  B200ATTN_E_WORKSPACE = -4,    /* workspace too small or misaligned */
  B200ATTN_E_CUDA = -5,         /* CUDA runtime / driver call failed */
  B200ATTN_E_DEVICE = -6        /* a kernel reported a bounded-wait expiry or bounds violation */
};

typedef struct b200attn_device_info_t {
  int32_t sm_count;
  int32_t cc_major;
  int32_t cc_minor;
  int32_t max_smem_optin;  /* bytes */
} b200attn_device_info_t;

/*
 * Prefill (many query rows per sequence).
 *
 *  DENSE : q [B,QH,M,D]  k,v [B,KVH,N,D]                       out [B,QH,M,D]
 *  RAGGED: q [total_q,QH,D]  k,v [total_kv,KVH,D]  q_indptr,kv_indptr [B+1] prefix sums
 *          out [total_q,QH,D]
 *  PAGED : q [B,QH,M,D]  k,v cache [cache_tokens,KVH,D]  kv_indptr [B] = lengths,
 *          k_table,v_table [B,table_stride] int32 physical page numbers
 *
 * All tensors contiguous, 16-byte aligned.  Causal masking is top-left aligned
 * on per-sequence indices (key j visible to query i iff j <= i).  scale = sm_scale.
 */
typedef struct b200attn_prefill_args_t {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const void* q_indptr;   /* RAGGED only */
  const void* kv_indptr;  /* RAGGED: prefix sums [B+1]; PAGED: lengths [B] */
  const int32_t* k_table; /* PAGED only */
  const int32_t* v_table; /* PAGED only */
  void* workspace;        /* >= b200attn_prefill_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  int64_t total_q;        /* RAGGED: rows of q */
  int64_t total_kv;       /* RAGGED: rows of k/v; PAGED: rows of the cache */
  int64_t table_stride;   /* PAGED: entries per table row */
  int32_t dtype;
  int32_t layout;
  int32_t indptr_is_i64;  /* width of q_indptr / kv_indptr entries */
  int32_t batch;
  int32_t q_heads;
  int32_t kv_heads;
  int32_t max_q;          /* DENSE/PAGED: M */
  int32_t max_kv;         /* DENSE: N */
  int32_t head_dim;       /* 64 or 128 */
  int32_t page_size;      /* PAGED */
  int32_t is_causal;
  int32_t device;         /* CUDA ordinal that owns the pointers */
  float sm_scale;
} b200attn_prefill_args_t;

/*
 * Decode / speculative decode (q_len = M <= 16 query tokens per sequence).
 *
 *  q, out [B,QH,M,D] (decode_attention's [B,QH,D] is M == 1)
 *  DENSE : k,v [B,KVH,N,D]
 *  RAGGED: k,v [total_kv,KVH,D], kv_indptr [B+1] prefix sums
 *  PAGED : k,v cache [cache_tokens,KVH,D], kv_indptr [B] lengths, tables as above
 *
 * causal_drafts != 0: the last M keys of each sequence are the draft tokens'
 * own keys and draft row i does not see draft keys i+1..M-1.
 *
 * Arithmetic: 16-bit inputs are multiplied on the tensor cores with fp32
 * accumulation.  fp32 inputs with M == 1 (and at most 16 q rows per KV head)
 * are multiplied in fp32 FMAs, as the reference's decode kernel does
 * (kernels/decode.py:146-160); fp32 inputs with M > 1 are rounded to fp16
 * copies in the workspace and multiplied on the tensor cores - the ten
 * mantissa bits of the TF32 tl.dot the reference's speculative-decode kernel
 * runs on fp32 operands (kernels/speculative_decode.py:153,175), but fp16's
 * range: magnitudes beyond 65504 become infinite.  The workspace holds those
 * copies (2 bytes per element of q, k and v as passed: a paged cache is copied
 * whole; when k and v together would need more than 8 GiB of copies the call
 * keeps fp32 FMAs instead).  b200attn_decode_static has no room for them and
 * keeps fp32 FMAs.
 */
typedef struct b200attn_decode_args_t {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const void* kv_indptr;
  const int32_t* k_table;
  const int32_t* v_table;
  void* workspace;        /* >= b200attn_decode_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  int64_t total_kv;       /* RAGGED: rows of k/v; PAGED: rows of the cache */
  int64_t table_stride;
  int32_t dtype;
  int32_t layout;
  int32_t indptr_is_i64;
  int32_t batch;
  int32_t q_heads;
  int32_t kv_heads;
  int32_t q_len;          /* M, 1..16 */
  int32_t max_kv;         /* DENSE: N; PAGED: table_stride * page_size */
  int32_t head_dim;
  int32_t page_size;
  int32_t causal_drafts;
  int32_t device;
  float sm_scale;
} b200attn_decode_args_t;

int b200attn_abi_version(void);
const char* b200attn_last_error(void);
int b200attn_device_info(int device, b200attn_device_info_t* info);

/*
 * Workspace rules (all entry points): the caller zero-fills the workspace once after allocating it and then
 * leaves its first 256 bytes (error word, scheduling counters that every launch returns to zero) alone; one
 * workspace serves one stream at a time.
 */
size_t b200attn_prefill_workspace_bytes(const b200attn_prefill_args_t* args);
size_t b200attn_decode_workspace_bytes(const b200attn_decode_args_t* args);

int b200attn_prefill(const b200attn_prefill_args_t* args, void* cuda_stream);
int b200attn_decode(const b200attn_decode_args_t* args, void* cuda_stream);

/*
 * Decode / speculative decode for callers that cannot hand over device memory for scratch and
 * must not trigger an allocation: a server that gave all of its HBM to the KV cache at start-up,
 * a plug-in living inside another framework's memory pool, code that runs while that framework
 * has frozen its allocator.  Same arguments, kernels and results as b200attn_decode, except that
 * `workspace` / `workspace_bytes` are ignored: the planner tables, merge tickets and split-KV
 * partials live in an 8 MiB array built into the library (each GPU that loads the library holds
 * those 8 MiB until the process exits).  Calls cudaMalloc / cudaFree or any allocating routine: never.
 *
 *  - Problems whose scratch need (b200attn_decode_workspace_bytes) exceeds 8 MiB are refused with
 *    B200ATTN_E_WORKSPACE; use b200attn_decode for those.
 *  - The first call on each device loads the library's device code on that GPU (which is what reserves
 *    the 8 MiB there) and looks up the array's device address; it takes device memory and it may fail
 *    once a framework has frozen its allocator or is capturing a stream.  Make that first call at
 *    start-up, before any stream capture; b200attn_decode_static_check on the device does the same
 *    set-up and is a convenient way to pay for it early.  Later calls allocate nothing.
 *  - All calls on a device share the one array.  Calls must not overlap on the GPU (two streams,
 *    two threads): they would overwrite each other's partials.  Back-to-back calls on one stream
 *    are fine; nothing needs clearing in between.
 *  - Device-side error codes (1 bounded wait expired, 2 block-table entry out of range, 3 planner
 *    overflow) land in word 0 of the array, where the caller cannot see them: read them with
 *    b200attn_decode_static_check.  The word is sticky until that call clears it.  A CTA whose
 *    wait expired writes NaN rows, so the failure also shows in the output; out-of-range block-table
 *    entries are skipped, never dereferenced.
 *
 * This function has no counterpart in the reference.
 */
int b200attn_decode_static(const b200attn_decode_args_t* args, void* cuda_stream);

/*
 * Reads and clears the device error word of b200attn_decode_static's built-in array on `device`
 * (one 4-byte copy on `cuda_stream`, which it synchronises; allocates nothing).  Returns 0, or
 * B200ATTN_E_DEVICE with the code in *code.  No counterpart in the reference.
 */
int b200attn_decode_static_check(int device, void* cuda_stream, int32_t* code);

/*
 * Self-test of the bounded waits: launches one warp that waits on a barrier nothing completes, with the
 * kernels' own wait loop limited to `tries` attempts (1..2^20; the kernels use 2^22), so that it gives up
 * after a fraction of a second, records code 1 in word 0 of `workspace` (>= 256 bytes, zeroed) and
 * returns.  b200attn_check_workspace then reports B200ATTN_E_DEVICE / code 1 and the context stays
 * usable.  No counterpart in the reference.
 */
int b200attn_selftest_wait_expiry(int device, void* workspace, uint32_t tries, void* cuda_stream);

/*
 * Paged KV-cache append: copies the new rows of every sequence into the pages its block table names.
 *   src        [total_rows, heads, head_dim]  new K (or V) rows of all sequences, packed
 *   src_indptr [B+1] prefix sums over src rows;  dst_pos [B] position in each sequence of its first new row
 *              (NULL = 0: build the cache from scratch); both share the width given by indptr_is_i64
 *   cache      [cache_rows, heads, head_dim], cache_rows = pages * page_size;  table [B, table_stride] int32
 * Row r of sequence b lands in cache row table[b][(dst_pos[b]+r) / page_size] * page_size + (dst_pos[b]+r) % page_size.
 * row_bytes = heads * head_dim * element size must be a multiple of 16; src and cache 16-byte aligned.
 * Table entries outside the cache are reported through the workspace error word and skipped.
 * Replaces the Python scatter loops of the reference's fixtures (tests/test_attention.py:101-134,
 * tests/test_decode.py:93-130, benchmarks/attention.py:351-431).
 */
typedef struct b200attn_paged_append_args_t {
  const void* src;
  void* cache;
  const void* src_indptr;
  const void* dst_pos;
  const int32_t* table;
  void* workspace;        /* >= 256 bytes, 256-byte aligned; word 0 is the device error code */
  size_t workspace_bytes;
  int64_t total_rows;
  int64_t cache_rows;
  int64_t table_stride;
  int32_t row_bytes;
  int32_t indptr_is_i64;
  int32_t batch;
  int32_t page_size;
  int32_t device;
} b200attn_paged_append_args_t;

int b200attn_paged_append(const b200attn_paged_append_args_t* args, void* cuda_stream);

/*
 * Softmax or log-softmax over the last dimension of a contiguous [rows, cols] tensor (any leading shape flattened
 * into rows), fp32 arithmetic, same dtype out.  `out` may be `x` (in place).  No workspace.
 * Replaces kernels/softmax.py:152-236 `softmax` (small :18-32, medium :35-66, partial / merge / finalize :69-150)
 * and :378-462 `log_softmax` (:239-375).
 */
typedef struct b200attn_softmax_args_t {
  const void* x;
  void* out;
  int64_t rows;
  int64_t cols;
  int32_t dtype;          /* B200ATTN_F16 / BF16 / F32 */
  int32_t log_softmax;    /* 0: softmax, 1: log-softmax */
  int32_t device;
} b200attn_softmax_args_t;

int b200attn_softmax(const b200attn_softmax_args_t* args, void* cuda_stream);

/*
 * Reads the error word a kernel of an earlier call may have set in `workspace` (bounded wait expired,
 * page index out of range, planner overflow).  Synchronises `cuda_stream`.  Returns 0, or
 * B200ATTN_E_DEVICE with the code in *code; in that case the 256-byte header is zeroed again, so that
 * the workspace can be used for the next call.
 */
int b200attn_check_workspace(void* workspace, void* cuda_stream, int32_t* code);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
