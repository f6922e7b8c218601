/*
 * pthb200_attn.h - C ABI of libpthb200_attn.so, the sm_100a (B200) implementation of
 * paged int8_per_token_head attention forward.
 *
 * This is the drop-in boundary: a plain-C interface (pointers, sizes, byte
 * strides; no torch types) that an engine binds through ctypes / cffi / dlsym.
 * The two launch structs are binary-compatible with the structs the reference
 * project passes to its own launcher, so a caller that fills the reference's
 * structs can call this library unchanged:
 *
 *   PthAttnArgs / PthAttnStream / PthAttnCombineArgs
 *       replace  csrc/pth_attn/attn_args.h:65-171  (same field order and types,
 *       ABI version 2; ctypes mirror python/pth_testing/ref_capi.py:38-119).
 *   pthb200_attention / pthb200_combine / pthb200_last_error
 *       replace  launch_attention / launch_combine / last_launch_error
 *       (csrc/pth_attn/attn_launch.h:46-52) and their C wrappers
 *       pth_attn_attention / pth_attn_combine / pth_attn_last_error
 *       (csrc/pth_attn/attn_capi.h:98-103).
 *   pthb200_abi_version / *_bytes getters
 *       replace  pth_attn_abi_version etc. (csrc/pth_attn/attn_capi.h:80-87).
 *   pthb200_attention_ex + PthB200Options
 *       replaces pth_attn_attention_ex + PthAttnOptions (attn_capi.h:32-39,
 *       100-101); the option block additionally carries the final
 *       log-sum-exp output this implementation can produce.
 *   pthb200_check_call
 *       replaces the host-side argument checks of the op
 *       (csrc/pth_attn/launch.cu:315-346,380-399): tile height from (wm, G,
 *       max_query_len) and alignment rules, without touching a device.
 *
 * Units: every stride is in BYTES except block_table_row_stride (int32
 * ELEMENTS).  All pointers are device pointers.  No entry point allocates
 * device memory, copies to the host or synchronises; a launch only enqueues
 * kernels on `stream`, so it can be captured in a CUDA graph.
 *
 * Semantics (identical to the reference, attn_args.h:20-51): query token i of
 * request r (q_len = qsl[r+1]-qsl[r], L = seq_lens[r], both read on the device)
 * sits at KV position p = L - q_len + i and sees keys [lo, hi] with
 *   lo = window > 0 ? max(0, p - window + 1) : 0
 *   hi = causal ? p : (window > 0 ? min(L-1, p + window - 1) : L-1).
 * Query head h reads KV head h / (num_q_heads / num_kv_heads).  The result is
 * softmax(softmax_scale * q . k_scale*k) applied to v_scale*v.
 *   num_splits == 1: out[token, head, :] is written (out_dtype).
 *   num_splits  > 1: ws_o[s, token, head, :] (fp32, the split's own normalised
 *       output) and ws_lse[s, token, head] (log2-sum-exp of the split's scaled
 *       scores; -inf for a split without keys, whose ws_o must not be read)
 *       are written for every s < num_splits; `out` is written by the combine.
 * Rows >= qsl[num_reqs] are never written.  How the keys of a row are divided
 * among the splits is this library's choice (any disjoint cover is valid input
 * to the combine).
 */
#ifndef PTHB200_ATTN_H_
#define PTHB200_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTH_ATTN_ABI_VERSION 2

/* q / out element types. */
enum { PTH_ATTN_F32 = 0, PTH_ATTN_F16 = 1, PTH_ATTN_BF16 = 2 };

/* Return codes. */
enum {
  PTH_ATTN_OK = 0,
  PTH_ATTN_EINVAL = -1,  /* an argument check failed; see pthb200_last_error() */
  PTH_ATTN_ECUDA = -2,   /* a CUDA runtime call or the launch failed */
  PTH_ATTN_ENOCUDA = -3  /* kept for code compatibility; never returned here */
};

/* A cache stream: logical [num_blocks, block_size, num_kv_heads, row], row
 * contiguous (head_size int8 for K/V, one fp32 for a scale). */
typedef struct PthAttnStream {
  const void* data;
  int64_t stride_block;
  int64_t stride_slot;
  int64_t stride_head;
} PthAttnStream;

typedef struct PthAttnArgs {
  int32_t abi_version;  /* PTH_ATTN_ABI_VERSION */
  int32_t struct_bytes; /* sizeof(PthAttnArgs) of the caller */

  const void* q; /* [num_tokens, num_q_heads, head_size] */
  int32_t q_dtype;
  int64_t q_stride_token;
  int64_t q_stride_head;

  void* out; /* [num_tokens, num_q_heads, head_size]; num_splits == 1 */
  int32_t out_dtype;
  int64_t out_stride_token;
  int64_t out_stride_head;

  PthAttnStream k_cache;
  PthAttnStream v_cache;
  PthAttnStream k_scale;
  PthAttnStream v_scale;
  int32_t num_blocks;
  int32_t block_size;
  int32_t num_kv_heads;
  int32_t head_size; /* 64, 128 or 256 */

  const int32_t* block_table; /* [>= num_reqs, *] physical block ids */
  int64_t block_table_row_stride;
  const int32_t* seq_lens;        /* [num_reqs] */
  const int32_t* query_start_loc; /* [num_reqs + 1] */

  int32_t num_reqs;
  int32_t num_tokens;
  int32_t num_q_heads;
  int32_t bq;          /* query tokens per row tile, >= 1 */
  int32_t num_q_tiles; /* 0 = num_tokens / bq + num_reqs */
  int32_t num_splits;
  float softmax_scale;

  float* ws_o; /* [>= num_splits, >= num_tokens, num_q_heads, head_size] */
  int64_t ws_o_stride_split;
  int64_t ws_o_stride_token;
  int64_t ws_o_stride_head;
  float* ws_lse; /* [>= num_splits, >= num_tokens, num_q_heads] */
  int64_t ws_lse_stride_split;
  int64_t ws_lse_stride_token;
  int64_t ws_lse_stride_head;

  int32_t window; /* 0 = none */
  int32_t causal; /* 1 = bottom-right causal, 0 = non-causal */
} PthAttnArgs;

typedef struct PthAttnCombineArgs {
  int32_t abi_version;
  int32_t struct_bytes;

  const float* ws_o;
  int64_t ws_o_stride_split;
  int64_t ws_o_stride_token;
  int64_t ws_o_stride_head;
  const float* ws_lse;
  int64_t ws_lse_stride_split;
  int64_t ws_lse_stride_token;
  int64_t ws_lse_stride_head;

  void* out;
  int32_t out_dtype;
  int64_t out_stride_token;
  int64_t out_stride_head;

  const int32_t* query_start_loc;
  int32_t num_reqs;
  int32_t num_tokens;
  int32_t num_q_heads;
  int32_t head_size;
  int32_t num_splits;
} PthAttnCombineArgs;

/* Kernel family of pthb200_attention_ex. */
enum {
  PTHB200_KERNEL_AUTO = 0,   /* the shipped choice */
  PTHB200_KERNEL_SCALAR = 1, /* CUDA-core kernel: every head size, layout, dtype */
  PTHB200_KERNEL_UMMA = 2,   /* tcgen05 int8 kernel (kind::i8, cache bytes used as stored);
                                EINVAL where it does not apply */
  PTHB200_KERNEL_UMMA_BF16 = 3, /* tcgen05 kernel that widens the cache to bf16 (kind::f16) */
  PTHB200_KERNEL_UMMA_ROWS = 4  /* tcgen05 kernel with query rows on the MMA M dimension
                                   (prefill, wide verification); bf16 operands */
};

/* options.flags: the caller promises that no request of the launch has more than
 * args.bq query tokens (max_query_len <= bq, e.g. every pure decode step), so each
 * request is exactly one row tile: the grid is num_reqs tiles wide instead of the
 * padded num_tokens / bq + num_reqs, and a CTA finds its request without a search.
 * Same results; query tokens past bq of a request that breaks the promise are not
 * computed. */
#define PTHB200_FLAG_ONE_TILE_PER_REQUEST 1

/* Options of the _ex entry points.  Zero-initialise, then set abi_version and
 * struct_bytes.  lse_out (optional) receives the natural-log log-sum-exp of the
 * scaled scores per (token, head), -inf for a row without keys: from the
 * attention launch when num_splits == 1, from the combine otherwise. */
typedef struct PthB200Options {
  int32_t abi_version;
  int32_t struct_bytes;
  int32_t kernel;
  int32_t flags; /* PTHB200_FLAG_* bits */
  float* lse_out; /* [num_tokens, num_q_heads] fp32 or NULL */
  int64_t lse_stride_token;
  int64_t lse_stride_head;
} PthB200Options;

/* Library identity for binding layers. */
int32_t pthb200_abi_version(void);
int32_t pthb200_attn_args_bytes(void);
int32_t pthb200_combine_args_bytes(void);
int32_t pthb200_options_bytes(void);
int32_t pthb200_has_cuda(void); /* always 1 */
/* Message of the calling thread's last failed call ("" after a success). */
const char* pthb200_last_error(void);

/* Enqueue the attention kernel(s) on `stream` (a cudaStream_t). */
int32_t pthb200_attention(const PthAttnArgs* args, void* stream);
int32_t pthb200_attention_ex(const PthAttnArgs* args, const PthB200Options* options,
                             void* stream);
/* Enqueue the split combine on `stream`. */
int32_t pthb200_combine(const PthAttnCombineArgs* args, void* stream);
int32_t pthb200_combine_ex(const PthAttnCombineArgs* args, const PthB200Options* options,
                           void* stream);

/* Attention + combine in one call that performs NO allocation: the split partials
 * live in a fixed 8 MiB array inside this library (a __device__ array of the loaded
 * module, one instance per GPU; the instance used is that of the CURRENT device of the
 * calling thread, which must be the device `stream` belongs to) instead of a caller
 * workspace; args->ws_o / ws_lse
 * and their strides are ignored.  It has no counterpart in the reference, whose op
 * always takes the workspace from its caller.  It is for callers that have no way
 * to obtain device memory at the point of the call: an engine that has handed all
 * free memory to its KV-cache pool after profiling and forbids allocation inside
 * forward (the reference's backend must reserve its workspace up front for this
 * reason), or a binding in a language with no route to the framework's allocator.
 * Limits and rules:
 *   - num_splits * num_tokens * num_q_heads * (head_size + 1) * 4 bytes (o rounded up
 *     to 256 bytes) must fit 8 MiB, else PTH_ATTN_EINVAL with both numbers in the
 *     message; with num_splits == 1 the array is not used;
 *   - the first call on a device looks the array up (cudaGetSymbolAddress, which may
 *     load the module there): make that call before any stream capture; later calls
 *     only launch kernels;
 *   - every call on a device uses the same array, so calls whose kernels can overlap
 *     (two streams, or unordered host threads) race on it: keep them on one stream or
 *     order them yourself.  Nothing in the array needs clearing between calls.
 * Results are those of pthb200_attention + pthb200_combine with a dense workspace. */
int32_t pthb200_attention_noalloc(const PthAttnArgs* args, void* stream);

/* ---- paged-copy ceiling ---------------------------------------------------------
 * Enqueues a kernel that fetches exactly the cache bytes pthb200_attention would fetch for
 * these arguments on the integer kernel - same persistent CTAs, same work-item schedule,
 * same TMA page copies into the same three-stage ring - and discards them.  Its time is the
 * memory-side floor of the attention launch: eta_mem = T_copy / T_attention, the measure the
 * reference reports against its own copy-ceiling program (bench/sol_copy.cu:424-512,
 * docs/benchmark-methodology.md:60-63).  Writes nothing.  PTH_ATTN_EINVAL where the integer
 * kernel does not apply. */
int32_t pthb200_copy_ceiling(const PthAttnArgs* args, void* stream);

/* ---- quantising cache writer --------------------------------------------------
 * The step in front of the attention path: stores the K and V rows of new tokens in the
 * cache's int8_per_token_head form.  It stands where vLLM's own per-token-head writer stands
 * for the reference (the reference calls it at python/pth_testing/reference.py:301-307 and
 * 461-473, and inherits it in production, python/pth_flash_attn/vllm_backend.py:10-14); the
 * arithmetic is the one the reference documents and mirrors (docs/integration.md:73-117,
 * python/pth_testing/reference.py:76-103), bit for bit:
 *   scale = max(absmax / 127, 1e-6);  q = clamp(trunc(x * (1 / scale) +- 0.5), -128, 127).
 * key / value: [num_tokens, num_kv_heads, head_size] of src_dtype (F32, F16 or BF16), byte
 * strides given, rows contiguous.  The four streams are the ones PthAttnArgs describes (the
 * data pointers are written through).  slot_mapping [num_tokens] int64: slot = block *
 * block_size + position; a negative value skips the token. */
typedef struct PthB200WriteArgs {
  int32_t abi_version;  /* PTH_ATTN_ABI_VERSION */
  int32_t struct_bytes; /* sizeof(PthB200WriteArgs) of the caller */
  const void* key;
  const void* value;
  int32_t src_dtype;
  int64_t key_stride_token;
  int64_t key_stride_head;
  int64_t value_stride_token;
  int64_t value_stride_head;
  PthAttnStream k_cache;
  PthAttnStream v_cache;
  PthAttnStream k_scale;
  PthAttnStream v_scale;
  int32_t num_blocks;
  int32_t block_size;
  int32_t num_kv_heads;
  int32_t head_size; /* 64, 128 or 256 */
  int32_t num_tokens;
  const int64_t* slot_mapping;
} PthB200WriteArgs;
int32_t pthb200_write_args_bytes(void);
/* Enqueue the writer on `stream`.  No allocation, no synchronisation. */
int32_t pthb200_write_kv(const PthB200WriteArgs* args, void* stream);

/* Host-only helpers of the op layer (no device access).
 * pthb200_tile_tokens: query tokens per row tile for a launch planned with `wm`
 * (1, 2 or 4), group size G and host bound max_query_len; returns -1 if wm is
 * not the tile height those rows need (the op's "wm is not the tile height"
 * refusal). */
int32_t pthb200_tile_tokens(int32_t wm, int32_t group, int32_t max_query_len);
/* Validates a filled PthAttnArgs exactly as pthb200_attention would, without
 * launching.  Returns PTH_ATTN_OK or PTH_ATTN_EINVAL (+ last error). */
int32_t pthb200_check_call(const PthAttnArgs* args);

/* Work a launch will enqueue, for callers that account for launches:
 * *attention_kernels and *combine_kernels receive the number of kernels
 * pthb200_attention + pthb200_combine enqueue for these arguments. */
int32_t pthb200_launch_count(const PthAttnArgs* args, int32_t* attention_kernels,
                             int32_t* combine_kernels);

/* ---- test hooks (counterparts of the reference's fragment unit tests,
 * csrc/pth_attn/attn_capi.h:41-78,102-105) ---------------------------------- */

/* One CTA runs the tensor-core building blocks on one 128-key tile:
 *   s_out[key][n] = sum_d k[key][d] * q[n][d]      (fp32 [128][16])
 *   o_out[d][n]   = sum_key v[key][d] * pm[key][n] (fp32 [128][16])
 * k, v: int8 [128][128]; q: bf16 [16][128]; pm: bf16 [128][16]; all dense on the
 * device.  variant bit 0: the padded operand image of the attention kernel (else
 * dense). */
int32_t pthb200_test_tile(const void* k, const void* q, const void* v, const void* pm,
                          float* s_out, float* o_out, int32_t variant, void* stream);
/* The integer counterpart: k, v int8 [128][128]; q int8 [32][128] (rows 0-15 high
 * digits, 16-31 low digits); pm int8 [128][48]; s_out int32 [128][32],
 * o_out int32 [128][48]. */
int32_t pthb200_test_tile_i8(const void* k, const void* q, const void* v, const void* pm,
                             int32_t* s_out, int32_t* o_out, void* stream);
/* The row-major counterpart (query rows on the MMA M dimension): k, v int8 [128][128];
 * q bf16 [128 rows][128]; pm bf16 [128 rows][128 keys], handed to the MMA through
 * TMEM; s_out fp32 [128 rows][128 keys] = q k^T, o_out fp32 [128 rows][128] = pm v. */
int32_t pthb200_test_tile_rows(const void* k, const void* q, const void* v, const void* pm,
                               float* s_out, float* o_out, void* stream);
/* The work-item schedule of the persistent integer kernel, computed on the HOST from host
 * copies of query_start_loc [num_reqs + 1] and seq_lens [num_reqs] by the same functions
 * the device runs: out [max_items][8] int32 receives, CTA by CTA and in running order,
 * {cta, request, row tile, KV head, split, splits of the request, first KV tile, end KV
 * tile}.  Returns the number of items (only the first max_items are stored), or
 * PTH_ATTN_EINVAL.  Counterpart of the reference's geometry unit tests
 * (tests/cpp/test_geometry.cpp:298-451: split partition, tile numbering). */
int32_t pthb200_test_schedule(const int32_t* query_start_loc, const int32_t* seq_lens, int32_t num_reqs,
                              int32_t group, int32_t num_kv_heads, int32_t bq, int32_t num_splits,
                              int32_t window, int32_t causal, int32_t row_class, int32_t class_rows,
                              int32_t num_ctas, int32_t* out, int32_t max_items);
/* Synchronises the device, returns and clears the status word in which a
 * kernel records a bounded wait that gave up (0 = none). */
int32_t pthb200_device_status(int32_t* status);

#ifdef __cplusplus
}
#endif

#endif /* PTHB200_ATTN_H_ */
