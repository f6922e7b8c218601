// Kernel parameters and launch geometry shared by every kernel of the library.
//
// Terms: a "row" is one (query token, query head) pair; the G = Hq / Hkv query
// heads that share a KV head are packed token-major (row n of a row tile is
// token n / G, head n % G).  A "row tile" is up to bq query tokens of ONE
// request; a "KV tile" is kKvTile consecutive KV positions.  A work item is
// (row tile, KV head, split).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pthb200_attn.h"

namespace pthb200 {

// KV positions per tile.  The split partition is made of whole tiles, so this
// constant is part of the meaning of a split for every kernel family.
constexpr int kKvTile = 128;

struct StreamParams {
  const uint8_t* data;
  int64_t stride_block;
  int64_t stride_slot;
  int64_t stride_head;
};

struct KernelParams {
  const uint8_t* q;
  int64_t q_stride_token, q_stride_head;
  uint8_t* out;
  int64_t out_stride_token, out_stride_head;
  StreamParams k, v, ks, vs;
  const int32_t* block_table;
  int64_t block_table_row_stride;
  const int32_t* seq_lens;
  const int32_t* query_start_loc;
  float* ws_o;
  int64_t ws_o_stride_split, ws_o_stride_token, ws_o_stride_head;
  float* ws_lse;
  int64_t ws_lse_stride_split, ws_lse_stride_token, ws_lse_stride_head;
  float* lse_out;  // optional natural-log LSE (num_splits == 1 only)
  int64_t lse_stride_token, lse_stride_head;
  int32_t q_dtype, out_dtype;
  int32_t block_size, num_kv_heads, head_size;
  int32_t block_shift;  // log2(block_size) if it is a power of two, else -1
  // TMA kernels: slots one page copy brings in (a power of two from 16 to 128 that divides
  // block_size; a page of more slots is fetched in several copies) and its log2
  int32_t copy_slots = 0, copy_shift = -1;
  int32_t num_reqs, num_tokens, num_q_heads, group;
  int32_t bq, num_q_tiles, num_splits;
  int32_t window, causal;
  float scale_log2;  // softmax_scale * log2(e)
  // integer kernel: how the raw cache bytes are fetched (set by its launcher)
  int32_t raw_mode;        // 1 = tiled TMA box per page, 2 = bulk copy per contiguous page run
  int32_t num_blocks;      // blocks in the cache views
  // How grid index x maps to a row tile, and which requests this launch serves.
  int32_t tile_map;    // 0 = padded tile grid (bisection over query_start_loc); 1 = row tile x is request x
                       //     (valid when no request has more than bq query tokens): num_q_tiles = num_reqs
  int32_t num_sms;     // SMs of the device (set by the launchers whose kernels choose splits on the device)
  int32_t row_class;   // 0 = every request; 1 = only requests with q_len * group <= class_rows; 2 = only the others
  int32_t class_rows;
};

// Re-tiles a launch to `bq` query tokens per row tile.  The caller's promise behind
// tile_map = 1 (no request longer than its bq) survives only while bq does not shrink.
inline void set_row_tile(KernelParams& p, int bq) {
  if (bq < p.bq) p.tile_map = 0;
  p.bq = bq;
  p.num_q_tiles = p.tile_map == 1 ? p.num_reqs : p.num_tokens / p.bq + p.num_reqs;
}

// A row tile resolved on the device.
struct RowTile {
  int32_t req;        // request index, -1 if the tile is surplus
  int32_t tok0;       // first query token (global row of q/out)
  int32_t ntok;       // query tokens in the tile (1..bq)
  int32_t q_len;      // query tokens of the request
  int32_t seq_len;    // KV length of the request
  int32_t first_idx;  // index of tok0 inside the request
};

// Row tile x of the grid: request r owns tiles [qsl[r]/bq + r, ... + ceil(q_len/bq)).
// The start index is strictly increasing in r, so the owner is found by
// bisection; tiles that fall between two requests are surplus (req = -1).
// `qsl(i)` reads query_start_loc[i] and `len(r)` seq_lens[r] (from global memory, or from
// copies of them).  With tile_map = 1 the caller has promised that no request has more than
// bq query tokens, so tile x is simply request x (tokens past bq would be left out, never
// written past the tile).  row_class filters requests by their row count, which lets two
// kernels share one launch: each resolves every tile and drops the other's requests.
template <class LoadQsl, class LoadLen>
__device__ __forceinline__ RowTile resolve_row_tile_with(const KernelParams& p, int x, LoadQsl qsl, LoadLen len) {
  RowTile t;
  t.req = -1;
  int lo = 0, hi = p.num_reqs - 1;
  if (p.tile_map == 1) {
    if (x >= p.num_reqs) return t;
    lo = x;
  } else {
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      const int first = qsl(mid) / p.bq + mid;
      if (first <= x) lo = mid; else hi = mid - 1;
    }
  }
  const int q0 = qsl(lo);
  const int q1 = qsl(lo + 1);
  const int seq_len = len(lo);  // issued with the two loads above, not after the checks below
  const int j = p.tile_map == 1 ? 0 : x - (q0 / p.bq + lo);
  const int q_len = q1 - q0;
  if (j < 0 || j * p.bq >= q_len) return t;
  if (p.row_class != 0 && (((int64_t)q_len * p.group <= p.class_rows) != (p.row_class == 1))) return t;
  t.req = lo;
  t.first_idx = j * p.bq;
  t.tok0 = q0 + t.first_idx;
  t.ntok = min(p.bq, q_len - t.first_idx);
  t.q_len = q_len;
  t.seq_len = seq_len;
  return t;
}

__device__ __forceinline__ RowTile resolve_row_tile(const KernelParams& p, int x) {
  return resolve_row_tile_with(
      p, x, [&](int i) { return __ldg(p.query_start_loc + i); }, [&](int r) { return __ldg(p.seq_lens + r); });
}

// Inclusive visible key range of the query token with index i inside its
// request (bottom-right aligned: KV position pos = L - q_len + i).
__device__ __forceinline__ void visible_range(const KernelParams& p, const RowTile& t, int i,
                                              int* lo, int* hi) {
  const int pos = t.seq_len - t.q_len + i;
  *lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  if (p.causal) {
    *hi = pos;
  } else {
    *hi = p.window > 0 ? min(t.seq_len - 1, (int)min((int64_t)pos + p.window - 1, (int64_t)INT32_MAX))
                       : t.seq_len - 1;
  }
  *hi = min(*hi, t.seq_len - 1);
}

// KV tiles [tile_begin, tile_end) that split `split` of this row tile reads:
// the tiles touched by the union of the rows' visible ranges, divided into
// num_splits runs whose sizes differ by at most one (num_splits: the launch's, or the number
// of pieces the kernel has chosen for this request).
__device__ __forceinline__ void split_tiles(const KernelParams& p, const RowTile& t, int split, int num_splits,
                                            int* tile_begin, int* tile_end, int* range_begin,
                                            int* range_end) {
  int lo_first, hi_first, lo_last, hi_last;
  visible_range(p, t, t.first_idx, &lo_first, &hi_first);
  visible_range(p, t, t.first_idx + t.ntok - 1, &lo_last, &hi_last);
  const int rb = lo_first;                 // lo is non-decreasing in i
  const int re = max(hi_last, hi_first) + 1;  // hi is non-decreasing in i
  *range_begin = rb;
  *range_end = re;
  if (re <= rb) {
    *tile_begin = *tile_end = 0;
    return;
  }
  const int t0 = rb / kKvTile;
  const int t1 = (re + kKvTile - 1) / kKvTile;
  const int64_t n = t1 - t0;
  *tile_begin = t0 + (int)((int64_t)split * n / num_splits);
  *tile_end = t0 + (int)((int64_t)(split + 1) * n / num_splits);
}
__device__ __forceinline__ void split_tiles(const KernelParams& p, const RowTile& t, int split,
                                            int* tile_begin, int* tile_end, int* range_begin,
                                            int* range_end) {
  split_tiles(p, t, split, p.num_splits, tile_begin, tile_end, range_begin, range_end);
}

__device__ __forceinline__ float load_q_elem(const uint8_t* q_row, int d, int dtype) {
  if (dtype == PTH_ATTN_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q_row)[d]);
  return __half2float(reinterpret_cast<const __half*>(q_row)[d]);
}

__device__ __forceinline__ void store_out_elem(uint8_t* row, int d, int dtype, float v) {
  if (dtype == PTH_ATTN_BF16) {
    reinterpret_cast<__nv_bfloat16*>(row)[d] = __float2bfloat16_rn(v);
  } else if (dtype == PTH_ATTN_F16) {
    reinterpret_cast<__half*>(row)[d] = __float2half_rn(v);
  } else {
    reinterpret_cast<float*>(row)[d] = v;
  }
}

struct CombineParams {
  const float* ws_o;
  int64_t ws_o_stride_split, ws_o_stride_token, ws_o_stride_head;
  const float* ws_lse;
  int64_t ws_lse_stride_split, ws_lse_stride_token, ws_lse_stride_head;
  uint8_t* out;
  int64_t out_stride_token, out_stride_head;
  float* lse_out;
  int64_t lse_stride_token, lse_stride_head;
  const int32_t* query_start_loc;
  int32_t out_dtype, num_reqs, num_tokens, num_q_heads, head_size, num_splits;
};

constexpr float kLn2 = 0.69314718055994530942f;

// Host-side launchers of the kernel families (defined in their .cu files).
// Each returns cudaGetLastError() of its launch.
cudaError_t launch_scalar_attention(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_umma_attention(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_umma_i8_attention(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_umma_rows_attention(const KernelParams& p, cudaStream_t stream);
// CTAs the persistent integer kernel is launched with on a device of `sms` SMs (-1: too many items).
int umma_i8_max_rows(int head_size);
int umma_i8_num_ctas(const KernelParams& p, int sms);
cudaError_t read_i8_status(unsigned int* v);
cudaError_t read_rows_status(unsigned int* v);
cudaError_t read_rows256_status(unsigned int* v);
cudaError_t read_rows2_status(unsigned int* v);
cudaError_t launch_umma_rows2_attention(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_umma_rows256_attention(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_combine_kernel(const CombineParams& p, cudaStream_t stream);
cudaError_t launch_copy_ceiling(const KernelParams& p, cudaStream_t stream);
cudaError_t launch_kv_writer(const PthB200WriteArgs& a, cudaStream_t stream);
// True if the tcgen05 kernel handles these parameters.
bool umma_supports(const KernelParams& p, const char** why);
// True if the integer tcgen05 kernel handles these parameters.
bool umma_i8_supports(const KernelParams& p, const char** why);
// True if the row-major tcgen05 kernel handles these parameters.
bool umma_rows_supports(const KernelParams& p, const char** why);

}  // namespace pthb200
