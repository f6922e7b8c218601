// Split-KV combine: merges the per-split partial outputs of one (token, head)
// row by their log2-sum-exp weights.
//
//   M   = max_s lse_s            (splits with lse_s = -inf hold no keys)
//   w_s = exp2(lse_s - M)
//   out = (sum_s w_s * o_s) / (sum_s w_s)
//
// The order of the sums depends on the number of splits S alone, never on the
// number of rows or on timing.  Up to kWideSplits splits, one warp owns a row
// and sums s = 0..S-1.  Above, one CTA owns a row: its warps (4, or 16 beyond
// kVeryWideSplits) sum contiguous runs of the splits (each in ascending order)
// and warp 0 adds the run sums in ascending order -- a launch with many splits
// has few rows, and one warp walking 100+ dependent rows of partials is pure
// latency.
//
// A split with lse = -inf is skipped BEFORE its ws_o row is read, so garbage
// (NaN included) in the partial of an empty split never reaches the output.
// Lane j owns output columns 4j..4j+3 (+128, +256 for wider heads) and moves
// them as 16-byte vectors, eight splits in flight at a time.  A row whose
// splits are all empty gets out = 0 and lse = -inf.  Rows >=
// query_start_loc[num_reqs] are skipped.
#include "params.cuh"

namespace pthb200 {

namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kWideSplits = 16;      // more splits than this: one CTA of 4 warps per row
constexpr int kVeryWideSplits = 64;  // more than this: one CTA of 16 warps per row
constexpr int kBatch = 8;        // partial rows loaded before their sums start

template <int D>
struct RowSum {
  static constexpr int kCols = (D + 127) / 128;
  float acc[kCols][4];
  float den;
};

// Adds the splits [s_begin, s_end) to `r` in ascending order.
template <int D>
__device__ __forceinline__ void sum_splits(const CombineParams& p, const uint8_t* lse_base, const uint8_t* o_base,
                                           float mx, int s_begin, int s_end, int lane, RowSum<D>& r) {
  constexpr int kCols = RowSum<D>::kCols;
  for (int s0 = s_begin; s0 < s_end; s0 += 32) {
    const int s_mine = s0 + lane;
    float w_mine = 0.f;
    if (s_mine < s_end) {
      const float v = *reinterpret_cast<const float*>(lse_base + (int64_t)s_mine * p.ws_lse_stride_split);
      w_mine = (v > -INFINITY) ? exp2f(v - mx) : 0.f;
      if (!(w_mine >= 0.f)) w_mine = 0.f;  // NaN lse: treated as empty
    }
    const int n = min(32, s_end - s0);
    for (int j0 = 0; j0 < n; j0 += kBatch) {
      float w[kBatch];
      float4 v[kBatch][kCols];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        w[b] = __shfl_sync(0xffffffffu, w_mine, (j0 + b) & 31);  // lanes past n hold 0
        const uint8_t* o_row = o_base + (int64_t)(s0 + j0 + b) * p.ws_o_stride_split;
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
          const int d = c * 128 + lane * 4;
          v[b][c] = make_float4(0.f, 0.f, 0.f, 0.f);
          // empty split (or past the range): its partial is never read
          if (w[b] != 0.f && d < D) v[b][c] = *reinterpret_cast<const float4*>(o_row + (int64_t)d * 4);
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        if (w[b] != 0.f) {
          r.den += w[b];
#pragma unroll
          for (int c = 0; c < kCols; ++c) {
            r.acc[c][0] = fmaf(w[b], v[b][c].x, r.acc[c][0]);
            r.acc[c][1] = fmaf(w[b], v[b][c].y, r.acc[c][1]);
            r.acc[c][2] = fmaf(w[b], v[b][c].z, r.acc[c][2]);
            r.acc[c][3] = fmaf(w[b], v[b][c].w, r.acc[c][3]);
          }
        }
      }
    }
  }
}

// kWideWarps > 0: one CTA of kWideWarps warps per row (a run of the splits each); else one warp per row.
template <int D, int kWideWarps>
__global__ void __launch_bounds__(kWideWarps > 0 ? kWideWarps * 32 : kThreads)
combine_kernel(const __grid_constant__ CombineParams p) {
  constexpr bool kWide = kWideWarps > 0;
  constexpr int kCols = RowSum<D>::kCols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = kWide ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * kWarps + warp;
  const int valid_tokens = min(p.num_tokens, __ldg(p.query_start_loc + p.num_reqs));
  if (row >= (int64_t)valid_tokens * p.num_q_heads) return;  // the whole CTA when kWide
  const int token = (int)(row / p.num_q_heads);
  const int head = (int)(row % p.num_q_heads);
  const int S = p.num_splits;

  const uint8_t* lse_base = reinterpret_cast<const uint8_t*>(p.ws_lse) + (int64_t)token * p.ws_lse_stride_token +
                            (int64_t)head * p.ws_lse_stride_head;
  const uint8_t* o_base = reinterpret_cast<const uint8_t*>(p.ws_o) + (int64_t)token * p.ws_o_stride_token +
                          (int64_t)head * p.ws_o_stride_head;

  // Pass 1: the maximum over all splits (lanes stride over s; every warp of a wide row repeats it).
  float mx = -INFINITY;
  for (int s = lane; s < S; s += 32) {
    const float v = *reinterpret_cast<const float*>(lse_base + (int64_t)s * p.ws_lse_stride_split);
    if (v > mx) mx = v;  // NaN never raises the maximum
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  RowSum<D> r;
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) r.acc[c][e] = 0.f;
  r.den = 0.f;

  // Pass 2: every lane walks the same sequence of splits, so the sums are identical across lanes.
  if (kWide) {
    constexpr int kRunWarps = kWide ? kWideWarps : 1;
    __shared__ float part[kRunWarps > 1 ? kRunWarps - 1 : 1][kCols * 4 + 1][32];
    const int quarter = (S + kRunWarps - 1) / kRunWarps;
    if (mx > -INFINITY) sum_splits<D>(p, lse_base, o_base, mx, min(S, warp * quarter), min(S, (warp + 1) * quarter), lane, r);
    if (warp > 0) {
#pragma unroll
      for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) part[warp - 1][c * 4 + e][lane] = r.acc[c][e];
      part[warp - 1][kCols * 4][lane] = r.den;
    }
    __syncthreads();
    if (warp > 0) return;
#pragma unroll
    for (int w = 0; w < kRunWarps - 1; ++w) {
#pragma unroll
      for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) r.acc[c][e] += part[w][c * 4 + e][lane];
      r.den += part[w][kCols * 4][lane];
    }
  } else {
    if (mx > -INFINITY) sum_splits<D>(p, lse_base, o_base, mx, 0, S, lane, r);
  }
  const float den = r.den;
  float(&acc)[kCols][4] = r.acc;

  const float inv = den > 0.f ? 1.f / den : 0.f;
  uint8_t* out_row = p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head;
#pragma unroll
  for (int c = 0; c < kCols; ++c) {
    const int d = c * 128 + lane * 4;
    if (d < D) {
      const float r0 = acc[c][0] * inv, r1 = acc[c][1] * inv, r2 = acc[c][2] * inv, r3 = acc[c][3] * inv;
      if (p.out_dtype == PTH_ATTN_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(r0, r1), b = __floats2bfloat162_rn(r2, r3);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(out_row + (int64_t)d * 2) = pk;
      } else if (p.out_dtype == PTH_ATTN_F16) {
        __half2 a = __floats2half2_rn(r0, r1), b = __floats2half2_rn(r2, r3);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(out_row + (int64_t)d * 2) = pk;
      } else {
        *reinterpret_cast<float4*>(out_row + (int64_t)d * 4) = make_float4(r0, r1, r2, r3);
      }
    }
  }
  if (p.lse_out != nullptr && lane == 0) {
    const float lse2 = den > 0.f ? mx + log2f(den) : -INFINITY;
    *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                              (int64_t)head * p.lse_stride_head) = lse2 * kLn2;
  }
}

}  // namespace

cudaError_t launch_combine_kernel(const CombineParams& p, cudaStream_t stream) {
  const int64_t rows = (int64_t)p.num_tokens * p.num_q_heads;
  const int wide_warps = p.num_splits > kVeryWideSplits ? 16 : p.num_splits > kWideSplits ? 4 : 0;
  const unsigned grid = wide_warps > 0 ? (unsigned)rows : (unsigned)((rows + kWarps - 1) / kWarps);
#define PTHB200_COMBINE(D_)                                                  \
  if (wide_warps == 16)                                                      \
    combine_kernel<D_, 16><<<grid, 16 * 32, 0, stream>>>(p);                 \
  else if (wide_warps == 4)                                                  \
    combine_kernel<D_, 4><<<grid, 4 * 32, 0, stream>>>(p);                   \
  else                                                                       \
    combine_kernel<D_, 0><<<grid, kThreads, 0, stream>>>(p)
  switch (p.head_size) {
    case 64:
      PTHB200_COMBINE(64);
      break;
    case 128:
      PTHB200_COMBINE(128);
      break;
    default:
      PTHB200_COMBINE(256);
      break;
  }
#undef PTHB200_COMBINE
  return cudaGetLastError();
}

}  // namespace pthb200
