// Split-KV combine: merges the per-split partial outputs of one (token, head)
// row by their log2-sum-exp weights.
//
//   M   = max_s lse_s            (splits with lse_s = -inf hold no keys)
//   w_s = exp2(lse_s - M)
//   out = (sum_s w_s * o_s) / (sum_s w_s),  summed in the order s = 0..S-1
//
// A split with lse = -inf is skipped BEFORE its ws_o row is read, so garbage
// (NaN included) in the partial of an empty split never reaches the output.
// One warp per row; lane j owns output columns 4j..4j+3 (+128, +256 for wider
// heads) and moves them as 16-byte vectors.  A row whose splits are all empty
// gets out = 0 and lse = -inf.  Rows >= query_start_loc[num_reqs] are skipped.
#include "params.cuh"

namespace pthb200 {


namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

template <int D>
__global__ void __launch_bounds__(kThreads) combine_kernel(const __grid_constant__ CombineParams p) {
  constexpr int kCols = (D + 127) / 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
  const int valid_tokens = min(p.num_tokens, __ldg(p.query_start_loc + p.num_reqs));
  if (row >= (int64_t)valid_tokens * p.num_q_heads) return;
  const int token = (int)(row / p.num_q_heads);
  const int head = (int)(row % p.num_q_heads);
  const int S = p.num_splits;

  const uint8_t* lse_base = reinterpret_cast<const uint8_t*>(p.ws_lse) + (int64_t)token * p.ws_lse_stride_token +
                            (int64_t)head * p.ws_lse_stride_head;
  const uint8_t* o_base = reinterpret_cast<const uint8_t*>(p.ws_o) + (int64_t)token * p.ws_o_stride_token +
                          (int64_t)head * p.ws_o_stride_head;

  // Pass 1: the maximum over splits (lanes stride over s).
  float mx = -INFINITY;
  for (int s = lane; s < S; s += 32) {
    const float v = *reinterpret_cast<const float*>(lse_base + (int64_t)s * p.ws_lse_stride_split);
    if (v > mx) mx = v;  // NaN never raises the maximum
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  float acc[kCols][4];
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
  float den = 0.f;

  if (mx > -INFINITY) {
    // Pass 2: fixed order s = 0..S-1, 32 splits per round; every lane walks the
    // same sequence, so the sum is deterministic and identical across lanes.
    for (int s0 = 0; s0 < S; s0 += 32) {
      const int s_mine = s0 + lane;
      float w_mine = 0.f;
      if (s_mine < S) {
        const float v = *reinterpret_cast<const float*>(lse_base + (int64_t)s_mine * p.ws_lse_stride_split);
        w_mine = (v > -INFINITY) ? exp2f(v - mx) : 0.f;
        if (!(w_mine >= 0.f)) w_mine = 0.f;  // NaN lse: treated as empty
      }
      const int n = min(32, S - s0);
      for (int j = 0; j < n; ++j) {
        const float w = __shfl_sync(0xffffffffu, w_mine, j);
        if (w == 0.f) continue;  // empty split: its partial is never read
        den += w;
        const uint8_t* o_row = o_base + (int64_t)(s0 + j) * p.ws_o_stride_split;
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
          const int d = c * 128 + lane * 4;
          if (d < D) {
            const float4 v = *reinterpret_cast<const float4*>(o_row + (int64_t)d * 4);
            acc[c][0] = fmaf(w, v.x, acc[c][0]);
            acc[c][1] = fmaf(w, v.y, acc[c][1]);
            acc[c][2] = fmaf(w, v.z, acc[c][2]);
            acc[c][3] = fmaf(w, v.w, acc[c][3]);
          }
        }
      }
    }
  }

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
  const unsigned grid = (unsigned)((rows + kWarps - 1) / kWarps);
  switch (p.head_size) {
    case 64:
      combine_kernel<64><<<grid, kThreads, 0, stream>>>(p);
      break;
    case 128:
      combine_kernel<128><<<grid, kThreads, 0, stream>>>(p);
      break;
    default:
      combine_kernel<256><<<grid, kThreads, 0, stream>>>(p);
      break;
  }
  return cudaGetLastError();
}

}  // namespace pthb200
