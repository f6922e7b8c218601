// CUDA-core attention kernel: every head size (64/128/256), q dtype, cache
// layout and alignment the C ABI admits.  It is the kernel family for shapes
// the tcgen05 kernel does not take, and the on-device cross-check for it.
//
// One CTA = one work item (row tile, KV head, split); one warp = one row at a
// time.  Per 32-key chunk, lane j scores key j (a full dot product over D from
// 4-byte cache words), the warp agrees on the running maximum, and every lane
// then accumulates its own D/32 output columns over the chunk's keys.  All
// arithmetic is fp32; exponentials are exp2 of log2-scaled scores.
#include "params.cuh"

namespace pthb200 {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int D>
__global__ void __launch_bounds__(kThreads) scalar_attention_kernel(const __grid_constant__ KernelParams p) {
  constexpr int kCols = (D + 127) / 128;  // 4-column groups per lane
  __shared__ float q_smem[kWarps][D];

  const RowTile t = resolve_row_tile(p, blockIdx.x);
  if (t.req < 0) return;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  int tile_begin, tile_end, range_begin, range_end;
  split_tiles(p, t, split, &tile_begin, &tile_end, &range_begin, &range_end);
  const int kv_begin = max(range_begin, tile_begin * kKvTile);
  const int kv_end = min(range_end, tile_end * kKvTile);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = t.ntok * p.group;
  const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;

  for (int row = warp; row < rows; row += kWarps) {
    const int ti = row / p.group;
    const int head = kvh * p.group + row % p.group;
    const int token = t.tok0 + ti;
    int lo, hi;
    visible_range(p, t, t.first_idx + ti, &lo, &hi);
    const int begin = max(lo, kv_begin);
    const int end = min(hi + 1, kv_end);

    const uint8_t* q_row = p.q + (int64_t)token * p.q_stride_token + (int64_t)head * p.q_stride_head;
    __syncwarp();
    for (int d = lane; d < D; d += 32) q_smem[warp][d] = load_q_elem(q_row, d, p.q_dtype);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[kCols][4];
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;

    for (int base = begin; base < end; base += 32) {
      const int pos = base + lane;
      const bool live = pos < end;
      float s = -INFINITY, vscale = 0.f;
      int64_t v_off = 0;
      if (live) {
        const int64_t blk = __ldg(bt + pos / p.block_size);
        const int64_t slot = pos % p.block_size;
        const uint8_t* kp = p.k.data + blk * p.k.stride_block + slot * p.k.stride_slot +
                            (int64_t)kvh * p.k.stride_head;
        float dot = 0.f;
#pragma unroll 8
        for (int d = 0; d < D; d += 4) {
          const int w = *reinterpret_cast<const int*>(kp + d);
          dot = fmaf(q_smem[warp][d + 0], (float)(int8_t)(w & 0xff), dot);
          dot = fmaf(q_smem[warp][d + 1], (float)(int8_t)((w >> 8) & 0xff), dot);
          dot = fmaf(q_smem[warp][d + 2], (float)(int8_t)((w >> 16) & 0xff), dot);
          dot = fmaf(q_smem[warp][d + 3], (float)(int8_t)((w >> 24) & 0xff), dot);
        }
        const float kscale = *reinterpret_cast<const float*>(
            p.ks.data + blk * p.ks.stride_block + slot * p.ks.stride_slot + (int64_t)kvh * p.ks.stride_head);
        vscale = *reinterpret_cast<const float*>(
            p.vs.data + blk * p.vs.stride_block + slot * p.vs.stride_slot + (int64_t)kvh * p.vs.stride_head);
        v_off = blk * p.v.stride_block + slot * p.v.stride_slot + (int64_t)kvh * p.v.stride_head;
        s = dot * (kscale * p.scale_log2);
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float alpha = exp2f(m - m_new);  // m = -inf -> 0; m_new is finite here
      const float pr = live ? exp2f(s - m_new) : 0.f;
      l = l * alpha + warp_sum(pr);
      m = m_new;
#pragma unroll
      for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[c][e] *= alpha;
      const float pv = pr * vscale;
      const int n_live = min(32, end - base);
      for (int j = 0; j < n_live; ++j) {
        const float w = __shfl_sync(0xffffffffu, pv, j);
        const int64_t off = __shfl_sync(0xffffffffu, v_off, j);
        const uint8_t* vp = p.v.data + off;
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
          const int d = c * 128 + lane * 4;
          if (d < D) {
            const int x = *reinterpret_cast<const int*>(vp + d);
            acc[c][0] = fmaf(w, (float)(int8_t)(x & 0xff), acc[c][0]);
            acc[c][1] = fmaf(w, (float)(int8_t)((x >> 8) & 0xff), acc[c][1]);
            acc[c][2] = fmaf(w, (float)(int8_t)((x >> 16) & 0xff), acc[c][2]);
            acc[c][3] = fmaf(w, (float)(int8_t)((x >> 24) & 0xff), acc[c][3]);
          }
        }
      }
    }

    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float lse2 = l > 0.f ? m + log2f(l) : -INFINITY;
    if (p.num_splits == 1) {
      uint8_t* o_row = p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head;
#pragma unroll
      for (int c = 0; c < kCols; ++c) {
        const int d = c * 128 + lane * 4;
        if (d < D) {
#pragma unroll
          for (int e = 0; e < 4; ++e) store_out_elem(o_row, d + e, p.out_dtype, acc[c][e] * inv);
        }
      }
      if (p.lse_out != nullptr && lane == 0) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                  (int64_t)head * p.lse_stride_head) = lse2 * kLn2;
      }
    } else {
      uint8_t* o_row = reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                       (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head;
#pragma unroll
      for (int c = 0; c < kCols; ++c) {
        const int d = c * 128 + lane * 4;
        if (d < D) {
          *reinterpret_cast<float4*>(o_row + (int64_t)d * 4) =
              make_float4(acc[c][0] * inv, acc[c][1] * inv, acc[c][2] * inv, acc[c][3] * inv);
        }
      }
      if (lane == 0) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                  (int64_t)token * p.ws_lse_stride_token +
                                  (int64_t)head * p.ws_lse_stride_head) = lse2;
      }
    }
  }
}

}  // namespace

cudaError_t launch_scalar_attention(const KernelParams& p, cudaStream_t stream) {
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  switch (p.head_size) {
    case 64:
      scalar_attention_kernel<64><<<grid, kThreads, 0, stream>>>(p);
      break;
    case 128:
      scalar_attention_kernel<128><<<grid, kThreads, 0, stream>>>(p);
      break;
    default:
      scalar_attention_kernel<256><<<grid, kThreads, 0, stream>>>(p);
      break;
  }
  return cudaGetLastError();
}

}  // namespace pthb200
