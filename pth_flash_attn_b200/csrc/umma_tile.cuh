// Building blocks of the tcgen05 attention kernels at head size 128: the
// shared-memory image of a widened KV tile, the exact int8 -> bf16 widening,
// and the two MMA chains over one 128-key tile.  Both operands of a
// tcgen05.mma.kind::f16 must have the same format: an fp16 A operand with a bf16
// B operand raises an illegal-instruction fault on B200, so everything is bf16.
//
// "Token-major" orientation (keys on the MMA M dimension, query rows on N):
//   S^T[key, row] = sum_d K[key, d] * Q[row, d]      A = K tile (K-major), B = Q (K-major)
//   O^T[d,   row] += sum_key V[key, d] * P[key, row]  A = V tile (MN-major), B = P (MN-major)
// Both accumulators live in TMEM: 128 lanes (keys, resp. d) x NPAD fp32 columns.
//
// Widened tile image (identical for K and V): 16 d-chunks of 8 elements; chunk c
// holds, for key t = 0..127, the 8 bf16 values d = 8c..8c+7 in 16 bytes at
//   c * chunk_stride + t * 16.
// For K (K-major A) a core matrix is 8 keys x 8 d: SBO = 128 (next 8 keys),
// LBO = chunk_stride (next 8 d).  For V (MN-major A, M = d) a core matrix is
// 8 keys (K dim) x 8 d: SBO = chunk_stride (next 8 d), LBO = 128 (next 8 keys).
// kChunkStride carries 16 bytes of padding so that the 8 lanes of a quarter
// warp, which write 8 different chunks of one key, hit 8 different bank groups.
//
// Q image (K-major B): chunk c, row n at c * (NPAD * 16) + n * 16.
// P image (MN-major B): rows in groups of 8; group j, key t at j * 2048 + t * 16.
#pragma once

#include <cuda_bf16.h>

#include "tcgen05.cuh"

namespace pthb200 {

constexpr int kHeadDim = 128;
constexpr int kTileKeys = 128;
constexpr int kChunks = kHeadDim / 8;                  // 16 d-chunks of 8 elements
constexpr int kChunkStride = kTileKeys * 16 + 16;      // 2064 bytes
constexpr int kWideBytes = kChunks * kChunkStride;     // one widened K or V tile
constexpr int kPGroupStride = kTileKeys * 16;          // 2048 bytes

// 4 int8 (one 32-bit word) -> 4 bf16, exactly.  With l = x & 0x7f and s = x >> 7
// (the sign bit), x = l - 128 s.  The bf16 bit patterns 0x4300 | l and
// 0x4300 | (s << 7) are the integers 128 + l and 128 + 128 s, so one packed
// bf16 subtraction yields x without any integer-to-float conversion.
__device__ __forceinline__ void widen4_bf16(uint32_t w, uint32_t& out01, uint32_t& out23) {
  const uint32_t lo = w & 0x7F7F7F7Fu;
  const uint32_t hi = w & 0x80808080u;
  const uint32_t a01 = __byte_perm(lo, 0x43434343u, 0x5140);
  const uint32_t a23 = __byte_perm(lo, 0x43434343u, 0x7362);
  const uint32_t b01 = __byte_perm(hi, 0x43434343u, 0x5140);
  const uint32_t b23 = __byte_perm(hi, 0x43434343u, 0x7362);
  const __nv_bfloat162 r01 =
      __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a01), *reinterpret_cast<const __nv_bfloat162*>(&b01));
  const __nv_bfloat162 r23 =
      __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a23), *reinterpret_cast<const __nv_bfloat162*>(&b23));
  out01 = *reinterpret_cast<const uint32_t*>(&r01);
  out23 = *reinterpret_cast<const uint32_t*>(&r23);
}

__device__ __forceinline__ uint4 widen8_bf16(uint2 raw) {
  uint4 r;
  widen4_bf16(raw.x, r.x, r.y);
  widen4_bf16(raw.y, r.z, r.w);
  return r;
}

// S^T = K * Q^T over the full head dimension: 8 MMAs of K = 16.  One thread.
template <int NPAD>
__device__ __forceinline__ void issue_qk(uint32_t s_tmem, uint32_t kw_saddr, uint32_t q_saddr, uint32_t chunk_stride) {
  constexpr uint32_t idesc = tc::instr_desc(128, NPAD, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk) {
    const uint64_t a = tc::smem_desc(kw_saddr + kk * 2 * chunk_stride, chunk_stride, 128);
    const uint64_t b = tc::smem_desc(q_saddr + kk * 2 * (NPAD * 16), NPAD * 16, 128);
    tc::mma_ss(s_tmem, a, b, idesc, kk > 0);
  }
}

// O^T (+)= V^T * P over the 128 keys of the tile: 8 MMAs of K = 16 keys.  One thread.
template <int NPAD>
__device__ __forceinline__ void issue_pv(uint32_t o_tmem, uint32_t vw_saddr, uint32_t p_saddr, uint32_t chunk_stride,
                                         bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(128, NPAD, tc::kFmtBF16, tc::kFmtBF16, 1, 1);
#pragma unroll
  for (int kk = 0; kk < kTileKeys / 16; ++kk) {
    const uint64_t a = tc::smem_desc(vw_saddr + kk * 256, 128, chunk_stride);
    const uint64_t b = tc::smem_desc(p_saddr + kk * 256, 128, kPGroupStride);
    tc::mma_ss(o_tmem, a, b, idesc, accumulate || kk > 0);
  }
}

}  // namespace pthb200
