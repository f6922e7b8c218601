// Building blocks of the integer tcgen05 attention kernel: the raw-byte operand
// images of a 128-key KV tile, the int8 MMA chains over them, asynchronous
// global -> shared copies and small conversion helpers.
//
// Raw K / V image of a tile (the cache bytes as stored, no conversion): column
// block j (bytes 16 j .. 16 j + 15 of every key's 128-byte row) sits at
// j * kImgChunk, key t at + 16 t.  Read K-major (K: 8 keys x 16 d per core
// matrix, SBO = 128, LBO = kImgChunk) it is the A operand of S^T = K Q^T; read
// MN-major (V: 16 d x 8 keys per core matrix, SBO = kImgChunk, LBO = 128) it is
// the A operand of O^T = V^T P.  The 16 bytes of padding per column block spread
// the 8 blocks of one key row over all shared-memory banks, so a half warp that
// copies one 128-byte row writes without bank conflicts.
//
// Digit images (B operands): Q [8 column blocks][2 NPAD rows][16 B], K-major;
// P [PD NPAD / 16 column blocks][128 keys][16 B], MN-major, dense blocks of
// kDigitChunk bytes.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "tcgen05.cuh"

namespace pthb200 {

constexpr int kHeadDimI8 = 128;
constexpr int kKeys = 128;
constexpr int kDigitChunk = kKeys * 16;      // 2,048 B
constexpr int kImgChunk = kKeys * 16 + 16;   // 2,064 B
constexpr int kImgBytes = 8 * kImgChunk;     // 16,512 B (head size 128)

// Geometry of the raw cells and operand images for head size HD (64, 128 or 256).
template <int HD>
struct I8Geom {
  static_assert(HD == 64 || HD == 128 || HD == 256, "head size");
  static constexpr int chunks = HD / 16;                       // 16-byte column blocks of one key's K (or V) row
  static constexpr int img_bytes = chunks * kImgChunk;         // one K or V image of a tile
  static constexpr int cell = 2 * HD + 8;                      // K | k_scale | V | v_scale
  static constexpr int raw_row = (cell + 8 + 15) / 16 * 16;    // 16-byte aligned bytes that cover an 8-byte aligned cell
  static constexpr int raw_stage = kKeys * raw_row;            // raw cells of one tile
  static constexpr int part_words = HD / 4 + 4;                // words of the 16-byte pieces that cover K + k_scale (or V + v_scale)
  static constexpr int halves = HD > 128 ? 2 : 1;              // O^T accumulators of 128 dims (MMA M = 128)
};

// Order-preserving map float -> int, so an integer warp reduction finds a float maximum.
__device__ __forceinline__ int float_key(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// int32 with |x| < 2^22 -> float, exactly, without the conversion unit.
__device__ __forceinline__ float int_to_float(uint32_t x) {
  return __uint_as_float(0x4B400000u + x) - 12582912.0f;
}

// 8- and 4-byte asynchronous copies global -> shared; src_bytes = 0 zero-fills.
__device__ __forceinline__ void cp_async8(uint32_t dst, const uint8_t* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const uint8_t* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Streaming loads of cache bytes (read once: keep them out of L1).
__device__ __forceinline__ uint2 ldg8_stream(const uint8_t* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t ldg4_stream(const uint8_t* p) {
  uint32_t r;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

__device__ __forceinline__ uint4 ldg16_stream(const uint8_t* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}

// Instruction descriptor of tcgen05.mma.kind::i8: signed 8-bit operands, int32 accumulator.
__host__ __device__ constexpr uint32_t idesc_i8(uint32_t m, uint32_t n, uint32_t a_mn, uint32_t b_mn) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// S^T = K Q^T.  One MMA covers 32 d = two 16-byte column blocks.  One thread.
template <int NPAD>
__device__ __forceinline__ void issue_qk_i8(uint32_t s_tmem, uint32_t kimg, uint32_t qimg) {
  constexpr uint32_t idesc = idesc_i8(128, 2 * NPAD, 0, 0);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint64_t a = tc::smem_desc(kimg + kk * 2 * kImgChunk, kImgChunk, 128);
    const uint64_t b = tc::smem_desc(qimg + kk * 2 * (2 * NPAD * 16), 2 * NPAD * 16, 128);
    mma_i8(s_tmem, a, b, idesc, kk > 0);
  }
}

// O^T = V^T P.  One MMA covers 32 keys = four 8-key groups.  One thread.
template <int NPAD, int PD>
__device__ __forceinline__ void issue_pv_i8(uint32_t o_tmem, uint32_t vimg, uint32_t pimg) {
  constexpr uint32_t idesc = idesc_i8(128, PD * NPAD, 1, 1);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint64_t a = tc::smem_desc(vimg + kk * 4 * 128, 128, kImgChunk);
    const uint64_t b = tc::smem_desc(pimg + kk * 4 * 128, 128, kDigitChunk);
    mma_i8(o_tmem, a, b, idesc, kk > 0);
  }
}

// ---- the same MMA chains for an issuing thread that keeps its descriptors in registers ----
// The start address (in 16-byte units) sits in the low word of a shared-memory descriptor, so
// moving an operand by `bytes` (a multiple of 16, inside shared memory) adds bytes / 16 to
// that word.  Building four descriptors per chain from scratch costs the single issuing
// thread about a hundred dependent instructions; this form costs two additions per MMA.
struct DescWords {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescWords desc_words(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  const uint64_t d = tc::smem_desc(saddr, lbo_bytes, sbo_bytes);
  return DescWords{(uint32_t)d, (uint32_t)(d >> 32)};
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_i8_words(uint32_t d_tmem, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi,
                                             uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
// k = descriptor words of the K image (desc_words(kimg, kImgChunk, 128)), q = of the Q image
// (desc_words(qimg, 2 NPAD 16, 128)).  HD / 32 MMAs: one per 32 dims.
template <int NPAD, int HD = 128>
__device__ __forceinline__ void issue_qk_i8_words(uint32_t s_tmem, DescWords k, DescWords q) {
  constexpr uint32_t idesc = idesc_i8(128, 2 * NPAD, 0, 0);
  constexpr uint32_t ka = (2 * kImgChunk) >> 4, qa = (2 * (2 * NPAD * 16)) >> 4;
  mma_i8_words<false>(s_tmem, k.lo, k.hi, q.lo, q.hi, idesc);
#pragma unroll
  for (int kk = 1; kk < HD / 32; ++kk) mma_i8_words<true>(s_tmem, k.lo + kk * ka, k.hi, q.lo + kk * qa, q.hi, idesc);
}
// v = desc_words(vimg, 128, kImgChunk), pd = desc_words(pimg, 128, kDigitChunk).  One chain of four
// MMAs (32 keys each) per 128 dims of the head: dims 128 h ... land in the accumulator at
// o_tmem + h PD NPAD.  For a head of 64 dims the M = 128 instruction also reads the 64 "rows"
// after the V image (whatever bytes follow it in shared memory): integer garbage in TMEM lanes
// 64-127, which nothing reads.
template <int NPAD, int PD, int HD = 128>
__device__ __forceinline__ void issue_pv_i8_words(uint32_t o_tmem, DescWords v, DescWords pd) {
  constexpr uint32_t idesc = idesc_i8(128, PD * NPAD, 1, 1);
  constexpr uint32_t step = (4 * 128) >> 4;
#pragma unroll
  for (int h = 0; h < I8Geom<HD>::halves; ++h) {
    const uint32_t vlo = v.lo + h * ((8 * kImgChunk) >> 4), o = o_tmem + h * (PD * NPAD);
    mma_i8_words<false>(o, vlo, v.hi, pd.lo, pd.hi, idesc);
    mma_i8_words<true>(o, vlo + step, v.hi, pd.lo + step, pd.hi, idesc);
    mma_i8_words<true>(o, vlo + 2 * step, v.hi, pd.lo + 2 * step, pd.hi, idesc);
    mma_i8_words<true>(o, vlo + 3 * step, v.hi, pd.lo + 3 * step, pd.hi, idesc);
  }
}

}  // namespace pthb200
