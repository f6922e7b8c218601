// Building blocks of the row-major tcgen05 attention kernel (head size 128): query
// rows on the MMA M dimension, as a prefill or a wide verification step wants them.
//
//   S[row, key] = sum_d   Q[row, d] * K[key, d]     A = Q image (K-major), B = K tile (K-major)
//   O[row, d]  += sum_key P[row, key] * V[key, d]   A = P in TMEM,         B = V tile (MN-major)
//
// K and V tiles are the widened bf16 images of umma_tile.cuh (chunk c of 8 d, key t at
// c * kChunkStride + t * 16), which serve as B operands unchanged: for K (N = keys,
// K-major) LBO = chunk stride, SBO = 128; for V (N = d, MN-major) LBO = 128 (next 8
// keys), SBO = chunk stride (next 8 d).  The Q image has the same form with rows in
// place of keys.  P never touches shared memory: the softmax thread of a row writes
// its probabilities as packed bf16 pairs into TMEM (lane = row, 32-bit column j =
// keys 2j, 2j + 1) and the PV MMA reads its A operand from there.
#pragma once

#include "umma_tile.cuh"

namespace pthb200 {

constexpr int kRowsPerTile = 128;                       // MMA M
constexpr int kQImageBytes = kChunks * kChunkStride;    // 33,024 B

namespace tc {

// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

}  // namespace tc

// S = Q K^T over the full head dimension: 8 MMAs of K = 16, N = 128 keys.  One thread.
__device__ __forceinline__ void issue_qk_rows(uint32_t s_tmem, uint32_t q_saddr, uint32_t kw_saddr) {
  constexpr uint32_t idesc = tc::instr_desc(kRowsPerTile, kTileKeys, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk) {
    const uint64_t a = tc::smem_desc(q_saddr + kk * 2 * kChunkStride, kChunkStride, 128);
    const uint64_t b = tc::smem_desc(kw_saddr + kk * 2 * kChunkStride, kChunkStride, 128);
    tc::mma_ss(s_tmem, a, b, idesc, kk > 0);
  }
}

// O (+)= P V over the 128 keys of the tile: 8 MMAs of K = 16 keys, N = 128 (d).  P is read
// from TMEM: 16 keys = 8 columns per step.  One thread.
__device__ __forceinline__ void issue_pv_rows(uint32_t o_tmem, uint32_t p_tmem, uint32_t vw_saddr, bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(kRowsPerTile, kHeadDim, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
#pragma unroll
  for (int kk = 0; kk < kTileKeys / 16; ++kk) {
    const uint64_t b = tc::smem_desc(vw_saddr + kk * 256, 128, kChunkStride);
    tc::mma_ts(o_tmem, p_tmem + kk * 8, b, idesc, accumulate || kk > 0);
  }
}

// ---- the same chains for an issuing thread that keeps its descriptors in registers ----
// (low word = start address in 16-byte units: moving an operand by `bytes` adds bytes / 16)
struct RowsDesc {
  uint32_t lo, hi;
};
__device__ __forceinline__ RowsDesc rows_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  const uint64_t d = tc::smem_desc(saddr, lbo_bytes, sbo_bytes);
  return RowsDesc{(uint32_t)d, (uint32_t)(d >> 32)};
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ss_words(uint32_t d_tmem, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi,
                                             uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
__device__ __forceinline__ void mma_ts_words(uint32_t d_tmem, uint32_t a_tmem, uint32_t blo, uint32_t bhi, uint32_t idesc,
                                             bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(blo), "r"(bhi), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// q = rows_desc(Q image, kChunkStride, 128), k = rows_desc(K image, kChunkStride, 128)
__device__ __forceinline__ void issue_qk_rows_words(uint32_t s_tmem, RowsDesc q, RowsDesc k) {
  constexpr uint32_t idesc = tc::instr_desc(kRowsPerTile, kTileKeys, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
  constexpr uint32_t step = (2 * kChunkStride) >> 4;
  mma_ss_words<false>(s_tmem, q.lo, q.hi, k.lo, k.hi, idesc);
#pragma unroll
  for (int kk = 1; kk < kHeadDim / 16; ++kk)
    mma_ss_words<true>(s_tmem, q.lo + kk * step, q.hi, k.lo + kk * step, k.hi, idesc);
}
// v = rows_desc(V image, 128, kChunkStride)
__device__ __forceinline__ void issue_pv_rows_words(uint32_t o_tmem, uint32_t p_tmem, RowsDesc v, bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(kRowsPerTile, kHeadDim, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
#pragma unroll
  for (int kk = 0; kk < kTileKeys / 16; ++kk)
    mma_ts_words(o_tmem, p_tmem + kk * 8, v.lo + kk * (256 >> 4), v.hi, idesc, accumulate || kk > 0);
}

// PV of one tile as two chains: keys 0-63 (P columns 0-31 of the S buffer, V rows 0-63) into the
// accumulator at o_tmem, keys 64-127 (P columns 64-95, V rows 64-127) into the one at o_tmem + 128.
__device__ __forceinline__ void issue_pv_halves_words(uint32_t o_tmem, uint32_t s_tmem, RowsDesc v, bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(kRowsPerTile, kHeadDim, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int kk = 0; kk < kTileKeys / 32; ++kk)
      mma_ts_words(o_tmem + h * 128, s_tmem + h * 64 + kk * 8, v.lo + (h * 4 + kk) * (256 >> 4), v.hi, idesc,
                   accumulate || kk > 0);
}

}  // namespace pthb200
