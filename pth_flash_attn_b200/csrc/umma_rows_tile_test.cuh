// Unit kernel for the row-major building blocks (umma_rows.cuh): one CTA widens one
// 128-key K tile and V tile, stages a 128-row Q image, and returns
//   s_out[row][key] = sum_d Q[row][d] * K[key][d]           (128 x 128 fp32)
//   o_out[row][d]   = sum_key P[row][key] * V[key][d]       (128 x 128 fp32)
// with P taken from `pm` (bf16 [128 rows][128 keys]) and handed to the MMA through
// TMEM, as the attention kernel does.  Included at the end of umma_rows_kernel.cu.
#pragma once

namespace pthb200 {
namespace rows_tile_test {

__global__ void __launch_bounds__(128) umma_rows_tile_test_kernel(const int8_t* k, const __nv_bfloat16* q,
                                                                  const int8_t* v, const __nv_bfloat16* pm,
                                                                  float* s_out, float* o_out) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* kw = smem;
  uint8_t* vw = kw + kWideBytes;
  uint8_t* qs = vw + kWideBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(qs + kQImageBytes);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(bar + 2);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    tc::mbar_init(&bar[0], 1);
    tc::mbar_init(&bar[1], 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 512);
    tc::tmem_relinquish();
  }
  const int c = tid & 15, tsub = tid >> 4;
  for (int i = 0; i < 16; ++i) {
    const int key = tsub + 8 * i;
    const uint2 kr = *reinterpret_cast<const uint2*>(k + key * 128 + c * 8);
    const uint2 vr = *reinterpret_cast<const uint2*>(v + key * 128 + c * 8);
    *reinterpret_cast<uint4*>(kw + c * kChunkStride + key * 16) = widen8_bf16(kr);
    *reinterpret_cast<uint4*>(vw + c * kChunkStride + key * 16) = widen8_bf16(vr);
    // Q image: same form, rows in place of keys
    *reinterpret_cast<uint4*>(qs + c * kChunkStride + key * 16) = *reinterpret_cast<const uint4*>(q + key * 128 + c * 8);
  }
  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  const uint32_t s_col = 0, p_col = 128, o_col = 256;
  if (tid == 0) {
    issue_qk_rows(tmem_base + s_col, tc::smem_u32(qs), tc::smem_u32(kw));
    tc::mma_commit(&bar[0]);
  }
  bool ok = tc::mbar_wait_bounded(&bar[0], 0);
  tc::fence_after_sync();
  uint32_t r[32];
  for (int j = 0; j < 4; ++j) {
    tc::tmem_ld32(tmem_base + s_col + j * 32 + lane_addr, r);
    tc::tmem_ld_wait();
    for (int n = 0; n < 32; ++n) s_out[tid * 128 + j * 32 + n] = __uint_as_float(r[n]);
  }
  // P row of this thread -> TMEM, two bf16 per column
  const uint32_t* prow = reinterpret_cast<const uint32_t*>(pm + tid * 128);
  for (int j = 0; j < 2; ++j) {
    for (int n = 0; n < 32; ++n) r[n] = prow[j * 32 + n];
    tc::tmem_st32(tmem_base + p_col + j * 32 + lane_addr, r);
  }
  tc::tmem_st_wait();
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    tc::fence_after_sync();
    issue_pv_rows(tmem_base + o_col, tmem_base + p_col, tc::smem_u32(vw), false);
    tc::mma_commit(&bar[1]);
  }
  ok &= tc::mbar_wait_bounded(&bar[1], 0);
  tc::fence_after_sync();
  for (int j = 0; j < 4; ++j) {
    tc::tmem_ld32(tmem_base + o_col + j * 32 + lane_addr, r);
    tc::tmem_ld_wait();
    for (int n = 0; n < 32; ++n) o_out[tid * 128 + j * 32 + n] = __uint_as_float(r[n]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
  if (!ok && tid == 0) atomicOr(&g_rows_status, 2u);
}

}  // namespace rows_tile_test
}  // namespace pthb200

extern "C" int32_t pthb200_test_tile_rows(const void* k, const void* q, const void* v, const void* pm, float* s_out,
                                          float* o_out, void* stream) {
  using namespace pthb200;
  using namespace pthb200::rows_tile_test;
  const int smem = 2 * kWideBytes + kQImageBytes + 64;
  auto* fn = umma_rows_tile_test_kernel;
  cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return PTH_ATTN_ECUDA;
  fn<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int8_t*>(k), static_cast<const __nv_bfloat16*>(q), static_cast<const int8_t*>(v),
      static_cast<const __nv_bfloat16*>(pm), s_out, o_out);
  return cudaGetLastError() == cudaSuccess ? PTH_ATTN_OK : PTH_ATTN_ECUDA;
}
