// Included at the end of umma_i8_kernel.cu (shares its helpers and status word).
#pragma once

// ---- unit kernel of the integer building blocks ------------------------------
// One CTA copies one raw 128-key K tile and V tile into operand images, takes
// ready-made int8 digit images of Q ([32][128]: rows 0-15 high digit, 16-31 low)
// and P ([128 keys][48]), runs both MMA chains and returns the int32 accumulators:
//   s_out[key][n'] = sum_d k[key][d] * q[n'][d]       (128 x 32)
//   o_out[d][n']   = sum_key v[key][d] * pm[key][n']  (128 x 48)
namespace pthb200 {
namespace {

__global__ void __launch_bounds__(128) i8_tile_test_kernel(const int8_t* k, const int8_t* q, const int8_t* v,
                                                           const int8_t* pm, int32_t* s_out, int32_t* o_out) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* kimg = smem;
  uint8_t* vimg = kimg + kImgBytes;
  uint8_t* qimg = vimg + kImgBytes;        // [8][32][16]
  uint8_t* pimg = qimg + 8 * 32 * 16;      // [3][128][16]
  uint64_t* bar = reinterpret_cast<uint64_t*>(pimg + 3 * kDigitChunk);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(bar + 2);
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    tc::mbar_init(bar, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 128);
    tc::tmem_relinquish();
  }
  for (int j = 0; j < 8; ++j) {
    *reinterpret_cast<uint4*>(kimg + j * kImgChunk + tid * 16) = *reinterpret_cast<const uint4*>(k + tid * 128 + j * 16);
    *reinterpret_cast<uint4*>(vimg + j * kImgChunk + tid * 16) = *reinterpret_cast<const uint4*>(v + tid * 128 + j * 16);
  }
  for (int idx = tid; idx < 32 * 8; idx += 128) {
    const int n = idx >> 3, j = idx & 7;
    *reinterpret_cast<uint4*>(qimg + j * (32 * 16) + n * 16) = *reinterpret_cast<const uint4*>(q + n * 128 + j * 16);
  }
  for (int c = 0; c < 3; ++c)
    *reinterpret_cast<uint4*>(pimg + c * kDigitChunk + tid * 16) = *reinterpret_cast<const uint4*>(pm + tid * 48 + c * 16);
  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  if (tid == 0) {
    issue_qk_i8<16>(tmem_base, tc::smem_u32(kimg), tc::smem_u32(qimg));
    issue_pv_i8<16, 3>(tmem_base + 32, tc::smem_u32(vimg), tc::smem_u32(pimg));
    tc::mma_commit(bar);
  }
  const bool ok = tc::mbar_wait_bounded(bar, 0);
  tc::fence_after_sync();
  for (int g = 0; g < 8; ++g) {
    uint32_t r[4];
    tmem_ld4(tmem_base + lane_addr + g * 4, r);
    tc::tmem_ld_wait();
    for (int e = 0; e < 4; ++e) s_out[tid * 32 + g * 4 + e] = (int32_t)r[e];
  }
  for (int g = 0; g < 12; ++g) {
    uint32_t r[4];
    tmem_ld4(tmem_base + 32 + lane_addr + g * 4, r);
    tc::tmem_ld_wait();
    for (int e = 0; e < 4; ++e) o_out[tid * 48 + g * 4 + e] = (int32_t)r[e];
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 128);
  if (!ok && tid == 0) atomicOr(&g_i8_status, 8u);
}

}  // namespace
}  // namespace pthb200

extern "C" int32_t pthb200_test_tile_i8(const void* k, const void* q, const void* v, const void* pm, int32_t* s_out,
                                        int32_t* o_out, void* stream) {
  using namespace pthb200;
  const int smem = 2 * kImgBytes + 8 * 32 * 16 + 3 * kDigitChunk + 64;
  if (cudaFuncSetAttribute(i8_tile_test_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return PTH_ATTN_ECUDA;
  i8_tile_test_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int8_t*>(k), static_cast<const int8_t*>(q), static_cast<const int8_t*>(v),
      static_cast<const int8_t*>(pm), s_out, o_out);
  return cudaGetLastError() == cudaSuccess ? PTH_ATTN_OK : PTH_ATTN_ECUDA;
}
