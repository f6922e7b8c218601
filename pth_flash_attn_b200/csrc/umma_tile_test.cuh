// Unit kernel for the tcgen05 building blocks (umma_tile.cuh): one CTA widens
// one 128-key K tile and V tile, stages Q and P, runs the two MMA chains of
// the attention kernel and returns the raw accumulators:
//   s_out[key][n] = sum_d K[key][d] * Q[n][d]        (128 x 16 fp32)
//   o_out[d][n]   = sum_key V[key][d] * P[key][n]    (128 x 16 fp32)
// Bit 0 of `variant` selects the chunk stride of the widened image (2064 bytes as
// the attention kernel uses, or the dense 2048), so a test can tell a layout
// mistake from a padding mistake.
// Included at the end of umma_kernel.cu (it shares that file's status word).
#pragma once

namespace pthb200 {
namespace tile_test {

constexpr int NPAD = 16;

__global__ void __launch_bounds__(128) umma_tile_test_kernel(const int8_t* k, const __nv_bfloat16* q, const int8_t* v,
                                                             const __nv_bfloat16* pm, float* s_out, float* o_out,
                                                             int chunk_stride) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* kw = smem;
  uint8_t* vw = kw + kWideBytes;
  uint8_t* qs = vw + kWideBytes;
  uint8_t* ps = qs + NPAD * 256;
  uint64_t* bar = reinterpret_cast<uint64_t*>(ps + NPAD * 256);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(bar + 2);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    tc::mbar_init(bar, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 32);
    tc::tmem_relinquish();
  }
  const int c = tid & 15, tsub = tid >> 4;
  for (int i = 0; i < 16; ++i) {
    const int key = tsub + 8 * i;
    const uint2 kr = *reinterpret_cast<const uint2*>(k + key * 128 + c * 8);
    const uint2 vr = *reinterpret_cast<const uint2*>(v + key * 128 + c * 8);
    *reinterpret_cast<uint4*>(kw + c * chunk_stride + key * 16) = widen8_bf16(kr);
    *reinterpret_cast<uint4*>(vw + c * chunk_stride + key * 16) = widen8_bf16(vr);
  }
  for (int idx = tid; idx < NPAD * kChunks; idx += 128) {
    const int n = idx >> 4, cc = idx & 15;
    *reinterpret_cast<uint4*>(qs + cc * (NPAD * 16) + n * 16) = *reinterpret_cast<const uint4*>(q + n * 128 + cc * 8);
  }
  for (int j = 0; j < NPAD / 8; ++j) {
    *reinterpret_cast<uint4*>(ps + j * kPGroupStride + tid * 16) = *reinterpret_cast<const uint4*>(pm + tid * NPAD + j * 8);
  }
  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  if (tid == 0) {
    issue_qk<NPAD>(tmem_base, tc::smem_u32(kw), tc::smem_u32(qs), chunk_stride);
    issue_pv<NPAD>(tmem_base + NPAD, tc::smem_u32(vw), tc::smem_u32(ps), chunk_stride, false);
    tc::mma_commit(bar);
  }
  const bool ok = tc::mbar_wait_bounded(bar, 0);
  tc::fence_after_sync();
  uint32_t r[16];
  tc::tmem_ld16(tmem_base + lane_addr, r);
  tc::tmem_ld_wait();
  for (int n = 0; n < 16; ++n) s_out[tid * 16 + n] = __uint_as_float(r[n]);
  tc::tmem_ld16(tmem_base + NPAD + lane_addr, r);
  tc::tmem_ld_wait();
  for (int n = 0; n < 16; ++n) o_out[tid * 16 + n] = __uint_as_float(r[n]);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 32);
  if (!ok && tid == 0) atomicOr(&g_umma_status, 2u);
}

}  // namespace tile_test
}  // namespace pthb200

extern "C" int32_t pthb200_test_tile(const void* k, const void* q, const void* v, const void* pm, float* s_out,
                                     float* o_out, int32_t variant, void* stream) {
  using namespace pthb200;
  using namespace pthb200::tile_test;
  const int smem = 2 * kWideBytes + 2 * NPAD * 256 + 64;
  auto* fn = umma_tile_test_kernel;
  cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return PTH_ATTN_ECUDA;
  fn<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int8_t*>(k), static_cast<const __nv_bfloat16*>(q), static_cast<const int8_t*>(v),
      static_cast<const __nv_bfloat16*>(pm), s_out, o_out, (variant & 1) ? kChunkStride : 2048);
  return cudaGetLastError() == cudaSuccess ? PTH_ATTN_OK : PTH_ATTN_ECUDA;
}

// Reads (and clears) the status word that kernels set when a bounded wait gave
// up.  Synchronises the device; meant for tests and debugging.
extern "C" int32_t pthb200_device_status(int32_t* status) {
  unsigned int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return PTH_ATTN_ECUDA;
  if (cudaMemcpyFromSymbol(&v, pthb200::g_umma_status, sizeof(v)) != cudaSuccess) return PTH_ATTN_ECUDA;
  if (cudaMemcpyToSymbol(pthb200::g_umma_status, &zero, sizeof(zero)) != cudaSuccess) return PTH_ATTN_ECUDA;
  unsigned int w = 0;
  if (pthb200::read_i8_status(&w) != cudaSuccess) return PTH_ATTN_ECUDA;
  v |= w;
  if (pthb200::read_rows_status(&w) != cudaSuccess) return PTH_ATTN_ECUDA;
  v |= w;
  if (pthb200::read_rows256_status(&w) != cudaSuccess) return PTH_ATTN_ECUDA;
  v |= w;
  if (pthb200::read_rows2_status(&w) != cudaSuccess) return PTH_ATTN_ECUDA;
  v |= w;
  if (status) *status = (int32_t)v;
  return PTH_ATTN_OK;
}
