// Quantising KV-cache writer: the step in front of the attention path.
//
// For every new token and KV head it turns one K row and one V row (fp32 / fp16 / bf16) into
// the cache's int8_per_token_head form, with the arithmetic of the writer the cache format
// is defined by, step for step in fp32 so that the bytes are identical:
//   absmax = max |x_d|;   scale = max(absmax / 127, 1e-6);   inv = 1 / scale
//   q_d = clamp(trunc(x_d * inv +- 0.5), -128, 127)          (round half away from zero)
// and stores the D int8 values and the fp32 scale through the same four strided streams the
// attention op reads (K bytes, V bytes, K scales, V scales), at the slot slot_mapping names:
// block = slot / block_size, position = slot % block_size; a negative slot skips the token.
//
// One warp per row: lane l owns D / 32 consecutive elements, the row maximum is a warp
// reduction, and a row's bytes leave as one coalesced store.  The kernel is bound by HBM
// (it reads 2 T Hkv D source elements and writes T Hkv (2 D + 8) bytes).
#include "params.cuh"

namespace pthb200 {
namespace {

constexpr int kWriterThreads = 256;

struct WriterParams {
  const uint8_t* key;
  const uint8_t* value;
  int64_t key_stride_token, key_stride_head, value_stride_token, value_stride_head;
  StreamParams k, v, ks, vs;  // data pointers are written through
  const int64_t* slot_mapping;
  int32_t src_dtype, block_size, num_kv_heads, num_tokens;
};

template <int EPL>  // elements per lane = D / 32
__device__ __forceinline__ void load_row(const uint8_t* row, int lane, int dtype, float (&x)[EPL]) {
  if (dtype == PTH_ATTN_F32) {
    const float* p = reinterpret_cast<const float*>(row) + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = p[e];
  } else if (dtype == PTH_ATTN_BF16) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(row) + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(p[e]);
  } else {
    const __half* p = reinterpret_cast<const __half*>(row) + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = __half2float(p[e]);
  }
}

template <int EPL>
__global__ void __launch_bounds__(kWriterThreads) kv_writer_kernel(const WriterParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kWriterThreads + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * kWriterThreads) >> 5;
  const int64_t rows = 2ll * p.num_tokens * p.num_kv_heads;  // K rows, then V rows
  for (int64_t r = warp; r < rows; r += warps) {
    const bool is_v = r >= rows / 2;
    const int64_t tr = is_v ? r - rows / 2 : r;
    const int token = (int)(tr / p.num_kv_heads), head = (int)(tr % p.num_kv_heads);
    const int64_t slot = p.slot_mapping[token];
    if (slot < 0) continue;  // padding token
    const int64_t block = slot / p.block_size, pos = slot % p.block_size;
    const uint8_t* src = is_v ? p.value + token * p.value_stride_token + head * p.value_stride_head
                              : p.key + token * p.key_stride_token + head * p.key_stride_head;
    float x[EPL];
    load_row<EPL>(src, lane, p.src_dtype, x);
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-6f);
    const float inv = __fdiv_rn(1.0f, scale);
    uint8_t q[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      float v = __fmul_rn(x[e], inv);
      v = v >= 0.f ? __fadd_rn(v, 0.5f) : __fadd_rn(v, -0.5f);
      v = fminf(fmaxf(v, -128.0f), 127.0f);
      q[e] = (uint8_t)(int8_t)(int)truncf(v);
    }
    const StreamParams& rows_s = is_v ? p.v : p.k;
    const StreamParams& scale_s = is_v ? p.vs : p.ks;
    uint8_t* dst = const_cast<uint8_t*>(rows_s.data) + block * rows_s.stride_block + pos * rows_s.stride_slot +
                   head * rows_s.stride_head + lane * EPL;
    if constexpr (EPL == 2) {
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(q[0] | (q[1] << 8));
    } else {
#pragma unroll
      for (int w = 0; w < EPL / 4; ++w)
        reinterpret_cast<uint32_t*>(dst)[w] = (uint32_t)q[4 * w] | ((uint32_t)q[4 * w + 1] << 8) |
                                              ((uint32_t)q[4 * w + 2] << 16) | ((uint32_t)q[4 * w + 3] << 24);
    }
    if (lane == 0) {
      *reinterpret_cast<float*>(const_cast<uint8_t*>(scale_s.data) + block * scale_s.stride_block +
                                pos * scale_s.stride_slot + head * scale_s.stride_head) = scale;
    }
  }
}

}  // namespace

cudaError_t launch_kv_writer(const PthB200WriteArgs& a, cudaStream_t stream) {
  WriterParams p{};
  p.key = static_cast<const uint8_t*>(a.key);
  p.value = static_cast<const uint8_t*>(a.value);
  p.key_stride_token = a.key_stride_token;
  p.key_stride_head = a.key_stride_head;
  p.value_stride_token = a.value_stride_token;
  p.value_stride_head = a.value_stride_head;
  auto stream_of = [](const PthAttnStream& s) {
    return StreamParams{static_cast<const uint8_t*>(s.data), s.stride_block, s.stride_slot, s.stride_head};
  };
  p.k = stream_of(a.k_cache);
  p.v = stream_of(a.v_cache);
  p.ks = stream_of(a.k_scale);
  p.vs = stream_of(a.v_scale);
  p.slot_mapping = a.slot_mapping;
  p.src_dtype = a.src_dtype;
  p.block_size = a.block_size;
  p.num_kv_heads = a.num_kv_heads;
  p.num_tokens = a.num_tokens;
  const int64_t rows = 2ll * a.num_tokens * a.num_kv_heads;
  const int64_t want = (rows + kWriterThreads / 32 - 1) / (kWriterThreads / 32);
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));  // a few CTAs per SM, grid-stride
  switch (a.head_size) {
    case 64:
      kv_writer_kernel<2><<<grid, kWriterThreads, 0, stream>>>(p);
      break;
    case 128:
      kv_writer_kernel<4><<<grid, kWriterThreads, 0, stream>>>(p);
      break;
    default:
      kv_writer_kernel<8><<<grid, kWriterThreads, 0, stream>>>(p);
      break;
  }
  return cudaGetLastError();
}

}  // namespace pthb200
