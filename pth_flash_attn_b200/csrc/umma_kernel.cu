// tcgen05 attention kernel, head size 128, token-major ("swap-AB") orientation:
// the 128 keys of a KV tile sit on the MMA M dimension and the query rows of a
// row tile (G heads x up to bq tokens, padded to NPAD = 16/32/64) on N.  Decode,
// speculative verification and windowed drafters have few rows per KV head, so
// this orientation spends tensor work on keys instead of on padding, and the
// kernel stays bound by the HBM reads of the cache.
//
// One CTA (128 threads) = one work item (row tile, KV head, split).  Per tile:
//   0. thread t resolves key t of the tile after next through the block table
//      into one byte offset (shared by the four cache streams) in shared memory;
//   1. the raw cell bytes of the tile, prefetched one tile ahead into registers
//      with coalesced 8-byte (K) and 4-byte (V) loads, are widened int8 -> bf16
//      and stored as MMA operand images (umma_tile.cuh);
//   2. thread 0 issues S^T = K Q^T into TMEM; thread t then owns key t: it reads
//      the scores of the live rows, applies k_scale[t] * softmax_scale * log2(e)
//      and, on tiles that touch a row's range boundary, the visibility mask;
//   3. the running row maxima are agreed through warp reductions + shared
//      memory; p = exp2(s - m); P[t, :] = bf16(p * v_scale[t]) goes to the P image,
//      the unscaled p is summed per thread;
//   4. O^T in TMEM is rescaled when a maximum grew, then thread 0 issues
//      O^T += V^T P.
// Epilogue: thread d owns output column d of every row: out = O^T / l.
//
// There is no dequantised copy of the cache anywhere but in shared memory.
// Every wait on an mbarrier is bounded; a wait that gives up sets bit 0 of the
// library's status word and the CTA finishes normally (its results are then
// meaningless, but nothing hangs and TMEM is released).
#include "params.cuh"
#include "umma_tile.cuh"

namespace pthb200 {

__device__ unsigned int g_umma_status = 0;

namespace {

constexpr int kThreads = 128;

template <int NPAD>
struct SmemLayout {
  static constexpr int kw = 0;
  static constexpr int vw = kw + kWideBytes;
  static constexpr int qs = vw + kWideBytes;
  static constexpr int ps = qs + NPAD * 256;
  static constexpr int offs = ps + NPAD * 256;        // int64 [2][128] key offsets
  static constexpr int wred = offs + 2 * 128 * 8;     // float [4][NPAD]
  static constexpr int mrun = wred + 4 * NPAD * 4;    // float [NPAD]
  static constexpr int rlo = mrun + NPAD * 4;         // int [NPAD]
  static constexpr int rhi = rlo + NPAD * 4;          // int [NPAD]
  static constexpr int bars = rhi + NPAD * 4;         // 2 x uint64
  static constexpr int tslot = bars + 16;             // uint32
  static constexpr int total = tslot + 16;
};

template <int NPAD>
__host__ __device__ constexpr uint32_t tmem_cols() {
  return 2 * NPAD < 32 ? 32 : 2 * NPAD;
}

// Order-preserving map float -> int so that an integer warp reduction finds the float maximum.
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

struct RawTile {
  uint2 k[16];
  uint2 v[16];
  float ks, vs;
};

__device__ __forceinline__ uint2 ldg8(const uint8_t* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t ldg4(const uint8_t* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

// Byte offset of KV position `pos` (block and slot terms; -1 if pos is outside [kv_lo, kv_hi)).
// The four cache streams share their block and slot strides (checked on the host).
__device__ __forceinline__ int64_t key_offset(const KernelParams& p, const int32_t* bt, int pos, int kv_lo, int kv_hi) {
  if (pos < kv_lo || pos >= kv_hi) return -1;
  int page, s;
  if (p.block_shift >= 0) {
    page = pos >> p.block_shift;
    s = pos & (p.block_size - 1);
  } else {
    page = pos / p.block_size;
    s = pos - page * p.block_size;
  }
  return (int64_t)__ldg(bt + page) * p.k.stride_block + (int64_t)s * p.k.stride_slot;
}

// Thread (tsub = tid / 16, c = tid % 16) fetches chunk c of keys tsub, tsub + 8, ...: the 16
// lanes of a half warp read one key's 128 K bytes (and 128 V bytes) contiguously.
__device__ __forceinline__ void load_tile(const int64_t* offs, const uint8_t* kb, const uint8_t* vb,
                                          const uint8_t* ksb, const uint8_t* vsb, int tid, RawTile& r) {
  const int tsub = tid >> 4;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t off = offs[tsub + 8 * i];
    if (off >= 0) {
      r.k[i] = ldg8(kb + off);
      r.v[i].x = ldg4(vb + off);
      r.v[i].y = ldg4(vb + off + 4);
    } else {
      r.k[i] = make_uint2(0u, 0u);
      r.v[i] = make_uint2(0u, 0u);
    }
  }
  const int64_t off = offs[tid];
  if (off >= 0) {
    r.ks = __uint_as_float(ldg4(ksb + off));
    r.vs = __uint_as_float(ldg4(vsb + off));
  } else {
    r.ks = 0.f;
    r.vs = 0.f;
  }
}

__device__ __forceinline__ void store_tile(uint8_t* kw, uint8_t* vw, int tid, const RawTile& r) {
  const int c = tid & 15, tsub = tid >> 4;
  const int base = c * kChunkStride + tsub * 16;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    *reinterpret_cast<uint4*>(kw + base + i * 128) = widen8_bf16(r.k[i]);
    *reinterpret_cast<uint4*>(vw + base + i * 128) = widen8_bf16(r.v[i]);
  }
}

// Rows of this work item: row n < rows is (token tok0 + n / G, head kvh * G + n % G).
__device__ __forceinline__ void row_target(const KernelParams& p, const RowTile& t, int kvh, int n, int* token, int* head) {
  *token = t.tok0 + n / p.group;
  *head = kvh * p.group + n % p.group;
}

template <int NPAD>
__global__ void __launch_bounds__(kThreads, (NPAD <= 32 ? 3 : 2))
umma_attention_kernel(const __grid_constant__ KernelParams p) {
  using L = SmemLayout<NPAD>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* kw = smem + L::kw;
  uint8_t* vw = smem + L::vw;
  uint8_t* qs = smem + L::qs;
  uint8_t* ps = smem + L::ps;
  int64_t* offs = reinterpret_cast<int64_t*>(smem + L::offs);
  float* wred = reinterpret_cast<float*>(smem + L::wred);
  float* mrun = reinterpret_cast<float*>(smem + L::mrun);
  int* rlo = reinterpret_cast<int*>(smem + L::rlo);
  int* rhi = reinterpret_cast<int*>(smem + L::rhi);
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + L::bars);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::tslot);

  const RowTile t = resolve_row_tile(p, blockIdx.x);
  if (t.req < 0) return;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows = t.ntok * p.group;  // <= NPAD by construction of bq
  int tile_begin, tile_end, range_begin, range_end;
  split_tiles(p, t, split, &tile_begin, &tile_end, &range_begin, &range_end);

  if (tile_begin >= tile_end) {
    // No keys for this work item: zero output, log-sum-exp -inf.
    for (int n = 0; n < rows; ++n) {
      int token, head;
      row_target(p, t, kvh, n, &token, &head);
      if (p.num_splits == 1) {
        store_out_elem(p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head, tid,
                       p.out_dtype, 0.f);
      } else {
        reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                 (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head)[tid] = 0.f;
      }
    }
    if (tid < rows) {
      int token, head;
      row_target(p, t, kvh, tid, &token, &head);
      if (p.num_splits > 1) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                  (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) =
            -INFINITY;
      } else if (p.lse_out != nullptr) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                  (int64_t)head * p.lse_stride_head) = -INFINITY;
      }
    }
    return;
  }

  const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;
  const int c = tid & 15;
  const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head + c * 8;
  const uint8_t* vb = p.v.data + (int64_t)kvh * p.v.stride_head + c * 8;
  const uint8_t* ksb = p.ks.data + (int64_t)kvh * p.ks.stride_head;
  const uint8_t* vsb = p.vs.data + (int64_t)kvh * p.vs.stride_head;

  // ---- set-up: row ranges, barriers, TMEM, Q image, zeroed P image, key offsets ----
  if (tid < NPAD) {
    int lo = 0, hi = -1;
    if (tid < rows) visible_range(p, t, t.first_idx + tid / p.group, &lo, &hi);
    rlo[tid] = lo;
    rhi[tid] = hi;
    mrun[tid] = -INFINITY;
  }
  if (tid == 0) {
    tc::mbar_init(bar_s, 1);
    tc::mbar_init(bar_o, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, tmem_cols<NPAD>());
    tc::tmem_relinquish();
  }
  for (int idx = tid; idx < NPAD * kChunks; idx += kThreads) {
    const int n = idx >> 4, cc = idx & 15;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (n < rows) {
      int token, head;
      row_target(p, t, kvh, n, &token, &head);
      val = *reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token + (int64_t)head * p.q_stride_head +
                                            cc * 16);
    }
    *reinterpret_cast<uint4*>(qs + cc * (NPAD * 16) + n * 16) = val;
  }
#pragma unroll
  for (int j = 0; j < NPAD / 8; ++j)
    *reinterpret_cast<uint4*>(ps + j * kPGroupStride + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
  offs[tid] = key_offset(p, bt, tile_begin * kTileKeys + tid, range_begin, range_end);
  offs[128 + tid] =
      tile_begin + 1 < tile_end ? key_offset(p, bt, (tile_begin + 1) * kTileKeys + tid, range_begin, range_end) : -1;
  // Tiles whose keys every live row sees need no mask: [mask_lo, mask_hi] is the
  // position range visible to all rows (lo and hi do not decrease with the row).
  int mask_lo, mask_hi, tmp;
  visible_range(p, t, t.first_idx + t.ntok - 1, &mask_lo, &tmp);
  visible_range(p, t, t.first_idx, &tmp, &mask_hi);

  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t s_tmem = tmem_base;          // columns [0, NPAD)
  const uint32_t o_tmem = tmem_base + NPAD;   // columns [NPAD, 2 NPAD)
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  const uint32_t kw_s = tc::smem_u32(kw), vw_s = tc::smem_u32(vw), qs_s = tc::smem_u32(qs), ps_s = tc::smem_u32(ps);

  RawTile raw;
  load_tile(offs, kb, vb, ksb, vsb, tid, raw);

  float l_part[NPAD];
#pragma unroll
  for (int n = 0; n < NPAD; ++n) l_part[n] = 0.f;
  bool ok = true;
  uint32_t it = 0;

  for (int tile = tile_begin; tile < tile_end; ++tile, ++it) {
    // The previous tile's PV MMA reads vw and ps: wait for it before overwriting them.
    if (it > 0) {
      ok &= tc::mbar_wait_bounded(bar_o, (it - 1) & 1);
      tc::fence_after_sync();
    }
    store_tile(kw, vw, tid, raw);
    const float ks_cur = raw.ks, vs_cur = raw.vs;
    if (tile + 1 < tile_end) load_tile(offs + ((it + 1) & 1) * 128, kb, vb, ksb, vsb, tid, raw);

    tc::fence_async_smem();
    __syncthreads();  // (A) operand images complete; the offsets of tile + 1 have been consumed
    if (tid == 0) {
      tc::fence_after_sync();
      issue_qk<NPAD>(s_tmem, kw_s, qs_s, kChunkStride);
      tc::mma_commit(bar_s);
    }
    // Offsets of the tile after next go where this tile's offsets were.
    if (tile + 2 < tile_end) offs[(it & 1) * 128 + tid] = key_offset(p, bt, (tile + 2) * kTileKeys + tid, range_begin, range_end);

    ok &= tc::mbar_wait_bounded(bar_s, it & 1);
    tc::fence_after_sync();

    uint32_t sr[NPAD];
#pragma unroll
    for (int g = 0; g < NPAD / 16; ++g)
      if (g * 16 < rows) tc::tmem_ld16(s_tmem + lane_addr + g * 16, sr + g * 16);
    tc::tmem_ld_wait();
    const int pos = tile * kTileKeys + tid;
    const bool interior = tile * kTileKeys >= mask_lo && tile * kTileKeys + (kTileKeys - 1) <= mask_hi;
    const float mult = ks_cur * p.scale_log2;
    float s[NPAD];
#pragma unroll
    for (int n = 0; n < NPAD; ++n) {
      if (n < rows) {
        const bool vis = interior || (pos >= rlo[n] && pos <= rhi[n]);
        s[n] = vis ? __uint_as_float(sr[n]) * mult : -INFINITY;
        const int key = __reduce_max_sync(0xffffffffu, float_key(s[n]));
        if (lane == (n & 31)) wred[warp * NPAD + n] = key_float(key);
      }
    }
    __syncthreads();  // (B) per-warp maxima visible

    bool grew = false;
#pragma unroll
    for (int n = 0; n < NPAD; ++n) {
      if (n < rows) {
        const float m_old = mrun[n];
        const float m_tile = fmaxf(fmaxf(wred[n], wred[NPAD + n]), fmaxf(wred[2 * NPAD + n], wred[3 * NPAD + n]));
        const float m_new = fmaxf(m_old, m_tile);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float a = fast_exp2(m_old - m_use);
        const float pr = fast_exp2(s[n] - m_use);
        l_part[n] = l_part[n] * a + pr;
        grew |= (m_new > m_old) && (m_old > -INFINITY);
        s[n] = pr * vs_cur;
      } else {
        s[n] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < NPAD / 8; ++j) {
      if (j * 8 < rows) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 b = __floats2bfloat162_rn(s[j * 8 + 2 * e], s[j * 8 + 2 * e + 1]);
          pk[e] = *reinterpret_cast<const uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(ps + j * kPGroupStride + tid * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }

    // A grown maximum rescales the accumulated O^T columns (thread = lane d of O^T).
    if (it > 0 && grew) {
#pragma unroll
      for (int g = 0; g < NPAD / 16; ++g) {
        if (g * 16 < rows) {
          uint32_t o[16];
          tc::tmem_ld16(o_tmem + lane_addr + g * 16, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int n = g * 16 + e;
            const float m_old = mrun[n];
            const float m_tile = fmaxf(fmaxf(wred[n], wred[NPAD + n]), fmaxf(wred[2 * NPAD + n], wred[3 * NPAD + n]));
            const float m_new = fmaxf(m_old, m_tile);
            const float a = (m_new == -INFINITY || n >= rows) ? 1.f : fast_exp2(m_old - m_new);
            o[e] = __float_as_uint(__uint_as_float(o[e]) * a);
          }
          tc::tmem_st16(o_tmem + lane_addr + g * 16, o);
        }
      }
      tc::tmem_st_wait();
    }

    tc::fence_before_sync();
    tc::fence_async_smem();
    __syncthreads();  // (C) P image and O^T rescale complete; mrun/wred reads done
    if (tid < rows) {
      const float m_tile =
          fmaxf(fmaxf(wred[tid], wred[NPAD + tid]), fmaxf(wred[2 * NPAD + tid], wred[3 * NPAD + tid]));
      mrun[tid] = fmaxf(mrun[tid], m_tile);
    }
    if (tid == 0) {
      tc::fence_after_sync();
      issue_pv<NPAD>(o_tmem, vw_s, ps_s, kChunkStride, it > 0);
      tc::mma_commit(bar_o);
    }
  }

  // ---- epilogue -------------------------------------------------------------
  ok &= tc::mbar_wait_bounded(bar_o, (it - 1) & 1);
  tc::fence_after_sync();
  __syncthreads();  // wred free for the row sums (its last readers are past barrier C)
#pragma unroll
  for (int n = 0; n < NPAD; ++n) {
    if (n < rows) {
      float v = l_part[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == (n & 31)) wred[warp * NPAD + n] = v;
    }
  }
  __syncthreads();

  uint32_t ot[NPAD];
#pragma unroll
  for (int g = 0; g < NPAD / 16; ++g)
    if (g * 16 < rows) tc::tmem_ld16(o_tmem + lane_addr + g * 16, ot + g * 16);
  tc::tmem_ld_wait();
#pragma unroll
  for (int n = 0; n < NPAD; ++n) {
    if (n < rows) {
      const float l = wred[n] + wred[NPAD + n] + wred[2 * NPAD + n] + wred[3 * NPAD + n];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float val = __uint_as_float(ot[n]) * inv;
      int token, head;
      row_target(p, t, kvh, n, &token, &head);
      if (p.num_splits == 1) {
        store_out_elem(p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head, tid,
                       p.out_dtype, val);
      } else {
        reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                 (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head)[tid] = val;
      }
    }
  }
  if (tid < rows) {
    const float l = wred[tid] + wred[NPAD + tid] + wred[2 * NPAD + tid] + wred[3 * NPAD + tid];
    const float lse2 = l > 0.f ? mrun[tid] + log2f(l) : -INFINITY;
    int token, head;
    row_target(p, t, kvh, tid, &token, &head);
    if (p.num_splits > 1) {
      *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) = lse2;
    } else if (p.lse_out != nullptr) {
      *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                (int64_t)head * p.lse_stride_head) = lse2 * kLn2;
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols<NPAD>());
  if (!ok && tid == 0) atomicOr(&g_umma_status, 1u);
}

template <int NPAD>
cudaError_t launch_variant(const KernelParams& p, cudaStream_t stream) {
  constexpr int smem = SmemLayout<NPAD>::total;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_attention_kernel<NPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  umma_attention_kernel<NPAD><<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int NPAD>
cudaError_t launch_npad(const KernelParams& p, cudaStream_t stream) {
  return launch_variant<NPAD>(p, stream);
}

}  // namespace

bool umma_supports(const KernelParams& p, const char** why) {
  auto mult8 = [](int64_t v) { return v % 8 == 0; };
  if (p.head_size != 128) {
    *why = "head_size is not 128";
    return false;
  }
  if (p.q_dtype != PTH_ATTN_BF16) {
    *why = "q is not bf16";
    return false;
  }
  if (reinterpret_cast<uintptr_t>(p.k.data) % 8 != 0 || !mult8(p.k.stride_block) || !mult8(p.k.stride_slot) ||
      !mult8(p.k.stride_head)) {
    *why = "k_cache rows are not 8-byte aligned";
    return false;
  }
  const StreamParams* others[3] = {&p.v, &p.ks, &p.vs};
  for (const StreamParams* s : others) {
    if (s->stride_block != p.k.stride_block || s->stride_slot != p.k.stride_slot) {
      *why = "the cache streams do not share their block and slot strides";
      return false;
    }
  }
  *why = "";
  return true;
}

cudaError_t launch_umma_attention(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  // Row tiles of at most 64 rows: shorten bq if the caller's tile is taller.
  const int cap = 64 / p.group;
  set_row_tile(p, p.bq > cap ? cap : p.bq);
  const int rows = p.bq * p.group;
  if (rows <= 16) return launch_npad<16>(p, stream);
  if (rows <= 32) return launch_npad<32>(p, stream);
  return launch_npad<64>(p, stream);
}

}  // namespace pthb200

#include "umma_tile_test.cuh"
