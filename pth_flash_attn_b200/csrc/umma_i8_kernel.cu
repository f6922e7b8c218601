// Integer tcgen05 attention kernel, head size 128, token-major orientation.
//
// The cache holds int8 K and V, so both contractions can run on the int8 tensor
// path (tcgen05.mma.kind::i8, int32 accumulators in TMEM) with the cache bytes
// used AS STORED: the raw bytes of a 128-key tile are copied global -> shared
// (cp.async, through the block table) straight into the MMA operand images.
// Nothing is widened, dequantised or converted on the way.
//
// The two floating-point operands become exact sums of int8 "digits":
//   Q row n:  q = sq[n] * (256 qh + ql),   qh, ql int8     (sq = absmax / 32512)
//   P key t:  p * v_scale[t] = u[n] * sum_k 128^k d_k,     0 <= d_k < 128
// with one unit u[n] per (KV tile, row), so the dynamic range that fixed point
// must cover is that of ONE tile; the digits sit side by side on the MMA N
// dimension:
//   S^T[key, (digit, row)]  = sum_d   K[key, d] * Qdigit[row, d]     (N = 2 NPAD)
//   O^T[d,   (digit, row)]  = sum_key V[key, d] * Pdigit[key, row]   (N = PD NPAD)
// Thread t owns key t when it turns S^T into probabilities and owns output
// column d = t when it folds O^T of a tile into its fp32 register accumulator
// (acc = acc * alpha + O^T * u), so TMEM never holds a value that needs
// rescaling.  Integer MMAs are exact; the only roundings are the 16-bit
// quantisation of q (relative 2^-16 of the row maximum) and the 7 PD-bit
// quantisation of p * v_scale (relative 2^-(7 PD + 1) of the tile maximum).
//
// Pipeline per CTA (128 threads, one work item = row tile x KV head x split):
// a ring of NS stages of raw K/V images filled NS - 1 tiles ahead; the QK MMA of
// tile i + 1 is issued before the softmax of tile i, the PV MMA of tile i runs
// under the loads and offset look-ups of later tiles.  Every mbarrier wait is
// bounded (a wait that gives up sets bit 2 of the status word; the CTA still
// finishes and frees its TMEM).
#include "params.cuh"
#include "tcgen05.cuh"

namespace pthb200 {

__device__ unsigned int g_i8_status = 0;

namespace {

constexpr int kThreads = 128;
constexpr int kKeys = 128;
constexpr int kDigitChunk = kKeys * 16;    // one 16-byte column block of all keys in the P image
// Raw K / V image: column block j (bytes 16 j .. 16 j + 15 of every key's row) at j * kImgChunk,
// key t at + 16 t.  The 16 bytes of padding per block spread the 8 blocks of one key row over
// all banks, so a half warp that copies one 128-byte row writes without conflicts.
constexpr int kImgChunk = kKeys * 16 + 16;
constexpr int kImgBytes = 8 * kImgChunk;   // 16,512 B
constexpr int kStageBytes = 2 * kImgBytes;

template <int NPAD, int PD, int NS>
struct Layout {
  static constexpr int stages = 0;
  static constexpr int qimg = stages + NS * kStageBytes;       // [8][2 NPAD][16]
  static constexpr int pimg = qimg + 8 * 2 * NPAD * 16;        // [PD NPAD / 16][128][16]
  static constexpr int offs = (pimg + PD * NPAD * kKeys + 15) / 16 * 16;        // int64 [128]
  static constexpr int wred = offs + kKeys * 8;                // float [4][NPAD + 1]
  static constexpr int mrun = wred + 4 * (NPAD + 1) * 4;       // float [NPAD]
  static constexpr int alpha = mrun + NPAD * 4;                // float [NPAD]
  static constexpr int unit = alpha + NPAD * 4;                // float [NPAD]
  static constexpr int sq = unit + NPAD * 4;                   // float [NPAD]
  static constexpr int rlo = sq + NPAD * 4;                    // int [NPAD]
  static constexpr int rhi = rlo + NPAD * 4;                   // int [NPAD]
  static constexpr int bars = (rhi + NPAD * 4 + 15) / 16 * 16; // 4 x uint64
  static constexpr int tslot = bars + 32;
  static constexpr int total = tslot + 16;
  // TMEM columns: two S^T buffers of 2 NPAD, two O^T buffers of PD NPAD.
  static constexpr int s_cols = 2 * NPAD;
  static constexpr int o_cols = PD * NPAD;
  static constexpr int tmem_need = 2 * s_cols + 2 * o_cols;
  static constexpr int tmem_alloc = tmem_need <= 32 ? 32 : tmem_need <= 64 ? 64 : tmem_need <= 128 ? 128
                                    : tmem_need <= 256 ? 256 : 512;
};

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

__device__ __forceinline__ uint32_t ldg4(const uint8_t* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
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

// S^T = K Q^T: A = raw K image (K-major: 8 keys x 16 d per core matrix), B = Q digit image
// (K-major, rows = (digit, row)).  One MMA covers 32 d = two 16-byte column blocks.
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

// O^T = V^T P: A = raw V image read MN-major (M = d: 16 d x 8 keys per core matrix), B = P digit
// image (MN-major, N = (digit, row)).  One MMA covers 32 keys = four 8-key groups.
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

// Byte offset of KV position `pos` (block and slot terms; -1 outside [kv_lo, kv_hi)).
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

// Copies the raw K and V rows of one tile into a stage.  K moves in 8-byte pieces: a half
// warp takes one key's 128-byte row (lane c -> bytes 8c .. 8c + 7).  V rows are only 4-byte
// aligned in the cache cell and move in 4-byte pieces: a whole warp takes one key's row.
__device__ __forceinline__ void issue_tile_loads(uint32_t stage, const int64_t* offs, const uint8_t* kb,
                                                 const uint8_t* vb, int tid) {
  {
    const int c = tid & 15, t0 = tid >> 4;
    const uint8_t* src0 = kb + c * 8;
    const uint32_t dst0 = stage + (c >> 1) * kImgChunk + (c & 1) * 8;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const int tok = t0 + 8 * r;
      const int64_t off = offs[tok];
      cp_async8(dst0 + tok * 16, src0 + (off >= 0 ? off : 0), off >= 0 ? 8u : 0u);
    }
  }
  {
    const int w = tid & 31, t0 = tid >> 5;
    const uint8_t* src0 = vb + w * 4;
    const uint32_t dst0 = stage + kImgBytes + (w >> 2) * kImgChunk + (w & 3) * 4;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const int tok = t0 + 4 * r;
      const int64_t off = offs[tok];
      cp_async4(dst0 + tok * 16, src0 + (off >= 0 ? off : 0), off >= 0 ? 4u : 0u);
    }
  }
}

__device__ __forceinline__ void row_target(const KernelParams& p, const RowTile& t, int kvh, int n, int* token, int* head) {
  *token = t.tok0 + n / p.group;
  *head = kvh * p.group + n % p.group;
}

template <int NPAD, int PD, int NS>
__global__ void __launch_bounds__(kThreads, (NPAD <= 16 ? 2 : 1))
umma_i8_attention_kernel(const __grid_constant__ KernelParams p) {
  using L = Layout<NPAD, PD, NS>;
  constexpr int XMAX = (1 << (7 * PD)) - 1;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* qimg = smem + L::qimg;
  uint8_t* pimg = smem + L::pimg;
  int64_t* offs = reinterpret_cast<int64_t*>(smem + L::offs);
  float* wred = reinterpret_cast<float*>(smem + L::wred);
  float* mrun = reinterpret_cast<float*>(smem + L::mrun);
  float* alpha_s = reinterpret_cast<float*>(smem + L::alpha);
  float* unit_s = reinterpret_cast<float*>(smem + L::unit);
  float* sq = reinterpret_cast<float*>(smem + L::sq);
  int* rlo = reinterpret_cast<int*>(smem + L::rlo);
  int* rhi = reinterpret_cast<int*>(smem + L::rhi);
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + L::bars);  // [2]
  uint64_t* bar_o = bar_s + 2;                                    // [2]
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::tslot);

  const RowTile t = resolve_row_tile(p, blockIdx.x);
  if (t.req < 0) return;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows = t.ntok * p.group;  // <= NPAD by construction of bq
  int tile_begin, tile_end, range_begin, range_end;
  split_tiles(p, t, split, &tile_begin, &tile_end, &range_begin, &range_end);

  if (tile_begin >= tile_end) {
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

  const int n_tiles = tile_end - tile_begin;
  const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;
  const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
  const uint8_t* vb = p.v.data + (int64_t)kvh * p.v.stride_head;
  const uint8_t* ksb = p.ks.data + (int64_t)kvh * p.ks.stride_head;
  const uint8_t* vsb = p.vs.data + (int64_t)kvh * p.vs.stride_head;
  const uint32_t stage0 = tc::smem_u32(smem + L::stages);

  // ---- set-up ---------------------------------------------------------------
  if (tid < NPAD) {
    int lo = 0, hi = -1;
    if (tid < rows) visible_range(p, t, t.first_idx + tid / p.group, &lo, &hi);
    rlo[tid] = lo;
    rhi[tid] = hi;
    mrun[tid] = -INFINITY;
  }
  if (tid == 0) {
    tc::mbar_init(&bar_s[0], 1);
    tc::mbar_init(&bar_s[1], 1);
    tc::mbar_init(&bar_o[0], 1);
    tc::mbar_init(&bar_o[1], 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, L::tmem_alloc);
    tc::tmem_relinquish();
  }
  // Q digits: 8 threads per row, 16 elements each.
  for (int base = 0; base < NPAD; base += kThreads / 8) {
    const int n = base + (tid >> 3), part = tid & 7;
    float v[16];
    if (n < rows) {
      int token, head;
      row_target(p, t, kvh, n, &token, &head);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token +
                                                        (int64_t)head * p.q_stride_head + part * 32);
      const uint4 a = src[0], b = src[1];
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[2 * e] = __uint_as_float(w[e] << 16);
        v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) v[e] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const bool finite_row = amax > 0.f && amax < INFINITY;
    const float inv = finite_row ? 32512.f / amax : 0.f;
    uint32_t hi_w[4] = {0, 0, 0, 0}, lo_w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      int qi = __float2int_rn(v[e] * inv);
      qi = max(-32512, min(32512, qi));
      const int qh = (qi + 128) >> 8;
      const int ql = qi - (qh << 8);
      hi_w[e >> 2] |= (uint32_t)(qh & 0xff) << (8 * (e & 3));
      lo_w[e >> 2] |= (uint32_t)(ql & 0xff) << (8 * (e & 3));
    }
    if (n < NPAD) {
      // image row of (digit, n) is digit * NPAD + n; column block `part`
      *reinterpret_cast<uint4*>(qimg + part * (2 * NPAD * 16) + n * 16) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
      *reinterpret_cast<uint4*>(qimg + part * (2 * NPAD * 16) + (NPAD + n) * 16) =
          make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
      if (part == 0) sq[n] = finite_row ? amax / 32512.f : 0.f;
    }
  }
  // P image: zero once (rows that are not live keep zero digits).
  for (int i = tid * 16; i < PD * NPAD * kKeys; i += kThreads * 16)
    *reinterpret_cast<uint4*>(pimg + i) = make_uint4(0u, 0u, 0u, 0u);

  // Tiles whose keys every live row sees need no mask.
  int mask_lo, mask_hi, tmp;
  visible_range(p, t, t.first_idx + t.ntok - 1, &mask_lo, &tmp);
  visible_range(p, t, t.first_idx, &tmp, &mask_hi);

  // Prologue: tiles 0 .. NS - 2 into stages 0 .. NS - 2 (one commit group each).
  float ks_next = 0.f, vs_next = 0.f;
#pragma unroll 1
  for (int j = 0; j < NS - 1; ++j) {
    __syncthreads();
    offs[tid] = j < n_tiles ? key_offset(p, bt, (tile_begin + j) * kKeys + tid, range_begin, range_end) : -1;
    __syncthreads();
    if (j < n_tiles) issue_tile_loads(stage0 + j * kStageBytes, offs, kb, vb, tid);
    cp_async_commit();
    if (j == 0) {
      const int64_t off = offs[tid];
      if (off >= 0) {
        ks_next = __uint_as_float(ldg4(ksb + off));
        vs_next = __uint_as_float(ldg4(vsb + off));
      }
    }
  }
  __syncthreads();  // the last round's readers of offs are done
  offs[tid] = NS - 1 < n_tiles ? key_offset(p, bt, (tile_begin + NS - 1) * kKeys + tid, range_begin, range_end) : -1;
  cp_async_wait<NS - 2>();
  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
  const uint32_t qimg_s = tc::smem_u32(qimg), pimg_s = tc::smem_u32(pimg);
  if (tid == 0) {
    issue_qk_i8<NPAD>(tmem_base, stage0, qimg_s);
    tc::mma_commit(&bar_s[0]);
  }

  float acc[NPAD], l_part[NPAD];
#pragma unroll
  for (int n = 0; n < NPAD; ++n) {
    acc[n] = 0.f;
    l_part[n] = 0.f;
  }
  bool ok = true;

  // Folds O^T of tile j (TMEM buffer j & 1) into the register accumulator.
  auto fold_o = [&](int j) {
    ok &= tc::mbar_wait_bounded(&bar_o[j & 1], (j >> 1) & 1);
    tc::fence_after_sync();
    const uint32_t o_tmem = tmem_base + 2 * L::s_cols + (j & 1) * L::o_cols + lane_addr;
#pragma unroll
    for (int g = 0; g < NPAD / 4; ++g) {
      if (g * 4 < rows) {
        uint32_t d[PD][4];
#pragma unroll
        for (int k = 0; k < PD; ++k) tmem_ld4(o_tmem + k * NPAD + g * 4, d[k]);
        tc::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = g * 4 + e;
          float o = int_to_float(d[PD - 1][e]);
#pragma unroll
          for (int k = PD - 2; k >= 0; --k) o = fmaf(o, 128.f, int_to_float(d[k][e]));
          acc[n] = fmaf(acc[n], alpha_s[n], o * unit_s[n]);
        }
      }
    }
  };

#pragma unroll 1
  for (int i = 0; i < n_tiles; ++i) {
    const uint32_t stage = stage0 + (i % NS) * kStageBytes;
    const float ks_cur = ks_next, vs_cur = vs_next;
    // (a) the next tile's bytes have landed: issue its QK MMA.
    if (i + 1 < n_tiles) {
      cp_async_wait<(NS >= 3 ? NS - 3 : 0)>();
      tc::fence_async_smem();
    }
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0 && i + 1 < n_tiles) {
      tc::fence_after_sync();
      issue_qk_i8<NPAD>(tmem_base + ((i + 1) & 1) * L::s_cols, stage0 + ((i + 1) % NS) * kStageBytes, qimg_s);
      tc::mma_commit(&bar_s[(i + 1) & 1]);
    }
    // O^T of the previous tile: after this the P image and stage (i - 1) % NS are free, and
    // that stage is refilled at once (tile i + NS - 1; its offsets were stored one iteration
    // ago), so the copy has a whole iteration to land before its QK MMA is issued.
    if (i > 0) fold_o(i - 1);
    {
      const int tile_new = i + NS - 1;
      if (tile_new < n_tiles) issue_tile_loads(stage0 + (tile_new % NS) * kStageBytes, offs, kb, vb, tid);
      cp_async_commit();
    }
    // Block-table look-up for the refill of the next iteration; scales of the next tile.
    const int64_t off_new =
        i + NS < n_tiles ? key_offset(p, bt, (tile_begin + i + NS) * kKeys + tid, range_begin, range_end) : -1;
    if (i + 1 < n_tiles) {
      const int64_t off = key_offset(p, bt, (tile_begin + i + 1) * kKeys + tid, range_begin, range_end);
      ks_next = 0.f;
      vs_next = 0.f;
      if (off >= 0) {
        ks_next = __uint_as_float(ldg4(ksb + off));
        vs_next = __uint_as_float(ldg4(vsb + off));
      }
    }

    // (b) scores of this tile.
    ok &= tc::mbar_wait_bounded(&bar_s[i & 1], (i >> 1) & 1);
    tc::fence_after_sync();
    const uint32_t s_tmem = tmem_base + (i & 1) * L::s_cols + lane_addr;
    const int pos = (tile_begin + i) * kKeys + tid;
    const bool interior = (tile_begin + i) * kKeys >= mask_lo && (tile_begin + i) * kKeys + (kKeys - 1) <= mask_hi;
    const float mult = ks_cur * p.scale_log2;
    float s[NPAD];
#pragma unroll
    for (int g = 0; g < NPAD / 4; ++g) {
      if (g * 4 < rows) {
        uint32_t hi[4], lo[4];
        tmem_ld4(s_tmem + g * 4, hi);
        tmem_ld4(s_tmem + NPAD + g * 4, lo);
        tc::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = g * 4 + e;
          const float sv = fmaf(int_to_float(hi[e]), 256.f, int_to_float(lo[e])) * (sq[n] * mult);
          const bool vis = interior || (pos >= rlo[n] && pos <= rhi[n]);
          s[n] = vis ? sv : -INFINITY;
          const int key = __reduce_max_sync(0xffffffffu, float_key(s[n]));
          if (lane == (n & 31)) wred[warp * (NPAD + 1) + n] = key_float(key);
        }
      }
    }
    {
      const int key = __reduce_max_sync(0xffffffffu, float_key(vs_cur));
      if (lane == 0) wred[warp * (NPAD + 1) + NPAD] = key_float(key);
    }
    __syncthreads();  // per-warp maxima are visible

    const float vs_max = fmaxf(fmaxf(wred[NPAD], wred[(NPAD + 1) + NPAD]),
                               fmaxf(wred[2 * (NPAD + 1) + NPAD], wred[3 * (NPAD + 1) + NPAD]));
#pragma unroll
    for (int g = 0; g < NPAD / 16; ++g) {
      if (g * 16 < rows) {
        uint32_t dig[PD][4] = {};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int n = g * 16 + e;
          if (n < rows) {
            const float m_old = mrun[n];
            const float m_tile = fmaxf(fmaxf(wred[n], wred[(NPAD + 1) + n]),
                                       fmaxf(wred[2 * (NPAD + 1) + n], wred[3 * (NPAD + 1) + n]));
            const float m_new = fmaxf(m_old, m_tile);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float a = fast_exp2(m_old - m_use);
            const float pr = fast_exp2(s[n] - m_use);
            l_part[n] = fmaf(l_part[n], a, pr);
            // largest p * v_scale of the tile bounds the fixed-point range
            const float bound = vs_max * fast_exp2(m_tile - m_use);
            const float inv_u = bound > 0.f ? (float)XMAX * __frcp_rn(bound) : 0.f;
            int x = __float2int_rn(pr * vs_cur * inv_u);
            x = min(x, XMAX);
#pragma unroll
            for (int k = 0; k < PD; ++k) dig[k][e >> 2] |= (uint32_t)((x >> (7 * k)) & 127) << (8 * (e & 3));
            if (tid == n) {
              alpha_s[n] = a;
              unit_s[n] = bound * (1.0f / (float)XMAX);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < PD; ++k)
          *reinterpret_cast<uint4*>(pimg + (k * (NPAD / 16) + g) * kDigitChunk + tid * 16) =
              make_uint4(dig[k][0], dig[k][1], dig[k][2], dig[k][3]);
      }
    }
    offs[tid] = off_new;  // read by the next iteration's refill; this iteration's refill is past barrier (b)
    tc::fence_before_sync();
    tc::fence_async_smem();
    __syncthreads();  // (c) P image, alpha, unit and the new offsets complete; mrun / wred reads done
    if (tid < rows) {
      const float m_tile = fmaxf(fmaxf(wred[tid], wred[(NPAD + 1) + tid]),
                                 fmaxf(wred[2 * (NPAD + 1) + tid], wred[3 * (NPAD + 1) + tid]));
      mrun[tid] = fmaxf(mrun[tid], m_tile);
    }
    if (tid == 0) {
      tc::fence_after_sync();
      issue_pv_i8<NPAD, PD>(tmem_base + 2 * L::s_cols + (i & 1) * L::o_cols, stage + kImgBytes, pimg_s);
      tc::mma_commit(&bar_o[i & 1]);
    }
  }
  fold_o(n_tiles - 1);

  // ---- epilogue -------------------------------------------------------------
  __syncthreads();
#pragma unroll
  for (int n = 0; n < NPAD; ++n) {
    if (n < rows) {
      float v = l_part[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == (n & 31)) wred[warp * (NPAD + 1) + n] = v;
    }
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < NPAD; ++n) {
    if (n < rows) {
      const float l = wred[n] + wred[(NPAD + 1) + n] + wred[2 * (NPAD + 1) + n] + wred[3 * (NPAD + 1) + n];
      const float val = l > 0.f ? acc[n] / l : 0.f;
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
    const float l = wred[tid] + wred[(NPAD + 1) + tid] + wred[2 * (NPAD + 1) + tid] + wred[3 * (NPAD + 1) + tid];
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

  cp_async_wait<0>();
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, L::tmem_alloc);
  if (!ok && tid == 0) atomicOr(&g_i8_status, 4u);
}

template <int NPAD, int PD, int NS>
cudaError_t launch_cfg(const KernelParams& p, cudaStream_t stream) {
  constexpr int smem = Layout<NPAD, PD, NS>::total;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_i8_attention_kernel<NPAD, PD, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  umma_i8_attention_kernel<NPAD, PD, NS><<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_umma_i8_attention(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  const int cap = 64 / p.group;
  if (p.bq > cap) p.bq = cap;
  p.num_q_tiles = p.num_tokens / p.bq + p.num_reqs;
  const int rows = p.bq * p.group;
  if (rows <= 16) return launch_cfg<16, 3, 3>(p, stream);
  if (rows <= 32) return launch_cfg<32, 2, 5>(p, stream);
  return launch_cfg<64, 2, 4>(p, stream);
}

// Reads and clears the integer kernel's status word (device must be idle).
cudaError_t read_i8_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_i8_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_i8_status, &zero, sizeof(zero));
}

}  // namespace pthb200

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
