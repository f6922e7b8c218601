// Row-major tcgen05 attention kernel for head size 256: query rows on the MMA M dimension,
// KV tiles of 64 keys.
//
// The 128-dim row-major kernel (umma_rows_kernel.cu) does not stretch to 256 dims: its bf16 K
// and V images of 128 keys would take 4 x 66 KB.  This kernel keeps the same roles and the
// same exact int8 -> bf16 widening, with other shapes:
//   tile       128 query rows x 64 keys; the split partition stays in units of 128 keys, a
//              CTA walks its range in steps of 64;
//   TMEM       S0 S1 (64 columns each: tile i uses buffer i % 2, so S(i + 1) is computed while
//              the softmax warps work on tile i), ONE accumulator O of 256 columns, and Q (128
//              columns, two bf16 per column): Q is the A operand of QK from TMEM like P is of
//              PV, which takes its 64 KB image out of shared memory;
//   MMAs       S = Q K^T: M 128, N 64, sixteen steps of 16 dims; O += P V: M 128, N 256, four
//              steps of 16 keys;
//   producers  thread (key, half) of the K set / V set widens 128 of the key's 256 dims; the
//              threads of the upper halves also carry the key's scale;
//   softmax    two groups of 4 warps; group g owns keys 32 g .. 32 g + 31 of EVERY tile and
//              columns 128 g .. 128 g + 127 of O.  The two threads of a row agree on the row's
//              reference maximum tile by tile (through shared memory and one named barrier), which
//              is what lets them share one accumulator; each rescales and finally writes its
//              half of the row's output.
// Raw ring: two units of 64 keys x 528 bytes.  Every mbarrier wait is bounded (page_copy.cuh).
#include <cuda.h>

#include <type_traits>

#include "params.cuh"
#include "sched.cuh"
#include "umma_rows.cuh"
#include "page_copy.cuh"

namespace pthb200 {

__device__ unsigned int g_rows256_status = 0;

namespace {

constexpr int kWDim = 256;                          // head size
constexpr int kWKeys = 64;                          // keys of a tile
constexpr int kWChunks = kWDim / 8;                 // 16-byte column blocks of a widened row: 8 bf16 each
constexpr int kWChunkStride = kWKeys * 16 + 16;     // 1,040 B: one column block of all keys, padded
constexpr int kWImage = kWChunks * kWChunkStride;   // 33,280 B: widened K or V of a tile
constexpr int kWRawRow = raw_row_for(kWDim);        // 528 B
constexpr int kWRawUnit = kWKeys * kWRawRow;        // 33,792 B: raw cells of a tile
constexpr int kWVStage = kWImage + kWKeys * 4;      // V image + v_scale[64]
constexpr int kWNK = 2, kWNS = 2, kWNR = 2;         // K images, V stages, raw units
constexpr int kWKsRing = 4;                         // tiles of scaled k_scale vectors kept
constexpr int kWGroup = 128;                        // threads of one softmax group = rows of a tile
constexpr int kWSoftmax = 2 * kWGroup;              // warps 0-3, 4-7
constexpr int kWGroupKeys = kWKeys / 2;             // 32 keys of a tile per group
constexpr int kWGroupDims = kWDim / 2;              // 128 columns of O per group
constexpr int kWProducers = 256;                    // warps 8-11 (K set) and 12-15 (V set)
constexpr int kWMmaWarp = 16, kWLoadWarp = 17;
constexpr int kWThreads = 576;
constexpr int kWProducerRegs = 72, kWSoftmaxRegs = 120;  // of the 96 per thread the CTA starts with
constexpr int kWSCol = 0, kWOCol = 128, kWQCol = 384;    // TMEM columns: S buffers at 0 and 64, O, Q
constexpr float kWRescaleGap = 8.0f;                // log2 units a row maximum may outgrow its reference

struct WLayout {
  static constexpr int kimg = 0;
  static constexpr int vst = kimg + kWNK * kWImage;
  static constexpr int raw = (vst + kWNS * kWVStage + 127) / 128 * 128;
  static constexpr int ksc = raw + kWNR * kWRawUnit;                 // float [kWKsRing][64]: k_scale * scale * log2 e
  static constexpr int tile_max = ksc + kWKsRing * kWKeys * 4;       // float [2 tiles][2 groups][128 rows]
  static constexpr int half_sum = tile_max + 2 * 2 * kWGroup * 4;    // float [2 groups][128 rows]
  static constexpr int bars = half_sum + 2 * kWGroup * 4;            // uint64 [...]
  static constexpr int n_bars = kWNS * 2 + 2 * kWNK + 6 + 2 * kWNR;
  static constexpr int misc = bars + n_bars * 8;
  static constexpr int total = misc + 32;
};

struct WBars {
  static constexpr int vfull = 0;                      // [NS] V producers -> softmax (pass 2) and PV
  static constexpr int vempty = kWNS;                  // [NS] PV commit -> V producers
  static constexpr int kempty = 2 * kWNS;              // [NK] QK commit -> K producers
  static constexpr int kfull = 2 * kWNS + kWNK;        // [NK] K producers -> QK
  static constexpr int s_ready = 2 * kWNS + 2 * kWNK;  // [2] QK commit -> softmax
  static constexpr int p_ready = s_ready + 2;          // [2] softmax -> PV
  static constexpr int pv_done = p_ready + 2;          // [2] PV commit -> QK, softmax
  static constexpr int raw_full = pv_done + 2;         // [NR]
  static constexpr int raw_free = raw_full + kWNR;     // [NR] producers -> loader
};

// Key of a tile held by row `r` of its images: with contiguous cells the even keys, then the odd ones.
__device__ __forceinline__ int tile_key_w(int raw_mode, int r) { return raw_mode == 2 ? 2 * (r & 31) + (r >> 5) : r; }

__device__ __forceinline__ uint32_t pack_bf16_w(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float ex2f_w(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// S(buffer) = Q K^T with Q in TMEM: 16 steps of 16 dims = two column blocks of the K image each.
__device__ __forceinline__ void issue_qk_w(uint32_t s_tmem, uint32_t q_tmem, RowsDesc k) {
  constexpr uint32_t idesc = tc::instr_desc(128, kWKeys, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
  constexpr uint32_t step = (2 * kWChunkStride) >> 4;
#pragma unroll
  for (int kk = 0; kk < kWDim / 16; ++kk) mma_ts_words(s_tmem, q_tmem + kk * 8, k.lo + kk * step, k.hi, idesc, kk > 0);
}
// O += P V: P in two pieces (keys 0-31 in columns 0-15 of the S buffer, keys 32-63 in columns
// 32-47: each softmax group writes P over its own half of S), four steps of 16 keys.
__device__ __forceinline__ void issue_pv_w(uint32_t o_tmem, uint32_t s_tmem, RowsDesc v, bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(128, kWDim, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int kk = 0; kk < kWGroupKeys / 16; ++kk)
      mma_ts_words(o_tmem, s_tmem + g * kWGroupKeys + kk * 8, v.lo + (g * (kWGroupKeys / 16) + kk) * (256 >> 4), v.hi, idesc,
                   accumulate || g > 0 || kk > 0);
}

__global__ void __launch_bounds__(kWThreads, 1)
umma_rows256_attention_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap tmap) {
  using L = WLayout;
  using B = WBars;
  static_assert(L::raw % 128 == 0 && kWRawUnit % 128 == 0 && (16 * kWRawRow) % 128 == 0, "TMA destinations");
  static_assert(L::vst % 16 == 0 && kWVStage % 16 == 0 && kWImage % 16 == 0, "image alignment");
  static_assert(L::total <= 227 * 1024, "shared memory of one CTA");
  extern __shared__ __align__(128) uint8_t smem[];
  float* tile_max = reinterpret_cast<float*>(smem + L::tile_max);
  float* half_sum = reinterpret_cast<float*>(smem + L::half_sum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::misc + 8);

  const int kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Row tile of this CTA: bisect a shared-memory copy of query_start_loc when it fits.
  constexpr int kQslCache = 4096;
  static_assert(kWNR * kWRawUnit >= 2 * kQslCache * 4, "the raw ring holds the copies of query_start_loc and seq_lens");
  RowTile t;
  if (p.tile_map == 0 && p.num_reqs + 1 <= kQslCache) {
    int* qsl_s = reinterpret_cast<int*>(smem + L::raw);
    int* len_s = qsl_s + kQslCache;
    for (int i = tid; i <= p.num_reqs; i += kWThreads) {
      qsl_s[i] = __ldg(p.query_start_loc + i);
      if (i < p.num_reqs) len_s[i] = __ldg(p.seq_lens + i);
    }
    __syncthreads();
    t = resolve_row_tile_with(p, blockIdx.x, [&](int i) { return qsl_s[i]; }, [&](int r) { return len_s[r]; });
    __syncthreads();
  } else {
    t = resolve_row_tile(p, blockIdx.x);
  }
  if (t.req < 0) return;
  const int rows = t.ntok * p.group;  // <= 128 by construction of bq
  // num_splits is a bound: the pieces a request is cut into are chosen here, from the lengths,
  // by the rule of the integer kernel (sched.cuh) - pieces of about equal length over the
  // whole launch, so a prefill chunk among long decode requests is not cut at all.  CTAs of
  // unused pieces leave at once; the CTA of piece 0 marks them as holding no keys.
  int nsplits = p.num_splits;
  if (p.num_splits > 1) {
    unsigned long long* total_s = reinterpret_cast<unsigned long long*>(smem + L::misc + 16);
    if (tid == 0) *total_s = 0ull;
    __syncthreads();
    SchedShape shape;
    shape.group = p.group;
    shape.num_kv_heads = p.num_kv_heads;
    shape.bq = p.bq;
    shape.num_splits = p.num_splits;
    shape.window = p.window;
    shape.causal = p.causal;
    shape.row_class = p.row_class;
    shape.class_rows = p.class_rows;
    unsigned long long w = 0;
    for (int r = tid; r < p.num_reqs; r += kWThreads) {
      const int q0 = __ldg(p.query_start_loc + r), q1 = __ldg(p.query_start_loc + r + 1);
      w += (unsigned long long)req_row_tiles(shape, q1 - q0) *
           (unsigned long long)req_kv_tiles(shape, q1 - q0, __ldg(p.seq_lens + r));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0 && w != 0) atomicAdd(total_s, w);
    __syncthreads();
    const int t_star = item_tiles(*total_s * (unsigned long long)p.num_kv_heads, p.num_sms);
    nsplits = req_splits(req_kv_tiles(shape, t.q_len, t.seq_len), t_star, p.num_splits);
    if (split >= nsplits) return;
    if (split == 0) {
      for (int i = tid; i < rows * (p.num_splits - nsplits); i += kWThreads) {
        int token, head;
        row_target(p, t, kvh, i % rows, &token, &head);
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)(nsplits + i / rows) * p.ws_lse_stride_split +
                                  (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) = -INFINITY;
      }
    }
    __syncthreads();  // the scratch word is part of a region the barriers are initialised in next
  }
  int tile_begin, tile_end, range_begin, range_end;
  split_tiles(p, t, split, nsplits, &tile_begin, &tile_end, &range_begin, &range_end);

  if (tile_begin >= tile_end) {
    // No keys for this work item: zero output, log-sum-exp -inf.
    for (int idx = tid; idx < rows * kWDim; idx += kWThreads) {
      const int n = idx / kWDim, d = idx % kWDim;
      int token, head;
      row_target(p, t, kvh, n, &token, &head);
      if (p.num_splits == 1) {
        store_out_elem(p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head, d, p.out_dtype, 0.f);
      } else {
        reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                 (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head)[d] = 0.f;
      }
    }
    if (tid < rows) {
      int token, head;
      row_target(p, t, kvh, tid, &token, &head);
      if (p.num_splits > 1) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                  (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) = -INFINITY;
      } else if (p.lse_out != nullptr) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                  (int64_t)head * p.lse_stride_head) = -INFINITY;
      }
    }
    return;
  }

  // the CTA walks its keys in tiles of 64: from the first 128-key tile of its piece to the end
  // of the keys its rows see (or of the piece)
  const int key_begin = tile_begin * 128;
  const int key_end = min(tile_end * 128, range_end);
  const int n_tiles = (key_end - key_begin + kWKeys - 1) / kWKeys;
  if (tid == 0) {
    for (int s = 0; s < kWNS; ++s) {
      tc::mbar_init(&bars[B::vfull + s], kWProducers / 2);
      tc::mbar_init(&bars[B::vempty + s], 1);
    }
    for (int s = 0; s < kWNK; ++s) {
      tc::mbar_init(&bars[B::kempty + s], 1);
      tc::mbar_init(&bars[B::kfull + s], kWProducers / 2);
    }
    for (int g = 0; g < 2; ++g) {
      tc::mbar_init(&bars[B::s_ready + g], 1);
      tc::mbar_init(&bars[B::p_ready + g], kWSoftmax);
      tc::mbar_init(&bars[B::pv_done + g], 1);
    }
    for (int s = 0; s < kWNR; ++s) {
      tc::mbar_init(&bars[B::raw_full + s], kWKeys >> p.copy_shift);  // page copies of a unit
      tc::mbar_init(&bars[B::raw_free + s], kWProducers);             // every producer thread reads every unit
    }
    *abort_flag = 0;
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const uint32_t kimg_s = tc::smem_u32(smem + L::kimg), vst_s = tc::smem_u32(smem + L::vst);
  bool ok = true;

  if (warp >= 8 && warp < kWMmaWarp) {
    // =========================== producers ====================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kWProducerRegs));
    // Warps 8-11 widen K, warps 12-15 V.  Thread pt of a set owns key pt % 64 and dims
    // 128 (pt / 64) .. + 127 of it: 128 bytes of the raw cell, which start 0 or 8 (K) or 4 or
    // 12 (V) bytes after a 16-byte boundary; the threads of the upper halves find the key's
    // scale right behind their bytes.
    const int pt = tid & 127;
    const bool v_part = warp >= 12;
    // Contiguous cells (raw_mode 2) alternate between the two 8-byte alignments: a warp takes
    // the even keys or the odd ones, so that it runs one instance of the widening below.  Row r
    // of the images (and of the scale vectors) then holds key tile_key_w(r): the order of the
    // keys inside a tile changes no sum, and the softmax masks by that key.
    const int img_row = pt & (kWKeys - 1), upper = pt >> 6;
    const int key = tile_key_w(p.raw_mode, img_row);
    const int bs = p.copy_slots;  // slots of one page copy
    const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
    const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
    const int row_pitch = p.raw_mode == 1 ? kWRawRow : 2 * kWDim + 8;
    const int my_page = key >> p.copy_shift, my_slot = key & (bs - 1);
    // first byte of this thread's 128 bytes inside a raw unit
    const uint32_t piece = my_page * bs * kWRawRow + my_slot * row_pitch + delta + (v_part ? kWDim + 4 : 0) + upper * 128;
    const int wo = (int)((piece & 15u) >> 2);  // first word of the piece in the 16-byte chunks read: 0 / 2 (K), 1 / 3 (V)
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int rs = j % kWNR;
      const int pos = key_begin + j * kWKeys + key;
      const bool valid = pos >= range_begin && pos < range_end;
      ok &= wait_or_abort(&bars[B::raw_full + rs], (j / kWNR) & 1, abort_flag);
      // nine 16-byte chunks from the boundary below the piece: its 32 words and the scale behind them
      uint32_t w[36];
      if (valid) {
        const uint4* row = reinterpret_cast<const uint4*>(smem + L::raw + rs * kWRawUnit + (piece & ~15u));
#pragma unroll
        for (int c = 0; c < 9; ++c) {
          const uint4 v = row[c];
          w[4 * c] = v.x;
          w[4 * c + 1] = v.y;
          w[4 * c + 2] = v.z;
          w[4 * c + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 36; ++c) w[c] = 0u;
      }
      mbar_arrive(&bars[B::raw_free + rs]);  // the bytes are in registers: the unit may be refilled
      uint8_t* dst;
      if (!v_part) {
        if (j >= kWNK) ok &= wait_or_abort(&bars[B::kempty + j % kWNK], ((j / kWNK) - 1) & 1, abort_flag);
        dst = smem + L::kimg + (j % kWNK) * kWImage;
      } else {
        if (j >= kWNS) ok &= wait_or_abort(&bars[B::vempty + j % kWNS], ((j / kWNS) - 1) & 1, abort_flag);
        dst = smem + L::vst + (j % kWNS) * kWVStage;
      }
      uint8_t* out16 = dst + (upper * 16) * kWChunkStride + img_row * 16;  // column blocks 16 upper .. 16 upper + 15
      uint32_t scale_bits;
      // (one instance per alignment: the words of w must be compile-time indices)
      auto widen_piece = [&](auto first_word) {
        constexpr int kW0 = decltype(first_word)::value;
#pragma unroll
        for (int c = 0; c < 16; ++c)
          *reinterpret_cast<uint4*>(out16 + c * kWChunkStride) = widen8_bf16(make_uint2(w[kW0 + 2 * c], w[kW0 + 2 * c + 1]));
        scale_bits = w[kW0 + 32];
      };
      if (wo == 0) widen_piece(std::integral_constant<int, 0>{});
      else if (wo == 1) widen_piece(std::integral_constant<int, 1>{});
      else if (wo == 2) widen_piece(std::integral_constant<int, 2>{});
      else widen_piece(std::integral_constant<int, 3>{});
      if (upper) {
        if (!v_part) {
          reinterpret_cast<float*>(smem + L::ksc)[(j % kWKsRing) * kWKeys + img_row] = __uint_as_float(scale_bits) * p.scale_log2;
        } else {
          *reinterpret_cast<uint32_t*>(dst + kWImage + img_row * 4) = scale_bits;
        }
      }
      tc::fence_async_smem();
      mbar_arrive(&bars[(v_part ? B::vfull + j % kWNS : B::kfull + j % kWNK)]);
    }
  } else if (warp == kWLoadWarp) {
    // =========================== loader =======================================
    // One TMA copy per run of copy_slots slots of a tile, issued by lane `copy`: a box of the
    // tensor map (raw_mode 1) or a bulk copy of a contiguous run of cells (raw_mode 2); the
    // next tile's block ids are fetched before waiting for the unit.
    const int copies = kWKeys >> p.copy_shift;
    if (lane < copies) {
      const int bs = p.copy_slots;
      const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;
      const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
      const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
      const int tma_x = (int)((reinterpret_cast<uintptr_t>(kb) - delta -
                               (reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15)) >> 2);
      const uint32_t raw_s = tc::smem_u32(smem + L::raw);
      auto page_block = [&](int j) -> int {
        const int pos0 = key_begin + j * kWKeys + lane * bs;
        if (j >= n_tiles || pos0 >= range_end || pos0 + bs <= range_begin) return -1;
        int page, slot;
        page_and_slot(p, pos0, &page, &slot);
        return __ldg(bt + page);
      };
      auto first_slot = [&](int j) -> int {
        int page, slot;
        page_and_slot(p, key_begin + j * kWKeys + lane * bs, &page, &slot);
        return slot;
      };
      int blk = page_block(0);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int blk_next = page_block(j + 1);
        const int rs = j % kWNR;
        if (j >= kWNR) ok &= wait_or_abort(&bars[B::raw_free + rs], ((j / kWNR) - 1) & 1, abort_flag);
        uint64_t* bar = &bars[B::raw_full + rs];
        if (blk >= 0 && ok) {
          const uint32_t dst = raw_s + rs * kWRawUnit + lane * bs * kWRawRow;
          if (p.raw_mode == 1) {
            mbar_arrive_expect_tx(bar, bs * kWRawRow);
            tma_load_3d(dst, &tmap, tma_x, first_slot(j), blk, bar);
          } else {
            const uint32_t bytes = bs * (2 * kWDim + 8);  // a multiple of 16, like the run's address
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy_g2s(dst, kb + (int64_t)blk * p.k.stride_block + (int64_t)first_slot(j) * (2 * kWDim + 8), bytes, bar);
          }
        } else {
          mbar_arrive(bar);
        }
        blk = blk_next;
      }
    }
  } else if (warp == kWMmaWarp) {
    // =========================== MMA issuer ===================================
    // ONE elected lane issues every tcgen05.mma of the CTA in one fixed order: QK(0), QK(1),
    // then PV(i), QK(i + 2).  QK(i + 2) overwrites the S buffer P(i) was written over: it
    // waits for PV(i) to have finished reading it, a whole tile of softmax after it is issued.
    named_barrier(5, kWSoftmax + 32);  // wait for Q in TMEM
    tc::fence_after_sync();
    {
      const RowsDesc kd = rows_desc(kimg_s, kWChunkStride, 128);
      const RowsDesc vd = rows_desc(vst_s, 128, kWChunkStride);
      auto issue_qk = [&](int q) {
        ok &= wait_or_abort(&bars[B::kfull + q % kWNK], (q / kWNK) & 1, abort_flag);
        if (ok && elect_one()) {
          tc::fence_after_sync();
          RowsDesc k = kd;
          k.lo += (uint32_t)(q % kWNK) * (kWImage >> 4);
          issue_qk_w(tmem_base + kWSCol + (q & 1) * kWKeys, tmem_base + kWQCol, k);
          tc::mma_commit(&bars[B::s_ready + (q & 1)]);
          tc::mma_commit(&bars[B::kempty + q % kWNK]);
        }
        __syncwarp();
      };
      issue_qk(0);
      if (n_tiles > 1) issue_qk(1);
#pragma unroll 1
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int sb = i & 1;
        ok &= wait_or_abort(&bars[B::p_ready + sb], (i >> 1) & 1, abort_flag);
        ok &= wait_or_abort(&bars[B::vfull + i % kWNS], (i / kWNS) & 1, abort_flag);
        if (ok && elect_one()) {
          tc::fence_after_sync();
          RowsDesc v = vd;
          v.lo += (uint32_t)(i % kWNS) * (kWVStage >> 4);
          issue_pv_w(tmem_base + kWOCol, tmem_base + kWSCol + sb * kWKeys, v, i > 0);
          tc::mma_commit(&bars[B::pv_done + sb]);
          tc::mma_commit(&bars[B::vempty + i % kWNS]);
        }
        __syncwarp();
        if (i + 2 < n_tiles) {
          ok &= wait_or_abort(&bars[B::pv_done + sb], (i >> 1) & 1, abort_flag);
          issue_qk(i + 2);
        }
      }
    }
  } else if (warp < 8) {
    // =========================== softmax ======================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kWSoftmaxRegs));
    const int g = warp >> 2;
    const int row = tid & 127;   // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_part = tmem_base + kWSCol + g * kWGroupKeys + lane_addr;   // this group's columns of S buffer 0
    const uint32_t o_part = tmem_base + kWOCol + g * kWGroupDims + lane_addr;   // this group's columns of O

    // ---- Q into TMEM: thread (row, g) stores dims 128 g .. 128 g + 127 of its row, two bf16 per column ----
    {
      int token, head;
      row_target(p, t, kvh, row, &token, &head);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token +
                                                        (int64_t)head * p.q_stride_head) + g * (kWGroupDims / 8);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t qw[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = row < rows ? __ldg(src + h * 8 + c) : make_uint4(0u, 0u, 0u, 0u);
          qw[4 * c] = v.x;
          qw[4 * c + 1] = v.y;
          qw[4 * c + 2] = v.z;
          qw[4 * c + 3] = v.w;
        }
        tc::tmem_st32(tmem_base + kWQCol + g * (kWGroupDims / 2) + h * 32 + lane_addr, qw);
      }
      tc::tmem_st_wait();
    }
    tc::fence_before_sync();
    named_barrier(5, kWSoftmax + 32);  // Q complete; the QK issuer may start

    int rlo = 0, rhi = -1;  // visible keys of this row (none for a padding row)
    if (row < rows) visible_range(p, t, t.first_idx + row / p.group, &rlo, &rhi);
    int mask_lo, mask_hi, tmp;  // key positions every live row sees: such tiles need no mask
    visible_range(p, t, t.first_idx + t.ntok - 1, &mask_lo, &tmp);
    visible_range(p, t, t.first_idx, &tmp, &mask_hi);
    float m_ref = -INFINITY;  // reference maximum of the row's exponentials (log2 units)
    float l = 0.f;            // sum of exp2(score - m_ref) over this group's keys
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
      const float* ksp = reinterpret_cast<const float*>(smem + L::ksc) + (i % kWKsRing) * kWKeys + g * kWGroupKeys;
      const float* vsp = reinterpret_cast<const float*>(smem + L::vst + (i % kWNS) * kWVStage + kWImage) + g * kWGroupKeys;
      const uint32_t s_tmem = s_part + (i & 1) * kWKeys;
      const int pos0 = key_begin + i * kWKeys;
      const bool interior = pos0 >= mask_lo && pos0 + (kWKeys - 1) <= mask_hi;
      ok &= wait_or_abort(&bars[B::s_ready + (i & 1)], (i >> 1) & 1, abort_flag);
      tc::fence_after_sync();
      uint32_t r[kWGroupKeys];  // the scores of this row and part, read once
      tc::tmem_ld32(s_tmem, r);
      tc::tmem_ld_wait();

      // ---- pass 1: scores in log2 units (kept in the registers) and their maximum ----
      float m_t;
      auto pass1 = [&](auto masked) {
        constexpr bool kMask = decltype(masked)::value;
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int n4 = 0; n4 < kWGroupKeys / 4; ++n4) {
          const float4 ks4 = reinterpret_cast<const float4*>(ksp)[n4];  // k_scale * scale * log2 e
          const float kk[4] = {ks4.x, ks4.y, ks4.z, ks4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n4 * 4 + e;
            float sc = __uint_as_float(r[n]) * kk[e];
            if constexpr (kMask) {
              const int pos = pos0 + tile_key_w(p.raw_mode, g * kWGroupKeys + n);  // key held by this column
              sc = (pos >= rlo && pos <= rhi) ? sc : -INFINITY;
            }
            r[n] = __float_as_uint(sc);
            mx[e] = fmaxf(mx[e], sc);
          }
        }
        m_t = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      };
      if (interior) pass1(std::false_type{}); else pass1(std::true_type{});
      // ---- the row's maximum over the whole tile: the other group has the other keys ----
      float* tm = tile_max + (i & 1) * 2 * kWGroup + row;
      tm[g * kWGroup] = m_t;
      named_barrier(4, kWSoftmax);
      m_t = fmaxf(m_t, tm[(g ^ 1) * kWGroup]);
      // ---- move the reference maximum if the row has outgrown it (both threads of a row decide alike) ----
      const float m_new = fmaxf(m_ref, m_t);
      const bool need = m_t > m_ref + kWRescaleGap;  // also true when m_ref is still -inf
      if (i == 0) {
        m_ref = m_new;  // nothing accumulated yet
      } else if (__any_sync(0xffffffffu, need)) {
        // O must be at rest: the PV of the previous tile has completed
        ok &= wait_or_abort(&bars[B::pv_done + ((i - 1) & 1)], ((i - 1) >> 1) & 1, abort_flag);
        tc::fence_after_sync();
        const float alpha = need ? ex2f_w(m_ref - m_new) : 1.0f;  // 0 when m_ref was -inf
#pragma unroll 1
        for (int j = 0; j < kWGroupDims / 16; ++j) {
          uint32_t o[16];
          tc::tmem_ld16(o_part + j * 16, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int n = 0; n < 16; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * alpha);
          tc::tmem_st16(o_part + j * 16, o);
        }
        tc::tmem_st_wait();
        l *= alpha;
        if (need) m_ref = m_new;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

      // ---- pass 2: p * v_scale as packed bf16 over the first columns of this part of S ----
      // (a masked score is -inf: its p is exp2(-inf) = 0)
      ok &= wait_or_abort(&bars[B::vfull + i % kWNS], (i / kWNS) & 1, abort_flag);  // v_scale of tile i
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[16];
#pragma unroll
      for (int n4 = 0; n4 < 8; ++n4) {
        const float4 vs4 = reinterpret_cast<const float4*>(vsp)[n4];
        const float vv[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pr = ex2f_w(__uint_as_float(r[n4 * 4 + e]) - m_use);
          ls[e] += pr;
          pv[e] = pr * vv[e];
        }
        pk[n4 * 2] = pack_bf16_w(pv[0], pv[1]);
        pk[n4 * 2 + 1] = pack_bf16_w(pv[2], pv[3]);
      }
      tc::tmem_st16(s_tmem, pk);
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc::tmem_st_wait();
      tc::fence_before_sync();
      mbar_arrive(&bars[B::p_ready + (i & 1)]);  // this group's part of P(i) is complete
    }

    // ---- epilogue: the row's sum is the two groups' sums; each group writes its half of the dims ----
    // (the commit after the last PV covers every MMA issued before it)
    ok &= wait_or_abort(&bars[B::pv_done + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1, abort_flag);
    tc::fence_after_sync();
    half_sum[g * kWGroup + row] = l;
    named_barrier(4, kWSoftmax);
    const float lsum = half_sum[row] + half_sum[kWGroup + row];  // the same order in both threads
    const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
    int token, head;
    row_target(p, t, kvh, row, &token, &head);
    uint8_t* out_row = p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head;
    float* ws_row = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                             (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head);
#pragma unroll 1
    for (int j = 0; j < kWGroupDims / 32; ++j) {
      uint32_t r[32];
      tc::tmem_ld32(o_part + j * 32, r);
      tc::tmem_ld_wait();
      float o[32];
#pragma unroll
      for (int n = 0; n < 32; ++n) o[n] = __uint_as_float(r[n]) * inv;
      const int d0 = g * kWGroupDims + j * 32;
      if (row < rows) {
        if (p.num_splits > 1) {
#pragma unroll
          for (int n = 0; n < 32; n += 4)
            *reinterpret_cast<float4*>(ws_row + d0 + n) = make_float4(o[n], o[n + 1], o[n + 2], o[n + 3]);
        } else if (p.out_dtype == PTH_ATTN_BF16) {
#pragma unroll
          for (int n = 0; n < 32; n += 8)
            *reinterpret_cast<uint4*>(out_row + (d0 + n) * 2) =
                make_uint4(pack_bf16_w(o[n], o[n + 1]), pack_bf16_w(o[n + 2], o[n + 3]), pack_bf16_w(o[n + 4], o[n + 5]),
                           pack_bf16_w(o[n + 6], o[n + 7]));
        } else {
#pragma unroll
          for (int n = 0; n < 32; ++n) store_out_elem(out_row, d0 + n, p.out_dtype, o[n]);
        }
      }
    }
    if (g == 0 && row < rows) {
      const float lse2 = lsum > 0.f ? m_ref + log2f(lsum) : -INFINITY;
      if (p.num_splits > 1) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                  (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) = lse2;
      } else if (p.lse_out != nullptr) {
        *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                  (int64_t)head * p.lse_stride_head) = lse2 * kLn2;
      }
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
  if (tid == 0 && *abort_flag) atomicOr(&g_rows256_status, 4u);
  (void)ok;
}

}  // namespace

cudaError_t launch_umma_rows256_attention(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  // Row tiles of 128 rows, whatever tile height the caller planned with.
  set_row_tile(p, 128 / p.group > 0 ? 128 / p.group : 1);
  set_copy_slots(p, kWKeys);  // a raw unit (64 keys) holds whole page copies
  p.raw_mode = raw_mode_for(p);
  p.num_sms = sm_count();
  if (p.num_sms <= 0) return cudaErrorInvalidDevice;
  static const CUtensorMap no_map{};
  const CUtensorMap* mapp = &no_map;
  if (p.raw_mode == 1) {
    mapp = cached_page_map(p);
    if (mapp == nullptr) return cudaErrorInvalidValue;
  }
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_rows256_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WLayout::total);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  umma_rows256_attention_kernel<<<grid, kWThreads, WLayout::total, stream>>>(p, *mapp);
  return cudaGetLastError();
}

// Reads and clears this kernel's status word (device must be idle).
cudaError_t read_rows256_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_rows256_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_rows256_status, &zero, sizeof(zero));
}

}  // namespace pthb200
