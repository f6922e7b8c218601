// Row-major tcgen05 attention kernel, head sizes 128 and 64, TWO row tiles per CTA: 256 query rows
// share every widened K / V tile.  (The shapes below are those of 128 dims; at 64 dims the images,
// the accumulators and the contraction steps over the head are half as large.)
//
// In the one-tile kernel (umma_rows_kernel.cu) every row tile of 128 rows widens the int8 keys
// and values of its whole context to bf16 for itself, and that widening and the shared-memory
// traffic around it - not the tensor core, not the softmax - take most of a tile's time.
// Here a CTA owns 256 rows (two MMA row tiles) and 64-key tiles:
//   TMEM       S(rt, b): 64 columns for row tile rt and buffer b = tile % 2 (256 columns), O(rt):
//              128 columns each (256 columns);
//   MMAs       per KV tile two QK (M 128, N 64, eight steps of 16 dims, Q images in shared
//              memory) on ONE K image and two PV (M 128, N 128, four steps of 16 keys, P from
//              TMEM) on ONE V stage;
//   producers  thread (key, half) of the K set / V set widens 64 of the key's 128 dims; the K
//              set's upper halves carry k_scale to the softmax, the V set multiplies its rows
//              by v_scale as it widens them (x * v_scale rounded once to bf16), so P is the
//              bare probability and the softmax spends nothing on v_scale;
//   softmax    256 threads, one per row: the row's maximum, sum and reference never leave the
//              thread, and there is nothing to merge at the end.
// Raw ring: four units of 64 keys x 272 bytes.  Every mbarrier wait is bounded (page_copy.cuh).
#include <cuda.h>

#include <type_traits>

#include "params.cuh"
#include "sched.cuh"
#include "umma_rows.cuh"
#include "page_copy.cuh"

namespace pthb200 {

__device__ unsigned int g_rows2_status = 0;

namespace {

constexpr int kXKeys = 64;                          // keys of a tile
constexpr int kXRows = 256;                         // rows of a CTA: two MMA row tiles
constexpr int kXChunkStride = kXKeys * 16 + 16;     // 1,040 B: one column block of all keys, padded
constexpr int kXQStride = 128 * 16 + 16;            // 2,064 B: one column block of the 128 rows of a Q image
// Sizes that follow the head size HD (figures for 128).
template <int HD>
struct XG {
  static_assert(HD == 64 || HD == 128, "head size");
  static constexpr int chunks = HD / 8;                    // 16-byte column blocks of a widened row: 8 bf16 each
  static constexpr int image = chunks * kXChunkStride;     // 16,640 B: widened K or V of a tile (V rows times v_scale)
  static constexpr int qimage = chunks * kXQStride;        // 33,024 B
  static constexpr int raw_row = raw_row_for(HD);          // 272 B
  static constexpr int raw_unit = kXKeys * raw_row;        // 17,408 B: raw cells of a tile
  static constexpr int piece = HD / 2;                     // bytes of a key a producer thread widens
  static constexpr int piece_chunks = piece / 8;           // column blocks it writes
  static constexpr int load_chunks = piece / 16 + 1;       // 16-byte chunks it reads: the piece, its misalignment, the scale
};
constexpr int kXNK = 2, kXNS = 2, kXNR = 4;         // K images, V stages, raw units
constexpr int kXKsRing = 4;                         // tiles of scaled k_scale vectors kept
constexpr int kXSoftmax = 256;                      // warps 0-3 (row tile 0), 4-7 (row tile 1)
constexpr int kXProducers = 256;                    // warps 8-11 (K set) and 12-15 (V set)
constexpr int kXMmaWarp = 16, kXLoadWarp = 17;
constexpr int kXThreads = 576;
constexpr int kXProducerRegs = 72, kXSoftmaxRegs = 120;  // of the 96 per thread the CTA starts with
constexpr int kXOCol = 256;                         // TMEM columns: S(rt, b) at (2 rt + b) 64, O(rt) at 256 + 128 rt
constexpr float kXRescaleGap = 8.0f;                // log2 units a row maximum may outgrow its reference

template <int HD>
struct XLayout {
  using G = XG<HD>;
  static constexpr int kimg = 0;
  static constexpr int vst = kimg + kXNK * G::image;
  static constexpr int qimg = vst + kXNS * G::image;                 // [2 row tiles] Q images
  static constexpr int raw = (qimg + 2 * G::qimage + 127) / 128 * 128;
  static constexpr int ksc = raw + kXNR * G::raw_unit;               // float [kXKsRing][64]: k_scale * scale * log2 e
  static constexpr int bars = ksc + kXKsRing * kXKeys * 4;           // uint64 [...]
  static constexpr int n_bars = 2 * kXNS + 2 * kXNK + 12 + 2 * kXNR;
  static constexpr int misc = bars + n_bars * 8;
  static constexpr int total = misc + 32;
};

struct XBars {
  static constexpr int vfull = 0;                      // [NS] V producers -> softmax (pass 2) and PV
  static constexpr int vempty = kXNS;                  // [NS] PV commit -> V producers
  static constexpr int kempty = 2 * kXNS;              // [NK] QK commit -> K producers
  static constexpr int kfull = 2 * kXNS + kXNK;        // [NK] K producers -> QK
  static constexpr int s_ready = 2 * kXNS + 2 * kXNK;  // [2 rt][2 b] QK commit -> softmax
  static constexpr int p_ready = s_ready + 4;          // [2 rt][2 b] softmax -> PV
  static constexpr int pv_done = p_ready + 4;          // [2 rt][2 b] PV commit -> QK, softmax
  static constexpr int raw_full = pv_done + 4;         // [NR]
  static constexpr int raw_free = raw_full + kXNR;     // [NR] producers -> loader
};

__device__ __forceinline__ uint32_t pack_bf16_x(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float ex2f_x(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Key of a tile held by row `r` of its images: with contiguous cells the even keys, then the odd ones.
__device__ __forceinline__ int tile_key_x(int raw_mode, int r) { return raw_mode == 2 ? 2 * (r & 31) + (r >> 5) : r; }

// S = Q K^T for one row tile: HD / 16 steps of 16 dims = two column blocks of either image each.
template <int HD>
__device__ __forceinline__ void issue_qk_x(uint32_t s_tmem, RowsDesc q, RowsDesc k) {
  constexpr uint32_t idesc = tc::instr_desc(128, kXKeys, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
  constexpr uint32_t qstep = (2 * kXQStride) >> 4, kstep = (2 * kXChunkStride) >> 4;
  mma_ss_words<false>(s_tmem, q.lo, q.hi, k.lo, k.hi, idesc);
#pragma unroll
  for (int kk = 1; kk < HD / 16; ++kk) mma_ss_words<true>(s_tmem, q.lo + kk * qstep, q.hi, k.lo + kk * kstep, k.hi, idesc);
}
// O += P V for one row tile: P (64 keys, two bf16 per column) in the first 32 columns of its S buffer.
template <int HD>
__device__ __forceinline__ void issue_pv_x(uint32_t o_tmem, uint32_t p_tmem, RowsDesc v, bool accumulate) {
  constexpr uint32_t idesc = tc::instr_desc(128, HD, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
#pragma unroll
  for (int kk = 0; kk < kXKeys / 16; ++kk) mma_ts_words(o_tmem, p_tmem + kk * 8, v.lo + kk * (256 >> 4), v.hi, idesc, accumulate || kk > 0);
}

template <int HD>
__global__ void __launch_bounds__(kXThreads, 1)
umma_rows2_attention_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap tmap) {
  using L = XLayout<HD>;
  using B = XBars;
  using G = XG<HD>;
  constexpr int kXDim = HD, kXChunks = G::chunks, kXImage = G::image, kXVStage = G::image, kXQImage = G::qimage;
  constexpr int kXRawRow = G::raw_row, kXRawUnit = G::raw_unit;
  static_assert(L::raw % 128 == 0 && kXRawUnit % 128 == 0 && (16 * kXRawRow) % 128 == 0, "TMA destinations");
  static_assert(L::vst % 16 == 0 && kXVStage % 16 == 0 && kXImage % 16 == 0 && L::qimg % 16 == 0 && kXQImage % 16 == 0,
                "image alignment");
  static_assert(L::bars % 8 == 0, "mbarriers");
  static_assert(L::total <= 227 * 1024, "shared memory of one CTA");
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::misc + 8);

  const int kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Row tile of this CTA: bisect a shared-memory copy of query_start_loc when it fits.
  constexpr int kQslCache = 4096;
  static_assert(kXNR * kXRawUnit >= 2 * kQslCache * 4, "the raw ring holds the copies of query_start_loc and seq_lens");
  RowTile t;
  if (p.tile_map == 0 && p.num_reqs + 1 <= kQslCache) {
    int* qsl_s = reinterpret_cast<int*>(smem + L::raw);
    int* len_s = qsl_s + kQslCache;
    for (int i = tid; i <= p.num_reqs; i += kXThreads) {
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
  const int rows = t.ntok * p.group;  // <= 256 by construction of bq
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
    for (int r = tid; r < p.num_reqs; r += kXThreads) {
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
      for (int i = tid; i < rows * (p.num_splits - nsplits); i += kXThreads) {
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
    for (int idx = tid; idx < rows * kXDim; idx += kXThreads) {
      const int n = idx / kXDim, d = idx % kXDim;
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
  const int n_tiles = (key_end - key_begin + kXKeys - 1) / kXKeys;
  // Row tiles with live rows: a CTA of at most 128 rows (the end of a chunk, a short request
  // inside a prefill launch) issues no MMA for its second row tile, whose softmax warps idle.
  const int n_rt = rows > 128 ? 2 : 1;
  if (tid == 0) {
    for (int s = 0; s < kXNS; ++s) {
      tc::mbar_init(&bars[B::vfull + s], kXProducers / 2);
      tc::mbar_init(&bars[B::vempty + s], n_rt);  // one commit per row tile's PV
    }
    for (int s = 0; s < kXNK; ++s) {
      tc::mbar_init(&bars[B::kempty + s], n_rt);  // one commit per row tile's QK
      tc::mbar_init(&bars[B::kfull + s], kXProducers / 2);
    }
    for (int g = 0; g < 4; ++g) {
      tc::mbar_init(&bars[B::s_ready + g], 1);
      tc::mbar_init(&bars[B::p_ready + g], 128);  // the threads of one row tile
      tc::mbar_init(&bars[B::pv_done + g], 1);
    }
    for (int s = 0; s < kXNR; ++s) {
      tc::mbar_init(&bars[B::raw_full + s], kXKeys >> p.copy_shift);  // page copies of a unit
      tc::mbar_init(&bars[B::raw_free + s], kXProducers);             // every producer thread reads every unit
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

  if (warp >= 8 && warp < kXMmaWarp) {
    // =========================== producers ====================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kXProducerRegs));
    // Warps 8-11 widen K, warps 12-15 V.  Thread pt of a set owns row pt % 64 of the images and
    // half of its key's dims (the lower or the upper): HD / 2 bytes of the raw cell, which start 0 or 8 (K) or
    // 4 or 12 (V) bytes after a 16-byte boundary; the threads of the upper halves find the key's
    // scale right behind their bytes.  Contiguous cells (raw_mode 2) alternate between the two
    // 8-byte alignments: a warp takes the even keys or the odd ones (one widening path per warp),
    // so the images hold a tile's even keys, then its odd ones; the softmax masks by that key.
    const int pt = tid & 127;
    const bool v_part = warp >= 12;
    const int img_row = pt & (kXKeys - 1), upper = pt >> 6;
    const int key = tile_key_x(p.raw_mode, img_row);
    const int bs = p.copy_slots;  // slots of one page copy
    const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
    const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
    const int row_pitch = p.raw_mode == 1 ? kXRawRow : 2 * kXDim + 8;
    const int my_page = key >> p.copy_shift, my_slot = key & (bs - 1);
    // first byte of this thread's bytes inside a raw unit
    const uint32_t piece = my_page * bs * kXRawRow + my_slot * row_pitch + delta + (v_part ? kXDim + 4 : 0) + upper * G::piece;
    const int wo = (int)((piece & 15u) >> 2);  // first word of the piece in the 16-byte chunks read: 0 / 2 (K), 1 / 3 (V)
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int rs = j % kXNR;
      const int pos = key_begin + j * kXKeys + key;
      const bool valid = pos >= range_begin && pos < range_end;
      ok &= wait_or_abort(&bars[B::raw_full + rs], (j / kXNR) & 1, abort_flag);
      // the 16-byte chunks from the boundary below the piece: its words and the scale behind them
      uint32_t w[4 * G::load_chunks];
      if (valid) {
        const uint4* row = reinterpret_cast<const uint4*>(smem + L::raw + rs * kXRawUnit + (piece & ~15u));
#pragma unroll
        for (int c = 0; c < G::load_chunks; ++c) {
          const uint4 v = row[c];
          w[4 * c] = v.x;
          w[4 * c + 1] = v.y;
          w[4 * c + 2] = v.z;
          w[4 * c + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4 * G::load_chunks; ++c) w[c] = 0u;
      }
      // The V set multiplies its row by the key's v_scale as it widens it (below): the scale word
      // sits behind the upper half of V, which only half of the threads of a key have read.
      float v_scale = 0.f;
      if (v_part && valid)
        v_scale = *reinterpret_cast<const float*>(smem + L::raw + rs * kXRawUnit + my_page * bs * kXRawRow + my_slot * row_pitch +
                                                  delta + 2 * kXDim + 4);
      mbar_arrive(&bars[B::raw_free + rs]);  // the bytes are in registers: the unit may be refilled
      uint8_t* dst;
      if (!v_part) {
        if (j >= kXNK) ok &= wait_or_abort(&bars[B::kempty + j % kXNK], ((j / kXNK) - 1) & 1, abort_flag);
        dst = smem + L::kimg + (j % kXNK) * kXImage;
      } else {
        if (j >= kXNS) ok &= wait_or_abort(&bars[B::vempty + j % kXNS], ((j / kXNS) - 1) & 1, abort_flag);
        dst = smem + L::vst + (j % kXNS) * kXVStage;
      }
      uint8_t* out16 = dst + (upper * G::piece_chunks) * kXChunkStride + img_row * 16;  // this half's column blocks
      uint32_t scale_bits;
      // (one instance per alignment: the words of w must be compile-time indices)
      // v_scale as the sum of two bf16 (hi + lo carries 16 bits of it): x * lo rounds a term 2^-9
      // of the product, the fused multiply-add then rounds x * v_scale once
      const __nv_bfloat16 vs_hi = __float2bfloat16_rn(v_scale);
      const __nv_bfloat162 hi2 = __bfloat162bfloat162(vs_hi);
      const __nv_bfloat162 lo2 = __bfloat162bfloat162(__float2bfloat16_rn(v_scale - __bfloat162float(vs_hi)));
      auto scale2 = [&](uint32_t x) -> uint32_t {
        const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&x);
        const __nv_bfloat162 y = __hfma2(xv, hi2, __hmul2(xv, lo2));
        return *reinterpret_cast<const uint32_t*>(&y);
      };
      auto widen_piece = [&](auto first_word) {
        constexpr int kW0 = decltype(first_word)::value;
#pragma unroll
        for (int c = 0; c < G::piece_chunks; ++c) {
          uint4 x = widen8_bf16(make_uint2(w[kW0 + 2 * c], w[kW0 + 2 * c + 1]));
          if (v_part) x = make_uint4(scale2(x.x), scale2(x.y), scale2(x.z), scale2(x.w));
          *reinterpret_cast<uint4*>(out16 + c * kXChunkStride) = x;
        }
        scale_bits = w[kW0 + G::piece / 4];
      };
      if (wo == 0) widen_piece(std::integral_constant<int, 0>{});
      else if (wo == 1) widen_piece(std::integral_constant<int, 1>{});
      else if (wo == 2) widen_piece(std::integral_constant<int, 2>{});
      else widen_piece(std::integral_constant<int, 3>{});
      if (upper && !v_part)
        reinterpret_cast<float*>(smem + L::ksc)[(j % kXKsRing) * kXKeys + img_row] = __uint_as_float(scale_bits) * p.scale_log2;
      tc::fence_async_smem();
      mbar_arrive(&bars[(v_part ? B::vfull + j % kXNS : B::kfull + j % kXNK)]);
    }
  } else if (warp == kXLoadWarp) {
    // =========================== loader =======================================
    // One TMA copy per run of copy_slots slots of a tile, issued by lane `copy`: a box of the
    // tensor map (raw_mode 1) or a bulk copy of a contiguous run of cells (raw_mode 2); the
    // next tile's block ids are fetched before waiting for the unit.
    const int copies = kXKeys >> p.copy_shift;
    if (lane < copies) {
      const int bs = p.copy_slots;
      const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;
      const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
      const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
      const int tma_x = (int)((reinterpret_cast<uintptr_t>(kb) - delta -
                               (reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15)) >> 2);
      const uint32_t raw_s = tc::smem_u32(smem + L::raw);
      auto page_block = [&](int j) -> int {
        const int pos0 = key_begin + j * kXKeys + lane * bs;
        if (j >= n_tiles || pos0 >= range_end || pos0 + bs <= range_begin) return -1;
        int page, slot;
        page_and_slot(p, pos0, &page, &slot);
        return __ldg(bt + page);
      };
      auto first_slot = [&](int j) -> int {
        int page, slot;
        page_and_slot(p, key_begin + j * kXKeys + lane * bs, &page, &slot);
        return slot;
      };
      int blk = page_block(0);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j) {
        const int blk_next = page_block(j + 1);
        const int rs = j % kXNR;
        if (j >= kXNR) ok &= wait_or_abort(&bars[B::raw_free + rs], ((j / kXNR) - 1) & 1, abort_flag);
        uint64_t* bar = &bars[B::raw_full + rs];
        if (blk >= 0 && ok) {
          const uint32_t dst = raw_s + rs * kXRawUnit + lane * bs * kXRawRow;
          if (p.raw_mode == 1) {
            mbar_arrive_expect_tx(bar, bs * kXRawRow);
            tma_load_3d(dst, &tmap, tma_x, first_slot(j), blk, bar);
          } else {
            const uint32_t bytes = bs * (2 * kXDim + 8);  // a multiple of 16, like the run's address
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy_g2s(dst, kb + (int64_t)blk * p.k.stride_block + (int64_t)first_slot(j) * (2 * kXDim + 8), bytes, bar);
          }
        } else {
          mbar_arrive(bar);
        }
        blk = blk_next;
      }
    }
  } else if (warp == kXMmaWarp) {
    // =========================== MMA issuer ===================================
    // ONE elected lane issues every tcgen05.mma of the CTA in one fixed order: the QK pairs of
    // tiles 0 and 1, then for every tile i the two PV(i) and the two QK(i + 2).  Row tile rt's
    // QK(i + 2) overwrites the S buffer its P(i) was written over: it waits for its PV(i) to have
    // finished reading it, a whole tile of softmax after it is issued.
    named_barrier(5, kXSoftmax + 32);  // wait for the Q images
    // (one instance per number of live row tiles: the loops over them unroll as constants)
    auto issue_all = [&](auto live_row_tiles) {
      constexpr int kRowTiles = decltype(live_row_tiles)::value;
      const RowsDesc qd = rows_desc(tc::smem_u32(smem + L::qimg), kXQStride, 128);
      const RowsDesc kd = rows_desc(kimg_s, kXChunkStride, 128);
      const RowsDesc vd = rows_desc(vst_s, 128, kXChunkStride);
      // both row tiles' QK of tile q; after_pv: each first waits for its row tile's PV of tile q - 2
      auto issue_qk_pair = [&](int q, bool after_pv) {
        const int b = q & 1;
        ok &= wait_or_abort(&bars[B::kfull + q % kXNK], (q / kXNK) & 1, abort_flag);
#pragma unroll
        for (int rt = 0; rt < kRowTiles; ++rt) {
          if (after_pv) ok &= wait_or_abort(&bars[B::pv_done + 2 * rt + b], ((q - 2) >> 1) & 1, abort_flag);
          if (ok && elect_one()) {
            tc::fence_after_sync();
            RowsDesc k = kd, qq = qd;
            k.lo += (uint32_t)(q % kXNK) * (kXImage >> 4);
            qq.lo += (uint32_t)rt * (kXQImage >> 4);
            issue_qk_x<HD>(tmem_base + (2 * rt + b) * kXKeys, qq, k);
            tc::mma_commit(&bars[B::s_ready + 2 * rt + b]);
            tc::mma_commit(&bars[B::kempty + q % kXNK]);  // (free once both row tiles' QK have read the K image)
          }
          __syncwarp();
        }
      };
      issue_qk_pair(0, false);
      if (n_tiles > 1) issue_qk_pair(1, false);
#pragma unroll 1
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int b = i & 1;
        ok &= wait_or_abort(&bars[B::vfull + i % kXNS], (i / kXNS) & 1, abort_flag);
#pragma unroll
        for (int rt = 0; rt < kRowTiles; ++rt) {
          ok &= wait_or_abort(&bars[B::p_ready + 2 * rt + b], (i >> 1) & 1, abort_flag);
          if (ok && elect_one()) {
            tc::fence_after_sync();
            RowsDesc v = vd;
            v.lo += (uint32_t)(i % kXNS) * (kXVStage >> 4);
            issue_pv_x<HD>(tmem_base + kXOCol + rt * kXDim, tmem_base + (2 * rt + b) * kXKeys, v, i > 0);
            tc::mma_commit(&bars[B::pv_done + 2 * rt + b]);
            tc::mma_commit(&bars[B::vempty + i % kXNS]);  // (free once both row tiles' PV have read the V stage)
          }
          __syncwarp();
        }
        if (i + 2 < n_tiles) issue_qk_pair(i + 2, true);
      }
    };
    if (n_rt == 2) issue_all(std::integral_constant<int, 2>{}); else issue_all(std::integral_constant<int, 1>{});
  } else if (warp < 8) {
    // =========================== softmax ======================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kXSoftmaxRegs));
    const int rt = warp >> 2;            // row tile of this thread
    const int row = tid;                 // row of the CTA's 256 (TMEM lane tid % 128 of row tile rt)
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_rt = tmem_base + 2 * rt * kXKeys + lane_addr;          // S(rt, 0)
    const uint32_t o_tmem = tmem_base + kXOCol + rt * kXDim + lane_addr;    // O(rt)

    // ---- Q image of this row tile: thread copies its row, 16 column blocks of 8 dims ----
    {
      int token, head;
      row_target(p, t, kvh, row, &token, &head);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token +
                                                        (int64_t)head * p.q_stride_head);
      uint8_t* qrow = smem + L::qimg + rt * kXQImage + (tid & 127) * 16;
#pragma unroll
      for (int c = 0; c < kXChunks; ++c) {
        const uint4 v = row < rows ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(qrow + c * kXQStride) = v;
      }
    }
    tc::fence_async_smem();
    named_barrier(5, kXSoftmax + 32);  // Q images complete; the QK issuer may start

    int rlo = 0, rhi = -1;  // visible keys of this row (none for a padding row)
    if (row < rows) visible_range(p, t, t.first_idx + row / p.group, &rlo, &rhi);
    int mask_lo, mask_hi, tmp;  // key positions every live row sees: such tiles need no mask
    visible_range(p, t, t.first_idx + t.ntok - 1, &mask_lo, &tmp);
    visible_range(p, t, t.first_idx, &tmp, &mask_hi);
    float m_ref = -INFINITY;  // reference maximum of the row's exponentials (log2 units)
    float l = 0.f;            // sum of exp2(score - m_ref)
    // A warp whose 32 rows are all padding (the last row tile of a chunk, a short request inside
    // a prefill launch) leaves the issue slots to the others; its rows end as rows without keys
    // (m = -inf, l = 0), which the epilogue never writes.
    // (Their loop is a separate one: the live warps' loop carries no trace of the case.)  A row
    // tile without any live row is never computed: its warps wait for nothing.
    if ((row & ~31) >= rows) {
      if (rt < n_rt) {
#pragma unroll 1
        for (int i = 0; i < n_tiles; ++i) {
          // the arrival keeps the barrier's count and, behind the wait, its phase: S(rt, i + 2) is
          // not ready before P(rt, i) has been used
          ok &= wait_or_abort(&bars[B::s_ready + 2 * rt + (i & 1)], (i >> 1) & 1, abort_flag);
          mbar_arrive(&bars[B::p_ready + 2 * rt + (i & 1)]);
        }
      }
    } else {  // warps with live rows (the loop keeps its indentation)
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      const float* ksp = reinterpret_cast<const float*>(smem + L::ksc) + (i % kXKsRing) * kXKeys;
      const uint32_t s_tmem = s_rt + b * kXKeys;
      const int pos0 = key_begin + i * kXKeys;
      const bool interior = pos0 >= mask_lo && pos0 + (kXKeys - 1) <= mask_hi;
      ok &= wait_or_abort(&bars[B::s_ready + 2 * rt + b], (i >> 1) & 1, abort_flag);
      tc::fence_after_sync();
      uint32_t r[kXKeys];  // the row's scores of this tile, read once: the second half arrives while
      tc::tmem_ld32(s_tmem, r);  // pass 1 works on the first
      tc::tmem_ld_wait();
      tc::tmem_ld32(s_tmem + 32, r + 32);

      // ---- pass 1: scores in log2 units (kept in the registers) and their maximum ----
      float m_t;
      auto pass1 = [&](auto masked) {
        constexpr bool kMask = decltype(masked)::value;
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int n4 = 0; n4 < kXKeys / 4; ++n4) {
          if (n4 == kXKeys / 8) tc::tmem_ld_wait();
          const float4 ks4 = reinterpret_cast<const float4*>(ksp)[n4];  // k_scale * scale * log2 e
          const float kk[4] = {ks4.x, ks4.y, ks4.z, ks4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n4 * 4 + e;
            float sc = __uint_as_float(r[n]) * kk[e];
            if constexpr (kMask) {
              const int pos = pos0 + tile_key_x(p.raw_mode, n);  // key held by this column
              sc = (pos >= rlo && pos <= rhi) ? sc : -INFINITY;
            }
            r[n] = __float_as_uint(sc);
            mx[e] = fmaxf(mx[e], sc);
          }
        }
        m_t = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      };
      if (interior) pass1(std::false_type{}); else pass1(std::true_type{});
      // ---- move the reference maximum if the row has outgrown it ----
      const float m_new = fmaxf(m_ref, m_t);
      const bool need = m_t > m_ref + kXRescaleGap;  // also true when m_ref is still -inf
      if (i == 0) {
        m_ref = m_new;  // nothing accumulated yet
      } else if (__any_sync(0xffffffffu, need)) {
        // O(rt) must be at rest: this row tile's PV of the previous tile has completed
        ok &= wait_or_abort(&bars[B::pv_done + 2 * rt + ((i - 1) & 1)], ((i - 1) >> 1) & 1, abort_flag);
        tc::fence_after_sync();
        const float alpha = need ? ex2f_x(m_ref - m_new) : 1.0f;  // 0 when m_ref was -inf
#pragma unroll 1
        for (int j = 0; j < kXDim / 16; ++j) {
          uint32_t o[16];
          tc::tmem_ld16(o_tmem + j * 16, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int n = 0; n < 16; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * alpha);
          tc::tmem_st16(o_tmem + j * 16, o);
        }
        tc::tmem_st_wait();
        l *= alpha;
        if (need) m_ref = m_new;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

      // ---- pass 2: p as packed bf16 over the first 32 columns of S (the V image carries v_scale) ----
      // (a masked score is -inf: its p is exp2(-inf) = 0)
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t pk[16];
#pragma unroll
        for (int n4 = 0; n4 < 8; ++n4) {
          float pv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pv[e] = ex2f_x(__uint_as_float(r[j * 32 + n4 * 4 + e]) - m_use);
            ls[e] += pv[e];
          }
          pk[n4 * 2] = pack_bf16_x(pv[0], pv[1]);
          pk[n4 * 2 + 1] = pack_bf16_x(pv[2], pv[3]);
        }
        tc::tmem_st16(s_tmem + j * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc::tmem_st_wait();
      tc::fence_before_sync();
      mbar_arrive(&bars[B::p_ready + 2 * rt + b]);  // P(rt, i) is complete
    }
    }  // warps with live rows

    // ---- epilogue: the row's output (the commit after the last PV covers every MMA issued before it) ----
    if (rt < n_rt) ok &= wait_or_abort(&bars[B::pv_done + 2 * rt + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1, abort_flag);
    tc::fence_after_sync();
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    int token, head;
    row_target(p, t, kvh, row, &token, &head);
    uint8_t* out_row = p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head;
    float* ws_row = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                             (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head);
#pragma unroll 1
    for (int j = 0; j < kXDim / 32; ++j) {
      uint32_t r[32];
      tc::tmem_ld32(o_tmem + j * 32, r);
      tc::tmem_ld_wait();
      float o[32];
#pragma unroll
      for (int n = 0; n < 32; ++n) o[n] = __uint_as_float(r[n]) * inv;
      const int d0 = j * 32;
      if (row < rows) {
        if (p.num_splits > 1) {
#pragma unroll
          for (int n = 0; n < 32; n += 4)
            *reinterpret_cast<float4*>(ws_row + d0 + n) = make_float4(o[n], o[n + 1], o[n + 2], o[n + 3]);
        } else if (p.out_dtype == PTH_ATTN_BF16) {
#pragma unroll
          for (int n = 0; n < 32; n += 8)
            *reinterpret_cast<uint4*>(out_row + (d0 + n) * 2) =
                make_uint4(pack_bf16_x(o[n], o[n + 1]), pack_bf16_x(o[n + 2], o[n + 3]), pack_bf16_x(o[n + 4], o[n + 5]),
                           pack_bf16_x(o[n + 6], o[n + 7]));
        } else {
#pragma unroll
          for (int n = 0; n < 32; ++n) store_out_elem(out_row, d0 + n, p.out_dtype, o[n]);
        }
      }
    }
    if (row < rows) {
      const float lse2 = l > 0.f ? m_ref + log2f(l) : -INFINITY;
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
  if (tid == 0 && *abort_flag) atomicOr(&g_rows2_status, 4u);
  (void)ok;
}

}  // namespace

namespace {
template <int HD>
cudaError_t launch_rows2(const KernelParams& p, const CUtensorMap& map, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_rows2_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, XLayout<HD>::total);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  umma_rows2_attention_kernel<HD><<<grid, kXThreads, XLayout<HD>::total, stream>>>(p, map);
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_umma_rows2_attention(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  // Row tiles of 256 rows, whatever tile height the caller planned with.
  set_row_tile(p, kXRows / p.group > 0 ? kXRows / p.group : 1);
  set_copy_slots(p, kXKeys);  // a raw unit (64 keys) holds whole page copies
  p.raw_mode = raw_mode_for(p);
  p.num_sms = sm_count();
  if (p.num_sms <= 0) return cudaErrorInvalidDevice;
  static const CUtensorMap no_map{};
  const CUtensorMap* mapp = &no_map;
  if (p.raw_mode == 1) {
    mapp = cached_page_map(p);
    if (mapp == nullptr) return cudaErrorInvalidValue;
  }
  return p.head_size == 64 ? launch_rows2<64>(p, *mapp, stream) : launch_rows2<128>(p, *mapp, stream);
}

// Reads and clears this kernel's status word (device must be idle).
cudaError_t read_rows2_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_rows2_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_rows2_status, &zero, sizeof(zero));
}

}  // namespace pthb200
