// Row-major tcgen05 attention kernel, head size 128: query rows on the MMA M dimension.
//
// For launches with many rows per KV head (prefill chunks, wide verification steps) the
// work per KV tile is dominated by the two contractions and by one exponential per
// (row, key).  This kernel gives every query row of a 128-row tile one softmax thread
// (TMEM lane = row), so the row maximum and sum never leave that thread's registers:
//
//   loader     (1 warp)   TMA page copies of the raw cache cells into a ring of raw half
//                         stages of 64 keys (same scheme as the integer kernel);
//   producers  (8 warps)  thread t of the K set / V set widens key t's int8 K / V bytes
//                         exactly to bf16 into the K image / the V stage (canonical
//                         no-swizzle layout), with k_scale * softmax_scale * log2 e and
//                         v_scale of the key;
//   MMA issuer (1 warp, one elected lane) S = Q K^T (M = 128 rows, N = 128 keys, fp32 in
//                         TMEM, two buffers: tile i uses buffer i % 2, so S(i + 1) is computed
//                         while the softmax warps work on tile i) and O(g) += P V for each
//                         softmax group g, with P read from TMEM (the A operand) and V from
//                         the V stage as an MN-major B operand;
//   softmax    (2 groups of 4 warps; group g owns keys 64 g .. 64 g + 63 of EVERY tile)
//                         thread r reads the 64 scores of row r and its half once, pass 1
//                         turns them into log2 units (score = S * k_scale * softmax_scale *
//                         log2 e) and finds their maximum, pass 2 writes p * v_scale as
//                         packed bf16 into TMEM over the columns of S it has read.  The
//                         reference maximum of a (row, half) moves only when the running
//                         maximum outgrows it by 2^8; then the thread rescales its row of
//                         O(g) in TMEM.  In steady state O is never touched by the softmax.
// The two groups' (m, l, O) are merged in the epilogue.  TMEM: S0 S1 O0 O1, 128 columns
// each.  The CTA starts with 96 registers per thread; the producer warpgroups hand part of
// theirs to the softmax warpgroups (setmaxnreg).  Every mbarrier wait is bounded (see
// page_copy.cuh).
#include <cuda.h>

#include <type_traits>

#include "params.cuh"
#include "sched.cuh"
#include "umma_rows.cuh"
#include "page_copy.cuh"

namespace pthb200 {

__device__ unsigned int g_rows_status = 0;

namespace {

constexpr int kRGroup = 128;             // threads of one softmax group = rows of a tile
constexpr int kRSoftmax = 2 * kRGroup;   // warps 0-3, 4-7
constexpr int kRProducers = 256;         // warps 8-11 (K half) and 12-15 (V half)
constexpr int kRMmaWarp = 16, kRLoadWarp = 17;
constexpr int kRThreads = 576;
constexpr int kRNS = 2;                  // V stages (V image + v_scale)
constexpr int kHalfKeys = 64;            // keys of one raw half stage
constexpr int kRawHalfBytes = kHalfKeys * kRawRow;   // 17,408 B
constexpr int kRVStage = kWideBytes + kTileKeys * 4;  // V image + v_scale[128]
constexpr int kRKsRing = 4;                          // tiles of scaled k_scale vectors kept
// Registers: the CTA starts with 96 per thread (18 warps: five on two of the SM's four schedulers, whose
// 16,384 registers that fills).  The two producer warpgroups hand 16 per thread to the two softmax
// warpgroups, which keep the 64 scores of a row and half tile in registers between the two passes;
// every scheduler has two warps of either kind.
constexpr int kRProducerRegs = 72, kRSoftmaxRegs = 120;
constexpr float kRescaleGap = 8.0f;      // log2 units a row maximum may outgrow its reference

template <int kRNK, int kRNR>  // K images, raw HALF stages (64 keys each)
struct RLayout {
  static constexpr int kimg = 0;
  static constexpr int vst = kimg + kRNK * kWideBytes;
  static constexpr int qimg = vst + kRNS * kRVStage;
  static constexpr int raw = qimg + kQImageBytes;
  static constexpr int ksc = raw + kRNR * kRawHalfBytes;       // float [kRKsRing][128]: k_scale * scale * log2 e
  static constexpr int park_m = ksc + kRKsRing * kTileKeys * 4; // float [128]
  static constexpr int park_l = park_m + kRGroup * 4;          // float [128]
  static constexpr int bars = park_l + kRGroup * 4;            // uint64 [...]
  static constexpr int n_bars = kRNS * 2 + 2 * kRNK + 6 + 2 * kRNR;
  static constexpr int misc = bars + n_bars * 8;
  static constexpr int total = misc + 32;
};

template <int kRNK, int kRNR>
struct RBars {
  static constexpr int vfull = 0;                      // [NS] V producers -> softmax (pass 2), 128 arrivals
  static constexpr int vempty = kRNS;                  // [NS] PV commit -> V producers
  static constexpr int kempty = 2 * kRNS;              // [NK] QK commit -> K producers
  static constexpr int kfull = 2 * kRNS + kRNK;        // [NK] K producers -> QK, 128 arrivals
  static constexpr int s_ready = 2 * kRNS + 2 * kRNK;  // [2] QK commit -> softmax
  static constexpr int p_ready = s_ready + 2;          // [2] softmax -> PV, 128 arrivals
  static constexpr int pv_done = p_ready + 2;          // [2] PV commit -> QK, softmax
  static constexpr int raw_full = pv_done + 2;         // [NR]
  static constexpr int raw_free = raw_full + kRNR;     // [NR] producers -> loader, 128 arrivals
};

// Key of a tile held by row `r` of its images: with contiguous cells the rows of a half tile
// hold its even keys, then its odd ones (see the producers).
__device__ __forceinline__ int tile_key_rows(int raw_mode, int r) {
  return raw_mode == 2 ? (r & 64) + 2 * (r & 31) + ((r >> 5) & 1) : r;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int kRNK, int kRNR>
__global__ void __launch_bounds__(kRThreads, 1)
umma_rows_attention_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap tmap) {
  using L = RLayout<kRNK, kRNR>;
  using B = RBars<kRNK, kRNR>;
  static_assert(L::raw % 128 == 0 && L::vst % 128 == 0 && L::qimg % 128 == 0, "TMA / image alignment");
  static_assert(L::total <= 227 * 1024, "shared memory of one CTA");
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* qimg = smem + L::qimg;
  float* park_m = reinterpret_cast<float*>(smem + L::park_m);
  float* park_l = reinterpret_cast<float*>(smem + L::park_l);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::misc + 8);

  const int kvh = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Row tile of this CTA: bisect a shared-memory copy of query_start_loc when it fits.
  constexpr int kQslCache = 4096;
  static_assert(kRNR * kRawHalfBytes >= 2 * kQslCache * 4, "the raw ring holds the copies of query_start_loc and seq_lens");
  RowTile t;
  if (p.tile_map == 0 && p.num_reqs + 1 <= kQslCache) {
    int* qsl_s = reinterpret_cast<int*>(smem + L::raw);
    int* len_s = qsl_s + kQslCache;
    for (int i = tid; i <= p.num_reqs; i += kRThreads) {
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
    for (int r = tid; r < p.num_reqs; r += kRThreads) {
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
      for (int i = tid; i < rows * (p.num_splits - nsplits); i += kRThreads) {
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
    for (int idx = tid; idx < rows * kHeadDim; idx += kRThreads) {
      const int n = idx >> 7, d = idx & 127;
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

  const int n_tiles = tile_end - tile_begin;
  if (tid == 0) {
    for (int s = 0; s < kRNS; ++s) {
      tc::mbar_init(&bars[B::vfull + s], kRProducers / 2);
      tc::mbar_init(&bars[B::vempty + s], 1);
    }
    for (int s = 0; s < kRNK; ++s) {
      tc::mbar_init(&bars[B::kempty + s], 1);
      tc::mbar_init(&bars[B::kfull + s], kRProducers / 2);
    }
    for (int g = 0; g < 2; ++g) {
      tc::mbar_init(&bars[B::s_ready + g], 1);
      tc::mbar_init(&bars[B::p_ready + g], kRSoftmax);
      tc::mbar_init(&bars[B::pv_done + g], 1);
    }
    for (int s = 0; s < kRNR; ++s) {
      tc::mbar_init(&bars[B::raw_full + s], kHalfKeys >> p.copy_shift);  // page copies of a half stage
      tc::mbar_init(&bars[B::raw_free + s], kRProducers / 2);             // 64 K-set + 64 V-set threads
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

  if (warp >= 8 && warp < kRMmaWarp) {
    // =========================== producers ====================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRProducerRegs));
    // Warps 8-11 widen the K half of the raw cells into the K image, warps 12-15 the V half
    // (and both scales) into the V stage; thread pt of either set owns key pt of the tile.
    const int pt = tid & 127;
    const bool v_part = warp >= 12;
    const int bs = p.copy_slots;  // slots of one page copy
    const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
    const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
    const int row_pitch = p.raw_mode == 1 ? kRawRow : 2 * kHeadDim + 8;
    // the raw ring is made of half stages of 64 keys: keys 0-63 of tile j are half stage
    // u = 2 j, keys 64-127 are u = 2 j + 1; half stage u sits in slot u % kRNR
    const int half = pt >> 6;
    // Contiguous cells (raw_mode 2) alternate between the two 8-byte alignments: a warp takes the
    // even keys or the odd ones of its half stage, so that it runs one of the two code paths
    // below.  Row pt of the images (and of the scale vectors) then holds key tile_key_rows(pt):
    // the order of the keys inside a tile changes no sum, and the softmax masks by that key.
    const int key = tile_key_rows(p.raw_mode, pt);
    const int my_page = (key & (kHalfKeys - 1)) >> p.copy_shift, my_slot = key & (bs - 1);
    const uint32_t cell_off = my_page * bs * kRawRow + my_slot * row_pitch + delta;  // inside a half stage
    const bool odd = (cell_off & 8u) != 0;
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int u = 2 * j + half;
      const int rs = u % kRNR;
      const int pos = (tile_begin + j) * kTileKeys + key;
      const bool valid = pos >= range_begin && pos < range_end;
      // A raw slot is used by the two halves in turn (kRNR is odd), and a parity wait only
      // tells apart two consecutive phases: this thread must not look at raw_full[rs] while
      // the slot's PREVIOUS half stage (the other half's) is still pending, or it would take
      // the phase before that one for its own, read stale bytes and release the slot early.
      // Page copies can complete out of order, so nothing else rules that out.  Wait first
      // until the previous occupant has been taken out of the slot.
      if (u >= kRNR) ok &= wait_or_abort(&bars[B::raw_free + rs], ((u / kRNR) - 1) & 1, abort_flag);
      ok &= wait_or_abort(&bars[B::raw_full + rs], (u / kRNR) & 1, abort_flag);
      // nine 16-byte chunks: raw words 0..35 (K half, k_scale) or 32..67 (k_scale, V half, v_scale)
      uint32_t w[36];
      if (valid) {
        const uint4* row = reinterpret_cast<const uint4*>(smem + L::raw + rs * kRawHalfBytes + (cell_off & ~15u)) +
                           (v_part ? 8 : 0);
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
      mbar_arrive(&bars[B::raw_free + rs]);  // the half row is in registers: the stage may be refilled
      const int st = j % kRNS;
      if (!v_part) {
        uint8_t* kdst = smem + L::kimg + (j % kRNK) * kWideBytes + pt * 16;
        if (j >= kRNK) ok &= wait_or_abort(&bars[B::kempty + j % kRNK], ((j / kRNK) - 1) & 1, abort_flag);
        float* ksc = reinterpret_cast<float*>(smem + L::ksc) + (j % kRKsRing) * kTileKeys;
        if (!odd) {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            *reinterpret_cast<uint4*>(kdst + c * kChunkStride) = widen8_bf16(make_uint2(w[2 * c], w[2 * c + 1]));
          ksc[pt] = __uint_as_float(w[32]) * p.scale_log2;
        } else {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            *reinterpret_cast<uint4*>(kdst + c * kChunkStride) = widen8_bf16(make_uint2(w[2 + 2 * c], w[3 + 2 * c]));
          ksc[pt] = __uint_as_float(w[34]) * p.scale_log2;
        }
        tc::fence_async_smem();
        mbar_arrive(&bars[B::kfull + j % kRNK]);
      } else {
        uint8_t* vstage = smem + L::vst + st * kRVStage;
        uint8_t* vdst = vstage + pt * 16;
        if (j >= kRNS) ok &= wait_or_abort(&bars[B::vempty + st], ((j / kRNS) - 1) & 1, abort_flag);
        if (!odd) {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            *reinterpret_cast<uint4*>(vdst + c * kChunkStride) = widen8_bf16(make_uint2(w[1 + 2 * c], w[2 + 2 * c]));
          *reinterpret_cast<uint32_t*>(vstage + kWideBytes + pt * 4) = w[33];
        } else {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            *reinterpret_cast<uint4*>(vdst + c * kChunkStride) = widen8_bf16(make_uint2(w[3 + 2 * c], w[4 + 2 * c]));
          *reinterpret_cast<uint32_t*>(vstage + kWideBytes + pt * 4) = w[35];
        }
        tc::fence_async_smem();
        mbar_arrive(&bars[B::vfull + st]);
      }
    }
  } else if (warp == kRLoadWarp) {
    // =========================== loader =======================================
    // One TMA copy per KV page of a tile, issued by lane `page`: a tiled tensor-map box of
    // [block_size slots] x [272 bytes] (raw_mode 1) or one bulk copy of a contiguous page
    // run (raw_mode 2); the next tile's block ids are fetched before waiting for the stage.
    const int pages_per_half = kHalfKeys >> p.copy_shift;
    if (lane < pages_per_half) {
      const int bs = p.copy_slots;
      const int32_t* bt = p.block_table + (int64_t)t.req * p.block_table_row_stride;
      const uint8_t* kb = p.k.data + (int64_t)kvh * p.k.stride_head;
      const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
      const int tma_x = (int)((reinterpret_cast<uintptr_t>(kb) - delta -
                               (reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15)) >> 2);
      const uint32_t raw_s = tc::smem_u32(smem + L::raw);
      const int n_halves = 2 * n_tiles;
      // block id of this lane's page of half stage u, -1 if no key of the page is in range
      auto page_block = [&](int u) -> int {
        const int pos0 = tile_begin * kTileKeys + u * kHalfKeys + lane * bs;
        if (u >= n_halves || pos0 >= range_end || pos0 + bs <= range_begin) return -1;
        int page, slot;
        page_and_slot(p, pos0, &page, &slot);
        return __ldg(bt + page);
      };
      // first slot, inside its page, of this lane's copy of half stage u
      auto first_slot = [&](int u) -> int {
        int page, slot;
        page_and_slot(p, tile_begin * kTileKeys + u * kHalfKeys + lane * bs, &page, &slot);
        return slot;
      };
      int blk = page_block(0);
#pragma unroll 1
      for (int u = 0; u < n_halves; ++u) {
        const int blk_next = page_block(u + 1);
        const int rs = u % kRNR;
        if (u >= kRNR) ok &= wait_or_abort(&bars[B::raw_free + rs], ((u / kRNR) - 1) & 1, abort_flag);
        uint64_t* bar = &bars[B::raw_full + rs];
        if (blk >= 0 && ok) {
          const uint32_t dst = raw_s + rs * kRawHalfBytes + lane * bs * kRawRow;
          if (p.raw_mode == 1) {
            mbar_arrive_expect_tx(bar, bs * kRawRow);
            tma_load_3d(dst, &tmap, tma_x, first_slot(u), blk, bar);
          } else {
            const uint32_t bytes = bs * (2 * kHeadDim + 8);  // a multiple of 16, like the run's address
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy_g2s(dst, kb + (int64_t)blk * p.k.stride_block + (int64_t)first_slot(u) * (2 * kHeadDim + 8), bytes, bar);
          }
        } else {
          mbar_arrive(bar);
        }
        blk = blk_next;
      }
    }
  } else if (warp == kRMmaWarp) {
    // =========================== MMA issuer ===================================
    // ONE thread (the lane elect.sync picks) issues every tcgen05.mma of the CTA, in one fixed
    // order: QK(0), QK(1), then PV(i), QK(i + 2) for i = 0, 1, ...  S has two buffers in TMEM
    // (tile i uses buffer i % 2), so QK(i + 1) runs while the softmax warps work on tile i.
    // P(i) is written over the columns of S(i) it was computed from: QK(i + 2), which
    // overwrites that buffer, waits for PV(i) to have finished reading them - one whole tile
    // of softmax later than it is issued, so the wait is not on the critical path.  PV(i) is
    // two chains: keys 0-63 of the tile into O(0), keys 64-127 into O(1), the accumulators of
    // the two softmax groups.  (A version with one issuing thread for QK and another for PV
    // produced results that varied from run to run; a version that polled the barriers and
    // issued whatever was ready first was slower.)  Operand descriptors are kept as register
    // word pairs.
    named_barrier(5, kRSoftmax + 32);  // wait for the Q image
    {
      const RowsDesc qd = rows_desc(tc::smem_u32(qimg), kChunkStride, 128);
      const RowsDesc kd = rows_desc(kimg_s, kChunkStride, 128);
      const RowsDesc vd = rows_desc(vst_s, 128, kChunkStride);
      auto issue_qk = [&](int q) {
        ok &= wait_or_abort(&bars[B::kfull + q % kRNK], (q / kRNK) & 1, abort_flag);
        if (ok && elect_one()) {
          tc::fence_after_sync();
          RowsDesc k = kd;
          k.lo += (uint32_t)(q % kRNK) * (kWideBytes >> 4);
          issue_qk_rows_words(tmem_base + (q & 1) * 128, qd, k);
          tc::mma_commit(&bars[B::s_ready + (q & 1)]);
          tc::mma_commit(&bars[B::kempty + q % kRNK]);
        }
        __syncwarp();
      };
      issue_qk(0);
      if (n_tiles > 1) issue_qk(1);
#pragma unroll 1
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int sb = i & 1;
        ok &= wait_or_abort(&bars[B::p_ready + sb], (i >> 1) & 1, abort_flag);
        if (ok && elect_one()) {
          tc::fence_after_sync();
          RowsDesc v = vd;
          v.lo += (uint32_t)(i % kRNS) * (kRVStage >> 4);
          issue_pv_halves_words(tmem_base + 256, tmem_base + sb * 128, v, i > 0);
          tc::mma_commit(&bars[B::pv_done + sb]);
          tc::mma_commit(&bars[B::vempty + i % kRNS]);
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRSoftmaxRegs));
    // Softmax group h (warps 4 h .. 4 h + 3) owns keys 64 h .. 64 h + 63 of EVERY tile: its thread
    // `row` keeps the running reference maximum and sum of that row over those keys and the
    // accumulator O(h) in TMEM; the two groups' results are merged at the end.  Both groups work
    // on tile i at the same time while the tensor core computes S(i + 1) into the other buffer.
    const int g = warp >> 2;
    const int row = tid & 127;   // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_half = tmem_base + g * 64 + lane_addr;         // this group's columns of S buffer 0
    const uint32_t o_tmem = tmem_base + 256 + g * 128 + lane_addr;  // O(g)

    // ---- Q image: thread (row, half) copies 8 of the 16 d-chunks of its row ----
    {
      const int half = tid >> 7;
      int token, head;
      row_target(p, t, kvh, row, &token, &head);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token +
                                                        (int64_t)head * p.q_stride_head);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int cc = half * 8 + c;
        const uint4 v = row < rows ? __ldg(src + cc) : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(qimg + cc * kChunkStride + row * 16) = v;
      }
    }
    tc::fence_async_smem();
    named_barrier(5, kRSoftmax + 32);  // Q image complete; the QK issuer may start

    int rlo = 0, rhi = -1;  // visible keys of this row (none for a padding row)
    if (row < rows) visible_range(p, t, t.first_idx + row / p.group, &rlo, &rhi);
    int mask_lo, mask_hi, tmp;  // key positions every live row sees: such tiles need no mask
    visible_range(p, t, t.first_idx + t.ntok - 1, &mask_lo, &tmp);
    visible_range(p, t, t.first_idx, &tmp, &mask_hi);
    float m_ref = -INFINITY;  // reference maximum of the row's exponentials (log2 units)
    float l = 0.f;            // sum of exp2(score - m_ref)
    // A warp whose 32 rows are all padding (a drafter step fills 64 of the 128 rows, a wide
    // verification step 32) leaves the issue slots to the others; its rows end as rows without
    // keys (m = -inf, l = 0), which the epilogue never writes.
    // (Their loop is a separate one: the live warps' loop carries no trace of the case.)
    if ((row & ~31) >= rows) {
#pragma unroll 1
      for (int i = 0; i < n_tiles; ++i) {
        // the arrival keeps the barrier's count and, behind the wait, its phase: S(i + 2) is not
        // ready before P(i) has been used
        ok &= wait_or_abort(&bars[B::s_ready + (i & 1)], (i >> 1) & 1, abort_flag);
        mbar_arrive(&bars[B::p_ready + (i & 1)]);
      }
    } else {  // warps with live rows (the loop keeps its indentation)
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
      const float* ksp = reinterpret_cast<const float*>(smem + L::ksc) + (i % kRKsRing) * kTileKeys + g * 64;
      const float* vsp = reinterpret_cast<const float*>(smem + L::vst + (i % kRNS) * kRVStage + kWideBytes) + g * 64;
      const uint32_t s_tmem = s_half + (i & 1) * 128;
      const int pos0 = (tile_begin + i) * kTileKeys;
      const bool interior = pos0 >= mask_lo && pos0 + (kTileKeys - 1) <= mask_hi;
      ok &= wait_or_abort(&bars[B::s_ready + (i & 1)], (i >> 1) & 1, abort_flag);
      tc::fence_after_sync();
      // the 64 scores of this row and half, read once
      uint32_t r[64];
      tc::tmem_ld32(s_tmem, r);
      tc::tmem_ld32(s_tmem + 32, r + 32);
      tc::tmem_ld_wait();

      // ---- pass 1: scores in log2 units (kept in the registers) and their maximum ----
      // (two instances: interior tiles, which every live row sees whole, skip the mask)
      float m_t;
      auto pass1 = [&](auto masked) {
        constexpr bool kMask = decltype(masked)::value;
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int n4 = 0; n4 < 16; ++n4) {
          const float4 ks4 = reinterpret_cast<const float4*>(ksp)[n4];  // k_scale * scale * log2 e
          const float kk[4] = {ks4.x, ks4.y, ks4.z, ks4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n4 * 4 + e;
            float sc = __uint_as_float(r[n]) * kk[e];
            if constexpr (kMask) {
              const int pos = pos0 + tile_key_rows(p.raw_mode, g * 64 + n);  // key held by column g 64 + n
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
      const bool need = m_t > m_ref + kRescaleGap;  // also true when m_ref is still -inf
      if (i == 0) {
        m_ref = m_new;  // nothing accumulated yet
      } else if (__any_sync(0xffffffffu, need)) {
        // O(g) must be at rest: the PV of the previous tile has completed
        ok &= wait_or_abort(&bars[B::pv_done + ((i - 1) & 1)], ((i - 1) >> 1) & 1, abort_flag);
        tc::fence_after_sync();
        const float alpha = need ? ex2f(m_ref - m_new) : 1.0f;  // 0 when m_ref was -inf
#pragma unroll 1
        for (int j = 0; j < 8; ++j) {
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

      // ---- pass 2: p * v_scale as packed bf16 over the first columns of this half of S ----
      // (a masked score is -inf: its p is exp2(-inf) = 0)
      ok &= wait_or_abort(&bars[B::vfull + i % kRNS], (i / kRNS) & 1, abort_flag);  // v_scale (and V) of tile i
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t pk[16];
#pragma unroll
        for (int n4 = 0; n4 < 8; ++n4) {
          const float4 vs4 = reinterpret_cast<const float4*>(vsp)[j * 8 + n4];
          const float vv[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
          float pv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float pr = ex2f(__uint_as_float(r[j * 32 + n4 * 4 + e]) - m_use);
            ls[e] += pr;
            pv[e] = pr * vv[e];
          }
          pk[n4 * 2] = pack_bf16(pv[0], pv[1]);
          pk[n4 * 2 + 1] = pack_bf16(pv[2], pv[3]);
        }
        tc::tmem_st16(s_tmem + j * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc::tmem_st_wait();
      tc::fence_before_sync();
      mbar_arrive(&bars[B::p_ready + (i & 1)]);  // this group's half of P(i) is complete
    }
    }  // warps with live rows

    // ---- epilogue: merge the two groups' (m, l, O) and write the rows ----
    // (the commit after the last PV covers every MMA issued before it)
    ok &= wait_or_abort(&bars[B::pv_done + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1, abort_flag);
    tc::fence_after_sync();
    // Group 1 hands its state to group 0 through 64 KB of shared memory that is idle by
    // now: the K images if they are large enough (every QK has completed once the last
    // tile's K image has been released), else the raw ring (every producer has read it
    // once the last tile's images are full).
    constexpr int kParkBytes = kRGroup * kHeadDim * 4;
    constexpr bool kParkInK = kRNK * kWideBytes >= kParkBytes;
    static_assert(kParkInK || kRNR * kRawHalfBytes >= kParkBytes, "no idle region holds the parked accumulator");
    float* park = reinterpret_cast<float*>(smem + (kParkInK ? L::kimg : L::raw));  // [d][row] fp32
    if (g == 1) {
      if constexpr (kParkInK) {
        ok &= wait_or_abort(&bars[B::kempty + (n_tiles - 1) % kRNK], ((n_tiles - 1) / kRNK) & 1, abort_flag);
      } else {
        ok &= wait_or_abort(&bars[B::vfull + (n_tiles - 1) % kRNS], ((n_tiles - 1) / kRNS) & 1, abort_flag);
        ok &= wait_or_abort(&bars[B::kfull + (n_tiles - 1) % kRNK], ((n_tiles - 1) / kRNK) & 1, abort_flag);
      }
      park_m[row] = m_ref;
      park_l[row] = l;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        uint32_t r[32];
        tc::tmem_ld32(o_tmem + j * 32, r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int n = 0; n < 32; ++n) park[(j * 32 + n) * kRGroup + row] = __uint_as_float(r[n]);
      }
    }
    named_barrier(4, kRSoftmax);
    if (g == 0) {
      const float m1 = park_m[row], l1 = park_l[row];
      const float m = fmaxf(m_ref, m1);
      const float c0 = m_ref == -INFINITY ? 0.f : ex2f(m_ref - m);
      const float c1 = m1 == -INFINITY ? 0.f : ex2f(m1 - m);
      const float lsum = l * c0 + l1 * c1;
      const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
      int token, head;
      row_target(p, t, kvh, row, &token, &head);
      uint8_t* out_row = p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head;
      float* ws_row = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                               (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head);
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        uint32_t r[32];
        tc::tmem_ld32(o_tmem + j * 32, r);
        tc::tmem_ld_wait();
        float o[32];
#pragma unroll
        for (int n = 0; n < 32; ++n) {
          const float o1 = c1 > 0.f ? park[(j * 32 + n) * kRGroup + row] * c1 : 0.f;
          o[n] = (__uint_as_float(r[n]) * c0 + o1) * inv;
        }
        if (row < rows) {
          if (p.num_splits > 1) {
#pragma unroll
            for (int n = 0; n < 32; n += 4)
              *reinterpret_cast<float4*>(ws_row + j * 32 + n) = make_float4(o[n], o[n + 1], o[n + 2], o[n + 3]);
          } else if (p.out_dtype == PTH_ATTN_BF16) {
#pragma unroll
            for (int n = 0; n < 32; n += 8)
              *reinterpret_cast<uint4*>(out_row + (j * 32 + n) * 2) =
                  make_uint4(pack_bf16(o[n], o[n + 1]), pack_bf16(o[n + 2], o[n + 3]), pack_bf16(o[n + 4], o[n + 5]),
                             pack_bf16(o[n + 6], o[n + 7]));
          } else {
#pragma unroll
            for (int n = 0; n < 32; ++n) store_out_elem(out_row, j * 32 + n, p.out_dtype, o[n]);
          }
        }
      }
      if (row < rows) {
        const float lse2 = lsum > 0.f ? m + log2f(lsum) : -INFINITY;
        if (p.num_splits > 1) {
          *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)split * p.ws_lse_stride_split +
                                    (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head) = lse2;
        } else if (p.lse_out != nullptr) {
          *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                    (int64_t)head * p.lse_stride_head) = lse2 * kLn2;
        }
      }
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
  if (tid == 0 && *abort_flag) atomicOr(&g_rows_status, 4u);
  (void)ok;
}

}  // namespace

// The row-major kernel reads the cache like the integer kernel (packed cells through TMA
// page copies) and takes bf16 queries.
bool umma_rows_supports(const KernelParams& p, const char** why) {
  if (!umma_i8_supports(p, why)) return false;
  // (this file: 128 dims; 256 dims: umma_rows256_kernel.cu; 64 dims: umma_rows2_kernel.cu)
  if (p.q_dtype != PTH_ATTN_BF16) {
    *why = "q is not bf16";  // the Q image is the query bits as they are, and K / V are widened to bf16
    return false;
  }
  return true;
}

namespace {
template <int NK, int NR>
cudaError_t launch_rows(const KernelParams& p, const CUtensorMap& map, dim3 grid, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_rows_attention_kernel<NK, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               RLayout<NK, NR>::total);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  umma_rows_attention_kernel<NK, NR><<<grid, kRThreads, RLayout<NK, NR>::total, stream>>>(p, map);
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_umma_rows_attention(const KernelParams& p_in, cudaStream_t stream) {
  if (p_in.head_size == 256) return launch_umma_rows256_attention(p_in, stream);
  if (p_in.head_size == 64) return launch_umma_rows2_attention(p_in, stream);  // the only row-major kernel for 64 dims
  // Launches whose requests have 256 rows or more on average (prefill chunks) run two row tiles
  // per CTA, which share every widened K / V tile (umma_rows2_kernel.cu); shorter ones (wide
  // verification, drafter steps) would leave its second row tile empty.
  if ((int64_t)p_in.num_tokens * p_in.group >= 256 * (int64_t)p_in.num_reqs) return launch_umma_rows2_attention(p_in, stream);
  KernelParams p = p_in;
  // Row tiles of 128 rows, whatever tile height the caller planned with: the partition of
  // the query tokens into row tiles is internal to a launch.
  set_row_tile(p, 128 / p.group > 0 ? 128 / p.group : 1);
  set_copy_slots(p, kHalfKeys);  // a raw half stage holds whole page copies
  p.raw_mode = raw_mode_for(p);
  p.num_sms = sm_count();
  if (p.num_sms <= 0) return cudaErrorInvalidDevice;
  static const CUtensorMap no_map{};
  const CUtensorMap* mapp = &no_map;
  if (p.raw_mode == 1) {
    mapp = cached_page_map(p);
    if (mapp == nullptr) return cudaErrorInvalidValue;
  }
  const CUtensorMap& map = *mapp;
  // Two K images and three raw half stages (64 keys each).  Consecutive QK MMAs must not read
  // their K operand from the same shared-memory addresses: with a single K image that the
  // producers rewrote between two QKs, results varied from run to run although every
  // producer / consumer edge was ordered by an mbarrier and a proxy fence.
  const dim3 grid(p.num_q_tiles, p.num_kv_heads, p.num_splits);
  return launch_rows<2, 3>(p, map, grid, stream);
}

// Reads and clears this file's status word (device must be idle).
cudaError_t read_rows_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_rows_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_rows_status, &zero, sizeof(zero));
}

}  // namespace pthb200


#include "umma_rows_tile_test.cuh"
