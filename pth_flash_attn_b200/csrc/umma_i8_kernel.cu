// Integer tcgen05 attention kernel, head sizes 64 / 128 / 256, token-major orientation, persistent CTAs.
//
// The cache holds int8 K and V, so both contractions run on the int8 tensor path
// (tcgen05.mma.kind::i8, int32 accumulators in TMEM) with the cache bytes used AS
// STORED: nothing is widened, dequantised or converted between HBM and the MMA.
//
// The two floating-point operands become exact sums of int8 "digits":
//   Q row n:  q = sq[n] * (256 qh + ql),   qh, ql int8     (sq = absmax / 32512)
//   P key t:  p * v_scale[t] = u[n] * sum_k 128^k d_k,     0 <= d_k < 128
// with one unit u[n] per (KV tile, row), so the dynamic range that fixed point
// must cover is that of ONE tile; the digits sit side by side on the MMA N
// dimension:
//   S^T[key, (digit, row)]  = sum_d   K[key, d] * Qdigit[row, d]     (N = 2 NPAD)
//   O^T[d,   (digit, row)]  = sum_key V[key, d] * Pdigit[key, row]   (N = PD NPAD)
// Integer MMAs are exact; the only roundings are the 16-bit quantisation of q
// (relative 2^-16 of the row maximum) and the 7 PD-bit quantisation of
// p * v_scale (relative 2^-(7 PD + 1) of the tile maximum).
//
// One CTA per SM runs work items (row tile x KV head x split) one after the other
// (sched.cuh says which).  Its warps have seven roles that meet only through mbarriers
// (tile = 128 consecutive keys); the rings of the data path are indexed by a tile count
// that runs on across items, so the copies of the next item's first tiles are in flight
// while the last tiles of the current item are still being computed:
//   scheduler  (1 warp)  walks the requests, finds this CTA's next item, writes -inf
//              markers for splits a request does not use and the result of an item
//              without keys, and for every other item publishes a descriptor together
//              with the item's Q digit image, row scales and row masks (two slots, so the
//              next item is staged while the current one runs);
//   loader     (1 warp)  lane `c` issues page copy c of a tile - a [copy_slots slots] x
//              [raw row] box of a tiled tensor map (raw row = the 16-byte aligned bytes
//              that cover a cell: 144 / 272 / 528 for head sizes 64 / 128 / 256), or a bulk
//              copy when the cells of a page are contiguous - into a ring of NR raw stages;
//              copy_slots is the largest power of two from 16 to 128 that divides the page
//              size, so a page of 816 slots is fetched 16 slots at a time and a tile may
//              straddle two pages; block ids are fetched one tile ahead;
//   producers  (NP groups of 4 warps; group k takes the tiles g with g % NP == k)
//              thread t reads the raw bytes around key t's cell into registers,
//              releases the raw stage, and writes them 16 bytes at a time into the
//              canonical (no-swizzle) operand images: K into a ring of NK K images,
//              V and the two scale vectors into a ring of NS V stages.  A cell is only
//              8-byte aligned and V starts D + 4 bytes into it, which is why the bytes
//              pass through registers once (a 256-dim row in two halves);
//   MMA issuer (1 thread) per item, in a fixed order: QK(0), QK(1), then QK(i + 2), PV(i);
//              S^T of a tile lands in one of SB buffers of the tile's softmax group, O^T in
//              the group's O^T buffer; its commits signal the softmax and free the images;
//   softmax    (2 groups of 4 warps; group g owns the tiles whose running count is g mod 2,
//              with its own running maximum, sum and accumulator) thread t owns key t of
//              S^T (scores -> tile maximum -> probabilities -> digits of P) and output
//              column d = t of O^T (and t + 128 of a 256-dim head, whose O^T is two
//              accumulators of 128 dims), which it folds tile by tile into an fp32 register
//              accumulator (acc = acc * alpha + O^T * u), so TMEM never holds a value
//              that needs rescaling.  Per-row factors live in lanes and travel by
//              shuffle.  The two groups' states are merged at the end of every item.
// Every mbarrier wait is bounded: a wait that gives up raises a CTA-wide abort
// flag (all later waits return at once), sets bit 2 of the status word, and the
// CTA still finishes and frees its TMEM.
#include <cuda.h>

#include "params.cuh"
#include "sched.cuh"
#include "umma_i8.cuh"
#include "page_copy.cuh"

namespace pthb200 {

__device__ unsigned int g_i8_status = 0;

namespace {

constexpr int kGroupThreads = 128;                      // one softmax warpgroup
constexpr int kSoftmaxThreads = 2 * kGroupThreads;      // warps 0-3 and 4-7
constexpr int kProducerThreads = 128;                   // one producer group: one thread per key of a tile
constexpr int kItemSlots = 2;                           // item descriptors (and Q images) in flight
// Warps after the softmax groups: NP producer groups of four warps, then the MMA issuer,
// the loader and the scheduler.
__host__ __device__ constexpr int threads_for(int np) { return kSoftmaxThreads + np * kProducerThreads + 96; }
constexpr int kStageScales = 2 * kKeys * 4;                 // k_scale[128], v_scale[128]

// What the scheduler publishes for one item (shared memory, one per slot).
struct ItemDesc {
  int32_t n_tiles;      // KV tiles of the item; 0 = no more items
  int32_t req, kvh, split;
  int32_t tok0, ntok;   // first query token (row of q / out) and query tokens of the row tile
  int32_t tile_begin;   // first KV tile
  int32_t range_begin, range_end;  // keys the rows of the tile see together
  int32_t mask_lo, mask_hi;        // keys EVERY live row sees: tiles inside need no mask
  int32_t pad;
};

template <int HD, int NPAD, int PD, int NS, int NK, int NR, int SB>
struct Layout {
  using G = I8Geom<HD>;
  static constexpr int img_bytes = G::img_bytes;
  static constexpr int vstage_bytes = G::img_bytes + kStageScales;  // V image and both scale vectors of one tile
  static constexpr int kstages = 0;                                 // [NK] K images
  static constexpr int vstages = kstages + NK * img_bytes;          // [NS] V image + scales
  static constexpr int qimg = vstages + NS * vstage_bytes;          // [slots][HD / 16][2 NPAD][16]
  static constexpr int qimg_bytes = G::chunks * 2 * NPAD * 16;
  static constexpr int pimg = qimg + kItemSlots * qimg_bytes;       // [2 groups][PD NPAD / 16][128][16]
  static constexpr int pimg_bytes = 2 * PD * NPAD * kKeys;
  // The raw ring is made of NR units of unit_keys keys: whole tiles, or - for 256 dims, whose
  // tile of raw rows is 66 KB - half tiles, so that a tile and a half can be in flight.
  static constexpr int raw_units = HD > 128 ? 2 : 1;                // units per tile
  static constexpr int unit_keys = kKeys / raw_units;
  static constexpr int unit_bytes = unit_keys * G::raw_row;
  static constexpr int raw = (pimg + pimg_bytes + 127) / 128 * 128; // [NR] raw units (TMA destinations: 128-byte aligned)
  static constexpr int wred = raw + NR * unit_bytes;                // float [2 groups][2][4][NPAD + 1]
  static constexpr int mrun = wred + 2 * 2 * 4 * (NPAD + 1) * 4;    // float [2 groups][2 NPAD], first NPAD used
  static constexpr int sq = mrun + 2 * 2 * NPAD * 4;                // float [slots][NPAD]
  static constexpr int rlo = sq + kItemSlots * NPAD * 4;            // int [slots][NPAD]
  static constexpr int rhi = rlo + kItemSlots * NPAD * 4;           // int [slots][NPAD]
  static constexpr int desc = (rhi + kItemSlots * NPAD * 4 + 15) / 16 * 16;  // ItemDesc [slots]
  static constexpr int bars = desc + kItemSlots * (int)sizeof(ItemDesc);
  static constexpr int n_bars = 2 * NS + 14 + 2 * NR + 2 * kItemSlots;
  static constexpr int misc = bars + n_bars * 8;                    // abort flag, TMEM slot, total work
  static constexpr int total = misc + 32;
  static constexpr int s_cols = 2 * NPAD;
  static constexpr int o_cols = G::halves * PD * NPAD;              // one O^T accumulator per 128 dims of the head
  static constexpr int s_total = 2 * SB * s_cols;                   // [2 groups][SB] S^T buffers
  static constexpr int tmem_need = s_total + 2 * o_cols;
  static constexpr int tmem_alloc = tmem_need <= 32 ? 32 : tmem_need <= 64 ? 64 : tmem_need <= 128 ? 128
                                    : tmem_need <= 256 ? 256 : 512;
  static_assert(sizeof(ItemDesc) % 16 == 0, "descriptor slots stay 16-byte aligned");
  static_assert(raw % 128 == 0 && unit_bytes % 128 == 0 && (16 * G::raw_row) % 128 == 0,
                "every page copy of 16 or more slots lands on a 128-byte boundary");
  static_assert(vstages % 16 == 0 && vstage_bytes % 16 == 0 && qimg % 16 == 0 && qimg_bytes % 16 == 0 && pimg % 16 == 0,
                "operand images start on 16-byte boundaries");
  static_assert(wred % 16 == 0 && bars % 8 == 0, "reduction buffers and mbarriers are aligned");
};

// Barrier indices inside the barrier array.
template <int NS, int NR>
struct Bars {
  static constexpr int full = 0;             // [NS] producers -> MMA, 128 arrivals
  static constexpr int empty = NS;           // [NS] PV issuer (tcgen05.commit) -> producers: V stage free
  static constexpr int s_ready = 2 * NS;      // [2 groups][2] MMA -> softmax (and producers: K image free)
  static constexpr int s_free = 2 * NS + 4;   // [2 groups][2] softmax -> MMA, 128 arrivals
  static constexpr int o_ready = 2 * NS + 8;  // [2] MMA -> softmax
  static constexpr int o_free = 2 * NS + 10;  // [2] softmax -> MMA, 128 arrivals
  static constexpr int p_ready = 2 * NS + 12; // [2] softmax -> MMA, 128 arrivals
  static constexpr int raw_full = 2 * NS + 14;// [NR] page copies -> producers
  static constexpr int raw_free = 2 * NS + 14 + NR;  // [NR] producers -> loader, 128 arrivals
  static constexpr int item_full = 2 * NS + 14 + 2 * NR;               // [slots] scheduler -> every other role
  static constexpr int item_empty = 2 * NS + 14 + 2 * NR + kItemSlots; // [slots] every other role -> scheduler
};

// Key of a tile held by row `r` of its operand images (see the producers).
__device__ __forceinline__ int tile_key(const KernelParams& p, int r) {
  return p.raw_mode == 2 ? 2 * (r & 63) + (r >> 6) : r;
}

// Barrier over `count` threads that also ORs a predicate over them (uniform result).
__device__ __forceinline__ bool named_barrier_or(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %3, 0;\n\t"
      "bar.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

template <int HD, int NPAD, int PD, int NS, int NK, int NR, int SB, int RQ, int NP>
__global__ void __launch_bounds__(threads_for(NP), 1)
umma_i8_attention_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap tmap) {
  using L = Layout<HD, NPAD, PD, NS, NK, NR, SB>;
  using B = Bars<NS, NR>;
  using G = I8Geom<HD>;
  constexpr int kRawRowHD = G::raw_row, kRawStageHD = L::unit_bytes, kImgHD = G::img_bytes;
  constexpr int RU = L::raw_units, kUnitKeys = L::unit_keys;  // raw units per tile, keys per unit
  // QK runs LA tiles ahead of PV: two when there is a V stage for it, else one
  constexpr int LA = NS >= 3 ? 2 : 1;
  constexpr int kVStageHD = L::vstage_bytes, kHalves = G::halves;
  constexpr int kRawStages = NR;
  constexpr int XMAX = (1 << (7 * PD)) - 1;
  constexpr int kThreads = threads_for(NP);
  constexpr int kMmaWarp = 8 + 4 * NP;     // lane 0 issues every MMA
  constexpr int kLoadWarp = kMmaWarp + 1;  // issues the page copies
  constexpr int kSchedWarp = kMmaWarp + 2; // finds and stages the items
  // arrivals that free an item slot: every softmax and producer thread, the issuer, the loader
  constexpr int kItemReaders = kSoftmaxThreads + NP * kProducerThreads + 2;
  static_assert(RQ >= 1 && 4 * RQ <= NPAD, "RQ = groups of four rows the softmax handles (rows <= 4 RQ)");
  // QK(i + LA) is issued before PV(i) (see the issuer) and needs the V stage of tile i + LA
  // filled: with LA + 1 stages or more that is never the one PV(i) has yet to free.
  static_assert(NS >= LA + 1 && NS >= 2, "tile i + LA needs a V stage of its own");
  static_assert(PD * NPAD >= 8 * RQ, "the P images hold 128 dims of the parked accumulator of one softmax group");
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* pimg = smem + L::pimg;
  float* wred = reinterpret_cast<float*>(smem + L::wred);
  float* mrun = reinterpret_cast<float*>(smem + L::mrun);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bars);
  volatile ItemDesc* descs = reinterpret_cast<volatile ItemDesc*>(smem + L::desc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + L::misc + 8);
  unsigned long long* total_s = reinterpret_cast<unsigned long long*>(smem + L::misc + 16);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  SchedShape shape;
  shape.group = p.group;
  shape.num_kv_heads = p.num_kv_heads;
  shape.bq = p.bq;
  shape.num_splits = p.num_splits;
  shape.window = p.window;
  shape.causal = p.causal;
  shape.row_class = p.row_class;
  shape.class_rows = p.class_rows;

  // ---- set-up by all threads -------------------------------------------------
  // (the loads of the total-work pass below are issued first: their latency hides behind the
  // barrier initialisation and the TMEM allocation)
  unsigned long long work = 0;
  for (int r = tid; r < p.num_reqs; r += kThreads) {
    const int q0 = __ldg(p.query_start_loc + r), q1 = __ldg(p.query_start_loc + r + 1);
    const int len = __ldg(p.seq_lens + r);
    work += (unsigned long long)req_row_tiles(shape, q1 - q0) * (unsigned long long)req_kv_tiles(shape, q1 - q0, len);
  }
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      tc::mbar_init(&bars[B::full + s], kProducerThreads);
      tc::mbar_init(&bars[B::empty + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      for (int k = 0; k < 2; ++k) {
        tc::mbar_init(&bars[B::s_ready + 2 * b + k], 1);
        tc::mbar_init(&bars[B::s_free + 2 * b + k], kGroupThreads);
      }
      tc::mbar_init(&bars[B::o_ready + b], 1);
      tc::mbar_init(&bars[B::o_free + b], kGroupThreads);
      tc::mbar_init(&bars[B::p_ready + b], kGroupThreads);
    }
    for (int s = 0; s < kRawStages; ++s) {
      tc::mbar_init(&bars[B::raw_full + s], kUnitKeys >> p.copy_shift);  // page copies of a unit
      tc::mbar_init(&bars[B::raw_free + s], kProducerThreads / RU);       // the threads whose keys are in the unit
    }
    for (int s = 0; s < kItemSlots; ++s) {
      tc::mbar_init(&bars[B::item_full + s], 32);
      tc::mbar_init(&bars[B::item_empty + s], kItemReaders);
    }
    *abort_flag = 0;
    *total_s = 0ull;
    tc::mbar_init_fence();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, L::tmem_alloc);
    tc::tmem_relinquish();
  }
  __syncthreads();
  {
    // total work of the launch in KV tiles (every CTA computes the same number)
    unsigned long long w = work;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0 && w != 0) atomicAdd(total_s, w);
  }
  tc::fence_before_sync();
  tc::fence_async_smem();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tslot;
  const int t_star = item_tiles(*total_s * (unsigned long long)p.num_kv_heads, (int)gridDim.x);
  const uint32_t kstage0 = tc::smem_u32(smem + L::kstages), vstage0 = tc::smem_u32(smem + L::vstages);
  bool ok = true;

  if (warp == kSchedWarp) {
    // =========================== scheduler ====================================
    // Walks the requests in blocks of 32 (lane l holds request base + l and the items of the
    // requests before it), so this CTA's items c, c + CTAs, ... are found in one pass.
    const int S = p.num_splits, hkv = p.num_kv_heads;
    int base = 0;
    long long blk_first = 0;
    int blk_total = 0;
    int my_q0 = 0, my_qlen = 0, my_len = 0, my_splits = 1, my_n = 0, my_excl = 0;
    auto load_block = [&](int b) {
      const int r = b + lane;
      my_n = 0;
      my_q0 = my_qlen = my_len = 0;
      my_splits = 1;
      if (r < p.num_reqs) {
        my_q0 = __ldg(p.query_start_loc + r);
        my_qlen = __ldg(p.query_start_loc + r + 1) - my_q0;
        my_len = __ldg(p.seq_lens + r);
        const int rt = req_row_tiles(shape, my_qlen);
        my_splits = req_splits(req_kv_tiles(shape, my_qlen, my_len), t_star, S);
        my_n = (int)req_items(rt, my_splits, hkv);
      }
      int v = my_n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      my_excl = v - my_n;
      blk_total = __shfl_sync(0xffffffffu, v, 31);
    };
    load_block(0);
    int pub = 0;  // items published so far
    for (long long idx = blockIdx.x;; idx += gridDim.x) {
      bool done = false;
      while (idx >= blk_first + blk_total) {
        blk_first += blk_total;
        base += 32;
        if (base >= p.num_reqs) {
          done = true;
          break;
        }
        load_block(base);
      }
      if (done) break;
      const int rel = (int)(idx - blk_first);
      const bool mine = rel >= my_excl && rel < my_excl + my_n;
      const int src = __ffs(__ballot_sync(0xffffffffu, mine)) - 1;
      const int req = base + src;
      const int q0 = __shfl_sync(0xffffffffu, my_q0, src), q_len = __shfl_sync(0xffffffffu, my_qlen, src);
      const int seq_len = __shfl_sync(0xffffffffu, my_len, src), splits = __shfl_sync(0xffffffffu, my_splits, src);
      const ItemCoord c = item_coord(rel - __shfl_sync(0xffffffffu, my_excl, src), hkv, splits);
      const int first_idx = c.row_tile * p.bq;
      const int ntok = min(p.bq, q_len - first_idx), tok0 = q0 + first_idx;
      const int rows = ntok * p.group;
      int lo_first, hi_first, lo_last, hi_last;
      visible_bounds(p.window, p.causal, seq_len, q_len, first_idx, &lo_first, &hi_first);
      visible_bounds(p.window, p.causal, seq_len, q_len, first_idx + ntok - 1, &lo_last, &hi_last);
      const int range_begin = lo_first, range_end = max(hi_first, hi_last) + 1;  // lo and hi grow with the token
      int tile_begin, tile_end;
      split_tile_span(range_begin, range_end, c.split, splits, &tile_begin, &tile_end);
      auto lse_slot = [&](int s, int n) -> float* {
        const int token = tok0 + n / p.group, head = c.kvh * p.group + n % p.group;
        return reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_lse) + (int64_t)s * p.ws_lse_stride_split +
                                        (int64_t)token * p.ws_lse_stride_token + (int64_t)head * p.ws_lse_stride_head);
      };
      // splits this request does not use hold no keys: marked by the CTA of split 0, once its
      // item has been handed to the other roles (the marks are off their critical path)
      auto mark_unused_splits = [&]() {
        if (c.split == 0 && S > splits) {
          for (int i = lane; i < rows * (S - splits); i += 32) *lse_slot(splits + i / rows, i % rows) = -INFINITY;
        }
      };
      if (tile_begin >= tile_end) {
        mark_unused_splits();
        // No keys for this item: zero output, log-sum-exp -inf.
        if (S == 1) {
          for (int i = lane; i < rows * HD; i += 32) {
            const int n = i / HD, token = tok0 + n / p.group, head = c.kvh * p.group + n % p.group;
            store_out_elem(p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head, i % HD,
                           p.out_dtype, 0.f);
          }
        }
        for (int n = lane; n < rows; n += 32) {
          if (S > 1) {
            *lse_slot(c.split, n) = -INFINITY;
          } else if (p.lse_out != nullptr) {
            const int token = tok0 + n / p.group, head = c.kvh * p.group + n % p.group;
            *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.lse_out) + (int64_t)token * p.lse_stride_token +
                                      (int64_t)head * p.lse_stride_head) = -INFINITY;
          }
        }
        continue;
      }
      const int slot = pub % kItemSlots;
      if (pub >= kItemSlots) {
        ok &= wait_or_abort(&bars[B::item_empty + slot], ((pub / kItemSlots) - 1) & 1, abort_flag);
        if (!ok) break;
      }
      if (lane == 0) {
        volatile ItemDesc* d = descs + slot;
        d->n_tiles = tile_end - tile_begin;
        d->req = req;
        d->kvh = c.kvh;
        d->split = c.split;
        d->tok0 = tok0;
        d->ntok = ntok;
        d->tile_begin = tile_begin;
        d->range_begin = range_begin;
        d->range_end = range_end;
        d->mask_lo = lo_last;
        d->mask_hi = hi_first;
      }
      {
        float* sq = reinterpret_cast<float*>(smem + L::sq) + slot * NPAD;
        int* rlo = reinterpret_cast<int*>(smem + L::rlo) + slot * NPAD;
        int* rhi = reinterpret_cast<int*>(smem + L::rhi) + slot * NPAD;
        uint8_t* qimg = smem + L::qimg + slot * L::qimg_bytes;
        for (int n = lane; n < NPAD; n += 32) {
          int lo = 0, hi = -1;
          if (n < rows) visible_bounds(p.window, p.causal, seq_len, q_len, first_idx + n / p.group, &lo, &hi);
          rlo[n] = lo;
          rhi[n] = hi;
        }
        // Q digits: HD / 16 lanes per row, 16 elements each (32 / (HD / 16) rows per pass).
        constexpr int kQLanes = G::chunks, kQRows = 32 / kQLanes;
        for (int nb = 0; nb < NPAD; nb += kQRows) {
          const int n = nb + lane / kQLanes, part = lane % kQLanes;
          float v[16];
          if (n < rows) {
            const int token = tok0 + n / p.group, head = c.kvh * p.group + n % p.group;
            const uint4* srcq = reinterpret_cast<const uint4*>(p.q + (int64_t)token * p.q_stride_token +
                                                               (int64_t)head * p.q_stride_head + part * 32);
            const uint4 a = __ldg(srcq), b = __ldg(srcq + 1);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            if (p.q_dtype == PTH_ATTN_BF16) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                v[2 * e] = __uint_as_float(w[e] << 16);
                v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                v[2 * e] = f.x;
                v[2 * e + 1] = f.y;
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = 0.f;
          }
          float amax = 0.f;
#pragma unroll
          for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
          for (int o = 1; o < kQLanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
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
          // image row of (digit, n) is digit * NPAD + n; 16-byte column block `part`
          *reinterpret_cast<uint4*>(qimg + part * (2 * NPAD * 16) + n * 16) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
          *reinterpret_cast<uint4*>(qimg + part * (2 * NPAD * 16) + (NPAD + n) * 16) =
              make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
          if (part == 0) sq[n] = finite_row ? amax / 32512.f : 0.f;
        }
      }
      tc::fence_async_smem();
      mbar_arrive(&bars[B::item_full + slot]);
      ++pub;
      mark_unused_splits();
    }
    // no more items for this CTA
    {
      const int slot = pub % kItemSlots;
      if (pub >= kItemSlots && ok) ok &= wait_or_abort(&bars[B::item_empty + slot], ((pub / kItemSlots) - 1) & 1, abort_flag);
      if (lane == 0) descs[slot].n_tiles = 0;
      __syncwarp();
      mbar_arrive(&bars[B::item_full + slot]);
    }
  } else if (warp == kLoadWarp) {
    // =========================== loader =======================================
    // The raw bytes of a tile arrive PAGE BY PAGE through TMA: one copy per KV page and head,
    // issued by lane `page` of this warp, completing on the raw stage's mbarrier.
    //   raw_mode 1 (slot stride a multiple of 16, e.g. NHD with several heads): a tiled
    //     tensor-map copy of a [block_size slots] x [272 bytes] box whose inner start is the
    //     cell address rounded down to 16 bytes;
    //   raw_mode 2 (cells of a page contiguous and 16-byte aligned: HND, or one KV head): a
    //     plain bulk copy of the page run.
    // TMA writes shared memory directly (no L1 staging) and a handful of 4 KB copies per tile
    // keeps tens of KB in flight per SM.  The block id of the next tile's page is fetched
    // before waiting for the raw stage, so the block-table latency is off the refill path.
    const int pages_per_unit = kUnitKeys >> p.copy_shift;  // page copies of a raw unit (a tile, or half of one)
    const int bs = p.copy_slots;                            // slots of one copy
    const uint32_t raw_s = tc::smem_u32(smem + L::raw);
    int g0 = 0;  // running tile count at the start of the item
#pragma unroll 1
    for (int item = 0;; ++item) {
      const int slot = item % kItemSlots;
      ok &= wait_or_abort(&bars[B::item_full + slot], (item / kItemSlots) & 1, abort_flag);
      if (!ok) break;
      const int n_tiles = descs[slot].n_tiles;
      if (n_tiles == 0) break;
      if (lane < pages_per_unit) {
        const int tile_begin = descs[slot].tile_begin, range_begin = descs[slot].range_begin,
                  range_end = descs[slot].range_end;
        const int n_units = n_tiles * RU;
        const int32_t* bt = p.block_table + (int64_t)descs[slot].req * p.block_table_row_stride;
        const uint8_t* kb = p.k.data + (int64_t)descs[slot].kvh * p.k.stride_head;
        const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
        // inner coordinate (4-byte elements) of this head's box: the tensor map starts at the
        // 16-byte boundary below head 0's first cell
        const int tma_x = (int)((reinterpret_cast<uintptr_t>(kb) - delta -
                                 (reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15)) >> 2);
        // block id of this lane's copy of unit v of the item, -1 if no key of the copy is in range
        auto page_block = [&](int v) -> int {
          const int pos0 = tile_begin * kKeys + v * kUnitKeys + lane * bs;
          if (v >= n_units || pos0 >= range_end || pos0 + bs <= range_begin) return -1;
          int page, slot;
          page_and_slot(p, pos0, &page, &slot);
          return __ldg(bt + page);
        };
        // first slot, inside its page, of this lane's copy of unit v
        auto first_slot = [&](int v) -> int {
          int page, slot;
          page_and_slot(p, tile_begin * kKeys + v * kUnitKeys + lane * bs, &page, &slot);
          return slot;
        };
        int blk = page_block(0);
#pragma unroll 1
        for (int v = 0; v < n_units; ++v) {
          const int blk_next = page_block(v + 1);
          const int u = g0 * RU + v, rs = u % kRawStages;  // running unit count, ring slot
          if (u >= kRawStages) ok &= wait_or_abort(&bars[B::raw_free + rs], ((u / kRawStages) - 1) & 1, abort_flag);
          uint64_t* bar = &bars[B::raw_full + rs];
          if (blk >= 0 && ok) {
            const uint32_t dst = raw_s + rs * kRawStageHD + lane * bs * kRawRowHD;
            if (p.raw_mode == 1) {
              mbar_arrive_expect_tx(bar, bs * kRawRowHD);
              tma_load_3d(dst, &tmap, tma_x, first_slot(v), blk, bar);
            } else {
              const uint32_t bytes = bs * G::cell;  // a multiple of 16, like the run's address
              mbar_arrive_expect_tx(bar, bytes);
              bulk_copy_g2s(dst, kb + (int64_t)blk * p.k.stride_block + (int64_t)first_slot(v) * G::cell, bytes, bar);
            }
          } else {
            mbar_arrive(bar);
          }
          blk = blk_next;
        }
      }
      g0 += n_tiles;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B::item_empty + slot]);
    }
  } else if (warp >= 8 && warp < kMmaWarp) {
    // =========================== producers ====================================
    const int pgrp = (warp - 8) >> 2;                              // producer group
    const int pt = (tid - kSoftmaxThreads) & (kProducerThreads - 1);  // row of the operand images this thread fills
    // The raw bytes of a tile are brought in by the loader warp (above), page by page; when a
    // raw tile has landed, producer thread t moves the words of its key into the operand
    // images: with delta = (cell address mod 16) in {0, 8} and D = head size, word w of K block
    // j is raw word delta / 4 + 4 j + w, of V block j raw word delta / 4 + D / 4 + 1 + 4 j + w;
    // the scales are raw words delta / 4 + D / 4 and + D / 2 + 1.
    const int bs = p.copy_slots;  // slots of one page copy
    const int row_pitch = p.raw_mode == 1 ? kRawRowHD : G::cell;
    // Row pt of the operand images holds key `key` of the tile.  With a 264-byte pitch
    // (raw_mode 2) consecutive cells alternate between the two 8-byte alignments: taking the
    // even cells in the first two warps and the odd ones in the last two keeps a warp on one
    // code path and its 16-byte loads 528 bytes apart (free of bank conflicts).  The order of
    // the keys inside a tile has no effect on the integer sums; the softmax masks by `key`.
    const int key = tile_key(p, pt);
    const int unit_of_key = key / kUnitKeys;  // raw unit of the tile that holds this key (warp-uniform)
    const int my_page = (key % kUnitKeys) >> p.copy_shift, my_slot = key & (bs - 1);
    int g0 = 0;
#pragma unroll 1
    for (int item = 0;; ++item) {
      const int slot = item % kItemSlots;
      ok &= wait_or_abort(&bars[B::item_full + slot], (item / kItemSlots) & 1, abort_flag);
      if (!ok) break;
      const int n_tiles = descs[slot].n_tiles;
      if (n_tiles == 0) break;
      const int tile_begin = descs[slot].tile_begin, range_begin = descs[slot].range_begin,
                range_end = descs[slot].range_end;
      const uint8_t* kb = p.k.data + (int64_t)descs[slot].kvh * p.k.stride_head;
      const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
      const uint32_t cell_off = my_page * bs * kRawRowHD + my_slot * row_pitch + delta;  // inside a raw stage
      const bool odd = (cell_off & 8u) != 0;
      int j = pgrp - g0 % NP;  // first tile of the item whose running count is pgrp mod NP
      if (j < 0) j += NP;
#pragma unroll 1
      for (; j < n_tiles; j += NP) {
        const int g = g0 + j;  // running tile count: indexes every ring
        const int u = g * RU + unit_of_key;  // running count of raw units
        const int rs = u % kRawStages;
        const int pos = (tile_begin + j) * kKeys + key;
        const bool valid = pos >= range_begin && pos < range_end;
        if constexpr (NP > 1 || RU > 1) {
          // A raw slot is used in turn by the producer groups (NR is not a multiple of NP) or by
          // the threads of the two half tiles (NR is odd).  A parity wait only tells apart two
          // consecutive phases, so these threads must not look at raw_full[rs] while the slot's
          // PREVIOUS occupant (somebody else's) is still pending: first wait until that one
          // has been taken out of the slot.
          if (u >= kRawStages) ok &= wait_or_abort(&bars[B::raw_free + rs], ((u / kRawStages) - 1) & 1, abort_flag);
        }
        ok &= wait_or_abort(&bars[B::raw_full + rs], (u / kRawStages) & 1, abort_flag);
        // The 16-byte pieces from the boundary below the cell: pieces 0 .. D / 16 hold K and
        // k_scale, pieces D / 16 .. D / 8 hold k_scale, V and v_scale.  Up to head size 128 both
        // sets are read before the raw stage is released; a 256-dim row is too long for that
        // (132 words), so its V set is read after the K image has been written.
        constexpr int PW = G::part_words, NCH = G::chunks;
        constexpr bool kTwoPhase = HD > 128;
        const uint4* row = reinterpret_cast<const uint4*>(smem + L::raw + rs * kRawStageHD + (cell_off & ~15u));
        auto load_part = [&](const uint4* src, uint32_t (&w)[PW]) {
          if (valid) {
#pragma unroll
            for (int c = 0; c < PW / 4; ++c) {
              const uint4 v = src[c];
              w[4 * c] = v.x;
              w[4 * c + 1] = v.y;
              w[4 * c + 2] = v.z;
              w[4 * c + 3] = v.w;
            }
          } else {
#pragma unroll
            for (int c = 0; c < PW; ++c) w[c] = 0u;
          }
        };
        uint32_t kw[PW], vw[PW];
        load_part(row, kw);
        if constexpr (!kTwoPhase) {
          load_part(row + NCH, vw);
          // this thread's row is in registers (the arrive orders the loads before it): once all
          // producers of the tile have arrived the loader may refill the raw stage
          mbar_arrive(&bars[B::raw_free + rs]);
        }
        const int st = g % NS;
        // K image g % NK is free once QK(g - NK) has completed, which is what S^T of that tile
        // being ready means: the producers wait on the s_ready barrier the softmax group waits
        // on (one commit less per tile for the issuing thread).  That barrier completes next
        // for a tile whose images this group writes after this wait, so the parity is unambiguous.
        if (g >= NK) {
          const int q = g - NK, qk = q >> 1;
          ok &= wait_or_abort(&bars[B::s_ready + 2 * (q & 1) + qk % SB], (qk / SB) & 1, abort_flag);
        }
        uint8_t* stage = smem + L::vstages + st * kVStageHD;  // V image, then the scales
        uint8_t* krow = smem + L::kstages + (g % NK) * kImgHD + pt * 16;
        uint8_t* vrow = stage + pt * 16;
        const int ko = odd ? 2 : 0, vo = odd ? 3 : 1;  // first word of K / V inside their sets of pieces
        if (!odd) {
#pragma unroll
          for (int b = 0; b < NCH; ++b)
            *reinterpret_cast<uint4*>(krow + b * kImgChunk) = make_uint4(kw[4 * b], kw[4 * b + 1], kw[4 * b + 2], kw[4 * b + 3]);
        } else {
#pragma unroll
          for (int b = 0; b < NCH; ++b)
            *reinterpret_cast<uint4*>(krow + b * kImgChunk) =
                make_uint4(kw[2 + 4 * b], kw[3 + 4 * b], kw[4 + 4 * b], kw[5 + 4 * b]);
        }
        const uint32_t k_scale_bits = odd ? kw[HD / 4 + 2] : kw[HD / 4];
        (void)ko;
        if constexpr (kTwoPhase) {
          load_part(row + NCH, vw);
          mbar_arrive(&bars[B::raw_free + rs]);
        }
        if (g >= NS) ok &= wait_or_abort(&bars[B::empty + st], ((g / NS) - 1) & 1, abort_flag);
        if (!odd) {
#pragma unroll
          for (int b = 0; b < NCH; ++b)
            *reinterpret_cast<uint4*>(vrow + b * kImgChunk) = make_uint4(vw[1 + 4 * b], vw[2 + 4 * b], vw[3 + 4 * b], vw[4 + 4 * b]);
        } else {
#pragma unroll
          for (int b = 0; b < NCH; ++b)
            *reinterpret_cast<uint4*>(vrow + b * kImgChunk) =
                make_uint4(vw[3 + 4 * b], vw[4 + 4 * b], vw[5 + 4 * b], vw[6 + 4 * b]);
        }
        (void)vo;
        *reinterpret_cast<uint32_t*>(stage + kImgHD + pt * 4) = k_scale_bits;
        *reinterpret_cast<uint32_t*>(stage + kImgHD + kKeys * 4 + pt * 4) = odd ? vw[HD / 4 + 3] : vw[HD / 4 + 1];
        tc::fence_async_smem();
        mbar_arrive(&bars[B::full + st]);
      }
      g0 += n_tiles;
      mbar_arrive(&bars[B::item_empty + slot]);
    }
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===================================
    // ONE thread (the lane elect.sync picks) issues every tcgen05.mma of the CTA, item after item, inside an item
    // in a fixed order (two issuing threads, one for QK and one for PV, produced rare
    // run-to-run differences):
    //   QK(0), QK(1), then for i = 0, 1, ...: QK(i + 2), PV(i)
    // (with only two V stages - the 256-dim instances - QK runs one tile ahead instead of two).
    // With g = running tile count of tile i:
    //   QK(i): the tile belongs to softmax group g & 1, is that group's k-th tile (k = g >> 1)
    //          and lands in its S^T buffer k % SB; needs the tile's images (full) and that
    //          buffer read by the softmax (s_free);
    //   PV(i): needs the group's P image (p_ready) and its O^T buffer folded (o_free); its
    //          completion frees the V stage.
    // Every condition of a step depends only on MMAs issued earlier in this order, so the
    // order cannot deadlock, and QK runs two tiles ahead of PV, which is as far as the S^T
    // buffers allow.  The next item's first QK follows the last PV of this item at once: its
    // images have long been filled, so S^T of the next item is ready while the softmax groups
    // still merge and write this one.  The two barriers of a step are waited for by lanes 0
    // and 1 in the same instruction: a look at an mbarrier costs 100-200 cycles on the busy
    // shared-memory pipe, and four looks in a row per tile made this thread the bottleneck.
    // This thread's own instruction stream is the narrowest part of the CTA (a few hundred
    // dependent instructions per tile took as long as the tile), so everything it needs is
    // kept in registers: barrier addresses as shared-memory offsets, operand descriptors as
    // word pairs that move by one addition per MMA.
    const uint32_t bars_s = tc::smem_u32(bars);
    const DescWords kd = desc_words(kstage0, kImgChunk, 128);
    const DescWords vd = desc_words(vstage0, 128, kImgChunk);
    const DescWords pd = desc_words(tc::smem_u32(pimg), 128, kDigitChunk);
    // lane 0 waits for barrier i0 (parity par0); lane 1 for barrier i1 if need1; true when both are complete
    auto wait_pair = [&](int i0, uint32_t par0, int i1, uint32_t par1, bool need1) -> bool {
      const uint32_t mine = bars_s + 8u * (uint32_t)(lane == 0 ? i0 : i1);
      const uint32_t par = lane == 0 ? par0 : par1;
      const bool need = lane == 0 || (lane == 1 && need1);
      const bool done = !need || wait_or_abort_s(mine, par, abort_flag);
      return __all_sync(0xffffffffu, done);
    };
    int g0 = 0;
    bool go = true;
#pragma unroll 1
    for (int item = 0; go; ++item) {
      const int slot = item % kItemSlots;
      go = wait_or_abort(&bars[B::item_full + slot], (item / kItemSlots) & 1, abort_flag);
      if (!go) break;
      const int n_tiles = descs[slot].n_tiles;
      if (n_tiles == 0) break;
      tc::fence_after_sync();
      const DescWords qd = desc_words(tc::smem_u32(smem + L::qimg + slot * L::qimg_bytes), 2 * NPAD * 16, 128);
      auto qk_step = [&](int q) -> bool {  // q = running tile count
        const int g = q & 1, k = q >> 1, sb = k % SB;
        const bool ready = wait_pair(B::full + q % NS, (q / NS) & 1, B::s_free + 2 * g + sb, ((k / SB) - 1) & 1, k >= SB);
        if (ready && elect_one()) {
          tc::fence_after_sync();
          DescWords kq = kd;
          kq.lo += (uint32_t)(q % NK) * (kImgHD >> 4);
          issue_qk_i8_words<NPAD, HD>(tmem_base + (g * SB + sb) * L::s_cols, kq, qd);
          tc::mma_commit_s(bars_s + 8u * (B::s_ready + 2 * g + sb));
        }
        return ready;
      };
      auto pv_step = [&](int i) -> bool {
        const int g = i & 1;
        const bool ready = wait_pair(B::p_ready + g, (i >> 1) & 1, B::o_free + g, ((i >> 1) - 1) & 1, i >= 2);
        if (ready && elect_one()) {
          tc::fence_after_sync();
          DescWords vi = vd, pi = pd;
          vi.lo += (uint32_t)(i % NS) * (kVStageHD >> 4);
          pi.lo += (uint32_t)g * ((PD * NPAD * kKeys) >> 4);
          issue_pv_i8_words<NPAD, PD, HD>(tmem_base + L::s_total + g * L::o_cols, vi, pi);
          tc::mma_commit_s(bars_s + 8u * (B::o_ready + g));
          tc::mma_commit_s(bars_s + 8u * (B::empty + i % NS));
        }
        return ready;
      };
#pragma unroll
      for (int a = 0; a < LA; ++a)
        if (go && a < n_tiles) go = qk_step(g0 + a);
#pragma unroll 1
      for (int i = 0; i < n_tiles && go; ++i) {
        if (i + LA < n_tiles) go = qk_step(g0 + i + LA);
        if (go) go = pv_step(g0 + i);
      }
      g0 += n_tiles;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B::item_empty + slot]);
    }
    ok &= go;
    __syncwarp();
  } else if (warp < 2 * 4) {
    // =========================== softmax ======================================
    // Two warpgroups: group g owns the tiles whose running count is g mod 2 and keeps its own
    // running maximum, sum and accumulator (as if the KV range were split in two inside the
    // CTA); the two states are merged at the end of every item.  Thread t of a group owns
    // key t of S^T and output column d = t of O^T.
    const int g = warp >> 2;
    const int gt = tid & 127;          // thread index inside the group
    const int gw = warp & 3;           // warp inside the group = TMEM lane quadrant
    const uint32_t lane_addr = (uint32_t)(gw * 32) << 16;
    uint8_t* pimg_g = pimg + g * (PD * NPAD * kKeys);
    float* wred_g = wred + g * (2 * 4 * (NPAD + 1));   // [2][4][NPAD + 1]
    float* mrun_g = mrun + g * (2 * NPAD);             // [2][NPAD]
    constexpr int NROW = 4 * RQ;  // rows this instance computes (live rows rounded up to four)
    constexpr int RL = (NPAD + 31) / 32;
    const int my_key = tile_key(p, gt);

    int g0 = 0, item = 0;
    ok &= wait_or_abort(&bars[B::item_full + 0], 0, abort_flag);
    bool stop = named_barrier_or(4, kSoftmaxThreads, !ok || descs[0].n_tiles == 0);
#pragma unroll 1
    while (!stop) {
      const int slot = item % kItemSlots;
      const int n_tiles = descs[slot].n_tiles, tile_begin = descs[slot].tile_begin;
      const int kvh = descs[slot].kvh, split = descs[slot].split, tok0 = descs[slot].tok0;
      const int rows = descs[slot].ntok * p.group;  // <= NROW by construction of bq
      const int mask_lo = descs[slot].mask_lo, mask_hi = descs[slot].mask_hi;
      const float* sq = reinterpret_cast<const float*>(smem + L::sq) + slot * NPAD;
      const int* rlo = reinterpret_cast<const int*>(smem + L::rlo) + slot * NPAD;
      const int* rhi = reinterpret_cast<const int*>(smem + L::rhi) + slot * NPAD;

      float acc[kHalves][NROW], l_part[NROW];  // thread t accumulates output columns t (and t + 128)
#pragma unroll
      for (int n = 0; n < NROW; ++n) {
#pragma unroll
        for (int h = 0; h < kHalves; ++h) acc[h][n] = 0.f;
        l_part[n] = 0.f;
      }
      // Per-row softmax state lives in LANES, not in shared memory: lane l of every warp holds,
      // for row l + 32 j, the running maximum and the factors of the latest tile (every warp
      // computes the same values), and the row loops fetch them with warp shuffles.
      float m_run[RL], a_l[RL], unit_l[RL], muse_l[RL], invu_l[RL];
#pragma unroll
      for (int j = 0; j < RL; ++j) {
        m_run[j] = -INFINITY;
        a_l[j] = 0.f;
        unit_l[j] = 0.f;
        muse_l[j] = 0.f;
        invu_l[j] = 0.f;
      }

      // Folds O^T of the tile with running count q (this group's TMEM buffer) into the register
      // accumulator, with the rescale factor and digit unit of that tile (still in a_l / unit_l).
      auto fold_o = [&](int q) {
        ok &= wait_or_abort(&bars[B::o_ready + g], (q >> 1) & 1, abort_flag);
        tc::fence_after_sync();
        const uint32_t o_tmem = tmem_base + L::s_total + g * L::o_cols + lane_addr;
        constexpr int FB = RQ < 2 ? RQ : 2;  // eight rows per round trip to TMEM
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
#pragma unroll
          for (int qb = 0; qb < RQ; qb += FB) {
            uint32_t d[FB][PD][4];
#pragma unroll
            for (int c = 0; c < FB; ++c)
#pragma unroll
              for (int k = 0; k < PD; ++k) tmem_ld4(o_tmem + h * (PD * NPAD) + k * NPAD + (qb + c) * 4, d[c][k]);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < FB; ++c) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int n = (qb + c) * 4 + e;
                const float alpha_n = __shfl_sync(0xffffffffu, a_l[n >> 5], n & 31);
                const float unit_n = __shfl_sync(0xffffffffu, unit_l[n >> 5], n & 31);
                float o = int_to_float(d[c][PD - 1][e]);
#pragma unroll
                for (int k = PD - 2; k >= 0; --k) o = fmaf(o, 128.f, int_to_float(d[c][k][e]));
                acc[h][n] = fmaf(acc[h][n], alpha_n, o * unit_n);
              }
            }
          }
        }
        tc::fence_before_sync();
        mbar_arrive(&bars[B::o_free + g]);
      };

      int lit = 0;                // tiles of this item this group has started
      int j = (g - g0) & 1;       // first tile of the item whose running count is g mod 2
#pragma unroll 1
      for (; j < n_tiles; j += 2, ++lit) {
        const int q = g0 + j;     // running tile count
        const int it = q >> 1;    // running count of this group's tiles; buffers alternate with it
        const int b = it & 1;
        float* wred_i = wred_g + b * 4 * (NPAD + 1);
        const uint8_t* scales = smem + L::vstages + (q % NS) * kVStageHD + kImgHD;
        const int sb = it % SB;
        ok &= wait_or_abort(&bars[B::s_ready + 2 * g + sb], (it / SB) & 1, abort_flag);
        tc::fence_after_sync();
        const float ks_cur = reinterpret_cast<const float*>(scales)[gt];
        const float vs_cur = reinterpret_cast<const float*>(scales)[kKeys + gt];
        const uint32_t s_tmem = tmem_base + (g * SB + sb) * L::s_cols + lane_addr;
        const int pos = (tile_begin + j) * kKeys + my_key;
        const bool interior = (tile_begin + j) * kKeys >= mask_lo && (tile_begin + j) * kKeys + (kKeys - 1) <= mask_hi;
        const float mult = ks_cur * p.scale_log2;
        float s[NROW];
        int mykey[RL];  // warp maximum of row lane + 32 j, as an ordered integer key
#pragma unroll
        for (int jj = 0; jj < RL; ++jj) mykey[jj] = float_key(-INFINITY);
        // up to sixteen rows per round trip to TMEM (one wait for the batch)
        constexpr int QB = RQ < 4 ? RQ : 4;
#pragma unroll
        for (int qb = 0; qb < RQ; qb += QB) {
          uint32_t hi[QB][4], lo[QB][4];
#pragma unroll
          for (int c = 0; c < QB; ++c) {
            tmem_ld4(s_tmem + (qb + c) * 4, hi[c]);
            tmem_ld4(s_tmem + NPAD + (qb + c) * 4, lo[c]);
          }
          tc::tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < QB; ++c) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int n = (qb + c) * 4 + e;
              const float sv = fmaf(int_to_float(hi[c][e]), 256.f, int_to_float(lo[c][e])) * (sq[n] * mult);
              const bool vis = interior || (pos >= rlo[n] && pos <= rhi[n]);
              s[n] = vis ? sv : -INFINITY;
              const int key = __reduce_max_sync(0xffffffffu, float_key(s[n]));
              if (lane == (n & 31)) mykey[n >> 5] = key;
            }
          }
        }
#pragma unroll
        for (int jj = 0; jj < RL; ++jj)
          if (lane + 32 * jj < NPAD) wred_i[gw * (NPAD + 1) + lane + 32 * jj] = key_float(mykey[jj]);
        tc::fence_before_sync();
        mbar_arrive(&bars[B::s_free + 2 * g + sb]);  // this S^T buffer may be overwritten by a later QK
        {
          const int key = __reduce_max_sync(0xffffffffu, float_key(vs_cur));
          if (lane == 0) wred_i[gw * (NPAD + 1) + NPAD] = key_float(key);
        }
        // O^T of this group's previous tile of the item; afterwards its P image is free.
        if (lit > 0) fold_o(q - 2);
        named_barrier(1 + g, kGroupThreads);  // per-warp maxima of the tile visible to the whole group
        const float vs_max = fmaxf(fmaxf(wred_i[NPAD], wred_i[(NPAD + 1) + NPAD]),
                                   fmaxf(wred_i[2 * (NPAD + 1) + NPAD], wred_i[3 * (NPAD + 1) + NPAD]));
#pragma unroll
        for (int jj = 0; jj < RL; ++jj) {
          const int r = (lane + 32 * jj) & (NPAD - 1);
          const float m_tile = fmaxf(fmaxf(wred_i[r], wred_i[(NPAD + 1) + r]),
                                     fmaxf(wred_i[2 * (NPAD + 1) + r], wred_i[3 * (NPAD + 1) + r]));
          const float m_old = m_run[jj];
          const float m_new = fmaxf(m_old, m_tile);
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          a_l[jj] = fast_exp2(m_old - m_use);
          // largest p * v_scale of the tile bounds the fixed-point range of its digits
          const float bound = vs_max * fast_exp2(m_tile - m_use);
          invu_l[jj] = bound > 0.f ? __fdividef((float)XMAX, bound) : 0.f;
          unit_l[jj] = bound * (1.0f / (float)XMAX);
          muse_l[jj] = m_use;
          m_run[jj] = m_new;
        }
#pragma unroll
        for (int q16 = 0; q16 < NPAD / 16; ++q16) {
          if (q16 * 4 < RQ) {
            uint32_t dig[PD][4] = {};
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              // Whole groups of four rows, padded rows included (their scores are finite
              // and their columns of O^T are never read): no branch per row, so the four
              // dependency chains overlap.
              if (q16 * 4 + q4 < RQ) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int n = q16 * 16 + q4 * 4 + e;
                  const float m_use = __shfl_sync(0xffffffffu, muse_l[n >> 5], n & 31);
                  const float a = __shfl_sync(0xffffffffu, a_l[n >> 5], n & 31);
                  const float inv_u = __shfl_sync(0xffffffffu, invu_l[n >> 5], n & 31);
                  const float pr = fast_exp2(s[n] - m_use);
                  l_part[n] = fmaf(l_part[n], a, pr);
                  int x = __float2int_rn(pr * vs_cur * inv_u);
                  x = min(x, XMAX);
#pragma unroll
                  for (int k = 0; k < PD; ++k) dig[k][q4] |= (uint32_t)((x >> (7 * k)) & 127) << (8 * e);
                }
              }
            }
#pragma unroll
            for (int k = 0; k < PD; ++k)
              *reinterpret_cast<uint4*>(pimg_g + (k * (NPAD / 16) + q16) * kDigitChunk + gt * 16) =
                  make_uint4(dig[k][0], dig[k][1], dig[k][2], dig[k][3]);
          }
        }
        tc::fence_async_smem();
        mbar_arrive(&bars[B::p_ready + g]);  // P image of the tile complete
      }
      if (lit > 0) fold_o(g0 + j - 2);  // the group's last tile of the item

      // ---- end of the item: reduce the row sums inside the group, merge the two groups ----
      // Every PV of the item has been folded by now, so the P images of both groups are idle:
      // group 1 parks its accumulator there ([row][d] fp32) for group 0 to pick up.
      named_barrier(4, kSoftmaxThreads);  // both groups have left their last tile
      float* wsum = wred_g;  // [4][NPAD + 1]
      if (gw == 0) {
#pragma unroll
        for (int jj = 0; jj < RL; ++jj)
          if (lane + 32 * jj < NPAD) mrun_g[lane + 32 * jj] = m_run[jj];
      }
#pragma unroll
      for (int n = 0; n < NROW; ++n) {
        if (n < rows) {
          float v = l_part[n];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == (n & 31)) wsum[gw * (NPAD + 1) + n] = v;
        }
      }
      // The P images hold 128 dims of a parked accumulator ([row][128] fp32): a head of 256 dims
      // goes through them in two rounds.
      float* park = reinterpret_cast<float*>(pimg);
#pragma unroll
      for (int h = 0; h < kHalves; ++h) {
        if (h > 0) named_barrier(4, kSoftmaxThreads);  // the previous round's parked values have been read
        if (g == 1) {
#pragma unroll
          for (int n = 0; n < NROW; ++n)
            if (n < rows) park[n * kKeys + gt] = acc[h][n];
        }
        named_barrier(4, kSoftmaxThreads);  // sums, maxima and the parked accumulator visible
        const int d = h * kKeys + gt;       // output column of this thread in this round
        if (g == 0) {
          const float* w0 = wred;
          const float* w1 = wred + 2 * 4 * (NPAD + 1);
          const float* m0p = mrun;             // running maxima published by the two groups
          const float* m1p = mrun + 2 * NPAD;
#pragma unroll
          for (int n = 0; n < NROW; ++n) {
            if (n < rows) {
              const float l0 = w0[n] + w0[(NPAD + 1) + n] + w0[2 * (NPAD + 1) + n] + w0[3 * (NPAD + 1) + n];
              const float l1 = w1[n] + w1[(NPAD + 1) + n] + w1[2 * (NPAD + 1) + n] + w1[3 * (NPAD + 1) + n];
              const float m0 = m0p[n], m1 = m1p[n];
              const float m = fmaxf(m0, m1);
              const float c0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - m);
              const float c1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - m);
              const float l = l0 * c0 + l1 * c1;
              const float o = acc[h][n] * c0 + (c1 > 0.f ? park[n * kKeys + gt] * c1 : 0.f);
              const float val = l > 0.f ? o / l : 0.f;
              const int token = tok0 + n / p.group, head = kvh * p.group + n % p.group;
              if (d < HD) {  // (a head of 64 dims uses half of the group's threads)
                if (p.num_splits == 1) {
                  store_out_elem(p.out + (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head, d,
                                 p.out_dtype, val);
                } else {
                  reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.ws_o) + (int64_t)split * p.ws_o_stride_split +
                                           (int64_t)token * p.ws_o_stride_token + (int64_t)head * p.ws_o_stride_head)[d] = val;
                }
              }
              if (h == 0 && gt == n) {
                const float lse2 = l > 0.f ? m + log2f(l) : -INFINITY;
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
        }
      }
      // ---- next item: the slot is released, and the barrier that protects the buffers of the
      // merge also makes "no more items" one decision of all 256 threads ----
      mbar_arrive(&bars[B::item_empty + slot]);
      g0 += n_tiles;
      ++item;
      const int nslot = item % kItemSlots;
      ok &= wait_or_abort(&bars[B::item_full + nslot], (item / kItemSlots) & 1, abort_flag);
      stop = named_barrier_or(4, kSoftmaxThreads, !ok || descs[nslot].n_tiles == 0);
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, L::tmem_alloc);
  if (tid == 0 && *abort_flag) atomicOr(&g_i8_status, 4u);
  (void)ok;
}

template <int HD, int NPAD, int PD, int NS, int NK, int NR, int SB, int RQ, int NP>
cudaError_t launch_cfg(const KernelParams& p, const CUtensorMap& map, int num_ctas, cudaStream_t stream) {
  constexpr int smem = Layout<HD, NPAD, PD, NS, NK, NR, SB>::total;
  static_assert(smem <= 227 * 1024, "shared memory of one CTA");
  static_assert(Layout<HD, NPAD, PD, NS, NK, NR, SB>::tmem_need <= 512, "TMEM columns");
  // a head of 64 dims makes the PV instruction read 64 image "rows" past the V image: they
  // must still be shared memory of this CTA
  static_assert(HD >= 128 || Layout<HD, NPAD, PD, NS, NK, NR, SB>::vstages + NS * Layout<HD, NPAD, PD, NS, NK, NR, SB>::vstage_bytes +
                                     8 * kImgChunk <= smem, "reads past the last V image stay inside the CTA's shared memory");
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    err = cudaFuncSetAttribute(umma_i8_attention_kernel<HD, NPAD, PD, NS, NK, NR, SB, RQ, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  umma_i8_attention_kernel<HD, NPAD, PD, NS, NK, NR, SB, RQ, NP><<<num_ctas, threads_for(NP), smem, stream>>>(p, map);
  return cudaGetLastError();
}

}  // namespace

// The integer kernel reads whole cache cells through TMA: it needs vLLM's packed cell
// (K | k_scale | V | v_scale contiguous, 2 D + 8 bytes, 8-byte aligned), pages of a multiple
// of 16 keys whose byte stride is a multiple of 16, and either a slot stride that is a multiple
// of 16 or cells that are contiguous inside a page, on top of what the tcgen05 kernels
// need in general.  Queries may be bf16 or fp16 (they become int8 digits either way).  Head
// sizes 64, 128 and 256; a head of 256 dims takes row tiles of at most 32 rows (its operand
// images leave room for no more), so at most 32 query heads per KV head.
bool umma_i8_supports(const KernelParams& p, const char** why) {
  KernelParams pq = p;
  if (pq.q_dtype == PTH_ATTN_F16) pq.q_dtype = PTH_ATTN_BF16;
  if (pq.head_size == 64 || pq.head_size == 256) pq.head_size = 128;  // the other conditions are the same
  if (!umma_supports(pq, why)) return false;
  const int D = p.head_size;
  if (p.group > umma_i8_max_rows(D)) {
    *why = "more query heads per KV head than a row tile of this head size holds";
    return false;
  }
  if (p.ks.data != p.k.data + D || p.v.data != p.k.data + D + 4 || p.vs.data != p.k.data + 2 * D + 4 ||
      p.ks.stride_head != p.k.stride_head || p.v.stride_head != p.k.stride_head ||
      p.vs.stride_head != p.k.stride_head) {
    *why = "the cache streams are not one packed K|k_scale|V|v_scale cell";
    return false;
  }
  if (raw_mode_for(p) == 0) {
    *why = "page geometry not supported by the TMA page copies";
    return false;
  }
  if (raw_mode_for(p) == 1 && encode_tiled_fn() == nullptr) {
    *why = "the driver does not provide cuTensorMapEncodeTiled";
    return false;
  }
  return true;
}

// Rows (query tokens x query heads per KV head) of the tallest row tile for a head size.
int umma_i8_max_rows(int head_size) { return head_size == 256 ? 32 : 64; }

// Kernels this launch enqueues and the CTAs of the attention kernel (no device access).
int umma_i8_num_ctas(const KernelParams& p_in, int sms) {
  KernelParams p = p_in;
  if (p.row_class == 1) {
    p.bq = p.class_rows / p.group > 0 ? p.class_rows / p.group : 1;
  } else {
    const int cap = umma_i8_max_rows(p.head_size) / p.group;
    if (p.bq > cap) p.bq = cap;
  }
  const long long items = ((long long)p.num_tokens / p.bq + p.num_reqs) * p.num_kv_heads * p.num_splits;
  if (items > 0x7fffffffll) return -1;
  return (int)(items < sms ? items : sms);
}

cudaError_t launch_umma_i8_attention(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  if (p.row_class == 1) {
    // Only requests of at most class_rows rows: each is one row tile.
    p.bq = p.class_rows / p.group > 0 ? p.class_rows / p.group : 1;
  } else {
    const int cap = umma_i8_max_rows(p.head_size) / p.group;
    if (p.bq > cap) p.bq = cap;
  }
  set_copy_slots(p, p.head_size == 256 ? 64 : 128);  // a raw unit (a tile; half a tile at 256 dims) holds whole copies
  p.raw_mode = raw_mode_for(p);
  const CUtensorMap* map = nullptr;
  static const CUtensorMap no_map{};
  if (p.raw_mode == 1) {
    map = cached_page_map(p);
    if (map == nullptr) return cudaErrorInvalidValue;
  } else {
    map = &no_map;
  }
  const int sms = sm_count();
  if (sms <= 0) return cudaErrorInvalidDevice;
  const int ctas = umma_i8_num_ctas(p_in, sms);
  if (ctas < 1) return cudaErrorInvalidValue;
  const int rows = p.bq * p.group;
  // Instances by live rows: the softmax code of each handles exactly ceil(rows / 4) row
  // groups, which keeps the decode loop small enough for the instruction cache.
  // The decode instance (rows <= 4) needs few registers and runs two producer groups.
  if (p.head_size == 128) {
    if (rows <= 4) return launch_cfg<128, 16, 3, 4, 2, 3, 2, 1, 2>(p, *map, ctas, stream);
    if (rows <= 8) return launch_cfg<128, 16, 3, 4, 2, 3, 2, 2, 1>(p, *map, ctas, stream);
    if (rows <= 16) return launch_cfg<128, 16, 3, 4, 2, 3, 2, 4, 1>(p, *map, ctas, stream);
    if (rows <= 32) return launch_cfg<128, 32, 2, 3, 2, 3, 1, 8, 1>(p, *map, ctas, stream);
    return launch_cfg<128, 64, 2, 3, 2, 2, 1, 16, 1>(p, *map, ctas, stream);
  }
  if (p.head_size == 64) {
    // half the bytes per tile: deeper rings keep as many bytes in flight
    if (rows <= 4) return launch_cfg<64, 16, 3, 4, 2, 6, 2, 1, 2>(p, *map, ctas, stream);
    if (rows <= 8) return launch_cfg<64, 16, 3, 4, 2, 6, 2, 2, 1>(p, *map, ctas, stream);
    if (rows <= 16) return launch_cfg<64, 16, 3, 4, 2, 6, 2, 4, 1>(p, *map, ctas, stream);
    if (rows <= 32) return launch_cfg<64, 32, 2, 3, 2, 6, 1, 8, 1>(p, *map, ctas, stream);
    return launch_cfg<64, 64, 2, 3, 2, 4, 1, 16, 1>(p, *map, ctas, stream);
  }
  // 256 dims: one K image, two V stages (QK one tile ahead of PV) and a raw ring of three half
  // tiles of 33 KB - a tile and a half of cache bytes in flight - fill the shared memory
  if (rows <= 4) return launch_cfg<256, 16, 2, 2, 1, 3, 2, 1, 1>(p, *map, ctas, stream);
  if (rows <= 8) return launch_cfg<256, 16, 2, 2, 1, 3, 2, 2, 1>(p, *map, ctas, stream);
  if (rows <= 16) return launch_cfg<256, 16, 2, 2, 1, 3, 2, 4, 1>(p, *map, ctas, stream);
  // up to 32 rows (prefill chunks cut into row tiles of 32 / G tokens): the wider Q and P images
  // leave room for two raw half tiles, one S^T buffer per group
  return launch_cfg<256, 32, 2, 2, 1, 2, 1, 8, 1>(p, *map, ctas, stream);
}

// Reads and clears the integer kernel's status word (device must be idle).
cudaError_t read_i8_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_i8_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_i8_status, &zero, sizeof(zero));
}

}  // namespace pthb200

#include "umma_i8_tile_test.cuh"
