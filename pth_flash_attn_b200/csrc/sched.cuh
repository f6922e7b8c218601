// Work-item schedule of the persistent integer kernel: which (row tile, KV head, split)
// items a launch consists of, how many splits a request gets, and which CTA runs which item.
//
// The host fixes only what a captured CUDA graph may bake in: the number of CTAs and the
// largest split count the workspace holds (num_splits).  Everything that depends on the
// lengths is decided on the device from seq_lens / query_start_loc, by every CTA alike:
//
//   request r     row_tiles(r) = ceil(q_len / bq) row tiles (0 if the launch does not serve
//                 the request), kv_tiles(r) = KV tiles its rows touch together;
//   total work    W = Hkv * sum_r row_tiles(r) * kv_tiles(r)   (KV tiles to read);
//   item size     t* = KV tiles an item should hold: W / (CTAs * m) with m <= 8 items per
//                 CTA, chosen so that t* stays near kItemTilesTarget when there is that much
//                 work, and never below kItemTilesMin;
//   splits        S(r) = round(kv_tiles(r) / t*) clamped to [1, num_splits]: every request is
//                 cut into pieces of about t* tiles, so the items of a launch are about
//                 equally long whatever the mix of context lengths;
//   item order    request-major; inside a request (row tile, split)-major and KV head
//                 fastest, so that the Hkv heads of the same pages are adjacent items;
//   assignment    CTA c runs items c, c + CTAs, c + 2 CTAs, ...: adjacent items (the heads of
//                 one page set) run at the same time on neighbouring CTAs, which lets the
//                 boundary sectors of neighbouring 264-byte cells be served from L2.
//
// Splits s >= S(r) of a request hold no keys: their log-sum-exp is set to -inf by the CTA
// that runs split 0 of the same rows, and the combine skips them.
//
// These functions compile for the host too (the schedule is tested without a GPU).
#pragma once

#include <stdint.h>

#include "params.cuh"

#if defined(__CUDACC__)
#define PTHB_HD __host__ __device__ __forceinline__
#else
#define PTHB_HD inline
#endif

namespace pthb200 {

constexpr int kItemTilesTarget = 24;  // KV tiles per item when a CTA has work for several items
constexpr int kItemsPerCtaMax = 8;    // items per CTA the split choice aims for at most
constexpr int kItemTilesMin = 4;      // an item is never planned shorter than this

struct SchedShape {
  int32_t group, num_kv_heads, bq, num_splits, window, causal, row_class, class_rows;
};

PTHB_HD int sched_min(int a, int b) { return a < b ? a : b; }
PTHB_HD int sched_max(int a, int b) { return a > b ? a : b; }

// Inclusive visible key range of query token i of a request (bottom-right aligned).
PTHB_HD void visible_bounds(int window, int causal, int seq_len, int q_len, int i, int* lo, int* hi) {
  const int pos = seq_len - q_len + i;
  *lo = window > 0 ? sched_max(0, pos - window + 1) : 0;
  int h;
  if (causal) {
    h = pos;
  } else if (window > 0) {
    const int64_t far = (int64_t)pos + window - 1;
    h = far > (int64_t)(seq_len - 1) ? seq_len - 1 : (int)far;
  } else {
    h = seq_len - 1;
  }
  *hi = sched_min(h, seq_len - 1);
}

// Row tiles of a request in this launch (0: the launch does not serve it).
PTHB_HD int req_row_tiles(const SchedShape& s, int q_len) {
  if (q_len <= 0) return 0;
  if (s.row_class != 0 && (((int64_t)q_len * s.group <= s.class_rows) != (s.row_class == 1))) return 0;
  return (q_len + s.bq - 1) / s.bq;
}

// KV tiles the rows of a request touch together.
PTHB_HD int req_kv_tiles(const SchedShape& s, int q_len, int seq_len) {
  if (q_len <= 0) return 0;
  int lo0, hi0, lo1, hi1;
  visible_bounds(s.window, s.causal, seq_len, q_len, 0, &lo0, &hi0);
  visible_bounds(s.window, s.causal, seq_len, q_len, q_len - 1, &lo1, &hi1);
  const int rb = lo0, re = sched_max(hi0, hi1) + 1;
  if (re <= rb) return 0;
  return (re + kKvTile - 1) / kKvTile - rb / kKvTile;
}

// t*: KV tiles an item should hold, from the total work and the number of CTAs.
PTHB_HD int item_tiles(unsigned long long total_tiles, int num_ctas) {
  const unsigned long long ctas = num_ctas > 0 ? (unsigned long long)num_ctas : 1ull;
  const unsigned long long per_cta = (total_tiles + ctas - 1) / ctas;
  unsigned long long m = per_cta / kItemTilesTarget;
  if (m < 1) m = 1;
  if (m > kItemsPerCtaMax) m = kItemsPerCtaMax;
  unsigned long long t = (per_cta + m - 1) / m;
  if (t < kItemTilesMin) t = kItemTilesMin;
  if (t > (1ull << 30)) t = 1ull << 30;
  return (int)t;
}

// S(r): splits of a request whose rows touch kv_tiles KV tiles.
PTHB_HD int req_splits(int kv_tiles, int t_star, int num_splits) {
  const int64_t s = ((int64_t)kv_tiles + t_star / 2) / t_star;
  return s < 1 ? 1 : (s > num_splits ? num_splits : (int)s);
}

// Items of a request, and the coordinates of its item `local`.
PTHB_HD int64_t req_items(int row_tiles, int splits, int num_kv_heads) {
  return (int64_t)row_tiles * splits * num_kv_heads;
}
struct ItemCoord {
  int32_t row_tile, split, kvh;
};
PTHB_HD ItemCoord item_coord(int local, int num_kv_heads, int splits) {
  ItemCoord c;
  c.kvh = local % num_kv_heads;
  const int rest = local / num_kv_heads;
  c.split = rest % splits;
  c.row_tile = rest / splits;
  return c;
}

// KV tiles [tile_begin, tile_end) of split `split` out of `splits` for a row tile whose
// rows see the keys [range_begin, range_end) together: whole tiles, sizes differ by <= 1.
PTHB_HD void split_tile_span(int range_begin, int range_end, int split, int splits, int* tile_begin, int* tile_end) {
  if (range_end <= range_begin) {
    *tile_begin = *tile_end = 0;
    return;
  }
  const int t0 = range_begin / kKvTile;
  const int t1 = (range_end + kKvTile - 1) / kKvTile;
  const int64_t n = t1 - t0;
  *tile_begin = t0 + (int)((int64_t)split * n / splits);
  *tile_end = t0 + (int)((int64_t)(split + 1) * n / splits);
}

}  // namespace pthb200
