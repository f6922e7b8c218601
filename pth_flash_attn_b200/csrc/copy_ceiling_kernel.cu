// Paged-copy ceiling: a kernel that fetches exactly the cache bytes the integer attention
// kernel fetches, in the same way, and throws them away.
//
// It is the measuring stick for the attention kernel's memory side (the counterpart of the
// reference's copy-ceiling program, bench/sol_copy.cu:424-512, whose ratio eta_mem = T_copy /
// T_kernel the reference reports for its decode shapes): same persistent CTAs (one per SM),
// same work-item schedule (sched.cuh), same TMA page copies (one [block_size slots] x
// [272 bytes] box of the page tensor map, or one bulk copy of a contiguous page run) into
// the same ring of three 34,816-byte raw stages in shared memory.  What is missing is
// everything after the copy: a stage is handed back as soon as its bytes have landed.  The
// time of this kernel on a launch is therefore the least the attention kernel could need
// for that launch with this access pattern and this many bytes in flight.
#include <cuda.h>

#include "params.cuh"
#include "sched.cuh"
#include "page_copy.cuh"

namespace pthb200 {
namespace {

constexpr int kCopyStages = 3;
constexpr int kCopyThreads = 64;  // warp 0 walks the items and issues the copies, warp 1 releases the stages

__global__ void __launch_bounds__(kCopyThreads, 1)
copy_ceiling_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kCopyStages * kRawStageBytes);  // [stages] full, [stages] free
  int* tiles_s = reinterpret_cast<int*>(bars + 2 * kCopyStages);                      // tiles of the next item (-1: end)
  uint64_t* item_bar = reinterpret_cast<uint64_t*>(tiles_s + 2);                      // [2] item published / consumed
  volatile int* abort_flag = reinterpret_cast<volatile int*>(item_bar + 2);
  unsigned long long* total_s = reinterpret_cast<unsigned long long*>(item_bar + 3);
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
  if (tid == 0) {
    for (int s = 0; s < kCopyStages; ++s) {
      tc::mbar_init(&bars[s], kKvTile >> p.copy_shift);
      tc::mbar_init(&bars[kCopyStages + s], 1);
    }
    tc::mbar_init(&item_bar[0], 1);
    tc::mbar_init(&item_bar[1], 1);
    *abort_flag = 0;
    *total_s = 0ull;
    tc::mbar_init_fence();
  }
  __syncthreads();
  {
    unsigned long long w = 0;
    for (int r = tid; r < p.num_reqs; r += kCopyThreads) {
      const int q0 = __ldg(p.query_start_loc + r), q1 = __ldg(p.query_start_loc + r + 1);
      w += (unsigned long long)req_row_tiles(shape, q1 - q0) *
           (unsigned long long)req_kv_tiles(shape, q1 - q0, __ldg(p.seq_lens + r));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0 && w != 0) atomicAdd(total_s, w);
  }
  tc::fence_async_smem();
  __syncthreads();
  const int t_star = item_tiles(*total_s * (unsigned long long)p.num_kv_heads, (int)gridDim.x);
  bool ok = true;

  if (warp == 0) {
    // ---- items (as the attention kernel's scheduler finds them) and their page copies ----
    const int S = p.num_splits, hkv = p.num_kv_heads, bs = p.copy_slots;
    const int pages_per_tile = kKvTile >> p.copy_shift;
    const uint32_t raw_s = tc::smem_u32(smem);
    int base = 0, blk_total = 0, my_q0 = 0, my_qlen = 0, my_len = 0, my_splits = 1, my_n = 0, my_excl = 0;
    long long blk_first = 0;
    auto load_block = [&](int b) {
      const int r = b + lane;
      my_n = my_q0 = my_qlen = my_len = 0;
      my_splits = 1;
      if (r < p.num_reqs) {
        my_q0 = __ldg(p.query_start_loc + r);
        my_qlen = __ldg(p.query_start_loc + r + 1) - my_q0;
        my_len = __ldg(p.seq_lens + r);
        my_splits = req_splits(req_kv_tiles(shape, my_qlen, my_len), t_star, S);
        my_n = (int)req_items(req_row_tiles(shape, my_qlen), my_splits, hkv);
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
    int g = 0, items = 0;  // running tile count, items published
    for (long long idx = blockIdx.x; ok; idx += gridDim.x) {
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
      const int src = __ffs(__ballot_sync(0xffffffffu, rel >= my_excl && rel < my_excl + my_n)) - 1;
      const int req = base + src;
      const int q_len = __shfl_sync(0xffffffffu, my_qlen, src), seq_len = __shfl_sync(0xffffffffu, my_len, src);
      const int splits = __shfl_sync(0xffffffffu, my_splits, src);
      const ItemCoord c = item_coord(rel - __shfl_sync(0xffffffffu, my_excl, src), hkv, splits);
      const int first_idx = c.row_tile * p.bq, ntok = min(p.bq, q_len - first_idx);
      int lo0, hi0, lo1, hi1, tile_begin, tile_end;
      visible_bounds(p.window, p.causal, seq_len, q_len, first_idx, &lo0, &hi0);
      visible_bounds(p.window, p.causal, seq_len, q_len, first_idx + ntok - 1, &lo1, &hi1);
      const int range_begin = lo0, range_end = max(hi0, hi1) + 1;
      split_tile_span(range_begin, range_end, c.split, splits, &tile_begin, &tile_end);
      const int n_tiles = tile_end - tile_begin;
      if (n_tiles <= 0) continue;
      // tell the releasing warp how many tiles follow
      if (items > 0) ok &= wait_or_abort(&item_bar[1], (items - 1) & 1, abort_flag);
      if (lane == 0) {
        tiles_s[0] = n_tiles;
        mbar_arrive(&item_bar[0]);
      }
      ++items;
      const int32_t* bt = p.block_table + (int64_t)req * p.block_table_row_stride;
      const uint8_t* kb = p.k.data + (int64_t)c.kvh * p.k.stride_head;
      const uint32_t delta = (uint32_t)(reinterpret_cast<uintptr_t>(kb) & 15);
      const int tma_x = (int)((reinterpret_cast<uintptr_t>(kb) - delta -
                               (reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15)) >> 2);
      auto page_block = [&](int tile) -> int {
        const int pos0 = (tile_begin + tile) * kKvTile + lane * bs;
        if (lane >= pages_per_tile || tile >= n_tiles || pos0 >= range_end || pos0 + bs <= range_begin) return -1;
        int page, slot;
        page_and_slot(p, pos0, &page, &slot);
        return __ldg(bt + page);
      };
      auto first_slot = [&](int tile) -> int {
        int page, slot;
        page_and_slot(p, (tile_begin + tile) * kKvTile + lane * bs, &page, &slot);
        return slot;
      };
      int blk = page_block(0);
#pragma unroll 1
      for (int j = 0; j < n_tiles; ++j, ++g) {
        const int blk_next = page_block(j + 1);
        const int rs = g % kCopyStages;
        if (g >= kCopyStages) ok &= wait_or_abort(&bars[kCopyStages + rs], ((g / kCopyStages) - 1) & 1, abort_flag);
        if (lane < pages_per_tile) {
          uint64_t* bar = &bars[rs];
          if (blk >= 0 && ok) {
            const uint32_t dst = raw_s + rs * kRawStageBytes + lane * bs * kRawRow;
            if (p.raw_mode == 1) {
              mbar_arrive_expect_tx(bar, bs * kRawRow);
              tma_load_3d(dst, &tmap, tma_x, first_slot(j), blk, bar);
            } else {
              const uint32_t bytes = bs * (2 * p.head_size + 8);
              mbar_arrive_expect_tx(bar, bytes);
              bulk_copy_g2s(dst, kb + (int64_t)blk * p.k.stride_block + (int64_t)first_slot(j) * (2 * p.head_size + 8), bytes, bar);
            }
          } else {
            mbar_arrive(bar);
          }
        }
        blk = blk_next;
      }
    }
    if (items > 0) ok &= wait_or_abort(&item_bar[1], (items - 1) & 1, abort_flag);
    if (lane == 0) {
      tiles_s[0] = -1;
      mbar_arrive(&item_bar[0]);
    }
  } else {
    // ---- the stand-in for the rest of the attention kernel: a landed stage is free again ----
    int g = 0;
    for (int item = 0; ok; ++item) {
      ok &= wait_or_abort(&item_bar[0], item & 1, abort_flag);
      const int n_tiles = *reinterpret_cast<volatile int*>(tiles_s);
      __syncwarp();
      if (lane == 0) mbar_arrive(&item_bar[1]);
      if (n_tiles < 0 || !ok) break;
      for (int j = 0; j < n_tiles; ++j, ++g) {
        const int rs = g % kCopyStages;
        ok &= wait_or_abort(&bars[rs], (g / kCopyStages) & 1, abort_flag);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[kCopyStages + rs]);
      }
    }
  }
  __syncthreads();
}

}  // namespace

cudaError_t launch_copy_ceiling(const KernelParams& p_in, cudaStream_t stream) {
  KernelParams p = p_in;
  if (p.row_class == 1) {
    p.bq = p.class_rows / p.group > 0 ? p.class_rows / p.group : 1;
  } else {
    const int cap = 64 / p.group;
    if (p.bq > cap) p.bq = cap;
  }
  set_copy_slots(p, 128);
  p.raw_mode = raw_mode_for(p);
  static const CUtensorMap no_map{};
  const CUtensorMap* map = &no_map;
  if (p.raw_mode == 1) {
    map = cached_page_map(p);
    if (map == nullptr) return cudaErrorInvalidValue;
  }
  const int sms = sm_count();
  if (sms <= 0) return cudaErrorInvalidDevice;
  const int ctas = umma_i8_num_ctas(p_in, sms);
  if (ctas < 1) return cudaErrorInvalidValue;
  constexpr int smem = kCopyStages * kRawStageBytes + 256;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    // the whole shared memory of the SM, as the attention kernel takes it: one CTA per SM
    err = cudaFuncSetAttribute(copy_ceiling_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  static_assert(smem <= 226 * 1024, "raw ring");
  copy_ceiling_kernel<<<ctas, kCopyThreads, 226 * 1024, stream>>>(p, *map);
  return cudaGetLastError();
}

}  // namespace pthb200
