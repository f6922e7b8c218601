// Shared by the tcgen05 attention kernels that fetch whole cache cells with TMA: the raw
// tile geometry, the mbarrier / bulk-copy wrappers of the loader and producer roles, the
// bounded wait, and the host side of the page tensor map.
//
// A raw tile holds, for each of the 128 keys of a KV tile, the 272 bytes from the 16-byte
// boundary below the key's 264-byte cell (K[128] | k_scale | V[128] | v_scale, 8-byte
// aligned): with delta = cell address mod 16 in {0, 8}, K is at raw bytes delta .. delta + 127,
// k_scale at delta + 128, V at delta + 132, v_scale at delta + 260.
#pragma once

#include <cuda.h>

#include <mutex>

#include "params.cuh"
#include "tcgen05.cuh"

namespace pthb200 {
namespace {

constexpr int kRawKeys = 128;                               // keys of one KV tile
constexpr int kRawRow = 272;                                // aligned bytes that cover a 264-byte cell
constexpr int kRawStageBytes = kRawKeys * kRawRow;          // 34,816 B
// The same for any head size: 144 bytes for 64, 272 for 128, 528 for 256.
__host__ __device__ constexpr int raw_row_for(int head_size) { return (2 * head_size + 8 + 8 + 15) / 16 * 16; }
static_assert(raw_row_for(128) == kRawRow, "raw row of head size 128");

// Slots one page copy brings in: the largest power of two from 16 to `most` that divides the
// page size (0 if there is none).  Pages of 16 to `most` slots that are a power of two are one
// copy; a page of 816 slots is 51 copies of 16, one of 256 slots two of 128.
__host__ __device__ inline int copy_slots_for(int block_size, int most) {
  for (int c = most; c >= 16; c >>= 1)
    if (block_size % c == 0) return c;
  return 0;
}
inline void set_copy_slots(KernelParams& p, int most) {
  p.copy_slots = copy_slots_for(p.block_size, most);
  p.copy_shift = -1;
  for (int sh = 4; sh <= 7; ++sh)
    if ((1 << sh) == p.copy_slots) p.copy_shift = sh;
}
// Page (row of the block table) and first slot inside it of KV position `pos`.
__device__ __forceinline__ void page_and_slot(const KernelParams& p, int pos, int* page, int* slot) {
  if (p.block_shift >= 0) {
    *page = pos >> p.block_shift;
    *slot = pos & (p.block_size - 1);
  } else {
    *page = pos / p.block_size;
    *slot = pos - *page * p.block_size;
  }
}

__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc::smem_u32(bar)), "r"(bytes) : "memory");
}
// Bulk copy global -> shared (both 16-byte aligned, size a multiple of 16); completion is
// signalled on the mbarrier as `bytes` of transaction count.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const uint8_t* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

// Tiled TMA load of one box of a rank-3 tensor map into shared memory.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(tc::smem_u32(bar))
      : "memory");
}

// Bounded wait with a CTA-wide abort flag: once any wait has given up, every wait returns.
// The thread sleeps inside try_wait (suspend hint) rather than spinning; the bound is a
// deadline of 2^32 SM cycles (about two seconds), checked between sleeps.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (tc::mbar_try_wait(bar, parity)) return true;
  const long long deadline = clock64() + (1ll << 32);
  for (;;) {
    if (tc::mbar_try_wait_hint(bar, parity, 100000u)) return true;
    if (*abort_flag) return false;
    if (clock64() > deadline) break;
  }
  *abort_flag = 1;
  return false;
}

// The same wait with the barrier given as a shared-memory address.
__device__ __forceinline__ bool wait_or_abort_s(uint32_t bar_s, uint32_t parity, volatile int* abort_flag) {
  if (tc::mbar_try_wait_s(bar_s, parity)) return true;
  const long long deadline = clock64() + (1ll << 32);
  for (;;) {
    if (tc::mbar_try_wait_hint_s(bar_s, parity, 100000u)) return true;
    if (*abort_flag) return false;
    if (clock64() > deadline) break;
  }
  *abort_flag = 1;
  return false;
}

// The same wait for a thread that others wait for (the MMA-issuing thread): it polls without
// a suspend hint, so it sees the phase complete as early as possible.
__device__ __forceinline__ bool wait_or_abort_spin_s(uint32_t bar_s, uint32_t parity, volatile int* abort_flag) {
  if (tc::mbar_try_wait_s(bar_s, parity)) return true;
  const long long deadline = clock64() + (1ll << 32);
  for (;;) {
    if (tc::mbar_try_wait_s(bar_s, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() > deadline) break;
  }
  *abort_flag = 1;
  return false;
}

// True in exactly one lane of a converged warp (elect.sync): the form in which the compiler
// knows that a single thread issues what follows.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void row_target(const KernelParams& p, const RowTile& t, int kvh, int n, int* token, int* head) {
  *token = t.tok0 + n / p.group;
  *head = kvh * p.group + n % p.group;
}

// cuTensorMapEncodeTiled, looked up once through the runtime (no link against libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &st) != cudaSuccess ||
        st != cudaDriverEntryPointSuccess) {
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Tensor map over the cache as 4-byte elements: [slot bytes / 4][block_size slots][num_blocks],
// starting at the 16-byte boundary below head 0's first cell; one box = copy_slots slots of one
// page x the raw row of the head size.  Returns false if the driver refuses the geometry.
bool make_page_map(const KernelParams& p, int num_blocks, CUtensorMap* map) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const uintptr_t base = reinterpret_cast<uintptr_t>(p.k.data) & ~(uintptr_t)15;
  // a slot's cells end (k.data - base) bytes after one slot stride from the row's start: the row
  // is that much longer, so the last head's cell is inside it (and no byte after the slot is)
  const uintptr_t lead = reinterpret_cast<uintptr_t>(p.k.data) - base;
  const cuuint64_t dims[3] = {(cuuint64_t)((p.k.stride_slot + lead) / 4), (cuuint64_t)p.block_size, (cuuint64_t)num_blocks};
  const cuuint64_t strides[2] = {(cuuint64_t)p.k.stride_slot, (cuuint64_t)p.k.stride_block};
  const cuuint32_t box[3] = {(cuuint32_t)(raw_row_for(p.head_size) / 4), (cuuint32_t)p.copy_slots, 1u};
  const cuuint32_t elem[3] = {1u, 1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, reinterpret_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The page map of a cache, built once and kept: encoding a map is a driver call of several
// microseconds, which a decode launch of some tens of microseconds pays on every call
// otherwise.  A map depends only on the cache view (address, strides, page size, block
// count), and a serving engine calls with the same few views for its whole life.  Returns
// nullptr if the driver refuses the geometry; the pointer stays valid (entries are only
// ever added; once the table is full, further views are encoded per call into a
// thread-local map).
const CUtensorMap* cached_page_map(const KernelParams& p) {
  struct Entry {
    uintptr_t base;
    int64_t stride_slot, stride_block;
    int32_t block_size, num_blocks, head_size, copy_slots;
    CUtensorMap map;
  };
  constexpr int kEntries = 64;
  static Entry entries[kEntries];
  static int used = 0;
  static std::mutex mu;
  const uintptr_t base = reinterpret_cast<uintptr_t>(p.k.data);
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i) {
      const Entry& e = entries[i];
      if (e.base == base && e.stride_slot == p.k.stride_slot && e.stride_block == p.k.stride_block &&
          e.block_size == p.block_size && e.num_blocks == p.num_blocks && e.head_size == p.head_size &&
          e.copy_slots == p.copy_slots) {
        return &e.map;
      }
    }
    if (used < kEntries) {
      Entry& e = entries[used];
      if (!make_page_map(p, p.num_blocks, &e.map)) return nullptr;
      e.base = base;
      e.stride_slot = p.k.stride_slot;
      e.stride_block = p.k.stride_block;
      e.block_size = p.block_size;
      e.num_blocks = p.num_blocks;
      e.head_size = p.head_size;
      e.copy_slots = p.copy_slots;
      ++used;
      return &e.map;
    }
  }
  thread_local CUtensorMap scratch;
  return make_page_map(p, p.num_blocks, &scratch) ? &scratch : nullptr;
}

// SMs of the current device (looked up once per device).
int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

// 1 = tiled TMA per page, 2 = bulk copy per contiguous page run, 0 = neither applies.
int raw_mode_for(const KernelParams& p) {
  const int slots = copy_slots_for(p.block_size, 128);  // pages are made of runs of 16 slots or more
  if (slots == 0) return 0;
  if (p.k.stride_block % 16 != 0) return 0;
  if (p.k.stride_slot == 2 * p.head_size + 8) {
    // A bulk copy starts and ends on 16-byte boundaries: the page run of every head must
    // itself be 16-byte aligned, so that the copy never reads a byte outside the run.
    const bool aligned_runs = reinterpret_cast<uintptr_t>(p.k.data) % 16 == 0 &&
                              (p.num_kv_heads == 1 || p.k.stride_head % 16 == 0) &&
                              ((int64_t)slots * p.k.stride_slot) % 16 == 0;
    return aligned_runs ? 2 : 0;
  }
  if (p.k.stride_slot % 16 == 0 && p.k.stride_slot >= raw_row_for(p.head_size)) return 1;
  return 0;
}

}  // namespace
}  // namespace pthb200
