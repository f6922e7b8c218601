// torch op library: registers pth_flash_attn::pth_flash_attn_fwd through the
// libtorch stable ABI and forwards to the C ABI of libpthb200_attn.so.
//
// The schema, the argument meaning, the order of the argument checks and their
// messages are those of the reference op (csrc/pth_attn/torch_bindings.cpp:20-38,
// csrc/pth_attn/launch.cu:166-346, docs/api.md), so a caller and its tests can
// switch libraries without edits.  What differs: the device check asks for
// compute capability 10.x, and an extra op, pth_flash_attn_fwd_lse, also returns
// the natural-log log-sum-exp per (token, head).
//
// The op allocates nothing, reads no device data on the host and does not
// synchronise; it launches on the current stream of q's device.
#include <cuda_runtime.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>
#include <torch/headeronly/util/Exception.h>

#include <climits>
#include <cmath>
#include <cstdint>

#include "../../include/pthb200_attn.h"

extern "C" int32_t aoti_torch_get_current_cuda_stream(int32_t device_index, void** ret_stream);

namespace {

using torch::headeronly::ScalarType;
using torch::stable::Tensor;

#define OP "pth_flash_attn_fwd: "

const char* type_name(ScalarType t) {
  switch (t) {
    case ScalarType::BFloat16: return "bfloat16";
    case ScalarType::Half: return "float16";
    case ScalarType::Float: return "float32";
    case ScalarType::Char: return "int8";
    case ScalarType::Int: return "int32";
    case ScalarType::Long: return "int64";
    default: return "an unsupported dtype";
  }
}

struct Checker {
  static void rank(const Tensor& t, int64_t want, const char* name) {
    STD_TORCH_CHECK(t.dim() == want, OP, name, " must be ", want, "-D, got ", t.dim(), "-D");
  }
  static void dtype(const Tensor& t, ScalarType want, const char* name) {
    STD_TORCH_CHECK(t.scalar_type() == want, OP, name, " must be ", type_name(want), ", got ",
                    type_name(t.scalar_type()));
  }
  static void size(const Tensor& t, int64_t dim, int64_t want, const char* name, const char* what) {
    STD_TORCH_CHECK(t.size(dim) == want, OP, name, ".size(", dim, ") must equal ", what, " = ", want, ", got ",
                    t.size(dim));
  }
  static void unit_inner_stride(const Tensor& t, const char* name) {
    STD_TORCH_CHECK(t.stride(t.dim() - 1) == 1, OP, name, " must have stride 1 in its last dimension, got ",
                    t.stride(t.dim() - 1));
  }
  static void same_device(const Tensor& t, const Tensor& q, const char* name) {
    STD_TORCH_CHECK(t.is_cuda() == q.is_cuda() && t.get_device_index() == q.get_device_index(), OP, name,
                    " must be on the same device as q");
  }
  // One past the last byte a view can touch must fit in int64 (and no negative strides).
  static void extent(const Tensor& t, const char* name) {
    int64_t total = static_cast<int64_t>(t.element_size());
    bool ok = true, empty = false;
    for (int64_t i = 0; i < t.dim(); ++i) {
      if (t.size(i) < 0 || t.stride(i) < 0) ok = false;
      if (t.size(i) == 0) empty = true;
    }
    if (ok && !empty) {
      for (int64_t i = 0; i < t.dim() && ok; ++i) {
        int64_t term = 0;
        ok = !__builtin_mul_overflow(t.size(i) - 1, t.stride(i), &term) &&
             !__builtin_mul_overflow(term, static_cast<int64_t>(t.element_size()), &term) &&
             !__builtin_add_overflow(total, term, &total);
      }
    }
    STD_TORCH_CHECK(ok, OP, name, " has negative strides or a byte extent that overflows int64");
  }
  static void alignment(const Tensor& t, int64_t align, const char* name) {
    STD_TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % static_cast<uintptr_t>(align) == 0, OP, name,
                    " data pointer must be ", align, "-byte aligned");
    const int64_t es = static_cast<int64_t>(t.element_size());
    for (int64_t i = 0; i + 1 < t.dim(); ++i) {
      STD_TORCH_CHECK((t.stride(i) * es) % align == 0, OP, name, " byte stride of dim ", i, " (", t.stride(i) * es,
                      ") must be a multiple of ", align);
    }
  }
};

void check_metadata(const Tensor& out, const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                    const Tensor& k_scale, const Tensor& v_scale, const Tensor& block_table, const Tensor& seq_lens,
                    const Tensor& query_start_loc, int64_t max_query_len, int64_t wm, int64_t num_splits,
                    double softmax_scale, const Tensor& ws_o, const Tensor& ws_lse, int64_t window, bool causal) {
  Checker::rank(q, 3, "q");
  STD_TORCH_CHECK(q.scalar_type() == ScalarType::BFloat16 || q.scalar_type() == ScalarType::Half, OP,
                  "q must be bfloat16 or float16, got ", type_name(q.scalar_type()));
  const int64_t T = q.size(0), Hq = q.size(1), D = q.size(2);
  STD_TORCH_CHECK(D == 64 || D == 128 || D == 256, OP, "head size D = q.size(2) must be 64, 128 or 256, got ", D);
  Checker::unit_inner_stride(q, "q");

  Checker::rank(out, 3, "out");
  Checker::dtype(out, q.scalar_type(), "out (same dtype as q)");
  Checker::size(out, 0, T, "out", "T");
  Checker::size(out, 1, Hq, "out", "Hq");
  Checker::size(out, 2, D, "out", "D");
  Checker::unit_inner_stride(out, "out");

  Checker::rank(k_cache, 4, "k_cache");
  Checker::rank(v_cache, 4, "v_cache");
  Checker::dtype(k_cache, ScalarType::Char, "k_cache");
  Checker::dtype(v_cache, ScalarType::Char, "v_cache");
  const int64_t NB = k_cache.size(0), BS = k_cache.size(1), Hkv = k_cache.size(2);
  Checker::size(k_cache, 3, D, "k_cache", "D");
  Checker::size(v_cache, 0, NB, "v_cache", "NB");
  Checker::size(v_cache, 1, BS, "v_cache", "BS");
  Checker::size(v_cache, 2, Hkv, "v_cache", "Hkv");
  Checker::size(v_cache, 3, D, "v_cache", "D");
  Checker::unit_inner_stride(k_cache, "k_cache");
  Checker::unit_inner_stride(v_cache, "v_cache");

  Checker::rank(k_scale, 3, "k_scale");
  Checker::rank(v_scale, 3, "v_scale");
  Checker::dtype(k_scale, ScalarType::Float, "k_scale");
  Checker::dtype(v_scale, ScalarType::Float, "v_scale");
  Checker::size(k_scale, 0, NB, "k_scale", "NB");
  Checker::size(k_scale, 1, BS, "k_scale", "BS");
  Checker::size(k_scale, 2, Hkv, "k_scale", "Hkv");
  Checker::size(v_scale, 0, NB, "v_scale", "NB");
  Checker::size(v_scale, 1, BS, "v_scale", "BS");
  Checker::size(v_scale, 2, Hkv, "v_scale", "Hkv");

  STD_TORCH_CHECK(Hkv >= 1 && Hq % Hkv == 0, OP, "Hq = ", Hq, " must be a positive multiple of Hkv = ", Hkv);
  const int64_t G = Hq / Hkv;
  STD_TORCH_CHECK(wm == 1 || wm == 2 || wm == 4, OP, "wm must be 1, 2 or 4, got ", wm);
  STD_TORCH_CHECK(G <= 64, OP, "G = Hq/Hkv = ", G, " exceeds the supported maximum ", 64);
  STD_TORCH_CHECK(G <= 16 * wm, OP, "G = Hq/Hkv = ", G, " must be <= 16*wm = ", 16 * wm);

  Checker::rank(block_table, 2, "block_table");
  Checker::rank(seq_lens, 1, "seq_lens");
  Checker::rank(query_start_loc, 1, "query_start_loc");
  Checker::dtype(block_table, ScalarType::Int, "block_table");
  Checker::dtype(seq_lens, ScalarType::Int, "seq_lens");
  Checker::dtype(query_start_loc, ScalarType::Int, "query_start_loc");
  Checker::unit_inner_stride(block_table, "block_table");
  Checker::unit_inner_stride(seq_lens, "seq_lens");
  Checker::unit_inner_stride(query_start_loc, "query_start_loc");
  const int64_t R = seq_lens.size(0);
  Checker::size(query_start_loc, 0, R + 1, "query_start_loc", "num_reqs + 1");
  STD_TORCH_CHECK(block_table.size(0) >= R, OP, "block_table has ", block_table.size(0),
                  " rows, fewer than num_reqs = ", R);

  STD_TORCH_CHECK(max_query_len >= 0 && max_query_len <= T, OP, "max_query_len must be in [0, T = ", T, "], got ",
                  max_query_len);
  STD_TORCH_CHECK(num_splits >= 1, OP, "num_splits must be >= 1, got ", num_splits);
  STD_TORCH_CHECK(std::isfinite(softmax_scale) && softmax_scale > 0.0, OP,
                  "softmax_scale must be finite and > 0, got ", softmax_scale);
  STD_TORCH_CHECK(window >= 0, OP, "window must be >= 0, got ", window);
  STD_TORCH_CHECK(!((window > 0 || !causal) && D != 128), OP,
                  "sliding-window and non-causal attention need head size D = 128, got ", D);

  Checker::same_device(out, q, "out");
  Checker::same_device(k_cache, q, "k_cache");
  Checker::same_device(v_cache, q, "v_cache");
  Checker::same_device(k_scale, q, "k_scale");
  Checker::same_device(v_scale, q, "v_scale");
  Checker::same_device(block_table, q, "block_table");
  Checker::same_device(seq_lens, q, "seq_lens");
  Checker::same_device(query_start_loc, q, "query_start_loc");

  if (num_splits > 1) {
    Checker::rank(ws_o, 4, "ws_o");
    Checker::rank(ws_lse, 3, "ws_lse");
    Checker::dtype(ws_o, ScalarType::Float, "ws_o");
    Checker::dtype(ws_lse, ScalarType::Float, "ws_lse");
    STD_TORCH_CHECK(ws_o.size(0) >= num_splits && ws_o.size(1) >= T, OP, "ws_o must have size(0) >= num_splits = ",
                    num_splits, " and size(1) >= T = ", T, ", got [", ws_o.size(0), ", ", ws_o.size(1), ", ...]");
    Checker::size(ws_o, 2, Hq, "ws_o", "Hq");
    Checker::size(ws_o, 3, D, "ws_o", "D");
    STD_TORCH_CHECK(ws_lse.size(0) >= num_splits && ws_lse.size(1) >= T, OP,
                    "ws_lse must have size(0) >= num_splits = ", num_splits, " and size(1) >= T = ", T, ", got [",
                    ws_lse.size(0), ", ", ws_lse.size(1), ", ...]");
    Checker::size(ws_lse, 2, Hq, "ws_lse", "Hq");
    Checker::unit_inner_stride(ws_o, "ws_o");
    Checker::unit_inner_stride(ws_lse, "ws_lse");
    Checker::same_device(ws_o, q, "ws_o");
    Checker::same_device(ws_lse, q, "ws_lse");
  }
}

void check_addresses(const Tensor& out, const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                     const Tensor& k_scale, const Tensor& v_scale, const Tensor& block_table, const Tensor& seq_lens,
                     const Tensor& query_start_loc, int64_t num_splits, const Tensor& ws_o, const Tensor& ws_lse) {
  Checker::extent(out, "out");
  Checker::extent(q, "q");
  Checker::extent(k_cache, "k_cache");
  Checker::extent(v_cache, "v_cache");
  Checker::extent(k_scale, "k_scale");
  Checker::extent(v_scale, "v_scale");
  Checker::extent(block_table, "block_table");
  Checker::extent(seq_lens, "seq_lens");
  Checker::extent(query_start_loc, "query_start_loc");
  Checker::alignment(k_cache, 4, "k_cache");
  Checker::alignment(v_cache, 4, "v_cache");
  Checker::alignment(k_scale, 4, "k_scale");
  Checker::alignment(v_scale, 4, "v_scale");
  Checker::alignment(q, 16, "q");
  Checker::alignment(out, 16, "out");
  if (num_splits > 1) {
    STD_TORCH_CHECK(ws_o.data_ptr() != nullptr && ws_lse.data_ptr() != nullptr, OP,
                    "workspace (ws_o, ws_lse) must be allocated when num_splits > 1");
    Checker::extent(ws_o, "ws_o");
    Checker::extent(ws_lse, "ws_lse");
    Checker::alignment(ws_o, 16, "ws_o");
  }
}

int64_t bytes(const Tensor& t, int64_t dim) { return t.stride(dim) * static_cast<int64_t>(t.element_size()); }

PthAttnStream as_stream(const Tensor& t) { return PthAttnStream{t.data_ptr(), bytes(t, 0), bytes(t, 1), bytes(t, 2)}; }

void run(Tensor& out, const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& k_scale,
         const Tensor& v_scale, const Tensor& block_table, const Tensor& seq_lens, const Tensor& query_start_loc,
         int64_t max_query_len, int64_t wm, int64_t num_splits, double softmax_scale, Tensor& ws_o, Tensor& ws_lse,
         int64_t window, bool causal, Tensor* lse) {
  check_metadata(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc, max_query_len,
                 wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal);
  if (lse != nullptr) {
    Checker::rank(*lse, 2, "lse");
    Checker::dtype(*lse, ScalarType::Float, "lse");
    Checker::size(*lse, 0, q.size(0), "lse", "T");
    Checker::size(*lse, 1, q.size(1), "lse", "Hq");
    Checker::same_device(*lse, q, "lse");
  }
  check_addresses(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc, num_splits, ws_o,
                  ws_lse);
  STD_TORCH_CHECK(q.is_cuda(), OP,
                  "arguments are valid, but the op computes on CUDA tensors only (the CPU registration exists to "
                  "test the argument checks)");
  const int32_t device = static_cast<int32_t>(q.get_device_index());
  int major = 0;
  const cudaError_t err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  STD_TORCH_CHECK(err == cudaSuccess, OP, "cannot query the compute capability: ", cudaGetErrorString(err));
  STD_TORCH_CHECK(major == 10, OP, "needs compute capability 10.x (sm_100a), device has major ", major);
  if (q.size(0) == 0 || seq_lens.size(0) == 0) return;

  const int64_t group = q.size(1) / k_cache.size(2);
  const int32_t bq = pthb200_tile_tokens(static_cast<int32_t>(wm), static_cast<int32_t>(group),
                                         static_cast<int32_t>(max_query_len > INT32_MAX ? INT32_MAX : max_query_len));
  STD_TORCH_CHECK(bq >= 1, OP, "wm = ", wm, " is not the tile height of G = ", group);

  PthAttnArgs a{};
  a.abi_version = PTH_ATTN_ABI_VERSION;
  a.struct_bytes = static_cast<int32_t>(sizeof(PthAttnArgs));
  const int32_t code = q.scalar_type() == ScalarType::Half ? PTH_ATTN_F16 : PTH_ATTN_BF16;
  a.q = q.data_ptr();
  a.q_dtype = code;
  a.q_stride_token = bytes(q, 0);
  a.q_stride_head = bytes(q, 1);
  a.out = out.data_ptr();
  a.out_dtype = code;
  a.out_stride_token = bytes(out, 0);
  a.out_stride_head = bytes(out, 1);
  a.k_cache = as_stream(k_cache);
  a.v_cache = as_stream(v_cache);
  a.k_scale = as_stream(k_scale);
  a.v_scale = as_stream(v_scale);
  a.num_blocks = static_cast<int32_t>(k_cache.size(0));
  a.block_size = static_cast<int32_t>(k_cache.size(1));
  a.num_kv_heads = static_cast<int32_t>(k_cache.size(2));
  a.head_size = static_cast<int32_t>(q.size(2));
  a.block_table = static_cast<const int32_t*>(block_table.data_ptr());
  a.block_table_row_stride = block_table.stride(0);
  a.seq_lens = static_cast<const int32_t*>(seq_lens.data_ptr());
  a.query_start_loc = static_cast<const int32_t*>(query_start_loc.data_ptr());
  a.num_reqs = static_cast<int32_t>(seq_lens.size(0));
  a.num_tokens = static_cast<int32_t>(q.size(0));
  a.num_q_heads = static_cast<int32_t>(q.size(1));
  a.bq = bq;
  a.num_q_tiles = 0;
  a.num_splits = static_cast<int32_t>(num_splits);
  a.softmax_scale = static_cast<float>(softmax_scale);
  a.window = window > INT32_MAX ? INT32_MAX : static_cast<int32_t>(window);
  a.causal = causal ? 1 : 0;
  if (num_splits > 1) {
    a.ws_o = static_cast<float*>(ws_o.data_ptr());
    a.ws_o_stride_split = bytes(ws_o, 0);
    a.ws_o_stride_token = bytes(ws_o, 1);
    a.ws_o_stride_head = bytes(ws_o, 2);
    a.ws_lse = static_cast<float*>(ws_lse.data_ptr());
    a.ws_lse_stride_split = bytes(ws_lse, 0);
    a.ws_lse_stride_token = bytes(ws_lse, 1);
    a.ws_lse_stride_head = bytes(ws_lse, 2);
  }
  PthB200Options opt{};
  opt.abi_version = PTH_ATTN_ABI_VERSION;
  opt.struct_bytes = static_cast<int32_t>(sizeof(PthB200Options));
  // max_query_len bounds every request: when it fits one row tile, each request is one tile
  if (max_query_len >= 1 && max_query_len <= bq) opt.flags |= PTHB200_FLAG_ONE_TILE_PER_REQUEST;
  if (lse != nullptr) {
    opt.lse_out = static_cast<float*>(lse->data_ptr());
    opt.lse_stride_token = bytes(*lse, 0);
    opt.lse_stride_head = bytes(*lse, 1);
  }

  const torch::stable::accelerator::DeviceGuard guard(device);
  void* stream = nullptr;
  STD_TORCH_CHECK(aoti_torch_get_current_cuda_stream(device, &stream) == 0, OP,
                  "cannot get the current CUDA stream of device ", device);
  int32_t rc = pthb200_attention_ex(&a, &opt, stream);
  STD_TORCH_CHECK(rc == PTH_ATTN_OK, OP, "attention launch: ", pthb200_last_error());
  if (num_splits == 1) return;
  PthAttnCombineArgs c{};
  c.abi_version = PTH_ATTN_ABI_VERSION;
  c.struct_bytes = static_cast<int32_t>(sizeof(PthAttnCombineArgs));
  c.ws_o = a.ws_o;
  c.ws_o_stride_split = a.ws_o_stride_split;
  c.ws_o_stride_token = a.ws_o_stride_token;
  c.ws_o_stride_head = a.ws_o_stride_head;
  c.ws_lse = a.ws_lse;
  c.ws_lse_stride_split = a.ws_lse_stride_split;
  c.ws_lse_stride_token = a.ws_lse_stride_token;
  c.ws_lse_stride_head = a.ws_lse_stride_head;
  c.out = a.out;
  c.out_dtype = a.out_dtype;
  c.out_stride_token = a.out_stride_token;
  c.out_stride_head = a.out_stride_head;
  c.query_start_loc = a.query_start_loc;
  c.num_reqs = a.num_reqs;
  c.num_tokens = a.num_tokens;
  c.num_q_heads = a.num_q_heads;
  c.head_size = a.head_size;
  c.num_splits = a.num_splits;
  rc = pthb200_combine_ex(&c, &opt, stream);
  STD_TORCH_CHECK(rc == PTH_ATTN_OK, OP, "combine launch: ", pthb200_last_error());
}

void pth_flash_attn_fwd(Tensor& out, const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                        const Tensor& k_scale, const Tensor& v_scale, const Tensor& block_table,
                        const Tensor& seq_lens, const Tensor& query_start_loc, int64_t max_query_len, int64_t wm,
                        int64_t num_splits, double softmax_scale, Tensor& ws_o, Tensor& ws_lse, int64_t window,
                        bool causal) {
  run(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc, max_query_len, wm,
      num_splits, softmax_scale, ws_o, ws_lse, window, causal, nullptr);
}

void pth_flash_attn_fwd_lse(Tensor& out, Tensor& lse, const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                            const Tensor& k_scale, const Tensor& v_scale, const Tensor& block_table,
                            const Tensor& seq_lens, const Tensor& query_start_loc, int64_t max_query_len, int64_t wm,
                            int64_t num_splits, double softmax_scale, Tensor& ws_o, Tensor& ws_lse, int64_t window,
                            bool causal) {
  run(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc, max_query_len, wm,
      num_splits, softmax_scale, ws_o, ws_lse, window, causal, &lse);
}

}  // namespace

STABLE_TORCH_LIBRARY(pth_flash_attn, m) {
  m.def(
      "pth_flash_attn_fwd(Tensor! out, Tensor q, Tensor k_cache, "
      "Tensor v_cache, Tensor k_scale, Tensor v_scale, Tensor block_table, "
      "Tensor seq_lens, Tensor query_start_loc, int max_query_len, int wm, "
      "int num_splits, float softmax_scale, Tensor! ws_o, Tensor! ws_lse, "
      "int window=0, bool causal=True) -> ()");
  m.def(
      "pth_flash_attn_fwd_lse(Tensor! out, Tensor! lse, Tensor q, Tensor k_cache, "
      "Tensor v_cache, Tensor k_scale, Tensor v_scale, Tensor block_table, "
      "Tensor seq_lens, Tensor query_start_loc, int max_query_len, int wm, "
      "int num_splits, float softmax_scale, Tensor! ws_o, Tensor! ws_lse, "
      "int window=0, bool causal=True) -> ()");
}

STABLE_TORCH_LIBRARY_IMPL(pth_flash_attn, CUDA, m) {
  m.impl("pth_flash_attn_fwd", TORCH_BOX(&pth_flash_attn_fwd));
  m.impl("pth_flash_attn_fwd_lse", TORCH_BOX(&pth_flash_attn_fwd_lse));
}

// CPU key: the same function, so the argument checks run without a GPU; after
// the checks a CPU call raises instead of computing.
STABLE_TORCH_LIBRARY_IMPL(pth_flash_attn, CPU, m) {
  m.impl("pth_flash_attn_fwd", TORCH_BOX(&pth_flash_attn_fwd));
  m.impl("pth_flash_attn_fwd_lse", TORCH_BOX(&pth_flash_attn_fwd_lse));
}
