// Host launcher and C ABI of libpthb200_attn.so (include/pthb200_attn.h).
//
// Every entry point validates its arguments (each failure names the field),
// converts the caller's struct into kernel parameters, chooses the kernel
// family and enqueues on the caller's stream.  Nothing here allocates device
// memory, reads device memory or synchronises.
#include <cmath>
#include <cstdio>
#include <string>

#include "params.cuh"
#include "sched.cuh"

namespace pthb200 {
namespace {

thread_local std::string g_last_error;

int32_t fail(int32_t code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

#define PTHB_REQUIRE(cond, msg)                      \
  do {                                               \
    if (!(cond)) return fail(PTH_ATTN_EINVAL, (msg)); \
  } while (0)

bool aligned(const void* ptr, int64_t a) { return reinterpret_cast<uintptr_t>(ptr) % (uintptr_t)a == 0; }

bool is_head_size(int32_t d) { return d == 64 || d == 128 || d == 256; }

int32_t check_stream(const PthAttnStream& s, const char* name) {
  PTHB_REQUIRE(s.data != nullptr, std::string(name) + ".data is NULL");
  PTHB_REQUIRE(aligned(s.data, 4), std::string(name) + ".data must be 4-byte aligned");
  PTHB_REQUIRE(s.stride_block >= 0 && s.stride_slot >= 0 && s.stride_head >= 0,
               std::string(name) + " strides must be >= 0");
  PTHB_REQUIRE(s.stride_block % 4 == 0 && s.stride_slot % 4 == 0 && s.stride_head % 4 == 0,
               std::string(name) + " byte strides must be multiples of 4");
  return PTH_ATTN_OK;
}

StreamParams to_stream(const PthAttnStream& s) {
  return StreamParams{static_cast<const uint8_t*>(s.data), s.stride_block, s.stride_slot, s.stride_head};
}

int32_t check_options(const PthB200Options* o) {
  if (o == nullptr) return PTH_ATTN_OK;
  PTHB_REQUIRE(o->abi_version == PTH_ATTN_ABI_VERSION, "options.abi_version does not match the library");
  PTHB_REQUIRE(o->struct_bytes == (int32_t)sizeof(PthB200Options), "options.struct_bytes != sizeof(PthB200Options)");
  PTHB_REQUIRE(o->kernel >= PTHB200_KERNEL_AUTO && o->kernel <= PTHB200_KERNEL_UMMA_ROWS, "options.kernel is not a kernel family");
  PTHB_REQUIRE((o->flags & ~PTHB200_FLAG_ONE_TILE_PER_REQUEST) == 0, "options.flags has unknown bits");
  if (o->lse_out != nullptr) {
    PTHB_REQUIRE(aligned(o->lse_out, 4), "options.lse_out must be 4-byte aligned");
    PTHB_REQUIRE(o->lse_stride_token % 4 == 0 && o->lse_stride_head % 4 == 0 && o->lse_stride_token >= 0 &&
                     o->lse_stride_head >= 0,
                 "options.lse strides must be non-negative multiples of 4");
  }
  return PTH_ATTN_OK;
}

// Argument checks of an attention launch; fills *kp on success.
int32_t build_attention(const PthAttnArgs* a, const PthB200Options* opt, KernelParams* kp) {
  PTHB_REQUIRE(a != nullptr, "args is NULL");
  PTHB_REQUIRE(a->abi_version == PTH_ATTN_ABI_VERSION, "args.abi_version does not match the library");
  PTHB_REQUIRE(a->struct_bytes == (int32_t)sizeof(PthAttnArgs), "args.struct_bytes != sizeof(PthAttnArgs)");
  if (int32_t rc = check_options(opt)) return rc;

  PTHB_REQUIRE(is_head_size(a->head_size), "head_size must be 64, 128 or 256");
  PTHB_REQUIRE(a->num_kv_heads >= 1 && a->num_q_heads >= 1 && a->num_q_heads % a->num_kv_heads == 0,
               "num_q_heads must be a positive multiple of num_kv_heads");
  const int32_t group = a->num_q_heads / a->num_kv_heads;
  PTHB_REQUIRE(group <= 64, "num_q_heads / num_kv_heads must be <= 64");
  PTHB_REQUIRE(a->num_reqs >= 1, "num_reqs must be >= 1");
  PTHB_REQUIRE(a->num_tokens >= 1, "num_tokens must be >= 1");
  PTHB_REQUIRE(a->bq >= 1, "bq must be >= 1");
  PTHB_REQUIRE(a->num_q_tiles >= 0, "num_q_tiles must be >= 0");
  PTHB_REQUIRE(a->num_splits >= 1 && a->num_splits <= 65535, "num_splits must be in [1, 65535]");
  PTHB_REQUIRE(a->num_kv_heads <= 65535, "num_kv_heads must be <= 65535");
  PTHB_REQUIRE(a->block_size >= 1, "block_size must be >= 1");
  PTHB_REQUIRE(a->num_blocks >= 1, "num_blocks must be >= 1");
  PTHB_REQUIRE(std::isfinite(a->softmax_scale) && a->softmax_scale > 0.f, "softmax_scale must be finite and > 0");
  PTHB_REQUIRE(a->window >= 0, "window must be >= 0");
  PTHB_REQUIRE(a->causal == 0 || a->causal == 1, "causal must be 0 or 1");
  PTHB_REQUIRE(a->q_dtype == PTH_ATTN_F16 || a->q_dtype == PTH_ATTN_BF16, "q_dtype must be F16 or BF16");

  PTHB_REQUIRE(a->q != nullptr, "q is NULL");
  PTHB_REQUIRE(aligned(a->q, 16), "q must be 16-byte aligned");
  PTHB_REQUIRE(a->q_stride_token % 16 == 0 && a->q_stride_head % 16 == 0 && a->q_stride_token >= 0 &&
                   a->q_stride_head >= 0,
               "q byte strides must be non-negative multiples of 16");
  if (int32_t rc = check_stream(a->k_cache, "k_cache")) return rc;
  if (int32_t rc = check_stream(a->v_cache, "v_cache")) return rc;
  if (int32_t rc = check_stream(a->k_scale, "k_scale")) return rc;
  if (int32_t rc = check_stream(a->v_scale, "v_scale")) return rc;
  PTHB_REQUIRE(a->block_table != nullptr && a->seq_lens != nullptr && a->query_start_loc != nullptr,
               "block_table, seq_lens and query_start_loc must not be NULL");
  PTHB_REQUIRE(a->block_table_row_stride >= 0, "block_table_row_stride must be >= 0");

  if (a->num_splits == 1) {
    PTHB_REQUIRE(a->out != nullptr, "out is NULL (num_splits == 1 writes out)");
    PTHB_REQUIRE(a->out_dtype == PTH_ATTN_F32 || a->out_dtype == PTH_ATTN_F16 || a->out_dtype == PTH_ATTN_BF16,
                 "out_dtype must be F32, F16 or BF16");
    PTHB_REQUIRE(aligned(a->out, 16), "out must be 16-byte aligned");
    PTHB_REQUIRE(a->out_stride_token % 16 == 0 && a->out_stride_head % 16 == 0 && a->out_stride_token >= 0 &&
                     a->out_stride_head >= 0,
                 "out byte strides must be non-negative multiples of 16");
  } else {
    PTHB_REQUIRE(a->ws_o != nullptr && a->ws_lse != nullptr, "ws_o and ws_lse must not be NULL when num_splits > 1");
    PTHB_REQUIRE(aligned(a->ws_o, 16), "ws_o must be 16-byte aligned");
    PTHB_REQUIRE(a->ws_o_stride_split % 16 == 0 && a->ws_o_stride_token % 16 == 0 && a->ws_o_stride_head % 16 == 0 &&
                     a->ws_o_stride_split >= 0 && a->ws_o_stride_token >= 0 && a->ws_o_stride_head >= 0,
                 "ws_o byte strides must be non-negative multiples of 16");
    PTHB_REQUIRE(aligned(a->ws_lse, 4), "ws_lse must be 4-byte aligned");
    PTHB_REQUIRE(a->ws_lse_stride_split % 4 == 0 && a->ws_lse_stride_token % 4 == 0 && a->ws_lse_stride_head % 4 == 0 &&
                     a->ws_lse_stride_split >= 0 && a->ws_lse_stride_token >= 0 && a->ws_lse_stride_head >= 0,
                 "ws_lse byte strides must be non-negative multiples of 4");
  }

  KernelParams& p = *kp;
  p = KernelParams{};
  p.q = static_cast<const uint8_t*>(a->q);
  p.q_stride_token = a->q_stride_token;
  p.q_stride_head = a->q_stride_head;
  p.out = static_cast<uint8_t*>(a->out);
  p.out_stride_token = a->out_stride_token;
  p.out_stride_head = a->out_stride_head;
  p.k = to_stream(a->k_cache);
  p.v = to_stream(a->v_cache);
  p.ks = to_stream(a->k_scale);
  p.vs = to_stream(a->v_scale);
  p.block_table = a->block_table;
  p.block_table_row_stride = a->block_table_row_stride;
  p.seq_lens = a->seq_lens;
  p.query_start_loc = a->query_start_loc;
  p.ws_o = a->ws_o;
  p.ws_o_stride_split = a->ws_o_stride_split;
  p.ws_o_stride_token = a->ws_o_stride_token;
  p.ws_o_stride_head = a->ws_o_stride_head;
  p.ws_lse = a->ws_lse;
  p.ws_lse_stride_split = a->ws_lse_stride_split;
  p.ws_lse_stride_token = a->ws_lse_stride_token;
  p.ws_lse_stride_head = a->ws_lse_stride_head;
  if (opt != nullptr && opt->lse_out != nullptr && a->num_splits == 1) {
    p.lse_out = opt->lse_out;
    p.lse_stride_token = opt->lse_stride_token;
    p.lse_stride_head = opt->lse_stride_head;
  }
  p.q_dtype = a->q_dtype;
  p.out_dtype = a->out_dtype;
  p.block_size = a->block_size;
  p.num_blocks = a->num_blocks;
  p.block_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == a->block_size) p.block_shift = sh;
  p.num_kv_heads = a->num_kv_heads;
  p.head_size = a->head_size;
  p.num_reqs = a->num_reqs;
  p.num_tokens = a->num_tokens;
  p.num_q_heads = a->num_q_heads;
  p.group = group;
  p.bq = a->bq;
  p.tile_map = (opt != nullptr && (opt->flags & PTHB200_FLAG_ONE_TILE_PER_REQUEST) != 0) ? 1 : 0;
  p.num_q_tiles = p.tile_map == 1 ? a->num_reqs : a->num_tokens / a->bq + a->num_reqs;
  p.num_splits = a->num_splits;
  p.window = a->window;
  p.causal = a->causal;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  return PTH_ATTN_OK;
}

// Internal family of the automatic choice: integer kernel for the short requests of the
// launch, then the row-major kernel for the others.
constexpr int32_t kFamilyPair = 100;

// Rows up to which a request of a pair launch belongs to the integer kernel.
int32_t pair_class_rows(const KernelParams& p) { return p.group > 16 ? p.group : 16; }

// Kernel family for these parameters (a PTHB200_KERNEL_* value other than AUTO, or kFamilyPair).
int32_t choose_family(const KernelParams& p, const PthB200Options* opt, int32_t* family) {
  const int32_t want = opt ? opt->kernel : PTHB200_KERNEL_AUTO;
  const char* why = "";
  const char* why_i8 = "";
  const bool umma_ok = umma_supports(p, &why);
  const bool i8_ok = umma_i8_supports(p, &why_i8);
  if (want == PTHB200_KERNEL_UMMA) {
    PTHB_REQUIRE(i8_ok, std::string("options.kernel = UMMA does not apply: ") + why_i8);
    *family = want;
  } else if (want == PTHB200_KERNEL_UMMA_BF16) {
    PTHB_REQUIRE(umma_ok, std::string("options.kernel = UMMA_BF16 does not apply: ") + why);
    *family = want;
  } else if (want == PTHB200_KERNEL_UMMA_ROWS) {
    const char* why_rows = "";
    PTHB_REQUIRE(umma_rows_supports(p, &why_rows), std::string("options.kernel = UMMA_ROWS does not apply: ") + why_rows);
    *family = want;
  } else if (want == PTHB200_KERNEL_SCALAR) {
    *family = PTHB200_KERNEL_SCALAR;
  } else {
    // Tall row tiles (prefill chunks, wide verification: more than 16 rows per KV head and
    // tile) go to the row-major kernel, short ones (decode, narrow verification) to the
    // token-major integer kernel.  A launch that may hold both (its tile height only bounds
    // the longest request) runs the two kernels one after the other, each serving its own
    // requests: a decode request inside a prefill batch is not padded to a 128-row tile.
    // A launch whose requests all hold the same number of tokens as far as the host can tell
    // (tokens = requests x q, q within one row tile, more than 16 rows each: a drafter or wide
    // verification step) has nothing for the integer kernel: the row-major kernel serves it
    // alone.  A shorter request hiding behind such numbers is still served, only on the taller tile.
    const char* why_rows = "";
    const bool tall = (int64_t)p.bq * p.group > 16;
    const int64_t q_each = p.num_reqs > 0 && p.num_tokens % p.num_reqs == 0 ? p.num_tokens / p.num_reqs : 0;
    const bool all_tall = q_each > 0 && q_each <= p.bq && q_each * p.group > pair_class_rows(p);
    *family = (tall && umma_rows_supports(p, &why_rows)) ? (i8_ok && !all_tall ? kFamilyPair : PTHB200_KERNEL_UMMA_ROWS)
              : i8_ok                                   ? PTHB200_KERNEL_UMMA
              : umma_ok                                 ? PTHB200_KERNEL_UMMA_BF16
                                                        : PTHB200_KERNEL_SCALAR;
  }
  return PTH_ATTN_OK;
}

int32_t attention_impl(const PthAttnArgs* a, const PthB200Options* opt, void* stream, bool launch,
                       int32_t* kernels = nullptr) {
  g_last_error.clear();
  KernelParams p;
  if (int32_t rc = build_attention(a, opt, &p)) return rc;
  int32_t family = 0;
  if (int32_t rc = choose_family(p, opt, &family)) return rc;
  if (kernels != nullptr) *kernels = family == kFamilyPair ? 2 : 1;
  if (!launch) return PTH_ATTN_OK;
  cudaError_t err;
  if (family == kFamilyPair) {
    KernelParams ps = p;
    ps.row_class = 1;
    ps.class_rows = pair_class_rows(p);
    err = launch_umma_i8_attention(ps, static_cast<cudaStream_t>(stream));
    if (err == cudaSuccess) {
      ps.row_class = 2;
      err = launch_umma_rows_attention(ps, static_cast<cudaStream_t>(stream));
    }
  } else if (family == PTHB200_KERNEL_UMMA) {
    err = launch_umma_i8_attention(p, static_cast<cudaStream_t>(stream));
  } else if (family == PTHB200_KERNEL_UMMA_ROWS) {
    err = launch_umma_rows_attention(p, static_cast<cudaStream_t>(stream));
  } else if (family == PTHB200_KERNEL_UMMA_BF16) {
    err = launch_umma_attention(p, static_cast<cudaStream_t>(stream));
  } else {
    PTHB_REQUIRE((int64_t)p.num_q_tiles <= 0x7fffffff, "too many row tiles");
    err = launch_scalar_attention(p, static_cast<cudaStream_t>(stream));
  }
  if (err != cudaSuccess) return fail(PTH_ATTN_ECUDA, std::string("attention launch failed: ") + cudaGetErrorString(err));
  return PTH_ATTN_OK;
}

int32_t combine_impl(const PthAttnCombineArgs* a, const PthB200Options* opt, void* stream, bool launch = true) {
  g_last_error.clear();
  PTHB_REQUIRE(a != nullptr, "args is NULL");
  PTHB_REQUIRE(a->abi_version == PTH_ATTN_ABI_VERSION, "args.abi_version does not match the library");
  PTHB_REQUIRE(a->struct_bytes == (int32_t)sizeof(PthAttnCombineArgs), "args.struct_bytes != sizeof(PthAttnCombineArgs)");
  if (int32_t rc = check_options(opt)) return rc;
  PTHB_REQUIRE(is_head_size(a->head_size), "head_size must be 64, 128 or 256");
  PTHB_REQUIRE(a->num_reqs >= 1 && a->num_tokens >= 1 && a->num_q_heads >= 1, "num_reqs, num_tokens and num_q_heads must be >= 1");
  PTHB_REQUIRE(a->num_splits >= 1, "num_splits must be >= 1");
  PTHB_REQUIRE(a->ws_o != nullptr && a->ws_lse != nullptr && a->out != nullptr && a->query_start_loc != nullptr,
               "ws_o, ws_lse, out and query_start_loc must not be NULL");
  PTHB_REQUIRE(a->out_dtype == PTH_ATTN_F32 || a->out_dtype == PTH_ATTN_F16 || a->out_dtype == PTH_ATTN_BF16,
               "out_dtype must be F32, F16 or BF16");
  PTHB_REQUIRE(aligned(a->ws_o, 16) && aligned(a->out, 16), "ws_o and out must be 16-byte aligned");
  PTHB_REQUIRE(a->ws_o_stride_split % 16 == 0 && a->ws_o_stride_token % 16 == 0 && a->ws_o_stride_head % 16 == 0,
               "ws_o byte strides must be multiples of 16");
  PTHB_REQUIRE(a->out_stride_token % 16 == 0 && a->out_stride_head % 16 == 0, "out byte strides must be multiples of 16");
  PTHB_REQUIRE(aligned(a->ws_lse, 4) && a->ws_lse_stride_split % 4 == 0 && a->ws_lse_stride_token % 4 == 0 &&
                   a->ws_lse_stride_head % 4 == 0,
               "ws_lse must be 4-byte aligned with strides that are multiples of 4");
  PTHB_REQUIRE(a->ws_o_stride_split >= 0 && a->ws_o_stride_token >= 0 && a->ws_o_stride_head >= 0 &&
                   a->ws_lse_stride_split >= 0 && a->ws_lse_stride_token >= 0 && a->ws_lse_stride_head >= 0 &&
                   a->out_stride_token >= 0 && a->out_stride_head >= 0,
               "strides must be >= 0");
  CombineParams c{};
  c.ws_o = a->ws_o;
  c.ws_o_stride_split = a->ws_o_stride_split;
  c.ws_o_stride_token = a->ws_o_stride_token;
  c.ws_o_stride_head = a->ws_o_stride_head;
  c.ws_lse = a->ws_lse;
  c.ws_lse_stride_split = a->ws_lse_stride_split;
  c.ws_lse_stride_token = a->ws_lse_stride_token;
  c.ws_lse_stride_head = a->ws_lse_stride_head;
  c.out = static_cast<uint8_t*>(a->out);
  c.out_stride_token = a->out_stride_token;
  c.out_stride_head = a->out_stride_head;
  if (opt != nullptr && opt->lse_out != nullptr) {
    c.lse_out = opt->lse_out;
    c.lse_stride_token = opt->lse_stride_token;
    c.lse_stride_head = opt->lse_stride_head;
  }
  c.query_start_loc = a->query_start_loc;
  c.out_dtype = a->out_dtype;
  c.num_reqs = a->num_reqs;
  c.num_tokens = a->num_tokens;
  c.num_q_heads = a->num_q_heads;
  c.head_size = a->head_size;
  c.num_splits = a->num_splits;
  if (!launch) return PTH_ATTN_OK;
  const cudaError_t err = launch_combine_kernel(c, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(PTH_ATTN_ECUDA, std::string("combine launch failed: ") + cudaGetErrorString(err));
  return PTH_ATTN_OK;
}

int32_t wm_for_rows(int32_t rows) {
  int32_t wm = 1;
  while (wm < 4 && rows > 16 * wm) wm *= 2;
  return wm;
}

}  // namespace
}  // namespace pthb200

extern "C" {

int32_t pthb200_abi_version(void) { return PTH_ATTN_ABI_VERSION; }
int32_t pthb200_attn_args_bytes(void) { return (int32_t)sizeof(PthAttnArgs); }
int32_t pthb200_combine_args_bytes(void) { return (int32_t)sizeof(PthAttnCombineArgs); }
int32_t pthb200_options_bytes(void) { return (int32_t)sizeof(PthB200Options); }
int32_t pthb200_has_cuda(void) { return 1; }
const char* pthb200_last_error(void) { return pthb200::g_last_error.c_str(); }

int32_t pthb200_attention(const PthAttnArgs* args, void* stream) {
  return pthb200::attention_impl(args, nullptr, stream, true);
}
int32_t pthb200_attention_ex(const PthAttnArgs* args, const PthB200Options* options, void* stream) {
  return pthb200::attention_impl(args, options, stream, true);
}
int32_t pthb200_combine(const PthAttnCombineArgs* args, void* stream) {
  return pthb200::combine_impl(args, nullptr, stream);
}
int32_t pthb200_combine_ex(const PthAttnCombineArgs* args, const PthB200Options* options, void* stream) {
  return pthb200::combine_impl(args, options, stream);
}

// Rows of a tile planned with `wm`: 16 * wm.  The tile holds floor(16 wm / G)
// tokens, or max_query_len tokens when that is fewer and still needs this wm.
int32_t pthb200_tile_tokens(int32_t wm, int32_t group, int32_t max_query_len) {
  if (!(wm == 1 || wm == 2 || wm == 4) || group < 1 || group > 16 * wm) return -1;
  const int32_t capacity = 16 * wm / group;
  int32_t bq = capacity;
  if (max_query_len >= 1 && max_query_len < capacity && pthb200::wm_for_rows(max_query_len * group) == wm) {
    bq = max_query_len;
  }
  return pthb200::wm_for_rows(bq * group) == wm ? bq : -1;
}

int32_t pthb200_check_call(const PthAttnArgs* args) { return pthb200::attention_impl(args, nullptr, nullptr, false); }

int32_t pthb200_launch_count(const PthAttnArgs* args, int32_t* attention_kernels, int32_t* combine_kernels) {
  int32_t kernels = 0;
  const int32_t rc = pthb200::attention_impl(args, nullptr, nullptr, false, &kernels);
  if (rc != PTH_ATTN_OK) return rc;
  if (attention_kernels) *attention_kernels = kernels;  // 2: short requests and tall ones on their own kernels
  if (combine_kernels) *combine_kernels = args->num_splits > 1 ? 1 : 0;
  return PTH_ATTN_OK;
}

int32_t pthb200_copy_ceiling(const PthAttnArgs* args, void* stream) {
  using namespace pthb200;
  g_last_error.clear();
  KernelParams p;
  if (int32_t rc = build_attention(args, nullptr, &p)) return rc;
  const char* why = "";
  PTHB_REQUIRE(umma_i8_supports(p, &why), std::string("the paged-copy ceiling follows the integer kernel, which does not apply: ") + why);
  PTHB_REQUIRE(p.head_size == 128, "the paged-copy ceiling is built for head size 128");
  const cudaError_t err = launch_copy_ceiling(p, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(PTH_ATTN_ECUDA, std::string("copy launch failed: ") + cudaGetErrorString(err));
  return PTH_ATTN_OK;
}

int32_t pthb200_write_args_bytes(void) { return (int32_t)sizeof(PthB200WriteArgs); }

int32_t pthb200_write_kv(const PthB200WriteArgs* a, void* stream) {
  using namespace pthb200;
  g_last_error.clear();
  PTHB_REQUIRE(a != nullptr, "args is NULL");
  PTHB_REQUIRE(a->abi_version == PTH_ATTN_ABI_VERSION, "args.abi_version does not match the library");
  PTHB_REQUIRE(a->struct_bytes == (int32_t)sizeof(PthB200WriteArgs), "args.struct_bytes != sizeof(PthB200WriteArgs)");
  PTHB_REQUIRE(is_head_size(a->head_size), "head_size must be 64, 128 or 256");
  PTHB_REQUIRE(a->num_kv_heads >= 1 && a->block_size >= 1 && a->num_blocks >= 1, "num_kv_heads, block_size and num_blocks must be >= 1");
  PTHB_REQUIRE(a->num_tokens >= 0, "num_tokens must be >= 0");
  PTHB_REQUIRE(a->src_dtype == PTH_ATTN_F32 || a->src_dtype == PTH_ATTN_F16 || a->src_dtype == PTH_ATTN_BF16,
               "src_dtype must be F32, F16 or BF16");
  if (a->num_tokens == 0) return PTH_ATTN_OK;
  PTHB_REQUIRE(a->key != nullptr && a->value != nullptr && a->slot_mapping != nullptr,
               "key, value and slot_mapping must not be NULL");
  const int64_t elem = a->src_dtype == PTH_ATTN_F32 ? 4 : 2;
  PTHB_REQUIRE(aligned(a->key, elem) && aligned(a->value, elem) && a->key_stride_token % elem == 0 &&
                   a->key_stride_head % elem == 0 && a->value_stride_token % elem == 0 &&
                   a->value_stride_head % elem == 0,
               "key / value must be aligned to their element size");
  PTHB_REQUIRE(aligned(a->slot_mapping, 8), "slot_mapping must be 8-byte aligned");
  if (int32_t rc = check_stream(a->k_cache, "k_cache")) return rc;
  if (int32_t rc = check_stream(a->v_cache, "v_cache")) return rc;
  if (int32_t rc = check_stream(a->k_scale, "k_scale")) return rc;
  if (int32_t rc = check_stream(a->v_scale, "v_scale")) return rc;
  const cudaError_t err = launch_kv_writer(*a, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(PTH_ATTN_ECUDA, std::string("writer launch failed: ") + cudaGetErrorString(err));
  return PTH_ATTN_OK;
}

// Host restatement of the persistent kernel's work-item schedule, built from the same
// functions the device runs (sched.cuh): the items each of `num_ctas` CTAs would run, in
// the order it would run them.
int32_t pthb200_test_schedule(const int32_t* query_start_loc, const int32_t* seq_lens, int32_t num_reqs,
                              int32_t group, int32_t num_kv_heads, int32_t bq, int32_t num_splits, int32_t window,
                              int32_t causal, int32_t row_class, int32_t class_rows, int32_t num_ctas, int32_t* out,
                              int32_t max_items) {
  using namespace pthb200;
  g_last_error.clear();
  PTHB_REQUIRE(query_start_loc != nullptr && seq_lens != nullptr && out != nullptr, "NULL argument");
  PTHB_REQUIRE(num_reqs >= 1 && group >= 1 && num_kv_heads >= 1 && bq >= 1 && num_splits >= 1 && num_ctas >= 1 &&
                   max_items >= 0,
               "counts must be >= 1");
  SchedShape sh{group, num_kv_heads, bq, num_splits, window, causal, row_class, class_rows};
  unsigned long long total = 0;
  for (int r = 0; r < num_reqs; ++r) {
    const int q_len = query_start_loc[r + 1] - query_start_loc[r];
    total += (unsigned long long)req_row_tiles(sh, q_len) * (unsigned long long)req_kv_tiles(sh, q_len, seq_lens[r]);
  }
  const int t_star = item_tiles(total * (unsigned long long)num_kv_heads, num_ctas);
  int32_t count = 0;
  for (int cta = 0; cta < num_ctas; ++cta) {
    int r = 0;
    long long first = 0;  // item index of request r's first item
    for (long long idx = cta;; idx += num_ctas) {
      int q_len = 0, splits = 1;
      long long n = 0;
      for (; r < num_reqs; ++r) {
        q_len = query_start_loc[r + 1] - query_start_loc[r];
        splits = req_splits(req_kv_tiles(sh, q_len, seq_lens[r]), t_star, num_splits);
        n = req_items(req_row_tiles(sh, q_len), splits, num_kv_heads);
        if (idx < first + n) break;
        first += n;
      }
      if (r >= num_reqs) break;
      const ItemCoord c = item_coord((int)(idx - first), num_kv_heads, splits);
      const int first_idx = c.row_tile * bq;
      const int ntok = sched_min(bq, q_len - first_idx);
      int lo0, hi0, lo1, hi1, tb, te;
      visible_bounds(window, causal, seq_lens[r], q_len, first_idx, &lo0, &hi0);
      visible_bounds(window, causal, seq_lens[r], q_len, first_idx + ntok - 1, &lo1, &hi1);
      split_tile_span(lo0, sched_max(hi0, hi1) + 1, c.split, splits, &tb, &te);
      if (count < max_items) {
        int32_t* o = out + (int64_t)count * 8;
        o[0] = cta;
        o[1] = r;
        o[2] = c.row_tile;
        o[3] = c.kvh;
        o[4] = c.split;
        o[5] = splits;
        o[6] = tb;
        o[7] = te;
      }
      ++count;
    }
  }
  return count;
}

}  // extern "C"

// ---- split attention without a caller workspace ---------------------------------
//
// pthb200_attention_noalloc runs attention + combine like the two calls above, but keeps
// the split partials in a fixed array inside this library instead of a workspace the
// caller allocated.  The array belongs to the loaded module (one instance per device),
// so the call performs no allocation of any kind.
//
// Nothing in the array has to start at zero: every partial (o and log-sum-exp) that the
// combine of a call reads is written by the attention launch of the same call, including
// the "-inf, no keys" marker of an empty split, so stale bytes of an earlier call are
// never read.  All calls on a device share the one array: two calls whose kernels may
// overlap (different streams, or different host threads without ordering between them)
// race on it.

#include <mutex>

// Capacity of the built-in array: split partials of one call, o and lse, fp32.
#define PTHB200_BUILTIN_WS_BYTES (8u * 1024u * 1024u)
static __device__ __align__(256) unsigned char g_pthb200_builtin_ws[PTHB200_BUILTIN_WS_BYTES];

namespace pthb200 {
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_builtin_ws_mutex;
unsigned char* g_builtin_ws_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device (cudaGetDevice), not on the device
// that owns `stream`: the caller makes the stream's device current before the call, as for
// every launch.  Looked up once per device (the lookup may load the module on that device,
// which is why a first call belongs before any stream capture); later calls only read the
// cached pointer.
int32_t builtin_ws(unsigned char** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(PTH_ATTN_ECUDA, std::string("cudaGetDevice failed: ") + cudaGetErrorString(err));
  PTHB_REQUIRE(dev >= 0 && dev < kMaxDevices, "pthb200_attention_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_builtin_ws_mutex);
  if (g_builtin_ws_ptr[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    err = cudaGetSymbolAddress((void**)&ptr, g_pthb200_builtin_ws);
    if (err != cudaSuccess || ptr == nullptr) {
      return fail(PTH_ATTN_ECUDA, std::string("pthb200_attention_noalloc: cudaGetSymbolAddress failed: ") +
                                      cudaGetErrorString(err));
    }
    g_builtin_ws_ptr[dev] = ptr;
  }
  *out = g_builtin_ws_ptr[dev];
  return PTH_ATTN_OK;
}

}  // namespace
}  // namespace pthb200

extern "C" int32_t pthb200_attention_noalloc(const PthAttnArgs* args, void* stream) {
  using namespace pthb200;
  g_last_error.clear();
  PTHB_REQUIRE(args != nullptr, "args is NULL");
  PTHB_REQUIRE(args->abi_version == PTH_ATTN_ABI_VERSION, "args.abi_version does not match the library");
  PTHB_REQUIRE(args->struct_bytes == (int32_t)sizeof(PthAttnArgs), "args.struct_bytes != sizeof(PthAttnArgs)");
  if (args->num_splits <= 1) return attention_impl(args, nullptr, stream, true);  // no partials at all
  PTHB_REQUIRE(args->num_splits <= 65535, "num_splits must be in [1, 65535]");
  PTHB_REQUIRE(args->num_tokens >= 1 && args->num_q_heads >= 1 && is_head_size(args->head_size),
               "num_tokens and num_q_heads must be >= 1 and head_size 64, 128 or 256");
  // dense partials: o [S][T][Hq][D] fp32, then lse [S][T][Hq] fp32 at the next 256-byte boundary.
  // The products are taken step by step so that no intermediate can overflow: S * T < 2^47,
  // and a row count beyond the array's capacity in floats ends the sum early.
  const int64_t cap = (int64_t)PTHB200_BUILTIN_WS_BYTES;
  int64_t rows = (int64_t)args->num_splits * args->num_tokens;
  if (rows <= cap) rows *= args->num_q_heads;
  const int64_t o_bytes = rows <= cap ? (rows * args->head_size * 4 + 255) / 256 * 256 : 0;
  const int64_t need = rows <= cap ? o_bytes + rows * 4 : INT64_MAX;
  if (need > cap) {
    return fail(PTH_ATTN_EINVAL,
                "pthb200_attention_noalloc: the split partials of this call need " +
                    (need == INT64_MAX ? std::string("more than 2^63") : std::to_string(need)) +
                    " bytes (num_splits * num_tokens * num_q_heads * (head_size + 1) * 4), the built-in array holds " +
                    std::to_string(cap) + "; use fewer splits, or pthb200_attention with a workspace of your own");
  }
  unsigned char* ws = nullptr;
  if (int32_t rc = builtin_ws(&ws)) return rc;
  PthAttnArgs a = *args;
  a.ws_o = reinterpret_cast<float*>(ws);
  a.ws_o_stride_head = (int64_t)a.head_size * 4;
  a.ws_o_stride_token = a.ws_o_stride_head * a.num_q_heads;
  a.ws_o_stride_split = a.ws_o_stride_token * a.num_tokens;
  a.ws_lse = reinterpret_cast<float*>(ws + o_bytes);
  a.ws_lse_stride_head = 4;
  a.ws_lse_stride_token = (int64_t)4 * a.num_q_heads;
  a.ws_lse_stride_split = a.ws_lse_stride_token * a.num_tokens;
  PthAttnCombineArgs c{};
  c.abi_version = PTH_ATTN_ABI_VERSION;
  c.struct_bytes = (int32_t)sizeof(PthAttnCombineArgs);
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
  // every check of both launches first: a refusal must not leave half the work enqueued
  if (int32_t rc = attention_impl(&a, nullptr, nullptr, false)) return rc;
  if (int32_t rc = combine_impl(&c, nullptr, nullptr, false)) return rc;
  if (int32_t rc = attention_impl(&a, nullptr, stream, true)) return rc;
  return combine_impl(&c, nullptr, stream);
}
