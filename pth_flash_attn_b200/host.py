"""Host-side helpers over the C ABI for callers that hold torch tensors.

``attention_forward`` is the call the torch op makes in C++, restated for Python
callers that want the C ABI directly (tests, benchmarks, engines without the op
library): it fills :class:`PthAttnArgs` from tensor pointers and byte strides and
enqueues the attention kernel and, for ``num_splits > 1``, the combine on the
current CUDA stream of ``q``'s device.  It allocates nothing and does not
synchronise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import capi

_DTYPE_CODE = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}


@dataclass
class CacheViews:
    """The four cache streams as raw device pointers + byte strides (block, slot, head)."""

    k: tuple[int, int, int, int]
    v: tuple[int, int, int, int]
    ks: tuple[int, int, int, int]
    vs: tuple[int, int, int, int]
    num_blocks: int
    block_size: int
    num_kv_heads: int
    head_size: int

    @staticmethod
    def from_tensors(k_cache, v_cache, k_scale, v_scale) -> "CacheViews":
        def geom(t):
            es = t.element_size()
            return (t.data_ptr(), t.stride(0) * es, t.stride(1) * es, t.stride(2) * es)

        return CacheViews(geom(k_cache), geom(v_cache), geom(k_scale), geom(v_scale),
                          k_cache.shape[0], k_cache.shape[1], k_cache.shape[2], k_cache.shape[3])


def _set_stream(dst: capi.PthAttnStream, g: tuple[int, int, int, int]) -> None:
    dst.data, dst.stride_block, dst.stride_slot, dst.stride_head = g


def fill_attn_args(q, out, cache: CacheViews, block_table, seq_lens, query_start_loc, *, bq: int,
                   num_splits: int, softmax_scale: float, ws_o=None, ws_lse=None, window: int = 0,
                   causal: bool = True) -> capi.PthAttnArgs:
    a = capi.new_attn_args()
    es = q.element_size()
    a.q = q.data_ptr()
    a.q_dtype = _DTYPE_CODE[q.dtype]
    a.q_stride_token, a.q_stride_head = q.stride(0) * es, q.stride(1) * es
    if out is not None:
        a.out = out.data_ptr()
        a.out_dtype = _DTYPE_CODE[out.dtype]
        a.out_stride_token = out.stride(0) * out.element_size()
        a.out_stride_head = out.stride(1) * out.element_size()
    _set_stream(a.k_cache, cache.k)
    _set_stream(a.v_cache, cache.v)
    _set_stream(a.k_scale, cache.ks)
    _set_stream(a.v_scale, cache.vs)
    a.num_blocks, a.block_size = cache.num_blocks, cache.block_size
    a.num_kv_heads, a.head_size = cache.num_kv_heads, cache.head_size
    a.block_table = block_table.data_ptr()
    a.block_table_row_stride = block_table.stride(0)
    a.seq_lens = seq_lens.data_ptr()
    a.query_start_loc = query_start_loc.data_ptr()
    a.num_reqs = seq_lens.shape[0]
    a.num_tokens, a.num_q_heads = q.shape[0], q.shape[1]
    a.bq, a.num_q_tiles, a.num_splits = bq, 0, num_splits
    a.softmax_scale = softmax_scale
    a.window, a.causal = window, int(causal)
    if ws_o is not None and ws_lse is not None and num_splits > 1:
        a.ws_o = ws_o.data_ptr()
        a.ws_o_stride_split, a.ws_o_stride_token, a.ws_o_stride_head = (s * 4 for s in ws_o.stride()[:3])
        a.ws_lse = ws_lse.data_ptr()
        a.ws_lse_stride_split, a.ws_lse_stride_token, a.ws_lse_stride_head = (
            s * 4 for s in ws_lse.stride()[:3])
    return a


def fill_combine_args(a: capi.PthAttnArgs) -> capi.PthAttnCombineArgs:
    c = capi.new_combine_args()
    for name in ("ws_o", "ws_o_stride_split", "ws_o_stride_token", "ws_o_stride_head", "ws_lse",
                 "ws_lse_stride_split", "ws_lse_stride_token", "ws_lse_stride_head", "out",
                 "out_dtype", "out_stride_token", "out_stride_head", "query_start_loc", "num_reqs",
                 "num_tokens", "num_q_heads", "head_size", "num_splits"):
        setattr(c, name, getattr(a, name))
    return c


def attention_forward(q, out, cache: CacheViews, block_table, seq_lens, query_start_loc, *, bq: int,
                      num_splits: int, softmax_scale: float, ws_o=None, ws_lse=None, window: int = 0,
                      causal: bool = True, lse_out=None, kernel: int = capi.KERNEL_AUTO, flags: int = 0,
                      lib: capi.B200Lib | None = None) -> None:
    """Attention (+ combine when ``num_splits > 1``) on the current stream; raises on a refusal."""
    lib = lib or capi.load_library()
    a = fill_attn_args(q, out, cache, block_table, seq_lens, query_start_loc, bq=bq,
                       num_splits=num_splits, softmax_scale=softmax_scale, ws_o=ws_o, ws_lse=ws_lse,
                       window=window, causal=causal)
    opt = capi.make_options(kernel, flags)
    if lse_out is not None:
        opt.lse_out = lse_out.data_ptr()
        opt.lse_stride_token, opt.lse_stride_head = lse_out.stride(0) * 4, lse_out.stride(1) * 4
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        rc = lib.attention(a, options=opt, stream=stream)
        if rc != capi.OK:
            raise RuntimeError(f"pthb200_attention: {lib.last_error()} (code {rc})")
        if num_splits > 1:
            rc = lib.combine(fill_combine_args(a), options=opt, stream=stream)
            if rc != capi.OK:
                raise RuntimeError(f"pthb200_combine: {lib.last_error()} (code {rc})")


def combine_partials(ws_o, ws_lse, out, query_start_loc, *, lse_out=None, lib: capi.B200Lib | None = None) -> None:
    """Merges ``S`` pieces of every row (``ws_o [S, T, Hq, D]`` fp32, each normalised by its own
    sum; ``ws_lse [S, T, Hq]`` in log2 units, -inf for a piece without keys) into ``out`` on the
    current stream: the combine step on its own, for pieces that did not come from one launch."""
    lib = lib or capi.load_library()
    S, T, Hq, D = ws_o.shape
    c = capi.new_combine_args()
    c.ws_o = ws_o.data_ptr()
    c.ws_o_stride_split, c.ws_o_stride_token, c.ws_o_stride_head = (s * 4 for s in ws_o.stride()[:3])
    c.ws_lse = ws_lse.data_ptr()
    c.ws_lse_stride_split, c.ws_lse_stride_token, c.ws_lse_stride_head = (s * 4 for s in ws_lse.stride()[:3])
    c.out, c.out_dtype = out.data_ptr(), _DTYPE_CODE[out.dtype]
    c.out_stride_token = out.stride(0) * out.element_size()
    c.out_stride_head = out.stride(1) * out.element_size()
    c.query_start_loc = query_start_loc.data_ptr()
    c.num_reqs, c.num_tokens, c.num_q_heads, c.head_size, c.num_splits = query_start_loc.shape[0] - 1, T, Hq, D, S
    opt = capi.make_options()
    if lse_out is not None:
        opt.lse_out = lse_out.data_ptr()
        opt.lse_stride_token, opt.lse_stride_head = lse_out.stride(0) * 4, lse_out.stride(1) * 4
    with torch.cuda.device(out.device):
        rc = lib.combine(c, options=opt, stream=torch.cuda.current_stream(out.device).cuda_stream)
    if rc != capi.OK:
        raise RuntimeError(f"pthb200_combine: {lib.last_error()} (code {rc})")


def write_kv(key, value, cache: CacheViews, slot_mapping, *, lib: capi.B200Lib | None = None) -> None:
    """Quantise ``key`` / ``value`` ``[T, Hkv, D]`` into the cache at ``slot_mapping`` (int64 ``[T]``;
    negative = skip) on the current stream, exactly as the cache format's own writer does."""
    lib = lib or capi.load_library()
    a = capi.new_write_args()
    es = key.element_size()
    a.key, a.value, a.src_dtype = key.data_ptr(), value.data_ptr(), _DTYPE_CODE[key.dtype]
    a.key_stride_token, a.key_stride_head = key.stride(0) * es, key.stride(1) * es
    a.value_stride_token, a.value_stride_head = value.stride(0) * es, value.stride(1) * es
    _set_stream(a.k_cache, cache.k)
    _set_stream(a.v_cache, cache.v)
    _set_stream(a.k_scale, cache.ks)
    _set_stream(a.v_scale, cache.vs)
    a.num_blocks, a.block_size = cache.num_blocks, cache.block_size
    a.num_kv_heads, a.head_size = cache.num_kv_heads, cache.head_size
    a.num_tokens = key.shape[0]
    a.slot_mapping = slot_mapping.data_ptr()
    with torch.cuda.device(key.device):
        rc = lib.write_kv(a, stream=torch.cuda.current_stream(key.device).cuda_stream)
    if rc != capi.OK:
        raise RuntimeError(f"pthb200_write_kv: {lib.last_error()} (code {rc})")
