"""The C ABI library loads without a GPU, exports every declared symbol, and refuses bad
arguments with messages that name the field (no device is touched by these calls)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from pth_flash_attn_b200 import capi

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    return capi.load_library()


def test_exports_every_declared_symbol(lib):
    header = (REPO / "include" / "pthb200_attn.h").read_text()
    declared = set(re.findall(r"\b(pthb200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(capi.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib.lib, name) is not None


def test_identity(lib):
    assert lib.lib.pthb200_abi_version() == 2
    assert lib.lib.pthb200_attn_args_bytes() == ctypes.sizeof(capi.PthAttnArgs)
    assert lib.lib.pthb200_combine_args_bytes() == ctypes.sizeof(capi.PthAttnCombineArgs)
    assert lib.has_cuda()
    assert lib.last_error() == ""


def test_struct_layout_matches_the_reference_mirror():
    # field order and sizes of the reference's ctypes mirror (ref_capi.py:49-119): 8-byte
    # pointers and int64 strides, int32 elsewhere; a change here breaks binary compatibility
    assert ctypes.sizeof(capi.PthAttnStream) == 32
    assert ctypes.sizeof(capi.PthAttnArgs) == 352
    assert ctypes.sizeof(capi.PthAttnCombineArgs) == 136
    assert capi.PthAttnArgs.k_cache.offset == 72 and capi.PthAttnArgs.window.offset == 344


def _valid_args():
    buf = np.zeros(1 << 16, dtype=np.uint8)
    base = (buf.ctypes.data + 255) & ~255
    a = capi.new_attn_args()
    a.q, a.q_dtype, a.q_stride_token, a.q_stride_head = base, capi.BF16, 8 * 128 * 2, 256
    a.out, a.out_dtype, a.out_stride_token, a.out_stride_head = base + 4096, capi.BF16, 8 * 128 * 2, 256
    for i, s in enumerate((a.k_cache, a.v_cache, a.k_scale, a.v_scale)):
        s.data, s.stride_block, s.stride_slot, s.stride_head = base + 8192 + 4 * i, 16 * 2 * 264, 2 * 264, 264
    a.num_blocks, a.block_size, a.num_kv_heads, a.head_size = 4, 16, 2, 128
    a.block_table, a.block_table_row_stride = base + 32768, 4
    a.seq_lens, a.query_start_loc = base + 33000, base + 33100
    a.num_reqs, a.num_tokens, a.num_q_heads, a.bq, a.num_splits = 1, 2, 8, 2, 1
    a.softmax_scale, a.window, a.causal = 0.088, 0, 1
    return a, buf


def test_check_call_accepts_a_valid_call(lib):
    a, keep = _valid_args()
    assert lib.check_call(a) == capi.OK, lib.last_error()
    assert lib.launch_count(a) == (1, 0)


@pytest.mark.parametrize("mutate,needle", [
    (lambda a: setattr(a, "abi_version", 1), "abi_version"),
    (lambda a: setattr(a, "struct_bytes", 8), "struct_bytes"),
    (lambda a: setattr(a, "head_size", 96), "head_size"),
    (lambda a: setattr(a, "num_q_heads", 7), "num_q_heads"),
    (lambda a: setattr(a, "bq", 0), "bq"),
    (lambda a: setattr(a, "num_splits", 0), "num_splits"),
    (lambda a: setattr(a, "softmax_scale", float("nan")), "softmax_scale"),
    (lambda a: setattr(a, "softmax_scale", 0.0), "softmax_scale"),
    (lambda a: setattr(a, "window", -1), "window"),
    (lambda a: setattr(a, "causal", 2), "causal"),
    (lambda a: setattr(a, "q_dtype", capi.F32), "q_dtype"),
    (lambda a: setattr(a, "q", a.q + 8), "q must be 16-byte aligned"),
    (lambda a: setattr(a, "q_stride_head", 250), "q byte strides"),
    (lambda a: setattr(a, "out", 0), "out is NULL"),
    (lambda a: setattr(a.k_cache, "data", a.k_cache.data + 1), "k_cache.data must be 4-byte aligned"),
    (lambda a: setattr(a.v_scale, "stride_slot", 522), "v_scale byte strides"),
    (lambda a: setattr(a, "num_splits", 2), "ws_o and ws_lse"),
    (lambda a: setattr(a, "seq_lens", 0), "seq_lens"),
])
def test_check_call_names_the_bad_field(lib, mutate, needle):
    a, keep = _valid_args()
    mutate(a)
    assert lib.check_call(a) == capi.EINVAL
    assert needle in lib.last_error(), lib.last_error()
    # a later valid call clears the message
    b, keep2 = _valid_args()
    assert lib.check_call(b) == capi.OK and lib.last_error() == ""


def test_tile_tokens_rule(lib):
    # floor(16 wm / G), or max_query_len when that is fewer and still needs this wm
    assert lib.tile_tokens(1, 4, 1) == 1
    assert lib.tile_tokens(1, 4, 16) == 4
    assert lib.tile_tokens(4, 4, 16) == 16
    assert lib.tile_tokens(4, 8, 2048) == 8
    assert lib.tile_tokens(4, 6, 300) == 10
    assert lib.tile_tokens(1, 6, 1) == 1
    assert lib.tile_tokens(4, 4, 1) == 16       # a short request keeps the planned capacity
    assert lib.tile_tokens(3, 4, 1) == -1 and lib.tile_tokens(1, 17, 1) == -1


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="not built"):
        capi.B200Lib(tmp_path / "libpthb200_attn.so")
