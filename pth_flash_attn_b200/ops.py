"""Python entry point of the op ``pth_flash_attn::pth_flash_attn_fwd`` and its fake kernel.

Mirrors the reference module python/pth_flash_attn/ops.py (same schema string,
same wrapper signature, same behaviour when the library is missing): the op is
C++ (``csrc/torch_op.cpp``, libtorch stable ABI) over the C ABI of
``libpthb200_attn.so``; this module loads ``_C.abi3.so``, registers the fake
(meta) kernel that ``torch.compile`` traces, and exposes typed wrappers.

The fake kernel returns ``None`` (the op is an out-variant) after running the
metadata checks of the C++ op in the same order with the same messages, so a bad
call fails at trace time with the reason it would fail with at run time.  Checks
that need addresses or a device stay in C++.

This module makes no ``torch.cuda`` call.
"""

from __future__ import annotations

import math
from pathlib import Path

import torch

OP_NAMESPACE = "pth_flash_attn"
OP_NAME = "pth_flash_attn_fwd"
OP_QUALNAME = f"{OP_NAMESPACE}::{OP_NAME}"
OP_SCHEMA = (
    "pth_flash_attn_fwd(Tensor! out, Tensor q, Tensor k_cache, "
    "Tensor v_cache, Tensor k_scale, Tensor v_scale, Tensor block_table, "
    "Tensor seq_lens, Tensor query_start_loc, int max_query_len, int wm, "
    "int num_splits, float softmax_scale, Tensor! ws_o, Tensor! ws_lse, "
    "int window=0, bool causal=True) -> ()"
)
LSE_OP_QUALNAME = f"{OP_NAMESPACE}::pth_flash_attn_fwd_lse"
LIBRARY_PATH = Path(__file__).with_name("_C.abi3.so")

_NAMES = {
    torch.bfloat16: "bfloat16",
    torch.float16: "float16",
    torch.float32: "float32",
    torch.int8: "int8",
    torch.int32: "int32",
    torch.int64: "int64",
}


class _Check:
    """The C++ checks, one static method per kind, raising the same text."""

    @staticmethod
    def fail(*parts: object) -> None:
        raise RuntimeError("pth_flash_attn_fwd: " + "".join(str(x) for x in parts))

    @staticmethod
    def name(dtype: torch.dtype) -> str:
        return _NAMES.get(dtype, "an unsupported dtype")

    @classmethod
    def rank(cls, t: torch.Tensor, want: int, name: str) -> None:
        if t.dim() != want:
            cls.fail(name, " must be ", want, "-D, got ", t.dim(), "-D")

    @classmethod
    def dtype(cls, t: torch.Tensor, want: torch.dtype, name: str) -> None:
        if t.dtype != want:
            cls.fail(name, " must be ", cls.name(want), ", got ", cls.name(t.dtype))

    @classmethod
    def size(cls, t: torch.Tensor, dim: int, want: int, name: str, what: str) -> None:
        if t.size(dim) != want:
            cls.fail(name, ".size(", dim, ") must equal ", what, " = ", want, ", got ", t.size(dim))

    @classmethod
    def unit_inner_stride(cls, t: torch.Tensor, name: str) -> None:
        if t.stride(-1) != 1:
            cls.fail(name, " must have stride 1 in its last dimension, got ", t.stride(-1))

    @classmethod
    def same_device(cls, t: torch.Tensor, q: torch.Tensor, name: str) -> None:
        if t.device != q.device:
            cls.fail(name, " must be on the same device as q")


def _fmt_float(x: float) -> str:
    # the C++ side streams a double: "nan", "inf", "0", "0.5" ...
    if math.isnan(x):
        return "nan"
    if math.isinf(x):
        return "inf" if x > 0 else "-inf"
    return f"{x:g}"


def _check_metadata(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc,
                    max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal) -> None:
    c = _Check
    c.rank(q, 3, "q")
    if q.dtype not in (torch.bfloat16, torch.float16):
        c.fail("q must be bfloat16 or float16, got ", c.name(q.dtype))
    T, Hq, D = q.size(0), q.size(1), q.size(2)
    if D not in (64, 128, 256):
        c.fail("head size D = q.size(2) must be 64, 128 or 256, got ", D)
    c.unit_inner_stride(q, "q")

    c.rank(out, 3, "out")
    c.dtype(out, q.dtype, "out (same dtype as q)")
    c.size(out, 0, T, "out", "T")
    c.size(out, 1, Hq, "out", "Hq")
    c.size(out, 2, D, "out", "D")
    c.unit_inner_stride(out, "out")

    c.rank(k_cache, 4, "k_cache")
    c.rank(v_cache, 4, "v_cache")
    c.dtype(k_cache, torch.int8, "k_cache")
    c.dtype(v_cache, torch.int8, "v_cache")
    NB, BS, Hkv = k_cache.size(0), k_cache.size(1), k_cache.size(2)
    c.size(k_cache, 3, D, "k_cache", "D")
    c.size(v_cache, 0, NB, "v_cache", "NB")
    c.size(v_cache, 1, BS, "v_cache", "BS")
    c.size(v_cache, 2, Hkv, "v_cache", "Hkv")
    c.size(v_cache, 3, D, "v_cache", "D")
    c.unit_inner_stride(k_cache, "k_cache")
    c.unit_inner_stride(v_cache, "v_cache")

    c.rank(k_scale, 3, "k_scale")
    c.rank(v_scale, 3, "v_scale")
    c.dtype(k_scale, torch.float32, "k_scale")
    c.dtype(v_scale, torch.float32, "v_scale")
    for t, name in ((k_scale, "k_scale"), (v_scale, "v_scale")):
        c.size(t, 0, NB, name, "NB")
        c.size(t, 1, BS, name, "BS")
        c.size(t, 2, Hkv, name, "Hkv")

    if Hkv < 1 or Hq % Hkv != 0:
        c.fail("Hq = ", Hq, " must be a positive multiple of Hkv = ", Hkv)
    G = Hq // Hkv
    if wm not in (1, 2, 4):
        c.fail("wm must be 1, 2 or 4, got ", wm)
    if G > 64:
        c.fail("G = Hq/Hkv = ", G, " exceeds the supported maximum ", 64)
    if G > 16 * wm:
        c.fail("G = Hq/Hkv = ", G, " must be <= 16*wm = ", 16 * wm)

    c.rank(block_table, 2, "block_table")
    c.rank(seq_lens, 1, "seq_lens")
    c.rank(query_start_loc, 1, "query_start_loc")
    c.dtype(block_table, torch.int32, "block_table")
    c.dtype(seq_lens, torch.int32, "seq_lens")
    c.dtype(query_start_loc, torch.int32, "query_start_loc")
    c.unit_inner_stride(block_table, "block_table")
    c.unit_inner_stride(seq_lens, "seq_lens")
    c.unit_inner_stride(query_start_loc, "query_start_loc")
    R = seq_lens.size(0)
    c.size(query_start_loc, 0, R + 1, "query_start_loc", "num_reqs + 1")
    if block_table.size(0) < R:
        c.fail("block_table has ", block_table.size(0), " rows, fewer than num_reqs = ", R)

    if not 0 <= max_query_len <= T:
        c.fail("max_query_len must be in [0, T = ", T, "], got ", max_query_len)
    if num_splits < 1:
        c.fail("num_splits must be >= 1, got ", num_splits)
    if not (math.isfinite(softmax_scale) and softmax_scale > 0.0):
        c.fail("softmax_scale must be finite and > 0, got ", _fmt_float(softmax_scale))
    if window < 0:
        c.fail("window must be >= 0, got ", window)
    if (window > 0 or not causal) and D != 128:
        c.fail("sliding-window and non-causal attention need head size D = 128, got ", D)

    for t, name in ((out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache"), (k_scale, "k_scale"),
                    (v_scale, "v_scale"), (block_table, "block_table"), (seq_lens, "seq_lens"),
                    (query_start_loc, "query_start_loc")):
        c.same_device(t, q, name)

    if num_splits > 1:
        c.rank(ws_o, 4, "ws_o")
        c.rank(ws_lse, 3, "ws_lse")
        c.dtype(ws_o, torch.float32, "ws_o")
        c.dtype(ws_lse, torch.float32, "ws_lse")
        if ws_o.size(0) < num_splits or ws_o.size(1) < T:
            c.fail("ws_o must have size(0) >= num_splits = ", num_splits, " and size(1) >= T = ", T,
                   ", got [", ws_o.size(0), ", ", ws_o.size(1), ", ...]")
        c.size(ws_o, 2, Hq, "ws_o", "Hq")
        c.size(ws_o, 3, D, "ws_o", "D")
        if ws_lse.size(0) < num_splits or ws_lse.size(1) < T:
            c.fail("ws_lse must have size(0) >= num_splits = ", num_splits, " and size(1) >= T = ", T,
                   ", got [", ws_lse.size(0), ", ", ws_lse.size(1), ", ...]")
        c.size(ws_lse, 2, Hq, "ws_lse", "Hq")
        c.unit_inner_stride(ws_o, "ws_o")
        c.unit_inner_stride(ws_lse, "ws_lse")
        c.same_device(ws_o, q, "ws_o")
        c.same_device(ws_lse, q, "ws_lse")


def pth_flash_attn_fwd_fake(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens,
                            query_start_loc, max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse,
                            window=0, causal=True) -> None:
    """Fake (meta) kernel: validate metadata like C++, write nothing, return None."""
    _check_metadata(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc,
                    max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal)


def pth_flash_attn_fwd_lse_fake(out, lse, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens,
                                query_start_loc, max_query_len, wm, num_splits, softmax_scale, ws_o,
                                ws_lse, window=0, causal=True) -> None:
    _check_metadata(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc,
                    max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal)
    _Check.rank(lse, 2, "lse")
    _Check.dtype(lse, torch.float32, "lse")
    _Check.size(lse, 0, q.size(0), "lse", "T")
    _Check.size(lse, 1, q.size(1), "lse", "Hq")
    _Check.same_device(lse, q, "lse")


def _load_library() -> bool:
    if not LIBRARY_PATH.is_file():
        return False
    torch.ops.load_library(str(LIBRARY_PATH))
    torch.library.register_fake(OP_QUALNAME)(pth_flash_attn_fwd_fake)
    torch.library.register_fake(LSE_OP_QUALNAME)(pth_flash_attn_fwd_lse_fake)
    return True


_LIBRARY_LOADED = _load_library()


def is_available() -> bool:
    """True if the op library was built and loaded (fake kernels registered)."""
    return _LIBRARY_LOADED


def _require_library() -> None:
    if not _LIBRARY_LOADED:
        raise RuntimeError(
            f"pth_flash_attn_fwd: op library {LIBRARY_PATH} is not built; run "
            "`python -m pth_flash_attn_b200.build` (there is no fallback implementation)"
        )


def pth_flash_attn_fwd(out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens,
                       query_start_loc, max_query_len: int, wm: int, num_splits: int,
                       softmax_scale: float, ws_o, ws_lse, window: int = 0, causal: bool = True) -> None:
    """Paged int8 attention for one launch, writing ``out`` in place (frozen schema).

    ``wm`` and ``num_splits`` come from :func:`planner.plan_launch`; ``ws_o`` / ``ws_lse`` are
    views of the caller's workspace of the plan's shapes (may be empty when ``num_splits == 1``).
    Allocates nothing, reads no device data on the host, does not synchronise.
    """
    _require_library()
    torch.ops.pth_flash_attn.pth_flash_attn_fwd.default(
        out, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc,
        max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal)


def pth_flash_attn_fwd_lse(out, lse, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens,
                           query_start_loc, max_query_len: int, wm: int, num_splits: int,
                           softmax_scale: float, ws_o, ws_lse, window: int = 0, causal: bool = True) -> None:
    """As :func:`pth_flash_attn_fwd`, also writing the natural-log log-sum-exp ``lse [T, Hq]`` fp32."""
    _require_library()
    torch.ops.pth_flash_attn.pth_flash_attn_fwd_lse.default(
        out, lse, q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, query_start_loc,
        max_query_len, wm, num_splits, softmax_scale, ws_o, ws_lse, window, causal)
