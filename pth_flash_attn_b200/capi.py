"""ctypes binding of ``libpthb200_attn.so`` (the C ABI declared in ``include/pthb200_attn.h``).

The struct mirrors below have the field order of the reference's launch structs
(csrc/pth_attn/attn_args.h:81-171; its own ctypes mirror is
python/pth_testing/ref_capi.py:38-119), so the same Python objects can be handed
to this library and to a library built from the reference.

There is no fallback: if the shared library has not been built,
:func:`load_library` raises.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

ABI_VERSION = 2
F32, F16, BF16 = 0, 1, 2
OK, EINVAL, ECUDA, ENOCUDA = 0, -1, -2, -3
KERNEL_AUTO, KERNEL_SCALAR, KERNEL_UMMA, KERNEL_UMMA_BF16, KERNEL_UMMA_ROWS = 0, 1, 2, 3, 4
# options.flags: no request has more than bq query tokens, so row tile x is request x
FLAG_ONE_TILE_PER_REQUEST = 1

LIBRARY_PATH = Path(__file__).with_name("libpthb200_attn.so")


class PthAttnStream(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("stride_block", ctypes.c_int64),
        ("stride_slot", ctypes.c_int64),
        ("stride_head", ctypes.c_int64),
    ]


class PthAttnArgs(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_int32),
        ("struct_bytes", ctypes.c_int32),
        ("q", ctypes.c_void_p),
        ("q_dtype", ctypes.c_int32),
        ("q_stride_token", ctypes.c_int64),
        ("q_stride_head", ctypes.c_int64),
        ("out", ctypes.c_void_p),
        ("out_dtype", ctypes.c_int32),
        ("out_stride_token", ctypes.c_int64),
        ("out_stride_head", ctypes.c_int64),
        ("k_cache", PthAttnStream),
        ("v_cache", PthAttnStream),
        ("k_scale", PthAttnStream),
        ("v_scale", PthAttnStream),
        ("num_blocks", ctypes.c_int32),
        ("block_size", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32),
        ("head_size", ctypes.c_int32),
        ("block_table", ctypes.c_void_p),
        ("block_table_row_stride", ctypes.c_int64),
        ("seq_lens", ctypes.c_void_p),
        ("query_start_loc", ctypes.c_void_p),
        ("num_reqs", ctypes.c_int32),
        ("num_tokens", ctypes.c_int32),
        ("num_q_heads", ctypes.c_int32),
        ("bq", ctypes.c_int32),
        ("num_q_tiles", ctypes.c_int32),
        ("num_splits", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("ws_o", ctypes.c_void_p),
        ("ws_o_stride_split", ctypes.c_int64),
        ("ws_o_stride_token", ctypes.c_int64),
        ("ws_o_stride_head", ctypes.c_int64),
        ("ws_lse", ctypes.c_void_p),
        ("ws_lse_stride_split", ctypes.c_int64),
        ("ws_lse_stride_token", ctypes.c_int64),
        ("ws_lse_stride_head", ctypes.c_int64),
        ("window", ctypes.c_int32),
        ("causal", ctypes.c_int32),
    ]


class PthAttnCombineArgs(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_int32),
        ("struct_bytes", ctypes.c_int32),
        ("ws_o", ctypes.c_void_p),
        ("ws_o_stride_split", ctypes.c_int64),
        ("ws_o_stride_token", ctypes.c_int64),
        ("ws_o_stride_head", ctypes.c_int64),
        ("ws_lse", ctypes.c_void_p),
        ("ws_lse_stride_split", ctypes.c_int64),
        ("ws_lse_stride_token", ctypes.c_int64),
        ("ws_lse_stride_head", ctypes.c_int64),
        ("out", ctypes.c_void_p),
        ("out_dtype", ctypes.c_int32),
        ("out_stride_token", ctypes.c_int64),
        ("out_stride_head", ctypes.c_int64),
        ("query_start_loc", ctypes.c_void_p),
        ("num_reqs", ctypes.c_int32),
        ("num_tokens", ctypes.c_int32),
        ("num_q_heads", ctypes.c_int32),
        ("head_size", ctypes.c_int32),
        ("num_splits", ctypes.c_int32),
    ]


class PthB200WriteArgs(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_int32),
        ("struct_bytes", ctypes.c_int32),
        ("key", ctypes.c_void_p),
        ("value", ctypes.c_void_p),
        ("src_dtype", ctypes.c_int32),
        ("key_stride_token", ctypes.c_int64),
        ("key_stride_head", ctypes.c_int64),
        ("value_stride_token", ctypes.c_int64),
        ("value_stride_head", ctypes.c_int64),
        ("k_cache", PthAttnStream),
        ("v_cache", PthAttnStream),
        ("k_scale", PthAttnStream),
        ("v_scale", PthAttnStream),
        ("num_blocks", ctypes.c_int32),
        ("block_size", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32),
        ("head_size", ctypes.c_int32),
        ("num_tokens", ctypes.c_int32),
        ("slot_mapping", ctypes.c_void_p),
    ]


class PthB200Options(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_int32),
        ("struct_bytes", ctypes.c_int32),
        ("kernel", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("lse_out", ctypes.c_void_p),
        ("lse_stride_token", ctypes.c_int64),
        ("lse_stride_head", ctypes.c_int64),
    ]


# Every symbol include/pthb200_attn.h declares (a test checks the library exports them all).
EXPORTED_SYMBOLS = (
    "pthb200_abi_version",
    "pthb200_attn_args_bytes",
    "pthb200_combine_args_bytes",
    "pthb200_options_bytes",
    "pthb200_has_cuda",
    "pthb200_last_error",
    "pthb200_attention",
    "pthb200_attention_ex",
    "pthb200_combine",
    "pthb200_combine_ex",
    "pthb200_attention_noalloc",
    "pthb200_copy_ceiling",
    "pthb200_write_args_bytes",
    "pthb200_write_kv",
    "pthb200_tile_tokens",
    "pthb200_check_call",
    "pthb200_launch_count",
    "pthb200_test_schedule",
    "pthb200_test_tile",
    "pthb200_test_tile_i8",
    "pthb200_test_tile_rows",
    "pthb200_device_status",
)


class B200Lib:
    """Loaded ``libpthb200_attn.so`` with typed entry points.

    Loading verifies the ABI version and the struct sizes against this mirror,
    so a stale mirror fails here instead of corrupting a launch.
    """

    def __init__(self, path: Path | str = LIBRARY_PATH) -> None:
        path = Path(path)
        if not path.is_file():
            raise RuntimeError(
                f"pth_flash_attn_b200: {path} is not built; run "
                "`python -m pth_flash_attn_b200.build` (needs nvcc). There is no fallback path."
            )
        self.path = path
        self.lib = ctypes.CDLL(str(path))
        lib = self.lib
        for name in ("pthb200_abi_version", "pthb200_attn_args_bytes",
                     "pthb200_combine_args_bytes", "pthb200_options_bytes", "pthb200_has_cuda"):
            getattr(lib, name).restype = ctypes.c_int32
            getattr(lib, name).argtypes = []
        lib.pthb200_last_error.restype = ctypes.c_char_p
        lib.pthb200_last_error.argtypes = []
        ap, cp, op = (ctypes.POINTER(PthAttnArgs), ctypes.POINTER(PthAttnCombineArgs),
                      ctypes.POINTER(PthB200Options))
        lib.pthb200_attention.restype = ctypes.c_int32
        lib.pthb200_attention.argtypes = [ap, ctypes.c_void_p]
        lib.pthb200_attention_ex.restype = ctypes.c_int32
        lib.pthb200_attention_ex.argtypes = [ap, op, ctypes.c_void_p]
        lib.pthb200_attention_noalloc.restype = ctypes.c_int32
        lib.pthb200_attention_noalloc.argtypes = [ap, ctypes.c_void_p]
        lib.pthb200_combine.restype = ctypes.c_int32
        lib.pthb200_combine.argtypes = [cp, ctypes.c_void_p]
        lib.pthb200_combine_ex.restype = ctypes.c_int32
        lib.pthb200_combine_ex.argtypes = [cp, op, ctypes.c_void_p]
        lib.pthb200_tile_tokens.restype = ctypes.c_int32
        lib.pthb200_tile_tokens.argtypes = [ctypes.c_int32] * 3
        lib.pthb200_check_call.restype = ctypes.c_int32
        lib.pthb200_check_call.argtypes = [ap]
        lib.pthb200_launch_count.restype = ctypes.c_int32
        lib.pthb200_launch_count.argtypes = [ap, ctypes.POINTER(ctypes.c_int32),
                                             ctypes.POINTER(ctypes.c_int32)]
        lib.pthb200_copy_ceiling.restype = ctypes.c_int32
        lib.pthb200_copy_ceiling.argtypes = [ap, ctypes.c_void_p]
        lib.pthb200_write_args_bytes.restype = ctypes.c_int32
        lib.pthb200_write_args_bytes.argtypes = []
        lib.pthb200_write_kv.restype = ctypes.c_int32
        lib.pthb200_write_kv.argtypes = [ctypes.POINTER(PthB200WriteArgs), ctypes.c_void_p]
        lib.pthb200_test_schedule.restype = ctypes.c_int32
        lib.pthb200_test_schedule.argtypes = ([ctypes.c_void_p] * 2 + [ctypes.c_int32] * 10
                                              + [ctypes.c_void_p, ctypes.c_int32])
        lib.pthb200_test_tile.restype = ctypes.c_int32
        lib.pthb200_test_tile.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int32, ctypes.c_void_p]
        lib.pthb200_test_tile_i8.restype = ctypes.c_int32
        lib.pthb200_test_tile_i8.argtypes = [ctypes.c_void_p] * 7
        lib.pthb200_test_tile_rows.restype = ctypes.c_int32
        lib.pthb200_test_tile_rows.argtypes = [ctypes.c_void_p] * 7
        lib.pthb200_device_status.restype = ctypes.c_int32
        lib.pthb200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
        if lib.pthb200_abi_version() != ABI_VERSION:
            raise RuntimeError(f"{path}: ABI {lib.pthb200_abi_version()} != mirror {ABI_VERSION}")
        if lib.pthb200_attn_args_bytes() != ctypes.sizeof(PthAttnArgs):
            raise RuntimeError(f"{path}: PthAttnArgs size differs from the ctypes mirror")
        if lib.pthb200_combine_args_bytes() != ctypes.sizeof(PthAttnCombineArgs):
            raise RuntimeError(f"{path}: PthAttnCombineArgs size differs from the ctypes mirror")
        if lib.pthb200_write_args_bytes() != ctypes.sizeof(PthB200WriteArgs):
            raise RuntimeError(f"{path}: PthB200WriteArgs size differs from the ctypes mirror")
        if lib.pthb200_options_bytes() != ctypes.sizeof(PthB200Options):
            raise RuntimeError(f"{path}: PthB200Options size differs from the ctypes mirror")

    def has_cuda(self) -> bool:
        return bool(self.lib.pthb200_has_cuda())

    def last_error(self) -> str:
        return self.lib.pthb200_last_error().decode()

    def attention(self, args: PthAttnArgs, *, options: PthB200Options | None = None,
                  stream: int = 0) -> int:
        if options is None:
            return int(self.lib.pthb200_attention(ctypes.byref(args), stream or None))
        return int(self.lib.pthb200_attention_ex(ctypes.byref(args), ctypes.byref(options),
                                                 stream or None))

    def attention_noalloc(self, args: PthAttnArgs, *, stream: int = 0) -> int:
        """Attention + combine with the split partials in the library's built-in array."""
        return int(self.lib.pthb200_attention_noalloc(ctypes.byref(args), stream or None))

    def combine(self, args: PthAttnCombineArgs, *, options: PthB200Options | None = None,
                stream: int = 0) -> int:
        if options is None:
            return int(self.lib.pthb200_combine(ctypes.byref(args), stream or None))
        return int(self.lib.pthb200_combine_ex(ctypes.byref(args), ctypes.byref(options),
                                               stream or None))

    def copy_ceiling(self, args: PthAttnArgs, *, stream: int = 0) -> int:
        """The paged-copy ceiling of an attention launch: same bytes, same copies, no compute."""
        return int(self.lib.pthb200_copy_ceiling(ctypes.byref(args), stream or None))

    def write_kv(self, args: "PthB200WriteArgs", *, stream: int = 0) -> int:
        """Quantise and store the K / V rows of new tokens (the cache writer)."""
        return int(self.lib.pthb200_write_kv(ctypes.byref(args), stream or None))

    def tile_tokens(self, wm: int, group: int, max_query_len: int) -> int:
        return int(self.lib.pthb200_tile_tokens(wm, group, max_query_len))

    def check_call(self, args: PthAttnArgs) -> int:
        return int(self.lib.pthb200_check_call(ctypes.byref(args)))

    def device_status(self) -> int:
        v = ctypes.c_int32(0)
        rc = self.lib.pthb200_device_status(ctypes.byref(v))
        if rc != OK:
            raise RuntimeError("pthb200_device_status failed")
        return v.value

    def schedule(self, query_start_loc, seq_lens, *, group: int, num_kv_heads: int, bq: int,
                 num_splits: int, num_ctas: int, window: int = 0, causal: bool = True,
                 row_class: int = 0, class_rows: int = 0):
        """The persistent kernel's work-item schedule, computed on the host (no device access).

        Returns an int32 array ``[items, 8]`` of ``(cta, request, row tile, KV head, split,
        splits of the request, first KV tile, end KV tile)`` in the order the CTAs run them.
        """
        import numpy as np

        qsl = np.ascontiguousarray(query_start_loc, dtype=np.int32)
        lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        args = (qsl.ctypes.data, lens.ctypes.data, len(lens), group, num_kv_heads, bq, num_splits, window,
                int(causal), row_class, class_rows, num_ctas)
        probe = np.zeros((1, 8), dtype=np.int32)
        n = int(self.lib.pthb200_test_schedule(*args, probe.ctypes.data, 0))
        if n < 0:
            raise RuntimeError(self.last_error())
        out = np.zeros((max(n, 1), 8), dtype=np.int32)
        self.lib.pthb200_test_schedule(*args, out.ctypes.data, n)
        return out[:n]

    def launch_count(self, args: PthAttnArgs) -> tuple[int, int]:
        a, c = ctypes.c_int32(0), ctypes.c_int32(0)
        rc = self.lib.pthb200_launch_count(ctypes.byref(args), ctypes.byref(a), ctypes.byref(c))
        if rc != OK:
            raise RuntimeError(self.last_error())
        return a.value, c.value


_LIB: B200Lib | None = None


def load_library() -> B200Lib:
    """Return the process-wide :class:`B200Lib` (raises if the library is not built)."""
    global _LIB
    if _LIB is None:
        _LIB = B200Lib()
    return _LIB


def make_options(kernel: int = KERNEL_AUTO, flags: int = 0) -> PthB200Options:
    o = PthB200Options()
    o.abi_version = ABI_VERSION
    o.struct_bytes = ctypes.sizeof(PthB200Options)
    o.kernel = kernel
    o.flags = flags
    return o


def new_attn_args() -> PthAttnArgs:
    a = PthAttnArgs()
    a.abi_version = ABI_VERSION
    a.struct_bytes = ctypes.sizeof(PthAttnArgs)
    return a


def new_write_args() -> PthB200WriteArgs:
    a = PthB200WriteArgs()
    a.abi_version = ABI_VERSION
    a.struct_bytes = ctypes.sizeof(PthB200WriteArgs)
    return a


def new_combine_args() -> PthAttnCombineArgs:
    a = PthAttnCombineArgs()
    a.abi_version = ABI_VERSION
    a.struct_bytes = ctypes.sizeof(PthAttnCombineArgs)
    return a
