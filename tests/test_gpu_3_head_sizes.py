"""GPU parity of the integer tcgen05 kernel at head sizes 64 and 256.

The reference ships its tensor path for all three head sizes (csrc/pth_attn/instantiate_d64.cu,
instantiate_d256.cu; its grid sweeps D in tests/gpu/grid_cases.py); its production shape is
D = 256 with 6 query heads per KV head.  The cases here force the integer kernel
(``KERNEL_UMMA``: a launch it does not support fails instead of falling back) and hold it to
the same gate against the fp64 oracle as head size 128: decode, verification and drafter
shapes, split-KV partials, sliding windows and non-causal ranges, both page layouts and both
TMA paths (tensor-map boxes and bulk copies of a contiguous page run), fp16 queries, page
sizes that are multiples of 16, and row tiles up to what each head size holds (64 rows at
D = 64, 32 at D = 256).
"""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi
from tests.helpers import check_lse, check_out

pytestmark = pytest.mark.gpu


def _seeded(lens, qlens, Hq, Hkv, D, seed, block_size=16, **kw):
    c = orc.make_paged_cache(lens, Hkv, D, block_size, seed=seed, **kw)
    rng = np.random.default_rng(seed + 1)
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int64)
    return c, q, qsl


def _check(c, q, qsl, D, what, *, bq, S=1, window=0, causal=True, kernel=capi.KERNEL_UMMA, q_dtype=torch.bfloat16,
           out_dtype=torch.bfloat16):
    from tests.gpu_util import run_case

    scale = D ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale, window=window, causal=causal)
    res = run_case(c, q, qsl, scale, bq=bq, num_splits=S, window=window, causal=causal, kernel=kernel,
                   q_dtype=q_dtype, out_dtype=out_dtype)
    assert capi.load_library().device_status() == 0
    check_out(res["out"], ref.out, what=what)
    check_lse(res["lse"], ref.lse, what=what)
    assert res["tail_intact"]
    if S > 1:
        o, _ = orc.combine_partials(res["ws_o"], res["ws_lse"])
        # (fp32 partials; the bf16-P kernel rounds p * v_scale to 8 bits, which a row that sees a
        # single key shows in full: relative gate)
        check_out(o, ref.out, max_tol=1e-2, mean_tol=1e-3, what=what + " partials", relative=True)
    return res


@pytest.mark.parametrize("S", [1, 3])
@pytest.mark.parametrize("qlen,G,bq", [(1, 4, 1), (1, 6, 1), (4, 4, 4), (2, 8, 2), (1, 16, 1)])
@pytest.mark.parametrize("D", [64, 256])
def test_decode_and_verify_shapes(D, qlen, G, bq, S):
    lens = [1000, 257, 128, qlen + 2, 1]
    qlens = [qlen] * 4 + [1]
    c, q, qsl = _seeded(lens, qlens, 2 * G, 2, D, seed=300 + D + qlen + G)
    _check(c, q, qsl, D, f"D{D} q{qlen} G{G} S{S}", bq=bq, S=S)


@pytest.mark.parametrize("qlen,G,bq", [(16, 4, 16), (40, 8, 8), (8, 2, 8)])
def test_tall_row_tiles_at_64_dims(qlen, G, bq):
    """Row tiles of 16 to 64 rows (the instances with 32 and 64 padded rows)."""
    lens = [700, 300 + qlen, qlen]
    c, q, qsl = _seeded(lens, [qlen] * 3, 2 * G, 2, 64, seed=411 + qlen)
    _check(c, q, qsl, 64, f"D64 rows {bq * G}", bq=bq, S=2)


def test_prefill_chunk_at_256_dims_is_cut_into_row_tiles_of_32_rows():
    """A chunk of 37 tokens x 6 heads: the kernel lowers the tile height to five tokens."""
    lens = [500, 90]
    c, q, qsl = _seeded(lens, [37, 5], 12, 2, 256, seed=77)
    _check(c, q, qsl, 256, "D256 chunk", bq=8, S=1)
    _check(c, q, qsl, 256, "D256 chunk through the library's own choice", bq=8, S=2, kernel=capi.KERNEL_AUTO)


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("layout,Hkv", [("HND", 2), ("NHD", 1), ("NHD", 4)])
def test_layouts_reach_both_copy_paths(D, layout, Hkv):
    """HND pages and a single KV head are contiguous page runs (bulk copies, keys of a tile
    interleaved by cell alignment); NHD with several heads goes through the tensor map."""
    lens = [900, 130, 17]
    c, q, qsl = _seeded(lens, [2, 2, 2], 4 * Hkv, Hkv, D, seed=500 + D + Hkv, layout=layout)
    _check(c, q, qsl, D, f"D{D} {layout} Hkv{Hkv}", bq=2, S=2)


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("block_size", [32, 64, 128, 256, 816])
def test_page_sizes(D, block_size):
    """816 slots per page, 256 dims and 6 query heads per KV head is the reference's production
    shape (README.md:279-289)."""
    lens = [1000, 300]
    for layout in ("NHD", "HND"):
        c, q, qsl = _seeded(lens, [1, 3], 12, 2, D, seed=600 + block_size, block_size=block_size, layout=layout)
        _check(c, q, qsl, D, f"D{D} {layout} pages of {block_size}", bq=2, S=2)


@pytest.mark.parametrize("D", [64, 256])
def test_window_noncausal_and_padding(D):
    lens = [3000, 700]
    c, q, qsl = _seeded(lens, [4, 4], 8, 2, D, seed=700 + D, pad_page_bytes=64, storage_offset_bytes=8)
    _check(c, q, qsl, D, f"D{D} window", bq=4, S=3, window=512)
    _check(c, q, qsl, D, f"D{D} non-causal window", bq=4, S=1, window=300, causal=False)
    _check(c, q, qsl, D, f"D{D} non-causal", bq=4, S=2, causal=False)


@pytest.mark.parametrize("D", [64, 256])
def test_fp16_queries_and_fp32_output(D):
    lens = [1500, 64]
    c, q, qsl = _seeded(lens, [1, 1], 12, 2, D, seed=800 + D)
    q16 = q.astype(np.float16).astype(np.float32)
    _check(c, q16, qsl, D, f"D{D} fp16 q", bq=1, S=2, q_dtype=torch.float16, out_dtype=torch.float32)


@pytest.mark.parametrize("D", [64, 256])
def test_long_context_matches_the_cuda_core_kernel(D):
    """A context too long for a comfortable CPU oracle: every row against the CUDA-core kernel."""
    from tests.gpu_util import run_case

    lens = [40000, 8200, 33]
    c, q, qsl = _seeded(lens, [1, 1, 1], 12, 2, D, seed=900 + D, keep_sources=False)
    scale = D ** -0.5
    a = run_case(c, q, qsl, scale, bq=1, num_splits=7, kernel=capi.KERNEL_UMMA)
    b = run_case(c, q, qsl, scale, bq=1, num_splits=1, kernel=capi.KERNEL_SCALAR, out_dtype=torch.float32)
    assert capi.load_library().device_status() == 0
    check_out(a["out"], b["out"], what=f"D{D} long")
    check_lse(a["lse"], b["lse"], what=f"D{D} long")


@pytest.mark.parametrize("D", [64, 256])
def test_results_do_not_change_from_run_to_run(D):
    from tests.gpu_util import run_case

    lens = [5000, 2000, 777]
    c, q, qsl = _seeded(lens, [2, 2, 2], 12, 2, D, seed=1000 + D)
    first = None
    for _ in range(30):
        res = run_case(c, q, qsl, D ** -0.5, bq=2, num_splits=3, kernel=capi.KERNEL_UMMA)
        if first is None:
            first = res["out_bytes"].copy()
        assert (res["out_bytes"] == first).all()


def test_head_size_256_refuses_more_than_32_query_heads_per_kv_head():
    from tests.gpu_util import run_case

    c, q, qsl = _seeded([100], [1], 64, 1, 256, seed=5)
    with pytest.raises(Exception, match="row tile"):
        run_case(c, q, qsl, 256 ** -0.5, bq=1, kernel=capi.KERNEL_UMMA)
    # the library's own choice serves the launch on CUDA cores
    _check(c, q, qsl, 256, "G 64", bq=1, kernel=capi.KERNEL_AUTO)


@pytest.mark.parametrize("qlen,G,bq", [(1, 32, 1), (5, 6, 5), (8, 4, 8), (3, 8, 3)])
def test_row_tiles_of_17_to_32_rows_at_256_dims(qlen, G, bq):
    lens = [900, 300 + qlen, qlen]
    c, q, qsl = _seeded(lens, [qlen] * 3, 2 * G, 2, 256, seed=1200 + qlen)
    _check(c, q, qsl, 256, f"D256 rows {bq * G}", bq=bq, S=2)


# ---- the row-major kernel for 256 dims (tall row tiles: prefill chunks, wide verification) ----
@pytest.mark.parametrize("S", [1, 3])
@pytest.mark.parametrize("layout,block_size", [("NHD", 16), ("HND", 816), ("NHD", 64)])
def test_rows_kernel_at_256_dims_prefill_chunk(S, layout, block_size):
    """A prefill chunk longer than one 128-row tile, ragged ends, plus short requests."""
    lens = [700, 1500, 90, 64]
    qlens = [300, 37, 1, 64]
    c, q, qsl = _seeded(lens, qlens, 12, 2, 256, seed=1300 + block_size, block_size=block_size, layout=layout)
    _check(c, q, qsl, 256, f"rows256 {layout} {block_size} S{S}", bq=8, S=S, kernel=capi.KERNEL_UMMA_ROWS)


def test_rows_kernel_at_256_dims_window_noncausal_offset():
    lens = [3000, 700]
    c, q, qsl = _seeded(lens, [40, 40], 8, 2, 256, seed=1400, pad_page_bytes=64, storage_offset_bytes=8)
    _check(c, q, qsl, 256, "rows256 window", bq=8, S=2, window=512, kernel=capi.KERNEL_UMMA_ROWS)
    _check(c, q, qsl, 256, "rows256 non-causal", bq=8, S=1, causal=False, kernel=capi.KERNEL_UMMA_ROWS)
    _check(c, q, qsl, 256, "rows256 non-causal window", bq=8, S=1, window=300, causal=False, kernel=capi.KERNEL_UMMA_ROWS)


def test_mixed_launch_at_256_dims_runs_each_request_on_its_kernel():
    """Decode, narrow verification and prefill requests in one launch through the library's own
    choice: the integer kernel serves the short requests, the row-major kernel the tall ones."""
    lens = [5000, 800, 2000, 300, 1]
    qlens = [1, 2, 200, 64, 1]
    c, q, qsl = _seeded(lens, qlens, 12, 2, 256, seed=1500)
    lib = capi.load_library()
    _check(c, q, qsl, 256, "mixed D256", bq=10, S=1, kernel=capi.KERNEL_AUTO)
    _check(c, q, qsl, 256, "mixed D256 split", bq=10, S=4, kernel=capi.KERNEL_AUTO)


def test_rows_kernel_at_256_dims_is_deterministic():
    from tests.gpu_util import run_case

    lens = [4000, 900]
    c, q, qsl = _seeded(lens, [256, 100], 12, 2, 256, seed=1600)
    first = None
    for _ in range(20):
        res = run_case(c, q, qsl, 256 ** -0.5, bq=10, num_splits=2, kernel=capi.KERNEL_UMMA_ROWS)
        if first is None:
            first = res["out_bytes"].copy()
        assert (res["out_bytes"] == first).all()


# ---- the two-row-tile row-major kernel at 64 dims (every tall launch at that head size) ----
@pytest.mark.parametrize("S", [1, 3])
@pytest.mark.parametrize("layout,block_size", [("NHD", 16), ("HND", 816), ("NHD", 64)])
def test_rows_kernel_at_64_dims_prefill_chunk(S, layout, block_size):
    lens = [700, 1500, 90, 64]
    qlens = [300, 37, 1, 64]
    c, q, qsl = _seeded(lens, qlens, 16, 2, 64, seed=1700 + block_size, block_size=block_size, layout=layout)
    _check(c, q, qsl, 64, f"rows2 D64 {layout} {block_size} S{S}", bq=8, S=S, kernel=capi.KERNEL_UMMA_ROWS)


def test_rows_kernel_at_64_dims_window_noncausal_offset_and_mixed():
    lens = [3000, 700]
    c, q, qsl = _seeded(lens, [40, 40], 8, 2, 64, seed=1800, pad_page_bytes=64, storage_offset_bytes=8)
    _check(c, q, qsl, 64, "rows2 D64 window", bq=8, S=2, window=512, kernel=capi.KERNEL_UMMA_ROWS)
    _check(c, q, qsl, 64, "rows2 D64 non-causal", bq=8, S=1, causal=False, kernel=capi.KERNEL_UMMA_ROWS)
    lens = [5000, 800, 2000, 300, 1]
    qlens = [1, 2, 200, 64, 1]
    c, q, qsl = _seeded(lens, qlens, 16, 2, 64, seed=1900)
    _check(c, q, qsl, 64, "mixed D64", bq=10, S=1, kernel=capi.KERNEL_AUTO)
    _check(c, q, qsl, 64, "mixed D64 split", bq=10, S=4, kernel=capi.KERNEL_AUTO)
