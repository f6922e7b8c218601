"""GPU parity of the tcgen05 kernel family (head size 128, bf16 queries)."""
import numpy as np
import pytest

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi
from tests.helpers import check_lse, check_out, load_golden
from tests.test_gpu_1_scalar import cache_from_golden

pytestmark = pytest.mark.gpu

GOLDEN_D128 = ["attn_decode", "attn_verify4", "attn_window_causal", "attn_window_noncausal",
               "attn_noncausal", "attn_mixed"]


KERNELS = [capi.KERNEL_UMMA, capi.KERNEL_UMMA_BF16, capi.KERNEL_UMMA_ROWS]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", GOLDEN_D128)
def test_golden_attention_umma(name, kernel):
    from tests.gpu_util import run_case

    g = load_golden(name)
    Hq, Hkv, D, window, causal = (int(v) for v in g["meta"])
    G = Hq // Hkv
    q = orc.f32_from_bf16_bits(g["q_bits"])
    c = cache_from_golden(g)
    bq = max(1, min(64 // G, int(np.diff(g["qsl"]).max())))
    res = run_case(c, q, g["qsl"], float(g["softmax_scale"]), bq=bq, window=window,
                   causal=bool(causal), kernel=kernel)
    assert capi.load_library().device_status() == 0
    valid = g["valid"]
    check_out(res["out"], g["out"], valid, what=name)
    assert res["tail_intact"]
    assert (res["out_bytes"][~valid] == 0xFF).all(), "rows of no request were written"
    check_lse(np.where(valid[:, None], res["lse"], -np.inf), g["lse"], what=name)


def _seeded(lens, qlens, Hq, Hkv, seed, **kw):
    c = orc.make_paged_cache(lens, Hkv, 128, 16, seed=seed, **kw)
    rng = np.random.default_rng(seed + 1)
    T = sum(qlens)
    q = orc.round_to_bf16(rng.standard_normal((T, Hq, 128), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int64)
    return c, q, qsl


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("S", [1, 2, 5])
@pytest.mark.parametrize("qlen,G,bq", [(1, 4, 1), (4, 4, 4), (16, 4, 16), (4, 8, 4), (40, 8, 8)])
def test_seeded_shapes(S, qlen, G, bq, kernel):
    """Decode, verify, drafter and a short prefill chunk, with and without split-KV."""
    from tests.gpu_util import run_case

    lens = [1000, 257, 128, qlen + 2]
    qlens = [qlen] * 4
    c, q, qsl = _seeded(lens, qlens, 2 * G, 2, seed=50 + qlen + G)
    scale = 128 ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    res = run_case(c, q, qsl, scale, bq=bq, num_splits=S, kernel=kernel)
    assert capi.load_library().device_status() == 0
    check_out(res["out"], ref.out, what=f"S{S} q{qlen} G{G}")
    check_lse(res["lse"], ref.lse, what=f"S{S} q{qlen} G{G}")
    if S > 1:
        o, l2 = orc.combine_partials(res["ws_o"], res["ws_lse"])
        check_out(o, ref.out, max_tol=1e-2, mean_tol=1e-3, what="partials")


@pytest.mark.parametrize("layout,kernel", [("NHD", k) for k in KERNELS] + [("HND", capi.KERNEL_AUTO)])
def test_cache_that_starts_8_bytes_off_a_16_byte_boundary(kernel, layout):
    """Cells are 8-byte aligned, the page copies 16-byte aligned: with the cache 8 bytes off,
    the first head's cells are the odd ones and the last head's cell ends 8 bytes after the
    slot stride counted from the copy's first byte.  (Contiguous page runs that are not 16-byte
    aligned are refused by the TMA kernels: the library's own choice serves them elsewhere.)"""
    from tests.gpu_util import run_case

    lens, qlens = [700, 130, 20], [4, 4, 4]
    c = orc.make_paged_cache(lens, 2, 128, 16, layout=layout, pad_page_bytes=64, seed=31, storage_offset_bytes=8)
    rng = np.random.default_rng(32)
    q = orc.round_to_bf16(rng.standard_normal((12, 8, 128), dtype=np.float32))
    qsl = np.array([0, 4, 8, 12])
    ref = orc.ref_attention_paged(q, c, qsl, 128 ** -0.5)
    res = run_case(c, q, qsl, 128 ** -0.5, bq=4, num_splits=2, kernel=kernel)
    assert capi.load_library().device_status() == 0
    check_out(res["out"], ref.out, what=f"offset 8 {layout}")
    check_lse(res["lse"], ref.lse, what=f"offset 8 {layout}")


def test_matches_scalar_kernel_on_device():
    """The two kernel families agree on a case too large for a comfortable CPU oracle."""
    from tests.gpu_util import run_case

    lens = [20000, 4097, 33]
    c, q, qsl = _seeded(lens, [4, 4, 4], 32, 8, seed=77)
    scale = 128 ** -0.5
    a = run_case(c, q, qsl, scale, bq=4, num_splits=3, kernel=capi.KERNEL_UMMA)
    b = run_case(c, q, qsl, scale, bq=4, num_splits=1, kernel=capi.KERNEL_SCALAR, out_dtype=__import__("torch").float32)
    check_out(a["out"], b["out"], what="umma vs scalar")
    check_lse(a["lse"], b["lse"], what="umma vs scalar")


def test_window_drafter_long():
    from tests.gpu_util import run_case

    lens = [9000, 5000]
    c, q, qsl = _seeded(lens, [16, 16], 8, 2, seed=91)
    scale = 128 ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale, window=4096)
    res = run_case(c, q, qsl, scale, bq=16, num_splits=4, window=4096, kernel=capi.KERNEL_UMMA)
    check_out(res["out"], ref.out, what="window 4096")
    check_lse(res["lse"], ref.lse, what="window 4096")


@pytest.mark.parametrize("S", [1, 3])
def test_rows_kernel_prefill_chunk(S):
    """A prefill chunk longer than one 128-row tile, ragged ends, plus a decode request."""
    from tests.gpu_util import run_case

    lens = [700, 1500, 90]
    qlens = [300, 37, 1]
    c, q, qsl = _seeded(lens, qlens, 16, 2, seed=123)
    scale = 128 ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    res = run_case(c, q, qsl, scale, bq=8, num_splits=S, kernel=capi.KERNEL_UMMA_ROWS)
    assert capi.load_library().device_status() == 0
    check_out(res["out"], ref.out, what=f"rows prefill S{S}")
    check_lse(res["lse"], ref.lse, what=f"rows prefill S{S}")
    assert res["tail_intact"]


def test_rows_kernel_window_and_auto_choice():
    """Drafter-shaped launch (16 tokens, window) on the row-major kernel, and through AUTO."""
    from tests.gpu_util import run_case

    lens = [9000, 5000]
    c, q, qsl = _seeded(lens, [16, 16], 8, 2, seed=91)
    scale = 128 ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale, window=4096)
    for kernel in (capi.KERNEL_UMMA_ROWS, capi.KERNEL_AUTO):
        res = run_case(c, q, qsl, scale, bq=16, num_splits=2, window=4096, kernel=kernel)
        check_out(res["out"], ref.out, what="rows window 4096")
        check_lse(res["lse"], ref.lse, what="rows window 4096")


@pytest.mark.parametrize("kernel", [capi.KERNEL_SCALAR] + KERNELS + [capi.KERNEL_AUTO])
@pytest.mark.parametrize("qlens,bq,S", [([1, 1, 1, 1, 1], 1, 3), ([4, 1, 3, 4], 4, 1), ([16, 9, 16], 16, 2)])
def test_one_tile_per_request_flag_gives_the_same_bytes(qlens, bq, S, kernel):
    """The caller's promise that no request exceeds bq tokens only changes how a CTA finds its
    request (tile x = request x, no padded grid): outputs are byte-equal with and without it."""
    from tests.gpu_util import run_case

    lens = [700 + 300 * i for i in range(len(qlens))]
    c, q, qsl = _seeded(lens, qlens, 8, 2, seed=90 + bq)
    scale = 128 ** -0.5
    a = run_case(c, q, qsl, scale, bq=bq, num_splits=S, kernel=kernel)
    b = run_case(c, q, qsl, scale, bq=bq, num_splits=S, kernel=kernel, flags=capi.FLAG_ONE_TILE_PER_REQUEST)
    assert capi.load_library().device_status() == 0
    assert (a["out_bytes"] == b["out_bytes"]).all()
    assert np.array_equal(a["lse"], b["lse"])
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    check_out(b["out"], ref.out, what=f"flag q{qlens}")


@pytest.mark.parametrize("S", [1, 3])
@pytest.mark.parametrize("G", [4, 8])
def test_mixed_launch_runs_each_request_on_its_kernel(G, S):
    """Decode, verification and prefill requests in one launch: the automatic choice serves
    the requests of at most 16 rows with the integer kernel and the others with the row-major
    kernel, so each request's rows equal the bytes of the launch forced to that kernel (when
    the key range is not split; pieces are chosen per launch)."""
    from tests.gpu_util import run_case

    qlens = [1, 40, 16 // G, 1, 300, 16 // G + 1, 1]
    lens = [3000, 900, 2100, 64, 1500, 5000, 129]
    c, q, qsl = _seeded(lens, qlens, 2 * G, 2, seed=120 + G)
    scale = 128 ** -0.5
    bq = 64 // G
    auto = run_case(c, q, qsl, scale, bq=bq, num_splits=S)
    assert capi.load_library().device_status() == 0
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    check_out(auto["out"], ref.out, what=f"mixed G{G} S{S}")
    check_lse(auto["lse"], ref.lse, what=f"mixed G{G} S{S}")
    assert auto["tail_intact"]
    rows = run_case(c, q, qsl, scale, bq=bq, num_splits=S, kernel=capi.KERNEL_UMMA_ROWS)
    # the integer kernel alone, tiled as the mixed launch tiles its requests
    i8 = run_case(c, q, qsl, scale, bq=16 // G, num_splits=S, kernel=capi.KERNEL_UMMA)
    for r, ql in enumerate(qlens):
        sl = slice(int(qsl[r]), int(qsl[r + 1]))
        want = i8 if ql * G <= 16 else rows
        if S == 1:
            assert (auto["out_bytes"][sl] == want["out_bytes"][sl]).all(), (r, ql)
        else:
            # the kernels cut a request into pieces by the total work of the requests THEY serve,
            # which differs between the mixed launch and a launch forced to one kernel
            check_out(auto["out"][sl], want["out"][sl], max_tol=1e-2, mean_tol=1e-3, what=f"request {r}")


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("bs,kernel", [(32, capi.KERNEL_UMMA), (64, capi.KERNEL_UMMA), (128, capi.KERNEL_UMMA),
                                       (32, capi.KERNEL_UMMA_ROWS), (64, capi.KERNEL_UMMA_ROWS),
                                       (128, capi.KERNEL_UMMA_ROWS), (256, capi.KERNEL_UMMA), (256, capi.KERNEL_UMMA_ROWS),
                                       (528, capi.KERNEL_UMMA), (528, capi.KERNEL_UMMA_ROWS),
                                       (816, capi.KERNEL_UMMA), (816, capi.KERNEL_UMMA_ROWS),
                                       (864, capi.KERNEL_UMMA), (864, capi.KERNEL_UMMA_ROWS),
                                       (48, capi.KERNEL_UMMA), (48, capi.KERNEL_AUTO), (40, capi.KERNEL_AUTO)])
def test_other_page_sizes(bs, kernel, layout):
    """Every page size that is a multiple of 16 runs on the TMA page copies: a page is fetched
    in copies of 16 to 128 slots (the largest power of two that divides it), so the reference's
    production pages of 816 slots and its grid's 528 and 864 (tests/gpu/grid_cases.py:225-245)
    are 51, 33 and 27 copies; a tile of 128 keys may straddle two pages.  Other sizes are served
    by the kernels that gather key by key, chosen automatically."""
    from tests.gpu_util import run_case

    lens, qlens = [1500, 257, 40], [4, 4, 4]
    c = orc.make_paged_cache(lens, 2, 128, bs, layout=layout, seed=60 + bs)
    rng = np.random.default_rng(61)
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), 8, 128), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int64)
    scale = 128 ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    for S in (1, 3):
        res = run_case(c, q, qsl, scale, bq=4, num_splits=S, kernel=kernel)
        assert capi.load_library().device_status() == 0
        check_out(res["out"], ref.out, what=f"block size {bs} S{S}")
        check_lse(res["lse"], ref.lse, what=f"block size {bs} S{S}")
        assert res["tail_intact"]


def test_launch_count_of_tall_launches():
    """Tall row tiles: the integer kernel (short requests) and the row-major kernel (the others)
    one after the other, unless the launch's numbers leave no room for a short request.  (The
    count is computed without touching the pointers; it needs the driver's tensor-map encoder.)"""
    from tests.test_capi_cpu import _valid_args

    lib = capi.load_library()
    a, keep = _valid_args()
    cells = a.k_cache.data            # one cell per slot and head: K | k_scale | V | v_scale
    for s, off in ((a.k_cache, 0), (a.k_scale, 128), (a.v_cache, 132), (a.v_scale, 260)):
        s.data = cells + off
    a.bq, a.num_reqs, a.num_tokens = 16, 2, 31
    assert lib.launch_count(a) == (2, 0), lib.last_error()
    a.num_tokens = 32          # 2 requests x 16 tokens x 4 heads per KV head: 64 rows each
    assert lib.launch_count(a) == (1, 0), lib.last_error()
    a.num_tokens = 8           # 4 tokens each: 16 rows, the integer kernel's own
    assert lib.launch_count(a) == (2, 0), lib.last_error()
    a.bq, a.num_tokens = 4, 8  # short tiles
    assert lib.launch_count(a) == (1, 0), lib.last_error()
