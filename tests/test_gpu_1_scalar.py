"""GPU parity of the CUDA-core kernel family against the oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi
from tests.helpers import check_lse, check_out, golden_dense, load_golden

pytestmark = pytest.mark.gpu

GOLDEN_ATTN = ["attn_decode", "attn_verify4", "attn_window_causal", "attn_window_noncausal",
               "attn_noncausal", "attn_mixed", "attn_d64_g6", "attn_d256_g6"]


def cache_from_golden(g, layout="NHD", pad=0, offset=0, seed=3):
    """Re-page the golden per-request ints/scales: dequantised sources re-quantise to the same
    bytes only approximately, so the cells are written directly."""
    from tests.gpu_util import CANARY  # noqa: F401

    Hq, Hkv, D = (int(v) for v in g["meta"][:3])
    lens = g["seq_lens"].tolist()
    c = orc.make_paged_cache(lens, Hkv, D, 16, layout, pad, seed=seed, storage_offset_bytes=offset)
    for r, L in enumerate(lens):
        if L == 0:
            continue
        pos = np.arange(L)
        blk = c.block_table[r].astype(np.int64)[pos // 16]
        sl = pos % 16
        c.k_cache[blk, sl] = g[f"k_int{r}"]
        c.v_cache[blk, sl] = g[f"v_int{r}"]
        c.k_scale[blk, sl] = g[f"k_scale{r}"]
        c.v_scale[blk, sl] = g[f"v_scale{r}"]
    return c


@pytest.mark.parametrize("name", GOLDEN_ATTN)
@pytest.mark.parametrize("kernel", [capi.KERNEL_SCALAR, capi.KERNEL_AUTO])
def test_golden_attention(name, kernel):
    from tests.gpu_util import run_case

    g = load_golden(name)
    Hq, Hkv, D, window, causal = (int(v) for v in g["meta"])
    G = Hq // Hkv
    q = orc.f32_from_bf16_bits(g["q_bits"])
    c = cache_from_golden(g)
    # verify the re-paged cache against the fixture before trusting the run
    for r, d in enumerate(golden_dense(g)):
        assert np.array_equal(c.dense(r).k_int, d.k_int)
    bq = max(1, min(16 // G if G <= 16 else 1, int(np.diff(g["qsl"]).max())))
    res = run_case(c, q, g["qsl"], float(g["softmax_scale"]), bq=bq, window=window,
                   causal=bool(causal), kernel=kernel)
    valid = g["valid"]
    # the d64/d256 fixtures use the reference's wide-range data (|v| up to ~18)
    check_out(res["out"], g["out"], valid, what=name, relative=name in ("attn_d64_g6", "attn_d256_g6"))
    # rows of an empty request / padding rows keep the canary; rows of requests are written
    assert res["tail_intact"]
    assert (res["out_bytes"][~valid] == 0xFF).all(), "rows of no request were written"
    lse = np.where(valid[:, None], res["lse"], -np.inf)
    check_lse(lse, g["lse"], what=name)


@pytest.mark.parametrize("S", [2, 3, 7])
def test_split_and_combine_scalar(S):
    from tests.gpu_util import run_case

    lens, qlens = [700, 129, 5], [3, 1, 2]
    Hq, Hkv, D = 8, 2, 128
    c = orc.make_paged_cache(lens, Hkv, D, 16, seed=41)
    rng = np.random.default_rng(42)
    T = sum(qlens)
    q = orc.round_to_bf16(rng.standard_normal((T, Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    scale = D ** -0.5
    ref = orc.ref_attention_paged(q, c, qsl, scale)
    res = run_case(c, q, qsl, scale, bq=4, num_splits=S, kernel=capi.KERNEL_SCALAR)
    check_out(res["out"], ref.out, what=f"S={S}")
    check_lse(res["lse"], ref.lse, what=f"S={S}")
    # partials merge to the same answer under the oracle's combine rule
    o, l2 = orc.combine_partials(res["ws_o"], res["ws_lse"])
    np.testing.assert_allclose(o, ref.out, atol=2e-5, rtol=1e-4)
    np.testing.assert_allclose(orc.log2_to_ln(l2), ref.lse, atol=1e-4)


@pytest.mark.parametrize("layout,pad,offset", [("HND", 0, 0), ("NHD", 72, 4), ("HND", 8, 12)])
def test_layouts_and_offsets(layout, pad, offset):
    from tests.gpu_util import run_case

    lens, qlens = [40, 0, 300], [2, 0, 1]
    Hq, Hkv, D = 4, 2, 128
    c = orc.make_paged_cache(lens, Hkv, D, 16, layout, pad, seed=5, storage_offset_bytes=offset)
    rng = np.random.default_rng(6)
    q = orc.round_to_bf16(rng.standard_normal((3, Hq, D), dtype=np.float32))
    qsl = [0, 2, 2, 3]
    ref = orc.ref_attention_paged(q, c, qsl, D ** -0.5)
    res = run_case(c, q, qsl, D ** -0.5, bq=2)
    check_out(res["out"], ref.out, what=layout)
    check_lse(res["lse"], ref.lse, what=layout)


@pytest.mark.parametrize("S,D", [(5, 128), (16, 128), (17, 128), (45, 64), (148, 128), (67, 256), (2, 256)])
def test_combine_skips_garbage_and_padding_rows(S, D):
    """Empty splits (-inf) may hold NaN partials; rows past qsl[R] keep their bytes.  Above
    16 splits one CTA owns a row (a quarter of the splits per warp), below one warp does."""
    lib = capi.load_library()
    T, Hq = 6, 4
    rng = np.random.default_rng(S * 1000 + D)
    ws_o = rng.standard_normal((S, T, Hq, D)).astype(np.float32)
    ws_lse = rng.standard_normal((S, T, Hq)).astype(np.float32) * 3
    ws_lse[1] = -np.inf
    ws_lse[S - 1, 0] = -np.inf
    if S > 40:
        ws_lse[9:31, 1] = -np.inf  # a whole quarter of the splits empty for one token
    ws_lse[:, 2] = -np.inf  # a row with no keys at all
    want, want_l2 = orc.combine_partials(ws_o, ws_lse)
    ws_o[np.isneginf(ws_lse)] = np.nan
    dev = "cuda"
    o_t, l_t = torch.from_numpy(ws_o).to(dev), torch.from_numpy(ws_lse).to(dev)
    out = torch.full((T, Hq, D), 7.0, dtype=torch.float32, device=dev)
    lse = torch.full((T, Hq), 7.0, dtype=torch.float32, device=dev)
    qsl = torch.tensor([0, 3, 5], dtype=torch.int32, device=dev)  # 5 valid tokens of 6
    a = capi.new_combine_args()
    a.ws_o, a.ws_lse, a.out = o_t.data_ptr(), l_t.data_ptr(), out.data_ptr()
    a.ws_o_stride_split, a.ws_o_stride_token, a.ws_o_stride_head = (s * 4 for s in o_t.stride()[:3])
    a.ws_lse_stride_split, a.ws_lse_stride_token, a.ws_lse_stride_head = (s * 4 for s in l_t.stride())
    a.out_dtype, a.out_stride_token, a.out_stride_head = capi.F32, Hq * D * 4, D * 4
    a.query_start_loc, a.num_reqs, a.num_tokens = qsl.data_ptr(), 2, T
    a.num_q_heads, a.head_size, a.num_splits = Hq, D, S
    opt = capi.make_options()
    opt.lse_out, opt.lse_stride_token, opt.lse_stride_head = lse.data_ptr(), Hq * 4, 4
    assert lib.combine(a, options=opt) == capi.OK, lib.last_error()
    torch.cuda.synchronize()
    got, got_l = out.cpu().numpy(), lse.cpu().numpy()
    np.testing.assert_allclose(got[:5], want[:5], rtol=4e-6, atol=4e-6)
    assert (got[2] == 0).all() and np.isneginf(got_l[2]).all()
    assert (got[5] == 7.0).all() and (got_l[5] == 7.0).all(), "padding row was written"
    fin = np.isfinite(want_l2[:5])
    np.testing.assert_allclose(got_l[:5][fin], orc.log2_to_ln(want_l2[:5])[fin], rtol=1e-5, atol=1e-5)


def test_combine_matches_reference_cpp_golden():
    g = load_golden("split_cpp")
    Hq, Hkv, D, window, causal, bq, S = (int(v) for v in g["meta"])
    lib = capi.load_library()
    dev = "cuda"
    o_t = torch.from_numpy(g["ws_o"]).to(dev)
    l_t = torch.from_numpy(g["ws_lse"]).to(dev)
    T = o_t.shape[1]
    out = torch.zeros((T, Hq, D), dtype=torch.float32, device=dev)
    qsl = torch.from_numpy(g["qsl"]).to(dev)
    a = capi.new_combine_args()
    a.ws_o, a.ws_lse, a.out = o_t.data_ptr(), l_t.data_ptr(), out.data_ptr()
    a.ws_o_stride_split, a.ws_o_stride_token, a.ws_o_stride_head = (s * 4 for s in o_t.stride()[:3])
    a.ws_lse_stride_split, a.ws_lse_stride_token, a.ws_lse_stride_head = (s * 4 for s in l_t.stride())
    a.out_dtype, a.out_stride_token, a.out_stride_head = capi.F32, Hq * D * 4, D * 4
    a.query_start_loc, a.num_reqs, a.num_tokens = qsl.data_ptr(), len(g["seq_lens"]), T
    a.num_q_heads, a.head_size, a.num_splits = Hq, D, S
    assert lib.combine(a) == capi.OK, lib.last_error()
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), g["combined"], rtol=2e-6, atol=2e-6)
