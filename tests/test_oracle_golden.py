"""Pins the numpy oracle to the reference project's own oracle.

Every fixture under tests/golden was produced by the reference's Python code
(tests/golden/make_golden.py); the known-answer values are those of the
reference's tests/cpu/test_reference.py.
"""
import numpy as np
import pytest

from oracle import paged_int8_attention as orc
from tests.helpers import golden_dense, load_golden


def test_writer_known_answers():
    # round half away from zero on exact ties (scale exactly 1.0)
    x = np.array([[127.0, 2.5, -2.5, 0.5, -0.5, 3.5, -126.5]], dtype=np.float32)
    q, s = orc.quantize_rows(x)
    assert s.tolist() == [1.0]
    assert q.tolist() == [[127, 3, -3, 1, -1, 4, -127]]
    # negative control: round-half-even differs on the same row
    assert np.rint(x).astype(np.int8).tolist() != q.tolist()
    # floor: zero rows and tiny rows sit on fp32(1e-6)
    q0, s0 = orc.quantize_rows(np.zeros((2, 16), np.float32))
    assert (s0 == np.float32(1e-6)).all() and (q0 == 0).all()
    # full-scale rows store +-127, never -128
    amp = np.float32(3.7)
    sg = np.where(np.arange(64) % 3 == 0, -amp, amp).astype(np.float32)[None]
    qe, _ = orc.quantize_rows(sg)
    assert (np.abs(qe) == 127).all()


def test_writer_golden():
    g = load_golden("writer")
    for tag in ("small", "rand"):
        q, s = orc.quantize_rows(g[f"x_{tag}"])
        assert np.array_equal(q, g[f"q_{tag}"])
        assert np.array_equal(s.view(np.uint32), g[f"s_{tag}"].view(np.uint32))


@pytest.mark.parametrize("name", ["cache_nhd", "cache_hnd_pad", "cache_nhd_d128"])
def test_cache_bytes_golden(name):
    """Same sources + same block ids => the reference's bytes in every written cell,
    the reference's stream geometry, and the same dense read-back."""
    g = load_golden(name)
    Hkv, D, bs, pad, off, nb, page = (int(v) for v in g["meta"])
    layout = str(g["layout"])
    lens = g["seq_lens"].tolist()
    sources = [(g[f"k_src{r}"], g[f"v_src{r}"]) for r in range(len(lens))]
    nblk = [-(-L // bs) for L in lens]
    block_ids = [g["block_table"][r, : nblk[r]].tolist() for r in range(len(lens))]
    c = orc.make_paged_cache(lens, Hkv, D, bs, layout, pad, seed=1, storage_offset_bytes=off,
                             sources=sources, block_ids=block_ids, num_blocks=nb)
    assert c.page_bytes == page
    # cell geometry: K at 0, ks at D, V at D+4, vs at 2D+4; strides from the views
    for view, key in ((c.k, "k_geom"), (c.v, "v_geom"), (c.ks, "ks_geom"), (c.vs, "vs_geom")):
        assert [view.offset, view.stride_block, view.stride_slot, view.stride_head] == \
            g[key].tolist(), key
    assert c.ks.offset - c.k.offset == D and c.v.offset - c.k.offset == D + 4
    assert c.vs.offset - c.k.offset == 2 * D + 4 and c.cell_bytes == 2 * (D + 4)
    # read the REFERENCE's bytes through this oracle's views
    ref = orc.PagedInt8Cache(
        storage=g["storage"].copy(), k=c.k, v=c.v, ks=c.ks, vs=c.vs,
        block_table=g["block_table"], seq_lens=g["seq_lens"], num_blocks=nb, block_size=bs,
        Hkv=Hkv, D=D, layout=layout, page_bytes=page, storage_offset_bytes=off)
    for r, L in enumerate(lens):
        mine, theirs = c.dense(r), ref.dense(r)
        for a, b, key in ((mine.k_int, theirs.k_int, "k_int"), (mine.v_int, theirs.v_int, "v_int"),
                          (mine.k_scale, theirs.k_scale, "k_scale"),
                          (mine.v_scale, theirs.v_scale, "v_scale")):
            assert np.array_equal(a, b), (r, key)
            assert np.array_equal(a, g[f"{key}{r}"]), (r, key)
    # unused slots of a used block hold the poison scale
    r = len(lens) - 1
    tail = lens[r] % bs
    if tail:
        last = int(c.block_table[r, (lens[r] - 1) // bs])
        assert (c.k_scale[last, tail:] == orc.POISON_SCALE).all()


ATTN_CASES = ["attn_decode", "attn_verify4", "attn_window_causal", "attn_window_noncausal",
              "attn_noncausal", "attn_mixed", "attn_d64_g6", "attn_d256_g6"]


@pytest.mark.parametrize("name", ATTN_CASES)
def test_attention_golden(name):
    g = load_golden(name)
    Hq, Hkv, D, window, causal = (int(v) for v in g["meta"])
    q = orc.f32_from_bf16_bits(g["q_bits"])
    res = orc.ref_attention(q, golden_dense(g), g["qsl"], float(g["softmax_scale"]),
                            window=window, causal=bool(causal))
    assert np.array_equal(res.valid, g["valid"])
    np.testing.assert_allclose(res.out, g["out"], rtol=1e-11, atol=1e-12)
    fin = np.isfinite(g["lse"])
    assert np.array_equal(np.isfinite(res.lse), fin)
    np.testing.assert_allclose(res.lse[fin], g["lse"][fin], rtol=1e-12, atol=1e-12)


def test_attention_mutants_are_caught():
    """Negative controls: an off-by-one causal limit or window must change the result."""
    g = load_golden("attn_window_causal")
    Hq, Hkv, D, window, causal = (int(v) for v in g["meta"])
    q = orc.f32_from_bf16_bits(g["q_bits"])
    kv = golden_dense(g)
    bad = orc.ref_attention(q, kv, g["qsl"], float(g["softmax_scale"]), window=window + 1,
                            causal=True)
    assert np.abs(bad.out - g["out"]).max() > 1e-6
    bad = orc.ref_attention(q, kv, g["qsl"], float(g["softmax_scale"]), window=window,
                            causal=False)
    assert np.abs(bad.out - g["out"]).max() > 1e-6


def test_visible_bounds_closed_form():
    for L in (1, 5, 40):
        for ql in (1, 3):
            if ql > L:
                continue
            for window in (0, 1, 4, 100):
                for causal in (True, False):
                    for i in range(ql):
                        p = L - ql + i
                        lo, hi = orc.visible_bounds(p, L, window, causal)
                        want = [k for k in range(L)
                                if (k <= p if causal else True)
                                and (abs(p - k) < window if window > 0 else True)]
                        assert list(range(lo, hi + 1)) == want


def test_split_combine_matches_reference_cpp():
    """The combine rule and partial semantics of the reference's C++ CPU path."""
    g = load_golden("split_cpp")
    Hq, Hkv, D, window, causal, bq, S = (int(v) for v in g["meta"])
    out, lse2 = orc.combine_partials(g["ws_o"], g["ws_lse"])
    np.testing.assert_allclose(out, g["combined"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(out, g["out"], rtol=1e-5, atol=1e-5)
    # log2 LSE of the partials merges to the natural-log LSE of the fp64 oracle
    np.testing.assert_allclose(orc.log2_to_ln(lse2), g["lse"], rtol=1e-5, atol=1e-5)
    # every split's partial is that split's own softmax over its 64-token tiles
    q = orc.f32_from_bf16_bits(g["q_bits"])
    kv = golden_dense(g)
    qsl = g["qsl"].tolist()
    G = Hq // Hkv
    for r, x in enumerate(kv):
        L, ql = x.seq_len, qsl[r + 1] - qsl[r]
        tiles = -(-L // 64)
        for s in range(S):
            t0, t1 = orc.split_tile_range(s, S, tiles)
            lo, hi = t0 * 64, min(t1 * 64, L)
            for i in range(ql):
                p = L - ql + i
                hi_i = min(hi, p + 1)
                tok = qsl[r] + i
                for h in range(Hq):
                    if hi_i <= lo:
                        assert np.isneginf(g["ws_lse"][s, tok, h])
                        continue
                    kd = x.k_deq()[lo:hi_i, h // G]
                    vd = x.v_deq()[lo:hi_i, h // G]
                    sc = kd @ q[tok, h].astype(np.float64) * float(g["softmax_scale"])
                    m = sc.max()
                    pr = np.exp(sc - m)
                    np.testing.assert_allclose(g["ws_o"][s, tok, h], pr @ vd / pr.sum(),
                                               rtol=1e-4, atol=1e-5)
                    np.testing.assert_allclose(g["ws_lse"][s, tok, h],
                                               (m + np.log(pr.sum())) / np.log(2.0),
                                               rtol=1e-5, atol=1e-5)


def test_combine_ignores_garbage_in_empty_splits():
    rng = np.random.default_rng(0)
    o = rng.standard_normal((3, 2, 2, 8))
    l2 = rng.standard_normal((3, 2, 2))
    l2[1] = -np.inf
    o2 = o.copy()
    o2[1] = np.nan
    a, la = orc.combine_partials(o, l2)
    b, lb = orc.combine_partials(o2, l2)
    assert np.array_equal(a, b) and np.array_equal(la, lb)
    l2[:] = -np.inf
    c, lc = orc.combine_partials(o2, l2)
    assert (c == 0).all() and np.isneginf(lc).all()


def test_bf16_round_trip():
    x = np.array([1.0, 1.00390625, 1.001953125, 3.1415926, -2.5e-8, 65504.0, 1e38], np.float32)
    b = orc.bf16_bits_from_f32(x)
    y = orc.f32_from_bf16_bits(b)
    assert y[0] == 1.0 and y[1] == 1.0  # tie rounds to even
    assert y[2] == 1.0
    import torch

    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(y, want)
