"""Host planner: same contract as the reference planner's CPU tests (no length parameter,
host ints only, S * T fits the workspace, split ranges partition the tiles)."""
import inspect
import random

import pytest

from pth_flash_attn_b200 import planner


def test_signature_is_the_descriptor():
    sig = inspect.signature(planner.plan_launch)
    assert tuple(sig.parameters) == planner.DESCRIPTOR_FIELDS
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in sig.parameters.values())
    assert not any("len" in name and name != "max_query_len" for name in sig.parameters)


def _plan(**kw):
    base = dict(num_tokens=64, num_reqs=64, max_query_len=1, G=4, Hkv=8, D=128, num_sms=148,
                is_prefill=False, ws_token_splits=1 << 20, window=0)
    base.update(kw)
    return planner.plan_launch(**base)


def test_rejects_non_host_ints():
    import torch

    with pytest.raises(TypeError):
        _plan(num_tokens=torch.tensor(64))
    with pytest.raises(TypeError):
        _plan(G=True)
    with pytest.raises(TypeError):
        _plan(is_prefill=1)
    with pytest.raises(TypeError):
        _plan(num_reqs=__import__("numpy").int64(64))
    with pytest.raises(ValueError):
        _plan(D=96)
    with pytest.raises(ValueError):
        _plan(G=65)
    with pytest.raises(ValueError):
        _plan(max_query_len=65)
    with pytest.raises(ValueError):
        _plan(num_tokens=200, num_reqs=64, max_query_len=3)


def test_plan_is_a_pure_function_of_the_descriptor():
    rnd = random.Random(0)
    for _ in range(200):
        G = rnd.choice([1, 2, 4, 6, 8, 16])
        q = rnd.choice([1, 2, 4, 8, 16])
        reqs = rnd.randint(1, 256)
        kw = dict(num_tokens=reqs * q, num_reqs=reqs, max_query_len=q, G=G, Hkv=rnd.choice([1, 2, 8]),
                  ws_token_splits=rnd.choice([0, 1000, 1 << 22]), window=rnd.choice([0, 4096]))
        a, b = _plan(**kw), _plan(**kw)
        assert a == b
        assert a.num_splits >= 1
        if a.num_splits > 1:
            assert a.num_splits * a.num_tokens <= kw["ws_token_splits"]
        assert a.bq * G <= 16 * a.wm <= 64
        assert a.q_tiles_upper >= reqs * -(-q // a.bq)
        assert a.ws_o_shape == ((a.num_splits if a.num_splits > 1 else 0), a.num_tokens, a.Hq, 128)


def test_baseline_shapes():
    # one request at any length must still spread over the machine: two pieces per SM
    one = _plan(num_tokens=1, num_reqs=1)
    assert one.wm == 1 and one.bq == 4 and one.num_splits == planner.s_alone(Hkv=8, D=128, num_sms=148) == 37
    # a full batch needs only a small bound (the device cuts 8,192-key requests in two)
    full = _plan()
    assert full.num_splits == 5
    # monotone in the machine size, never below one
    assert [_plan(num_sms=n).num_splits for n in (1, 32, 148, 1000)] == sorted(
        _plan(num_sms=n).num_splits for n in (1, 32, 148, 1000))
    # verify: 4 draft tokens x G = 4 -> 16 rows
    v = _plan(num_tokens=128, num_reqs=32, max_query_len=4)
    assert v.wm == 1 and v.bq == 4 and v.num_splits == 10
    # drafter: 16 tokens x 4 heads = 64 rows, window caps the splits
    d = _plan(num_tokens=512, num_reqs=32, max_query_len=16, window=4096)
    assert d.wm == 4 and d.bq == 16
    assert d.num_splits <= -(-(4096 + 16 - 2) // planner.KV_TILE_TOKENS) + 1
    # tall windowed tiles: pieces only to fill the SMs (256 unsplit items already do)
    assert d.num_splits == 1
    assert _plan(num_tokens=64, num_reqs=4, max_query_len=16, window=4096).num_splits == -(-148 // 32) == 5
    # short windowed tiles keep the generous bound of the persistent kernel
    assert _plan(num_tokens=128, num_reqs=32, max_query_len=4, window=4096).num_splits == 10
    tight = _plan(num_tokens=1, num_reqs=1, window=200)
    assert tight.num_splits == -(-(200 + 1 - 2) // planner.KV_TILE_TOKENS) + 1 == 3
    # prefill
    # prefill: full tiles; cut only if the caller reserved partials for the whole launch (the
    # bound then counts requests, which may be long decode requests inside a mixed launch)
    pf = _plan(num_tokens=8192, num_reqs=4, max_query_len=2048, G=8, is_prefill=True, ws_token_splits=4096)
    assert pf.wm == 4 and pf.bq == 8 and pf.num_splits == 1
    mixed = _plan(num_tokens=2128, num_reqs=58, max_query_len=1024, G=8, is_prefill=True, ws_token_splits=8 * 2128)
    assert mixed.num_splits == 8 and mixed.num_splits * mixed.num_tokens <= 8 * 2128
    # no reservation, no split
    assert _plan(num_tokens=1, num_reqs=1, ws_token_splits=0).num_splits == 1


def test_workspace_reservation_covers_every_plan():
    for Hkv in (1, 2, 8):
        w = planner.workspace_token_splits(max_num_seqs=64, q_dec_max=4, Hkv=Hkv, D=128, num_sms=148)
        for reqs in (1, 2, 7, 33, 64):
            for q in (1, 4):
                p = planner.plan_launch(num_tokens=reqs * q, num_reqs=reqs, max_query_len=q, G=4, Hkv=Hkv, D=128,
                                        num_sms=148, is_prefill=False, ws_token_splits=w)
                unclamped = planner.plan_launch(num_tokens=reqs * q, num_reqs=reqs, max_query_len=q, G=4, Hkv=Hkv,
                                                D=128, num_sms=148, is_prefill=False, ws_token_splits=1 << 40)
                assert p.num_splits == unclamped.num_splits, "the reservation clamped a plan"
        o, l = planner.workspace_shapes(ws_token_splits=w, Hq=4 * Hkv, D=128)
        assert planner.workspace_bytes(ws_token_splits=w, Hq=4 * Hkv, D=128) == (o[0] * o[1] * o[2] + l[0] * l[1]) * 4


def test_split_ranges_partition_the_tiles():
    for tiles in (0, 1, 5, 64, 1000):
        for S in (1, 2, 7, 64):
            ranges = [planner.split_tile_range(split=s, num_splits=S, num_tiles=tiles) for s in range(S)]
            assert ranges[0][0] == 0 and ranges[-1][1] == tiles
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        planner.split_tile_range(split=3, num_splits=3, num_tiles=9)


def test_helpers():
    assert planner.max_tokens_per_tile(4) == 16 and planner.max_tokens_per_tile(6) == 10
    assert [planner.wm_for_rows(r) for r in (1, 16, 17, 32, 33, 64)] == [1, 1, 2, 2, 4, 4]
    with pytest.raises(ValueError):
        planner.wm_for_rows(65)
    assert planner.c_target(D=128, num_sms=148) == 148 * planner.CTAS_PER_SM[128]
