"""The persistent kernel's work-item schedule, checked on the host.

``pthb200_test_schedule`` runs the functions the device scheduler runs (csrc/sched.cuh) on
host copies of the lengths.  The properties pinned here are the ones the reference pins for
its own scheduler (tests/cpp/test_geometry.cpp:298-451, tests/cpu/test_ref_capi_build.py:
323-363): the split partition of a row tile is a disjoint cover of its KV tiles with sizes
that differ by at most one, every (request, row tile, KV head) is served, surplus and empty
requests produce no work, and the plan depends on the lengths only through the device arrays.
"""
import numpy as np
import pytest

from pth_flash_attn_b200 import capi

KV_TILE = 128


def _lib():
    return capi.load_library()


def _visible(seq_len, q_len, i, window, causal):
    pos = seq_len - q_len + i
    lo = max(0, pos - window + 1) if window > 0 else 0
    if causal:
        hi = pos
    elif window > 0:
        hi = min(seq_len - 1, pos + window - 1)
    else:
        hi = seq_len - 1
    return lo, min(hi, seq_len - 1)


def _check_cover(items, qlens, lens, *, G, Hkv, bq, S, window=0, causal=True, row_class=0, class_rows=0):
    """Every served row tile x KV head has splits 0..s-1 exactly once and their tile spans
    chain from the first to the last tile its rows can see."""
    by_key = {}
    for cta, r, rt, kvh, split, splits, tb, te in items.tolist():
        assert 1 <= splits <= S
        by_key.setdefault((r, rt, kvh), []).append((split, splits, tb, te))
    expected = set()
    for r, (ql, L) in enumerate(zip(qlens, lens)):
        if ql == 0:
            continue
        if row_class and ((ql * G <= class_rows) != (row_class == 1)):
            continue
        for rt in range(-(-ql // bq)):
            for kvh in range(Hkv):
                expected.add((r, rt, kvh))
    assert set(by_key) == expected
    for (r, rt, kvh), lst in by_key.items():
        lst.sort()
        splits = lst[0][1]
        assert [s for s, *_ in lst] == list(range(splits)), (r, rt, kvh, lst)
        ql, L = qlens[r], lens[r]
        i0, i1 = rt * bq, min(ql, rt * bq + bq) - 1
        lo0, hi0 = _visible(L, ql, i0, window, causal)
        lo1, hi1 = _visible(L, ql, i1, window, causal)
        rb, re = lo0, max(hi0, hi1) + 1
        if re <= rb:
            assert all(tb >= te for _, _, tb, te in lst)
            continue
        t0, t1 = rb // KV_TILE, -(-re // KV_TILE)
        assert lst[0][2] == t0 and lst[-1][3] == t1
        sizes = []
        for k in range(splits - 1):
            assert lst[k][3] == lst[k + 1][2]
        for _, _, tb, te in lst:
            sizes.append(te - tb)
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("seed", range(6))
def test_random_batches_are_covered_exactly_once(seed):
    rng = np.random.default_rng(seed)
    R = int(rng.integers(1, 70))
    G, Hkv = int(rng.choice([1, 4, 8])), int(rng.choice([1, 2, 8]))
    bq = int(rng.choice([1, 2, 4, 16 // min(G, 16) or 1]))
    qlens = rng.integers(0, 3 * bq + 1, size=R).tolist()
    lens = [int(q + rng.integers(0, 9000)) if q else int(rng.integers(0, 50)) for q in qlens]
    S = int(rng.choice([1, 3, 37]))
    window = int(rng.choice([0, 0, 300]))
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    ctas = int(rng.choice([1, 7, 148]))
    items = _lib().schedule(qsl, lens, group=G, num_kv_heads=Hkv, bq=bq, num_splits=S, num_ctas=ctas, window=window)
    _check_cover(items, qlens, lens, G=G, Hkv=Hkv, bq=bq, S=S, window=window)
    # CTA c runs the items c, c + CTAs, ... of one global order
    order = {}
    for cta in range(ctas):
        mine = items[items[:, 0] == cta]
        order[cta] = len(mine)
    counts = np.array([order[c] for c in range(ctas)])
    assert counts.max() - counts.min() <= 1


def test_row_classes_partition_the_requests():
    qlens = [1, 40, 2, 1, 300, 3, 1]
    lens = [3000, 900, 2100, 64, 1500, 5000, 129]
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    lib = _lib()
    short = lib.schedule(qsl, lens, group=8, num_kv_heads=2, bq=2, num_splits=3, num_ctas=148, row_class=1,
                         class_rows=16)
    _check_cover(short, qlens, lens, G=8, Hkv=2, bq=2, S=3, row_class=1, class_rows=16)
    assert set(short[:, 1].tolist()) == {0, 2, 3, 6}


def test_split_choice_at_the_benchmark_shapes():
    """Equal requests are cut into equal items, a whole number of rounds over 148 CTAs."""
    lib = _lib()
    # 64 decode requests of 8,192 keys, 8 KV heads: 2 pieces of 32 tiles each, 1,024 items
    items = lib.schedule(np.arange(65), [8192] * 64, group=4, num_kv_heads=8, bq=1, num_splits=3, num_ctas=148)
    assert set(items[:, 5].tolist()) == {2} and len(items) == 1024
    assert set((items[:, 7] - items[:, 6]).tolist()) == {32}
    # one decode request of 131,072 keys: 37 pieces -> 296 items = two per CTA
    items = lib.schedule([0, 1], [131072], group=4, num_kv_heads=8, bq=1, num_splits=37, num_ctas=148)
    assert set(items[:, 5].tolist()) == {37} and len(items) == 296
    # the KV heads of one (request, split) are neighbours in the global order
    first = items[items[:, 0] < 8]
    first = first[np.argsort(first[:, 0], kind="stable")]
    round0 = np.array([row for row in first.tolist() if row[4] == 0])
    assert round0[:, 3].tolist() == list(range(8))
    # the caller's split count is a bound
    items = lib.schedule([0, 1], [131072], group=4, num_kv_heads=8, bq=1, num_splits=18, num_ctas=148)
    assert set(items[:, 5].tolist()) == {18}


def test_plan_ignores_requests_without_queries_and_keys():
    lib = _lib()
    items = lib.schedule([0, 0, 1, 1], [500, 0, 70], group=4, num_kv_heads=2, bq=1, num_splits=4, num_ctas=148)
    # request 0 and 2 have no query; request 1 has a query but no keys: it still gets items
    # (they write the zero output and the -inf log-sum-exp), with an empty tile span
    assert set(items[:, 1].tolist()) == {1}
    assert ((items[:, 7] - items[:, 6]) == 0).all()
