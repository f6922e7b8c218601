"""Negative controls of the parity gate: broken variants of the computation must fail it.

The reference pairs every guard of its test harness with a mutant that has to be caught
(tests/cpu/test_ref_capi_build.py:507-544, tests/cpu/test_grid.py:301-410): a causal limit
off by one, a window off by one, non-causal run as causal, V read four bytes early (onto
the K scale), the wrong KV head, the first token of every split lost, the last token of a
tile skipped, padding rows written.  Here each mutant is a small numpy variant of the
attention the oracle computes, run on the oracle's own cache image (poisoned slots
included), and the gate used by every GPU parity test - ``check_out`` / ``check_lse`` of
tests/helpers.py - must reject it while accepting the unmodified computation.
"""
import numpy as np
import pytest

from oracle import paged_int8_attention as orc
from tests.helpers import check_lse, check_out

HQ, HKV, D, BS = 8, 2, 128, 16
G = HQ // HKV
SCALE = D ** -0.5
LENS, QLENS = [300, 77, 129], [4, 3, 1]


def _case(seed=7):
    c = orc.make_paged_cache(LENS, HKV, D, BS, seed=seed)
    rng = np.random.default_rng(seed + 1)
    q = orc.round_to_bf16(rng.standard_normal((sum(QLENS), HQ, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(QLENS)])
    return c, q, qsl


def _attention(c, q, qsl, *, window=0, causal=True, hi_shift=0, lo_shift=0, v_byte_shift=0, kv_head=None,
               drop_first_of_split=0, drop_last_of_tile=0, extra_keys=0):
    """Dense fp64 attention over the cache image with the mutations switched on by the arguments."""
    T = q.shape[0]
    out = np.zeros((T, HQ, D))
    lse = np.full((T, HQ), -np.inf)
    raw = c.storage
    for r, L in enumerate(LENS):
        ql = int(qsl[r + 1] - qsl[r])
        span = L + extra_keys                     # reading past the request's end hits poison
        pos = np.arange(span)
        blk = c.block_table[r].astype(np.int64)[np.minimum(pos // BS, c.block_table.shape[1] - 1)]
        sl = pos % BS
        for i in range(ql):
            tok = int(qsl[r]) + i
            lo, hi = orc.visible_bounds(L - ql + i, L, window, causal)
            lo, hi = max(0, lo + lo_shift), min(span - 1, hi + hi_shift + extra_keys)
            keep = np.ones(span, dtype=bool)
            if drop_first_of_split:               # the first key of every split of `drop_first_of_split` tiles
                keep[::128 * drop_first_of_split] = False
            if drop_last_of_tile:
                keep[127::128] = False
            idx = np.nonzero(keep[lo:hi + 1])[0] + lo
            for h in range(HQ):
                kvh = h // G if kv_head is None else kv_head(h)
                K = c.k_cache[blk[idx], sl[idx], kvh].astype(np.float64) * c.k_scale[blk[idx], sl[idx], kvh][:, None]
                if v_byte_shift:
                    off = (c.v.offset + blk[idx] * c.v.stride_block + sl[idx] * c.v.stride_slot
                           + kvh * c.v.stride_head + v_byte_shift)
                    V = raw[off[:, None] + np.arange(D)[None, :]].view(np.int8).astype(np.float64)
                else:
                    V = c.v_cache[blk[idx], sl[idx], kvh].astype(np.float64)
                V = V * c.v_scale[blk[idx], sl[idx], kvh].astype(np.float64)[:, None]
                s = (K @ q[tok, h].astype(np.float64)) * SCALE
                m = s.max()
                p = np.exp(s - m)
                out[tok, h] = (p @ V) / p.sum()
                lse[tok, h] = m + np.log(p.sum())
    return out, lse


def _rejected(out, lse, ref):
    try:
        check_out(out, ref.out, what="mutant")
        check_lse(lse, ref.lse, what="mutant")
    except AssertionError:
        return True
    return False


def test_the_unmodified_computation_passes_the_gate():
    c, q, qsl = _case()
    ref = orc.ref_attention_paged(q, c, qsl, SCALE)
    out, lse = _attention(c, q, qsl)
    assert not _rejected(out, lse, ref)
    ref_w = orc.ref_attention_paged(q, c, qsl, SCALE, window=40)
    out, lse = _attention(c, q, qsl, window=40)
    assert not _rejected(out, lse, ref_w)


MUTANTS = {
    "causal limit one key short": dict(hi_shift=-1),
    "one token past the request (poisoned slot)": dict(extra_keys=1),
    "V read four bytes early (onto the K scale)": dict(v_byte_shift=-4),
    "query head h reads KV head h % Hkv": dict(kv_head=lambda h: h % HKV),
    "every head reads KV head 0": dict(kv_head=lambda h: 0),
    "first key of every 128-key split lost": dict(drop_first_of_split=1),
    "last key of every tile skipped": dict(drop_last_of_tile=1),
}


@pytest.mark.parametrize("name", sorted(MUTANTS))
def test_mutant_is_rejected(name):
    c, q, qsl = _case()
    ref = orc.ref_attention_paged(q, c, qsl, SCALE)
    out, lse = _attention(c, q, qsl, **MUTANTS[name])
    assert _rejected(out, lse, ref), name


def test_window_and_causal_mutants_are_rejected():
    c, q, qsl = _case()
    ref = orc.ref_attention_paged(q, c, qsl, SCALE, window=40)
    assert _rejected(*_attention(c, q, qsl, window=40, lo_shift=-1), ref), "window one key too wide"
    assert _rejected(*_attention(c, q, qsl, window=40, lo_shift=1), ref), "window one key too narrow"
    assert _rejected(*_attention(c, q, qsl, window=0), ref), "window ignored"
    ref_nc = orc.ref_attention_paged(q, c, qsl, SCALE, causal=False)
    assert _rejected(*_attention(c, q, qsl, causal=True), ref_nc), "non-causal run as causal"


def test_written_padding_rows_and_lost_rows_are_rejected():
    """Rows of no request must keep their canary, rows of a request must all be written."""
    c, q, qsl = _case()
    ref = orc.ref_attention_paged(q, c, qsl, SCALE)
    out, lse = _attention(c, q, qsl)
    lost = out.copy()
    lost[5] = np.nan                               # a row the kernel never wrote (canary / NaN fill)
    assert _rejected(lost, lse, ref)
    bad_lse = lse.copy()
    bad_lse[2, 3] += 2e-3                          # log-sum-exp off by more than 1e-3
    assert _rejected(out, bad_lse, ref)
    dead = lse.copy()
    dead[0, 0] = -np.inf                           # a live row reported as having no keys
    assert _rejected(out, dead, ref)
