"""Parity at the sizes the benchmark times.

Every workload of bench.py is built exactly as the benchmark builds it (its device cache
of quantised N(0, 1) values, its planner-chosen split bound and tile height, the flags the
torch op would set) and run once through the C ABI.  Two checks per launch:

* sampled (token, head) rows against the fp64 CPU oracle reading the same cache bytes
  (first, last and a random token of the longest, the shortest and random requests), with
  the gate of every parity test: bf16 output max |d| <= 2e-2, mean |d| <= 2e-3, natural-log
  LSE within 1e-3;
* EVERY row against the CUDA-core kernel of this library (itself checked against the
  oracle on small shapes), so that a wrong row the sample misses cannot hide.

The reference argues the same way for its long prefill cases: rows are independent, so
checking whole row tiles of a large launch is checking the launch
(tests/gpu/attn_prefill.py:3-30).
"""
import numpy as np
import pytest
import torch

import bench
from pth_flash_attn_b200 import capi, host
from tests.helpers import LSE_TOL, OUT_MAX_TOL, OUT_MEAN_TOL

pytestmark = pytest.mark.gpu

CASES = [
    # workload, world (KV-head shards), rank
    ("decode_small", 1, 0),
    ("long_decode", 1, 0),       # 1 x 131,072 with 37 pieces, 64 x 8,192
    ("long_decode", 8, 5),       # one KV head: contiguous pages, bulk-copy path
    ("long_decode", 2, 1),
    ("verify4", 1, 0),
    ("drafter16", 1, 0),
    ("chunked_prefill", 1, 0),
    ("mixed", 8, 2),
    ("mixed", 1, 0),
]


def _scalar_reference(dl):
    """The same launch on the CUDA-core kernel, unsplit: (out fp32, lse)."""
    s = dl.sets[0]
    out = torch.full((dl.T, dl.hq, bench.D), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((dl.T, dl.hq), float("nan"), dtype=torch.float32, device="cuda")
    host.attention_forward(s["q"], out, s["views"], s["bt"], s["lens"], s["qsl"], bq=dl.bq, num_splits=1,
                           softmax_scale=bench.D ** -0.5, window=dl.window, causal=dl.causal, lse_out=lse,
                           kernel=capi.KERNEL_SCALAR)
    torch.cuda.synchronize()
    return out, lse


@pytest.mark.parametrize("name,world,rank", CASES)
def test_benchmark_workload_matches_the_oracle(name, world, rank):
    props = torch.cuda.get_device_properties(0)
    lib = capi.load_library()
    for i, launch in enumerate(bench.workload_launches(name)):
        dl = bench.DeviceLaunch(torch, launch, rank, world, torch.device("cuda", 0), 4321 + 100 * i + rank,
                                props.multi_processor_count)
        r = dl.parity(picks_per_launch=10, seed=3 + i)
        what = f"{name} launch {i} shard {rank}/{world} (S <= {dl.S}, bq {dl.bq})"
        assert lib.device_status() == 0, what
        assert r["all_rows_written"], what
        assert r["max_abs"] <= OUT_MAX_TOL, (what, r)
        assert r["mean_abs"] <= OUT_MEAN_TOL, (what, r)
        assert r["lse_abs"] <= LSE_TOL, (what, r)
        # every row against the CUDA-core kernel
        lse = torch.full((dl.T, dl.hq), float("nan"), dtype=torch.float32, device="cuda")
        dl.launch(0, lse_out=lse)
        torch.cuda.synchronize()
        ref_out, ref_lse = _scalar_reference(dl)
        d = (dl.out.float() - ref_out).abs()
        assert float(d.max()) <= OUT_MAX_TOL, (what, float(d.max()))
        assert float(d.mean()) <= OUT_MEAN_TOL, (what, float(d.mean()))
        assert float((lse - ref_lse).abs().max()) <= LSE_TOL, what
        del dl
        torch.cuda.empty_cache()


def test_head_shards_concatenate_to_the_unsharded_launch():
    """KV-head shards of one batch, each on its own cache holding the same cells for its
    heads, give the head slices of the unsharded launch: byte for byte when the key range
    is not split, within the parity gate when it is."""
    from pth_flash_attn_b200 import planner, sharding

    dev = torch.device("cuda", 0)
    Hq, Hkv, Dh, BSz, CELL = 32, 8, bench.D, bench.BS, bench.CELL
    lens, qlens = [9000, 700, 4100, 33], [4, 4, 1, 3]
    full = bench.DeviceLaunch(torch, dict(seq_lens=lens, q_lens=qlens, Hq=Hq, Hkv=Hkv), 0, 1, dev, 99, 148)
    full.launch(0)
    torch.cuda.synchronize()
    s0 = full.sets[0]
    full_one = torch.zeros_like(full.out)
    host.attention_forward(s0["q"], full_one, s0["views"], s0["bt"], s0["lens"], s0["qsl"], bq=full.bq, num_splits=1,
                           softmax_scale=Dh ** -0.5, flags=full.flags)
    torch.cuda.synchronize()
    cells = s0["storage"].view(-1, BSz, Hkv, CELL)
    for world in (2, 4, 8):
        for rank in range(world):
            sh = sharding.head_shard(rank, world, Hq, Hkv)
            hkv = sh.num_kv_heads
            part = cells[:, :, sh.kv_begin:sh.kv_end, :].contiguous()
            base, page = part.data_ptr(), BSz * hkv * CELL
            slot, head = hkv * CELL, CELL
            views = host.CacheViews((base, page, slot, head), (base + Dh + 4, page, slot, head),
                                    (base + Dh, page, slot, head), (base + 2 * Dh + 4, page, slot, head),
                                    cells.shape[0], BSz, hkv, Dh)
            q = s0["q"][:, sh.q_begin:sh.q_end].contiguous()
            out = torch.zeros_like(q)
            # the unsharded launch's split bound, so that both cut the requests alike
            S = full.S
            ws_o = torch.empty((S, full.T, sh.num_q_heads, Dh), dtype=torch.float32, device=dev)
            ws_lse = torch.empty((S, full.T, sh.num_q_heads), dtype=torch.float32, device=dev)
            host.attention_forward(q, out, views, s0["bt"], s0["lens"], s0["qsl"], bq=full.bq, num_splits=S,
                                   softmax_scale=Dh ** -0.5, ws_o=ws_o, ws_lse=ws_lse, flags=full.flags)
            torch.cuda.synchronize()
            want = full.out[:, sh.q_begin:sh.q_end]
            # unsplit, the work of a (request, KV head) does not depend on the other heads at all
            one = torch.zeros_like(q)
            host.attention_forward(q, one, views, s0["bt"], s0["lens"], s0["qsl"], bq=full.bq, num_splits=1,
                                   softmax_scale=Dh ** -0.5, flags=full.flags)
            torch.cuda.synchronize()
            if hkv > 1:
                assert torch.equal(one.view(torch.int16), full_one[:, sh.q_begin:sh.q_end].view(torch.int16)), (world, rank)
            else:
                # one KV head per GPU: the pages are contiguous, the kernel copies them whole and
                # takes the keys of a tile in another order, so the fp32 row sums round differently
                d1 = (one.float() - full_one[:, sh.q_begin:sh.q_end].float()).abs()
                assert float(d1.max()) <= 2e-2 and float(d1.mean()) <= 1e-4, (world, rank, float(d1.max()))
            # a shard has fewer KV heads, so the device may cut its requests into a different
            # number of pieces than the unsharded launch: equal within the parity gate always,
            # byte for byte when the cuts agree
            d = (out.float() - want.float()).abs()
            assert float(d.max()) <= 2e-2 and float(d.mean()) <= 2e-3, (world, rank, float(d.max()))
    assert capi.load_library().device_status() == 0
    assert planner.plan_launch(num_tokens=sum(qlens), num_reqs=len(lens), max_query_len=4, G=4, Hkv=1, D=128,
                               num_sms=148, is_prefill=False, ws_token_splits=1 << 20).Hq == 4
