"""The geometry of the reference's GPU correctness grid, run through this library.

``tests/golden/grid_cases.json`` lists the 328 cases of the reference's grid
(tests/gpu/grid_cases.py ``all_cases()``: paging edges x page sizes x layouts, row counts x
group sizes, batches, split counts up to S_max, contexts up to 262,144, dtypes, padded rows,
strided q / out, sliding windows and non-causal ranges at D = 128), exported by
``tests/golden/make_grid_cases.py``.  Every case is built here with this repository's oracle
(seeded N(0, 1) sources quantised by the writer rule, poisoned unused slots, shuffled block
ids) and run through the C ABI with the kernel family the library chooses itself, then held
to the parity gate (bf16 / fp16 / fp32 output max |d| <= 2e-2, mean |d| <= 2e-3, LSE within
1e-3) against the fp64 oracle - dense where that is cheap, sampled rows plus a comparison of
EVERY row with the CUDA-core kernel where a context is long.  The gate is applied to
|d| / max(1, |ref|): it is stated for unit-scale outputs, and the kernel families that carry
p * v_scale as bf16 round it to 8 significant bits, which a row that sees a single key (the
grid has launches made of such rows, output in fp32) shows in full as 2^-9 of |v|, while
any longer row averages it away.  As in the reference's harness
(grid_cases.py:809-958), rows of no request and the bytes around the output keep their
canary bytes.
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host
from tests.helpers import LSE_TOL, OUT_MAX_TOL, OUT_MEAN_TOL, check_lse, check_out

pytestmark = pytest.mark.gpu

CASES = json.loads((Path(__file__).parent / "golden" / "grid_cases.json").read_text())["cases"]
FAMILIES = sorted({c["family"] for c in CASES})
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "f32": torch.float32}
DENSE_LIMIT = 3_000_000   # keys x KV heads up to which the dense fp64 oracle is used
CANARY = 0xFF


def _seed(name: str) -> int:
    return int(hashlib.sha256(name.encode()).hexdigest()[:8], 16) % (2 ** 31)


def _run(case):
    from tests.gpu_util import cache_to_device

    G, Hkv, D = case["G"], case["Hkv"], case["D"]
    Hq = G * Hkv
    qlens, lens = case["q_lens"], case["seq_lens"]
    seed = _seed(case["name"])
    c = orc.make_paged_cache(lens, Hkv, D, case["block_size"], layout=case["layout"],
                             pad_page_bytes=case["pad_page_bytes"], seed=seed,
                             storage_offset_bytes=case["storage_offset_bytes"], keep_sources=False)
    rng = np.random.default_rng(seed + 1)
    Tq, T = sum(qlens), sum(qlens) + case["pad_rows"]
    q_dt = DTYPES[case["q_dtype"]]
    out_dt = q_dt if case["out_dtype"] == "q" else DTYPES[case["out_dtype"]]
    q_f32 = rng.standard_normal((T, Hq, D), dtype=np.float32)
    # strided q / out: extra heads and extra elements per row around the views
    ph, pe = (1, 8) if case["strided_io"] else (0, 0)
    q_big = torch.zeros((T, Hq + ph, D + pe), dtype=q_dt, device="cuda")
    q_big[:, :Hq, :D] = torch.from_numpy(q_f32).cuda().to(q_dt)
    q = q_big[:, :Hq, :D]
    q_used = q.float().cpu().numpy()
    esz = torch.empty((), dtype=out_dt).element_size()
    out_buf = torch.full(((T + 2), Hq + ph, D + pe), 0, dtype=torch.uint8, device="cuda").repeat(1, 1, esz)
    out_buf.fill_(CANARY)
    out_all = out_buf.view(out_dt)                       # [T + 2, Hq + ph, D + pe]
    out = out_all[:T, :Hq, :D]
    lse = torch.full((T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    qsl_t = torch.from_numpy(qsl).cuda()
    storage, views, bt, lens_t = cache_to_device(c)
    S = case["num_splits"]
    ws_o = ws_lse = None
    if S > 1:
        ws_o = torch.full((S, T, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        ws_lse = torch.full((S, T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    kw = dict(bq=case["bq"], softmax_scale=D ** -0.5, window=case["window"], causal=case["causal"])
    host.attention_forward(q, out, views, bt, lens_t, qsl_t, num_splits=S, ws_o=ws_o, ws_lse=ws_lse, lse_out=lse, **kw)
    torch.cuda.synchronize()
    assert capi.load_library().device_status() == 0
    got = out.float().cpu().numpy()
    got_lse = lse.cpu().numpy()
    # canaries: rows of no request, the two rows behind the output, the padding around the views
    raw = out_buf.cpu().numpy()
    raw_rows = raw.reshape(T + 2, Hq + ph, (D + pe) * esz)
    assert (raw_rows[Tq:] == CANARY).all(), "rows of no request were written"
    if ph:
        assert (raw_rows[:, Hq:] == CANARY).all() and (raw_rows[:, :, D * esz:] == CANARY).all(), "write outside the view"
    assert np.isnan(got_lse[Tq:]).all()
    work = sum(lens) * Hkv
    what = case["name"]
    if work <= DENSE_LIMIT:
        ref = orc.ref_attention_paged(q_used[:Tq], c, qsl, D ** -0.5, window=case["window"], causal=case["causal"])
        check_out(got[:Tq], ref.out, what=what, relative=True)
        check_lse(got_lse[:Tq], ref.lse, what=what)
    else:
        picks = sorted({(int(t), int(h)) for t, h in zip(rng.integers(0, Tq, 16), rng.integers(0, Hq, 16))}
                       | {(0, 0), (Tq - 1, Hq - 1)})
        ref_out, ref_lse = orc.ref_attention_rows(q_used, c, qsl, D ** -0.5, picks, window=case["window"],
                                                  causal=case["causal"])
        sel = np.stack([got[t, h] for t, h in picks])
        check_out(sel, ref_out, what=what, relative=True)
        check_lse(np.array([got_lse[t, h] for t, h in picks]), ref_lse, what=what)
        # every row against the CUDA-core kernel
        out2 = torch.full((T, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        lse2 = torch.full((T, Hq), float("nan"), dtype=torch.float32, device="cuda")
        host.attention_forward(q, out2, views, bt, lens_t, qsl_t, num_splits=1, lse_out=lse2,
                               kernel=capi.KERNEL_SCALAR, **kw)
        torch.cuda.synchronize()
        d = (out.float()[:Tq] - out2[:Tq]).abs()
        assert float(d.max()) <= OUT_MAX_TOL and float(d.mean()) <= OUT_MEAN_TOL, (what, float(d.max()))
        live = torch.isfinite(lse2[:Tq])
        assert float((lse[:Tq][live] - lse2[:Tq][live]).abs().max()) <= LSE_TOL, what
    del storage


@pytest.mark.parametrize("family", FAMILIES)
def test_reference_grid_family(family):
    failures = []
    cases = [c for c in CASES if c["family"] == family]
    for case in cases:
        try:
            _run(case)
        except AssertionError as e:   # collect: one bad case must not hide the others
            failures.append(f"{case['name']}: {e}")
        torch.cuda.empty_cache()
    assert not failures, f"{len(failures)} of {len(cases)} cases failed:\n" + "\n".join(failures[:20])
