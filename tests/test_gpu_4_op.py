"""GPU tests of the torch op ``pth_flash_attn::pth_flash_attn_fwd`` (the reference-facing
boundary): parity with the oracle through the op, byte equality with the C ABI call,
``opcheck``, and CUDA-graph replay with lengths rewritten in place (the counterpart of
the reference's tests/gpu/test_backend_op.py and tests/gpu/test_attn_graph.py)."""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import ops, planner
from tests.helpers import check_out

pytestmark = pytest.mark.gpu


def _views(c: orc.PagedInt8Cache, dev="cuda"):
    """The four strided tensors the op takes, as views of one device buffer."""
    storage = torch.from_numpy(c.storage).to(dev)
    i8, f32 = storage.view(torch.int8), storage.view(torch.float32)
    shape = (c.num_blocks, c.block_size, c.Hkv)

    def rows(s):
        return torch.as_strided(i8, shape + (c.D,), (s.stride_block, s.stride_slot, s.stride_head, 1), s.offset)

    def scal(s):
        assert s.offset % 4 == 0 and s.stride_block % 4 == 0 and s.stride_slot % 4 == 0 and s.stride_head % 4 == 0
        return torch.as_strided(f32, shape, (s.stride_block // 4, s.stride_slot // 4, s.stride_head // 4), s.offset // 4)

    return storage, rows(c.k), rows(c.v), scal(c.ks), scal(c.vs)


def _setup(lens, qlens, Hq=32, Hkv=8, seed=5):
    D = 128
    c = orc.make_paged_cache(lens, Hkv, D, 16, seed=seed)
    rng = np.random.default_rng(seed + 1)
    T = int(sum(qlens))
    q_f32 = orc.round_to_bf16(rng.standard_normal((T, Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    storage, kc, vc, ks, vs = _views(c)
    t = dict(
        c=c, q_f32=q_f32, qsl_np=qsl, storage=storage, k_cache=kc, v_cache=vc, k_scale=ks, v_scale=vs,
        q=torch.from_numpy(q_f32).cuda().to(torch.bfloat16), bt=torch.from_numpy(c.block_table).cuda(),
        lens=torch.from_numpy(c.seq_lens).cuda(), qsl=torch.from_numpy(qsl).cuda(), T=T, Hq=Hq, Hkv=Hkv, D=D,
        scale=D ** -0.5, q_max=int(max(qlens)), R=len(lens),
    )
    return t


def _plan(t, num_splits=None):
    plan = planner.plan_launch(num_tokens=t["T"], num_reqs=t["R"], max_query_len=t["q_max"], G=t["Hq"] // t["Hkv"],
                               Hkv=t["Hkv"], D=t["D"], num_sms=148, is_prefill=False,
                               ws_token_splits=64 * t["T"])
    S = plan.num_splits if num_splits is None else num_splits
    ws_o = torch.full((S if S > 1 else 0, t["T"], t["Hq"], t["D"]), float("nan"), dtype=torch.float32, device="cuda")
    ws_lse = torch.full((S if S > 1 else 0, t["T"], t["Hq"]), float("nan"), dtype=torch.float32, device="cuda")
    return plan.wm, S, ws_o, ws_lse


def _call(t, out, wm, S, ws_o, ws_lse, **kw):
    ops.pth_flash_attn_fwd(out, t["q"], t["k_cache"], t["v_cache"], t["k_scale"], t["v_scale"], t["bt"], t["lens"],
                           t["qsl"], t["q_max"], wm, S, t["scale"], ws_o, ws_lse, **kw)


@pytest.mark.parametrize("qlens,S", [([1, 1, 1], None), ([4, 4, 4], 3), ([16, 16, 16], 1), ([40, 3, 1], 2)])
def test_op_matches_oracle_and_c_abi(qlens, S):
    from pth_flash_attn_b200 import host

    t = _setup([900, 257, 4100], qlens)
    wm, S, ws_o, ws_lse = _plan(t, S)
    out = torch.full((t["T"], t["Hq"], t["D"]), float("nan"), dtype=torch.bfloat16, device="cuda")
    _call(t, out, wm, S, ws_o, ws_lse)
    torch.cuda.synchronize()
    ref = orc.ref_attention_paged(t["q_f32"], t["c"], t["qsl_np"], t["scale"])
    check_out(out.float().cpu().numpy(), ref.out, what=f"op q{qlens} S{S}")
    # the same launch through the C ABI gives the same bytes
    G = t["Hq"] // t["Hkv"]
    bq = max(1, min(16 * wm // G, t["q_max"]))
    out2 = torch.full_like(out, float("nan"))
    views = host.CacheViews.from_tensors(t["k_cache"], t["v_cache"], t["k_scale"], t["v_scale"])
    host.attention_forward(t["q"], out2, views, t["bt"], t["lens"], t["qsl"], bq=bq, num_splits=S,
                           softmax_scale=t["scale"], ws_o=ws_o if S > 1 else None, ws_lse=ws_lse if S > 1 else None)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_op_window_and_legacy_call():
    t = _setup([5000, 4200], [16, 16], Hq=8, Hkv=2)
    wm, S, ws_o, ws_lse = _plan(t, 2)
    out = torch.zeros((t["T"], t["Hq"], t["D"]), dtype=torch.bfloat16, device="cuda")
    _call(t, out, wm, S, ws_o, ws_lse, window=4096, causal=True)
    torch.cuda.synchronize()
    ref = orc.ref_attention_paged(t["q_f32"], t["c"], t["qsl_np"], t["scale"], window=4096)
    check_out(out.float().cpu().numpy(), ref.out, what="op window")
    # the 15-argument call is the explicit window=0, causal=True call
    a, b = torch.zeros_like(out), torch.zeros_like(out)
    _call(t, a, wm, S, ws_o, ws_lse)
    _call(t, b, wm, S, ws_o, ws_lse, window=0, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_opcheck():
    t = _setup([300, 77], [1, 1])
    wm, S, ws_o, ws_lse = _plan(t, 2)
    out = torch.zeros((t["T"], t["Hq"], t["D"]), dtype=torch.bfloat16, device="cuda")
    args = (out, t["q"], t["k_cache"], t["v_cache"], t["k_scale"], t["v_scale"], t["bt"], t["lens"], t["qsl"],
            t["q_max"], wm, S, t["scale"], ws_o, ws_lse)
    torch.library.opcheck(torch.ops.pth_flash_attn.pth_flash_attn_fwd.default, args,
                          test_utils=("test_schema", "test_faketensor"))


def test_graph_replay_with_lengths_rewritten_in_place():
    """Capture once; rewrite seq_lens in place (across page and tile edges, shrink, empty
    request); every replay equals the eager call on the same lengths byte for byte."""
    t = _setup([3000, 700, 129, 64], [4, 4, 4, 4])
    wm, S, ws_o, ws_lse = _plan(t, 3)
    out = torch.zeros((t["T"], t["Hq"], t["D"]), dtype=torch.bfloat16, device="cuda")
    _call(t, out, wm, S, ws_o, ws_lse)  # eager first: kernel attributes are set outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            _call(t, out, wm, S, ws_o, ws_lse)
    torch.cuda.synchronize()
    first = None
    for lens in ([3000, 700, 129, 64], [2999, 128, 17, 4], [16, 16, 16, 16], [1500, 4, 129, 63]):
        t["lens"].copy_(torch.tensor(lens, dtype=torch.int32))
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        replayed = out.clone()
        eager = torch.full_like(out, float("nan"))
        _call(t, eager, wm, S, ws_o, ws_lse)
        torch.cuda.synchronize()
        assert torch.equal(replayed.view(torch.int16), eager.view(torch.int16)), lens
        if first is None:
            first = replayed
    assert not torch.equal(first.view(torch.int16), replayed.view(torch.int16)), "stale lengths would pass"


def test_op_does_not_synchronise_or_allocate():
    """The op reads no device data on the host and allocates nothing (the reference pins both:
    tests/gpu/test_backend_impl.py:149-190): with the sync debug mode set to "error" a hidden
    synchronisation raises, and the allocator's counters do not move across the calls."""
    for qlens, S in (([1, 1, 1], 3), ([4, 4, 4], 1), ([40, 3, 1], 2)):
        t = _setup([3000, 700, 129], qlens)
        wm, S, ws_o, ws_lse = _plan(t, S)
        out = torch.zeros((t["T"], t["Hq"], t["D"]), dtype=torch.bfloat16, device="cuda")
        _call(t, out, wm, S, ws_o, ws_lse)   # first call: kernel attributes, page map
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats()
        torch.cuda.set_sync_debug_mode("error")
        try:
            for _ in range(3):
                _call(t, out, wm, S, ws_o, ws_lse)
        finally:
            torch.cuda.set_sync_debug_mode("default")
        torch.cuda.synchronize()
        after = torch.cuda.memory_stats()
        for key in ("allocation.all.allocated", "allocated_bytes.all.allocated", "segment.all.allocated",
                    "reserved_bytes.all.allocated"):
            assert after[key] == before[key], key
        ref = orc.ref_attention_paged(t["q_f32"], t["c"], t["qsl_np"], t["scale"])
        check_out(out.float().cpu().numpy(), ref.out, what=f"q {qlens} S {S}")


@pytest.mark.parametrize("qlens,S", [([1, 1, 1], 1), ([4, 4, 2], 3), ([16, 9], 2)])
def test_fp16_queries_and_output(qlens, S):
    """fp16 q / out through the op: the integer kernel turns the queries into int8 digits
    whatever their 16-bit format is."""
    lens = [2500, 300, 77][:len(qlens)]
    t = _setup(lens, qlens)
    q16 = torch.from_numpy(t["q_f32"]).cuda().to(torch.float16)
    t["q"] = q16
    wm, S, ws_o, ws_lse = _plan(t, S)
    out = torch.full((t["T"], t["Hq"], t["D"]), float("nan"), dtype=torch.float16, device="cuda")
    _call(t, out, wm, S, ws_o, ws_lse)
    torch.cuda.synchronize()
    ref = orc.ref_attention_paged(q16.float().cpu().numpy(), t["c"], t["qsl_np"], t["scale"])
    check_out(out.float().cpu().numpy(), ref.out, what=f"fp16 q {qlens} S {S}")
    from pth_flash_attn_b200 import capi
    assert capi.load_library().device_status() == 0
