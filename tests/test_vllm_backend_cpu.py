"""The vLLM backend on CPU tensors: builder, implementation, cache views, plugin.

No GPU and no vLLM engine: the op is replaced by a recorder, the vLLM configuration by a
namespace with exactly the fields the backend reads, and the workspace manager is vLLM's own
on the CPU device - the arrangement of the reference's backend tests
(tests/cpu/test_backend_builder.py:3-12).  What is pinned:

* graph level ``UNIFORM_BATCH`` and the decode threshold ``max(64 // G, 1 + k)``;
* every op call carries exactly ``planner.plan_launch`` of its own padded descriptor; a mixed
  step is the decode-like call followed by the prefill call, whose ``query_start_loc`` is
  rebased from the DEVICE values; a capture build sets the lengths to 1;
* the implementation reserves its workspace at construction, issues at most two op calls
  with views of the caller's tensors, and allocates nothing once the workspace is locked;
* the cache views address the same bytes as the oracle's cache image, for both physical
  layouts vLLM has used;
* everything the kernels do not serve is refused with its reason;
* the module makes no ``torch.cuda`` call.

Skipped as a whole when vLLM cannot be imported.
"""
from __future__ import annotations

import random
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytest.importorskip("vllm")

from vllm.v1.attention.backend import AttentionCGSupport, CommonAttentionMetadata  # noqa: E402
from vllm.v1.worker import workspace as vllm_workspace  # noqa: E402

from oracle import paged_int8_attention as orc  # noqa: E402
from pth_flash_attn_b200 import planner, plugin, vllm_backend  # noqa: E402
from pth_flash_attn_b200.vllm_backend import (  # noqa: E402
    PthFlashAttnBackend,
    PthFlashAttnImpl,
    PthFlashAttnMetadataBuilder,
    cache_views,
    reserved_token_splits,
    verify_query_len,
)

HQ, HKV, D, SMS = 32, 8, 128, 148
G = HQ // HKV


def make_config(*, k=3, max_num_seqs=8, heads=HQ, rswa=None, dbo=False):
    spec = None if k is None else SimpleNamespace(num_speculative_tokens=k, parallel_drafting=False)
    return SimpleNamespace(
        model_config=SimpleNamespace(rswa_window=rswa, get_num_attention_heads=lambda pc: heads),
        parallel_config=SimpleNamespace(use_ubatching=dbo, num_ubatches=2 if dbo else 1,
                                        decode_context_parallel_size=1),
        scheduler_config=SimpleNamespace(max_num_seqs=max_num_seqs),
        speculative_config=spec,
        compilation_config=SimpleNamespace(static_forward_context={}),
    )


def make_spec(num_kv_heads=HKV, head_size=D, sliding_window=None):
    spec = SimpleNamespace(num_kv_heads=num_kv_heads, head_size=head_size)
    if sliding_window is not None:
        spec.sliding_window = sliding_window
    return spec


@pytest.fixture(autouse=True)
def fixed_sm_count(monkeypatch):
    monkeypatch.setattr(vllm_backend, "_num_sms", lambda device=None: SMS)


def make_builder(**cfg):
    spec = make_spec(cfg.pop("num_kv_heads", HKV), cfg.pop("head_size", D), cfg.pop("sliding_window", None))
    return PthFlashAttnMetadataBuilder(spec, ["layers.0.attn"], make_config(**cfg), torch.device("cpu"))


def make_cam(q_lens, seq_lens=None, *, device_qsl=None, max_reqs=8, **kw):
    qsl = [0]
    for q in q_lens:
        qsl.append(qsl[-1] + q)
    seqs = seq_lens if seq_lens is not None else [q + 500 for q in q_lens]
    host = torch.tensor(qsl, dtype=torch.int32)
    dev = torch.tensor(device_qsl, dtype=torch.int32) if device_qsl else host
    seq_buf = torch.zeros(max_reqs, dtype=torch.int32)
    seq_buf[:len(seqs)] = torch.tensor(seqs, dtype=torch.int32)
    return CommonAttentionMetadata(
        query_start_loc=dev, query_start_loc_cpu=host, seq_lens=seq_buf[:len(q_lens)], num_reqs=len(q_lens),
        num_actual_tokens=qsl[-1], max_query_len=max(q_lens), max_seq_len=max(seqs),
        block_table_tensor=torch.zeros(max_reqs, 8, dtype=torch.int32),
        slot_mapping=torch.zeros(qsl[-1], dtype=torch.int64), **kw)


def plan_of(builder, tokens, reqs, q_max, is_prefill):
    return planner.plan_launch(num_tokens=tokens, num_reqs=reqs, max_query_len=q_max, G=builder.group,
                               Hkv=builder.num_kv_heads, D=builder.head_size, num_sms=SMS, is_prefill=is_prefill,
                               ws_token_splits=builder.ws_token_splits, window=builder.window)


# ------------------------------------------------------------------ builder
def test_graph_level_and_decode_threshold():
    assert PthFlashAttnBackend.get_builder_cls() is PthFlashAttnMetadataBuilder
    assert PthFlashAttnMetadataBuilder._cudagraph_support is AttentionCGSupport.UNIFORM_BATCH
    assert make_builder(k=3).reorder_batch_threshold == max(64 // G, 4) == 16
    assert make_builder(k=None, heads=64, num_kv_heads=1).reorder_batch_threshold == 1   # G = 64
    assert make_builder(k=7, heads=64, num_kv_heads=2).reorder_batch_threshold == 8      # G = 32: 1 + k wins
    cfg = make_config(k=7, heads=64)
    assert PthFlashAttnMetadataBuilder.get_varlen_cudagraph_max_query_len(cfg, make_spec(2)) == 8
    assert verify_query_len(make_config(k=None)) == 1 and verify_query_len(make_config(k=5)) == 6


def test_decode_step_is_one_call_with_its_plan():
    b = make_builder()
    cam = make_cam([4, 4, 4])
    md = b.build(0, cam)
    assert len(md.calls) == 1 and md.prefill is None
    call = md.decode
    assert call.plan == plan_of(b, 12, 3, 4, False)
    assert call.tokens == slice(0, 12) and call.max_query_len == 4
    assert call.query_start_loc.data_ptr() == cam.query_start_loc.data_ptr()
    assert call.seq_lens.data_ptr() == cam.seq_lens.data_ptr() and call.seq_lens.shape == (3,)
    assert call.block_table.shape[0] == 3


def test_mixed_step_is_decode_call_then_prefill_call_rebased_on_the_device():
    b = make_builder()
    # the device copy of the starts is behind the host one for the first request (adaptive verification)
    cam = make_cam([4, 1, 300, 40], device_qsl=[0, 2, 3, 303, 343])
    md = b.build(0, cam)
    assert [c.plan.is_prefill for c in md.calls] == [False, True]
    dec, pre = md.calls
    assert dec.plan == plan_of(b, 5, 2, 4, False) and dec.tokens == slice(0, 5)
    assert dec.query_start_loc.tolist() == [0, 2, 3]
    assert pre.plan == plan_of(b, 340, 2, 300, True) and pre.tokens == slice(5, 345)
    assert pre.query_start_loc.tolist() == [0, 300, 340]            # device values, rebased
    assert pre.query_start_loc.data_ptr() == b._rebased_qsl.data_ptr()  # the persistent buffer
    assert pre.seq_lens.tolist() == cam.seq_lens[2:].tolist()
    # a second build reuses the buffer
    again = b.build(0, make_cam([1, 200]))
    assert again.prefill.query_start_loc.data_ptr() == b._rebased_qsl.data_ptr()


def test_prefill_only_and_padded_decode_batches():
    b = make_builder()
    md = b.build(0, make_cam([100, 17]))
    assert len(md.calls) == 1 and md.decode is None and md.prefill.plan == plan_of(b, 117, 2, 100, True)
    assert md.prefill.query_start_loc.tolist() == [0, 100, 117]
    md = b.build(0, make_cam([1] * 8))
    assert len(md.calls) == 1 and md.decode.plan == plan_of(b, 8, 8, 1, False)


def test_capture_build_sets_lengths_to_one():
    b = make_builder()
    cam = make_cam([1, 1, 1], seq_lens=[4000, 9000, 77])
    md = b.build_for_cudagraph_capture(cam)
    assert md.seq_lens.tolist() == [1, 1, 1] and md.decode.plan == plan_of(b, 3, 3, 1, False)


def test_no_plan_exceeds_the_reservation():
    rnd = random.Random(1)
    for _ in range(100):
        k = rnd.choice([None, 1, 3, 7])
        b = make_builder(k=k, max_num_seqs=8)
        q = [rnd.randint(1, (k or 0) + 1) for _ in range(rnd.randint(1, 8))]
        for call in b.build(0, make_cam(q)).calls:
            assert call.plan.ws_token_splits_used <= b.ws_token_splits
    cfg = make_config(k=3, max_num_seqs=8)
    assert make_builder(k=3).ws_token_splits == reserved_token_splits(cfg, num_kv_heads=HKV, head_size=D, num_sms=SMS)


def test_builder_refusals():
    with pytest.raises(NotImplementedError, match="dual-batch"):
        make_builder(dbo=True)
    with pytest.raises(NotImplementedError, match="R-SWA"):
        make_builder(rswa=128)
    with pytest.raises(NotImplementedError, match="head size 96"):
        make_builder(head_size=96)
    with pytest.raises(NotImplementedError, match="sliding window at head size 256"):
        make_builder(head_size=256, sliding_window=2048)
    with pytest.raises(ValueError, match="multiple"):
        make_builder(heads=30)
    b = make_builder()
    with pytest.raises(NotImplementedError, match="cascade"):
        b.build(16, make_cam([1, 1]))
    with pytest.raises(NotImplementedError, match="per-request causal"):
        b.build(0, make_cam([1, 1], causal=torch.ones(2, dtype=torch.bool)))
    with pytest.raises(NotImplementedError, match="non-causal attention at head size 64"):
        make_builder(head_size=64).build(0, make_cam([1, 1], causal=False))
    assert make_builder(sliding_window=4096).window == 4096
    assert make_builder(sliding_window=4096).build(0, make_cam([1] * 2)).decode.plan.num_splits <= 34


# ------------------------------------------------------------------ implementation
class Recorder:
    def __init__(self):
        self.calls = []

    def __call__(self, *args):
        self.calls.append(args)


@pytest.fixture
def cpu_workspace():
    vllm_workspace.reset_workspace_manager()
    vllm_workspace.init_workspace_manager(torch.device("cpu"))
    yield vllm_workspace.current_workspace_manager()
    vllm_workspace.reset_workspace_manager()


def make_impl(monkeypatch, config=None, **kw):
    monkeypatch.setattr(vllm_backend, "get_current_vllm_config_or_none", lambda: config)
    args = dict(num_heads=HQ, head_size=D, scale=D ** -0.5, num_kv_heads=HKV, alibi_slopes=None,
                sliding_window=None, kv_cache_dtype="int8_per_token_head")
    args.update(kw)
    return PthFlashAttnImpl(**args)


def packed_cache(blocks=6, slots=16):
    return torch.zeros(blocks, HKV, slots, 2 * (D + 4), dtype=torch.int8)


def test_forward_issues_the_planned_calls_on_views(monkeypatch, cpu_workspace):
    rec = Recorder()
    monkeypatch.setattr(vllm_backend.ops, "pth_flash_attn_fwd", rec)
    cfg = make_config()
    impl = make_impl(monkeypatch, cfg)
    assert impl._ws_token_splits == reserved_token_splits(cfg, num_kv_heads=HKV, head_size=D, num_sms=SMS)
    b = make_builder()
    cam = make_cam([4, 1, 300])
    md = b.build(0, cam)
    T = 305
    q = torch.zeros(T, HQ, D, dtype=torch.bfloat16)
    out = torch.ones(T, HQ, D, dtype=torch.bfloat16)
    kv = packed_cache()
    cpu_workspace.lock()   # from here on a growing workspace would raise
    assert impl.forward(None, q, None, None, kv, md, out) is out
    assert len(rec.calls) == 2
    for got, call in zip(rec.calls, md.calls):
        o, qq, k, v, ks, vs, bt, lens, qsl, q_max, wm, S, scale, ws_o, ws_lse, window, causal = got
        assert o.data_ptr() == out[call.tokens].data_ptr() and o.shape[0] == call.tokens.stop - call.tokens.start
        assert qq.data_ptr() == q[call.tokens].data_ptr()
        assert k.shape == (6, 16, HKV, D) and ks.shape == (6, 16, HKV) and ks.dtype == torch.float32
        assert bt is call.block_table and lens is call.seq_lens and qsl is call.query_start_loc
        assert (q_max, wm, S) == (call.max_query_len, call.plan.wm, call.plan.num_splits)
        assert scale == pytest.approx(D ** -0.5) and window == 0 and causal is True
        if S > 1:
            assert tuple(ws_o.shape) == call.plan.ws_o_shape and tuple(ws_lse.shape) == call.plan.ws_lse_shape
        else:
            assert ws_o.numel() == 0 and ws_lse.numel() == 0
    # the views are built once per cache tensor
    first = impl._caches(kv)
    assert impl._caches(kv) is first and impl._caches(packed_cache()) is not first
    # the memory-profile run executes nothing
    n = len(rec.calls)
    assert impl.forward(None, q, None, None, kv, None, out).abs().sum() == 0 and len(rec.calls) == n


def test_forward_refuses_a_launch_beyond_the_reservation(monkeypatch, cpu_workspace):
    monkeypatch.setattr(vllm_backend.ops, "pth_flash_attn_fwd", Recorder())
    impl = make_impl(monkeypatch, make_config(max_num_seqs=1, k=None))
    b = make_builder(max_num_seqs=8, k=3)     # a builder configured for more than the layer reserved
    md = b.build(0, make_cam([4] * 8))
    if md.decode.plan.ws_token_splits_used > impl._ws_token_splits:
        with pytest.raises(RuntimeError, match="token-splits"):
            impl.forward(None, torch.zeros(32, HQ, D, dtype=torch.bfloat16), None, None, packed_cache(), md,
                         torch.zeros(32, HQ, D, dtype=torch.bfloat16))


def test_impl_refusals(monkeypatch):
    for kw, text in ((dict(alibi_slopes=[1.0] * HQ), "ALiBi"), (dict(logits_soft_cap=30.0), "soft cap"),
                     (dict(sinks=torch.zeros(HQ)), "sinks"), (dict(kv_cache_dtype="fp8"), "kv_cache_dtype fp8"),
                     (dict(head_size=96), "head size 96"), (dict(sliding_window=0), "sliding window 0"),
                     (dict(head_size=256, sliding_window=512), "sliding window at head size 256"),
                     (dict(attn_type="encoder"), "attention type")):
        with pytest.raises(NotImplementedError, match=text):
            make_impl(monkeypatch, None, **kw)
    impl = make_impl(monkeypatch, None, sliding_window=2048)
    assert impl.window == 2048
    with pytest.raises(NotImplementedError, match="fused output quantisation"):
        impl.forward(None, None, None, None, None, None, None, output_scale=torch.ones(1))


def test_backend_class_answers():
    B = PthFlashAttnBackend
    assert B.get_name() == "CUSTOM" and B.get_impl_cls() is PthFlashAttnImpl
    assert B.supports_block_size(None) and B.supports_block_size(816) and not B.supports_block_size(24)
    assert [B.supports_head_size(d) for d in (64, 96, 128, 256)] == [True, False, True, True]
    assert B.supports_attn_type("decoder") and not B.supports_attn_type("encoder")
    assert not B.supports_rswa() and not B.supports_sink() and not B.supports_batch_invariance()
    cap = lambda major: SimpleNamespace(major=major, minor=0)  # noqa: E731
    assert not B.supports_compute_capability(cap(8)) and not B.supports_compute_capability(cap(9))
    assert B.supports_compute_capability(cap(10)) == vllm_backend.ops.is_available()
    assert B.supported_kv_cache_dtypes == ["int8_per_token_head"]


# ------------------------------------------------------------------ cache views
@pytest.mark.parametrize("layout", ["packed_hnd", "split_halves"])
def test_cache_views_address_the_cells_of_the_oracle_image(layout):
    Hkv, Dh, BS, blocks = 2, 128, 16, 5
    c = orc.make_paged_cache([70, 9], Hkv, Dh, BS, layout="HND", seed=4)
    if layout == "packed_hnd":
        raw = torch.from_numpy(c.storage.copy()).view(torch.int8)
        kv = raw[: c.num_blocks * c.page_bytes].view(c.num_blocks, Hkv, BS, 2 * (Dh + 4))
    else:
        kv = torch.zeros(c.num_blocks, 2, BS, Hkv, Dh + 4, dtype=torch.int8)
        kv[:, 0, :, :, :Dh] = torch.from_numpy(c.k_cache.copy())
        kv[:, 1, :, :, :Dh] = torch.from_numpy(c.v_cache.copy())
        kv[:, 0, :, :, Dh:] = torch.from_numpy(c.k_scale.copy()).view(torch.int8).view(c.num_blocks, BS, Hkv, 4)
        kv[:, 1, :, :, Dh:] = torch.from_numpy(c.v_scale.copy()).view(torch.int8).view(c.num_blocks, BS, Hkv, 4)
    k, v, ks, vs = cache_views(kv, Dh)
    assert k.shape == (c.num_blocks, BS, Hkv, Dh) and ks.shape == (c.num_blocks, BS, Hkv)
    assert np.array_equal(k.numpy(), c.k_cache) and np.array_equal(v.numpy(), c.v_cache)
    assert np.array_equal(ks.numpy(), c.k_scale) and np.array_equal(vs.numpy(), c.v_scale)
    assert k.data_ptr() == kv.data_ptr()   # views, not copies
    with pytest.raises(NotImplementedError, match="unknown"):
        cache_views(torch.zeros(3, 4, 5, dtype=torch.int8), Dh)


# ------------------------------------------------------------------ plugin and module hygiene
def test_plugin_registers_custom_once_and_yields_to_others(monkeypatch):
    from vllm.v1.attention.backends import registry

    member = registry.AttentionBackendEnum.CUSTOM
    saved = dict(registry._ATTN_OVERRIDES) if hasattr(registry, "_ATTN_OVERRIDES") else None
    try:
        if member.is_overridden():
            member.clear_override()
        assert plugin.register() is True
        assert member.get_path() == plugin.BACKEND_CLASS_PATH == "pth_flash_attn_b200.vllm_backend.PthFlashAttnBackend"
        assert plugin.register() is True     # idempotent
        registry.register_backend(member, "someone.else.Backend")
        assert plugin.register() is False and member.get_path() == "someone.else.Backend"
    finally:
        if member.is_overridden():
            member.clear_override()
        if saved is not None:
            registry._ATTN_OVERRIDES.update(saved)


def test_backend_module_makes_no_torch_cuda_call():
    for name in ("vllm_backend.py", "plugin.py", "planner.py"):
        text = (Path(vllm_backend.__file__).parent / name).read_text()
        code = "\n".join(line.split("#")[0] for line in text.splitlines())
        code = code.replace("``torch.cuda``", "")
        assert "torch.cuda" not in code, name
