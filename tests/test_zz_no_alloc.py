"""GPU test of ``pthb200_attention_noalloc``: the split partials live in the library's
built-in device array instead of a caller workspace.

Collected last (file name), so it runs after every other GPU test has used the same
device, and it must also pass alone.  Each case calls the entry point twice in a row
through the C ABI and compares both results with ``pthb200_attention`` +
``pthb200_combine`` on a caller workspace, within the tolerances of the parity tests
(bf16 output max |d| <= 2e-2, mean |d| <= 2e-3), and with the oracle.
"""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host
from tests.helpers import check_out

pytestmark = pytest.mark.gpu


def _case(seed, lens, q_len, num_splits, Hq=32, Hkv=8, D=128):
    from tests.gpu_util import cache_to_device, q_to_device

    rng = np.random.default_rng(seed)
    c = orc.make_paged_cache(lens, Hkv, D, 16, seed=seed)
    R = len(lens)
    qsl = np.arange(R + 1, dtype=np.int32) * q_len
    T = int(qsl[-1])
    q_f32 = orc.round_to_bf16(rng.standard_normal((T, Hq, D), dtype=np.float32))
    scale = D ** -0.5
    ref = orc.ref_attention_paged(q_f32, c, qsl, scale)
    storage, views, bt, lens_t = cache_to_device(c)
    q = q_to_device(q_f32)
    qsl_t = torch.from_numpy(qsl).cuda()
    bq = max(1, min(64 // (Hq // Hkv), q_len))

    def fresh_out():
        return torch.full((T, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")

    # the existing entry points, on a workspace of the caller
    out_ws = fresh_out()
    ws_o = torch.full((num_splits, T, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    ws_lse = torch.full((num_splits, T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    host.attention_forward(q, out_ws, views, bt, lens_t, qsl_t, bq=bq, num_splits=num_splits,
                           softmax_scale=scale, ws_o=ws_o, ws_lse=ws_lse)
    torch.cuda.synchronize()

    lib = capi.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):  # two calls in a row share the built-in array
        out = fresh_out()
        a = host.fill_attn_args(q, out, views, bt, lens_t, qsl_t, bq=bq, num_splits=num_splits,
                                softmax_scale=scale)
        rc = lib.attention_noalloc(a, stream=stream)
        assert rc == capi.OK, lib.last_error()
        outs.append(out)
    torch.cuda.synchronize()
    assert lib.device_status() == 0
    want = out_ws.float().cpu().numpy()
    valid = np.ones(T, dtype=bool)
    for k, out in enumerate(outs):
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all(), f"call {k}: rows were left unwritten"
        check_out(got, want, valid, what=f"noalloc call {k} vs workspace call")
        check_out(got, ref.out, valid, what=f"noalloc call {k} vs oracle")
    del storage


def test_noalloc_decode_splits():
    _case(11, [700, 33, 1500, 129], q_len=1, num_splits=3)


def test_noalloc_verify_splits_then_unsplit():
    _case(12, [900, 257], q_len=4, num_splits=2)
    _case(13, [300, 40], q_len=1, num_splits=1)  # no partials: the array is not used


def test_noalloc_refuses_more_than_the_array_holds():
    from tests.gpu_util import cache_to_device, q_to_device

    Hq, Hkv, D, T = 32, 8, 128, 256
    c = orc.make_paged_cache([T], Hkv, D, 16, seed=3)
    storage, views, bt, lens_t = cache_to_device(c)
    q = q_to_device(np.zeros((T, Hq, D), dtype=np.float32))
    out = torch.zeros((T, Hq, D), dtype=torch.bfloat16, device="cuda")
    qsl_t = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    a = host.fill_attn_args(q, out, views, bt, lens_t, qsl_t, bq=16, num_splits=2, softmax_scale=1.0)
    lib = capi.load_library()
    rc = lib.attention_noalloc(a, stream=torch.cuda.current_stream().cuda_stream)
    assert rc == capi.EINVAL
    msg = lib.last_error()
    assert "8388608" in msg and str(2 * T * Hq * (D + 1) * 4) in msg, msg
    torch.cuda.synchronize()
    del storage
