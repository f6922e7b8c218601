"""The paged-copy ceiling kernel runs the schedule of the attention kernel to its end and
reports no give-up, for every cache geometry the integer kernel serves, and refuses what that
kernel refuses.  (It writes nothing, so there is nothing else to compare.)"""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout,Hkv,S", [("NHD", 8, 1), ("NHD", 8, 5), ("HND", 2, 3), ("NHD", 1, 37)])
def test_copy_ceiling_runs_to_completion(layout, Hkv, S):
    from tests.gpu_util import cache_to_device, q_to_device

    lens, qlens = [9000, 300, 0, 4100, 77], [1, 1, 1, 1, 1]
    lens[2] = 1
    c = orc.make_paged_cache(lens, Hkv, 128, 16, layout=layout, seed=8)
    storage, views, bt, lens_t = cache_to_device(c)
    T, Hq = sum(qlens), 4 * Hkv
    q = q_to_device(np.zeros((T, Hq, 128), dtype=np.float32))
    out = torch.zeros((T, Hq, 128), dtype=torch.bfloat16, device="cuda")
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32, device="cuda")
    ws_o = torch.zeros((S, T, Hq, 128), dtype=torch.float32, device="cuda") if S > 1 else None
    ws_lse = torch.zeros((S, T, Hq), dtype=torch.float32, device="cuda") if S > 1 else None
    a = host.fill_attn_args(q, out, views, bt, lens_t, qsl, bq=1, num_splits=S, softmax_scale=1.0, ws_o=ws_o,
                            ws_lse=ws_lse)
    lib = capi.load_library()
    for _ in range(3):
        assert lib.copy_ceiling(a, stream=torch.cuda.current_stream().cuda_stream) == capi.OK, lib.last_error()
    torch.cuda.synchronize()
    assert lib.device_status() == 0
    assert float(out.abs().sum()) == 0.0   # nothing is written
    del storage


def test_copy_ceiling_refuses_what_the_integer_kernel_refuses():
    from tests.gpu_util import cache_to_device, q_to_device

    lib = capi.load_library()
    # pages of 40 slots are not made of runs of 16: no TMA page copies, no integer kernel;
    # head size 64 has an integer kernel, but the ceiling program is built for 128
    for D, bs, reason in ((128, 40, "integer kernel"), (64, 16, "head size 128")):
        c = orc.make_paged_cache([100], 2, D, bs, seed=1)
        storage, views, bt, lens_t = cache_to_device(c)
        q = q_to_device(np.zeros((1, 8, D), dtype=np.float32))
        out = torch.zeros((1, 8, D), dtype=torch.bfloat16, device="cuda")
        qsl = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
        a = host.fill_attn_args(q, out, views, bt, lens_t, qsl, bq=1, num_splits=1, softmax_scale=1.0)
        assert lib.copy_ceiling(a) == capi.EINVAL and reason in lib.last_error(), lib.last_error()
        del storage
