"""Run-to-run determinism: the same launch repeated must give the same bytes.

The kernels have no atomics and a fixed reduction order, so any difference between
two runs is a synchronisation bug (one was found this way: two threads issuing
tcgen05.mma concurrently in the row-major kernel)."""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host

pytestmark = pytest.mark.gpu

CASES = [
    # kernel, seq_lens, q_lens, Hq, Hkv, bq, splits
    (capi.KERNEL_UMMA, [4100, 9000, 300], [1, 1, 1], 32, 8, 1, 1),
    (capi.KERNEL_UMMA, [4100, 9000, 300], [4, 4, 4], 32, 8, 4, 3),
    (capi.KERNEL_UMMA, [6000], [16], 32, 8, 16, 1),
    (capi.KERNEL_UMMA_ROWS, [4100], [16], 32, 8, 16, 1),
    (capi.KERNEL_UMMA_ROWS, [3000, 700], [200, 16], 16, 2, 8, 2),
    (capi.KERNEL_UMMA_BF16, [4100, 300], [4, 4], 32, 8, 4, 1),
]


@pytest.mark.parametrize("kernel,lens,qlens,Hq,Hkv,bq,S", CASES)
def test_repeated_launches_are_identical(kernel, lens, qlens, Hq, Hkv, bq, S):
    from tests.gpu_util import cache_to_device, q_to_device

    c = orc.make_paged_cache(lens, Hkv, 128, 16, seed=31)
    rng = np.random.default_rng(32)
    T = sum(qlens)
    q = q_to_device(orc.round_to_bf16(rng.standard_normal((T, Hq, 128), dtype=np.float32)))
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32, device="cuda")
    storage, views, bt, lens_t = cache_to_device(c)
    ws_o = torch.zeros((S, T, Hq, 128), dtype=torch.float32, device="cuda") if S > 1 else None
    ws_lse = torch.zeros((S, T, Hq), dtype=torch.float32, device="cuda") if S > 1 else None
    first = None
    for run in range(40):
        out = torch.full((T, Hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        host.attention_forward(q, out, views, bt, lens_t, qsl, bq=bq, num_splits=S, softmax_scale=128 ** -0.5,
                               ws_o=ws_o, ws_lse=ws_lse, kernel=kernel)
        torch.cuda.synchronize()
        if first is None:
            first = out
        else:
            assert torch.equal(first.view(torch.int16), out.view(torch.int16)), f"run {run} differs from run 0"
    assert capi.load_library().device_status() == 0
    del storage
