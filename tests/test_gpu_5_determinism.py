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

# kernel, seq_lens, q_lens, Hq, Hkv, bq, splits, repeats, head size: long runs of the tcgen05 families.
# Row-major launches: prefill chunks (256 rows or more per request on average: two row tiles per CTA at
# 128 dims), drafter / wide-verification sizes (the one-tile kernel, whose raw ring is shared by two
# producer halves), and the kernels of the other head sizes.
LONG_CASES = [
    (capi.KERNEL_UMMA_ROWS, [4096, 700], [2048, 40], 16, 2, 8, 1, 300, 128),
    (capi.KERNEL_UMMA_ROWS, [6000, 3000], [300, 16], 32, 8, 16, 3, 300, 128),
    (capi.KERNEL_UMMA_ROWS, [9000, 5000, 700], [16, 16, 40], 32, 8, 16, 2, 300, 128),
    (capi.KERNEL_UMMA, [20000, 9000, 300, 4100], [1, 1, 1, 1], 32, 8, 1, 4, 300, 128),
    (capi.KERNEL_UMMA, [9000, 2500], [4, 4], 32, 8, 4, 2, 300, 128),
    (capi.KERNEL_AUTO, [9000, 700, 3000, 64], [1, 300, 4, 1], 16, 2, 8, 2, 300, 128),
    (capi.KERNEL_UMMA_ROWS, [4096, 700], [1024, 40], 12, 2, 10, 2, 200, 256),
    (capi.KERNEL_UMMA, [20000, 9000, 300], [1, 2, 1], 12, 2, 2, 3, 200, 256),
    (capi.KERNEL_UMMA_ROWS, [4096, 700], [1024, 40], 16, 4, 16, 1, 200, 64),
    (capi.KERNEL_UMMA, [20000, 9000, 300], [1, 4, 1], 16, 4, 4, 3, 200, 64),
]

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


@pytest.mark.parametrize("kernel,lens,qlens,Hq,Hkv,bq,S,repeats,D", LONG_CASES)
def test_many_repeats_on_cold_and_warm_caches(kernel, lens, qlens, Hq, Hkv, bq, S, repeats, D):
    """A rare ordering bug shows as one launch in a hundred: repeat each launch 300 times, with
    a buffer larger than L2 written between some of them (so that page copies arrive in other
    orders), and compare every result with the first on the device."""
    from tests.gpu_util import cache_to_device, q_to_device

    c = orc.make_paged_cache(lens, Hkv, D, 16, seed=41)
    rng = np.random.default_rng(42)
    T = sum(qlens)
    q = q_to_device(orc.round_to_bf16(rng.standard_normal((T, Hq, D), dtype=np.float32)))
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32, device="cuda")
    storage, views, bt, lens_t = cache_to_device(c)
    ws_o = torch.zeros((S, T, Hq, D), dtype=torch.float32, device="cuda") if S > 1 else None
    ws_lse = torch.zeros((S, T, Hq), dtype=torch.float32, device="cuda") if S > 1 else None
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
    first = None
    differing = torch.zeros((), dtype=torch.int32, device="cuda")
    for run in range(repeats):
        if run % 7 == 3:
            flush.fill_(run & 0xFF)
        out = torch.full((T, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        host.attention_forward(q, out, views, bt, lens_t, qsl, bq=bq, num_splits=S, softmax_scale=D ** -0.5,
                               ws_o=ws_o, ws_lse=ws_lse, kernel=kernel)
        if first is None:
            first = out
        else:
            differing += (first.view(torch.int16) != out.view(torch.int16)).any().to(torch.int32)
    torch.cuda.synchronize()
    assert int(differing.item()) == 0, f"{int(differing.item())} of {repeats} launches differ from the first"
    assert capi.load_library().device_status() == 0
    ref = orc.ref_attention_paged(q.float().cpu().numpy(), c, qsl.cpu().numpy(), D ** -0.5)
    from tests.helpers import check_out
    check_out(first.float().cpu().numpy(), ref.out, what="repeated launch")
    del storage
