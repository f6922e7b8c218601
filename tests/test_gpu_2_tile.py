"""Unit test of the tcgen05 building blocks: widening, operand images, both MMA chains."""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("padded", [1, 0])
def test_umma_tile(padded):
    lib = capi.load_library()
    rng = np.random.default_rng(3)
    k = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    v = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    k[0, :4] = [-128, 127, 0, -1]
    q = orc.round_to_bf16(rng.standard_normal((16, 128), dtype=np.float32))
    pm = orc.round_to_bf16(rng.random((128, 16), dtype=np.float32))
    dev = "cuda"
    kt, vt = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    qt = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    pt = torch.from_numpy(pm).to(dev).to(torch.bfloat16)
    s_out = torch.full((128, 16), float("nan"), dtype=torch.float32, device=dev)
    o_out = torch.full((128, 16), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.lib.pthb200_test_tile(kt.data_ptr(), qt.data_ptr(), vt.data_ptr(), pt.data_ptr(),
                                   s_out.data_ptr(), o_out.data_ptr(), padded, None)
    assert rc == capi.OK
    assert lib.device_status() == 0, "a bounded wait gave up"
    s_want = k.astype(np.float64) @ q.astype(np.float64).T          # [key][n]
    o_want = v.astype(np.float64).T @ pm.astype(np.float64)         # [d][n]
    s_got, o_got = s_out.cpu().numpy(), o_out.cpu().numpy()
    # products are exact in fp32; only the accumulation order differs
    np.testing.assert_allclose(s_got, s_want, rtol=1e-5, atol=1e-2)
    np.testing.assert_allclose(o_got, o_want, rtol=1e-5, atol=1e-2)


def test_umma_tile_int8():
    """Raw int8 operand images, both integer MMA chains, int32 accumulators: exact."""
    lib = capi.load_library()
    rng = np.random.default_rng(8)
    k = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    v = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    q = rng.integers(-128, 128, size=(32, 128), dtype=np.int8)
    pm = rng.integers(0, 128, size=(128, 48), dtype=np.int8)
    dev = "cuda"
    kt, vt, qt, pt = (torch.from_numpy(a).to(dev) for a in (k, v, q, pm))
    s_out = torch.full((128, 32), -7, dtype=torch.int32, device=dev)
    o_out = torch.full((128, 48), -7, dtype=torch.int32, device=dev)
    rc = lib.lib.pthb200_test_tile_i8(kt.data_ptr(), qt.data_ptr(), vt.data_ptr(), pt.data_ptr(),
                                      s_out.data_ptr(), o_out.data_ptr(), None)
    assert rc == capi.OK
    assert lib.device_status() == 0, "a bounded wait gave up"
    s_want = k.astype(np.int64) @ q.astype(np.int64).T
    o_want = v.astype(np.int64).T @ pm.astype(np.int64)
    assert np.array_equal(s_out.cpu().numpy(), s_want)
    assert np.array_equal(o_out.cpu().numpy(), o_want)


def test_umma_tile_rows():
    """Row-major building blocks: S = Q K^T (rows on M) and O = P V with P read from TMEM."""
    lib = capi.load_library()
    rng = np.random.default_rng(21)
    k = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    v = rng.integers(-128, 128, size=(128, 128), dtype=np.int8)
    q = orc.round_to_bf16(rng.standard_normal((128, 128), dtype=np.float32))
    pm = orc.round_to_bf16(rng.random((128, 128), dtype=np.float32))
    dev = "cuda"
    kt, vt = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    qt = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    pt = torch.from_numpy(pm).to(dev).to(torch.bfloat16)
    s_out = torch.full((128, 128), float("nan"), dtype=torch.float32, device=dev)
    o_out = torch.full((128, 128), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.lib.pthb200_test_tile_rows(kt.data_ptr(), qt.data_ptr(), vt.data_ptr(), pt.data_ptr(),
                                        s_out.data_ptr(), o_out.data_ptr(), None)
    assert rc == capi.OK
    assert lib.device_status() == 0, "a bounded wait gave up"
    s_want = q.astype(np.float64) @ k.astype(np.float64).T          # [row][key]
    o_want = pm.astype(np.float64) @ v.astype(np.float64)           # [row][d]
    np.testing.assert_allclose(s_out.cpu().numpy(), s_want, rtol=1e-5, atol=1e-2)
    np.testing.assert_allclose(o_out.cpu().numpy(), o_want, rtol=1e-5, atol=1e-2)
