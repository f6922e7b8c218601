"""GPU test of the quantising cache writer (``pthb200_write_kv``).

Bit-exact against the oracle's writer (``quantize_rows``, itself pinned to the reference's
mirror of vLLM's writer by tests/golden/writer.npz): the int8 bytes and the fp32 scales the
kernel stores equal the oracle's for fp32, bf16 and fp16 sources, every head size, both page
layouts, padded pages and a storage offset; skipped tokens and every byte outside the
written rows keep their previous content; and a cache written by this kernel reads back
through the attention op like one written by the oracle.
"""
import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host
from tests.helpers import check_out, load_golden

pytestmark = pytest.mark.gpu

DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _empty_cache(num_blocks, Hkv, D, BS, layout, pad=0, offset=0, seed=0):
    page = Hkv * BS * 2 * (D + 4) + pad
    rng = np.random.default_rng(seed)
    storage = rng.integers(0, 256, size=offset + num_blocks * page, dtype=np.uint8)
    k, v, ks, vs = orc.stream_views(D, Hkv, BS, layout, page, offset)
    return orc.PagedInt8Cache(storage=storage, k=k, v=v, ks=ks, vs=vs, block_table=np.zeros((1, 1), np.int32),
                              seq_lens=np.zeros(1, np.int32), num_blocks=num_blocks, block_size=BS, Hkv=Hkv, D=D,
                              layout=layout, page_bytes=page, storage_offset_bytes=offset)


@pytest.mark.parametrize("src", sorted(DTYPES))
@pytest.mark.parametrize("D,layout,pad,offset", [(128, "NHD", 0, 0), (128, "HND", 64, 16), (64, "NHD", 0, 0),
                                                 (256, "HND", 0, 8), (128, "NHD", 32, 0)])
def test_writer_bytes_equal_the_oracle(D, layout, pad, offset, src):
    from tests.gpu_util import cache_to_device

    Hkv, BS, blocks, T = 4, 16, 9, 77
    rng = np.random.default_rng(D + len(layout) + pad)
    c = _empty_cache(blocks, Hkv, D, BS, layout, pad, offset, seed=5)
    dt = DTYPES[src]
    key = (torch.from_numpy(rng.standard_normal((T, Hkv, D), dtype=np.float32)) * 3).to(dt)
    val = torch.from_numpy(rng.standard_normal((T, Hkv, D), dtype=np.float32)).to(dt)
    key[3] = 0                     # an all-zero row: the scale floor
    key[5, 1, 7] = 1e4             # an outlier channel
    slots = rng.permutation(blocks * BS)[:T].astype(np.int64)
    slots[[2, 40]] = -1            # padding tokens
    # expected image: the oracle's writer on the very same (rounded) source values
    want = c.storage.copy()
    exp = orc.PagedInt8Cache(**{**c.__dict__, "storage": want})
    kq, kscale = orc.quantize_rows(key.float().numpy())
    vq, vscale = orc.quantize_rows(val.float().numpy())
    live = slots >= 0
    b, s = slots[live] // BS, slots[live] % BS
    exp.k_cache[b, s] = kq[live]
    exp.v_cache[b, s] = vq[live]
    exp.k_scale[b, s] = kscale[live]
    exp.v_scale[b, s] = vscale[live]

    storage, views, _, _ = cache_to_device(c)
    host.write_kv(key.cuda(), val.cuda(), views, torch.from_numpy(slots).cuda())
    torch.cuda.synchronize()
    got = storage.cpu().numpy()
    assert np.array_equal(got, want), f"{int((got != want).sum())} bytes differ"


def test_writer_golden_vectors_and_strided_sources():
    """The reference-generated vectors of tests/golden/writer.npz, through non-contiguous sources."""
    from tests.gpu_util import cache_to_device

    g = load_golden("writer")
    x = g["x_rand"]                                   # [64, 128] fp32
    T, Hkv, D, BS = 16, 4, 128, 16
    c = _empty_cache(2, Hkv, D, BS, "NHD", seed=1)
    big = torch.zeros((T, Hkv + 1, D + 32), dtype=torch.float32)
    big[:, :Hkv, :D] = torch.from_numpy(x.reshape(T, Hkv, D))
    key = big.cuda()[:, :Hkv, :D]                     # strided rows
    storage, views, _, _ = cache_to_device(c)
    slots = torch.arange(T, dtype=torch.int64, device="cuda")
    host.write_kv(key, key, views, slots)
    torch.cuda.synchronize()
    back = orc.PagedInt8Cache(**{**c.__dict__, "storage": storage.cpu().numpy()})
    assert np.array_equal(back.k_cache[0].reshape(-1, D), g["q_rand"])
    assert np.array_equal(back.v_cache[0].reshape(-1, D), g["q_rand"])
    assert np.array_equal(back.k_scale[0].reshape(-1), g["s_rand"])


def test_attention_reads_a_cache_this_writer_wrote():
    """Write with the kernel, read with the op: equal to the oracle's cache and attention."""
    from tests.gpu_util import cache_to_device, run_case

    Hq, Hkv, D, BS = 8, 2, 128, 16
    lens, qlens = [300, 77], [4, 1]
    ref_cache = orc.make_paged_cache(lens, Hkv, D, BS, seed=12)          # the oracle's writer
    mine = orc.PagedInt8Cache(**{**ref_cache.__dict__, "storage": ref_cache.storage.copy(), "k_src": [], "v_src": []})
    mine.k_cache[...] = 0
    mine.v_cache[...] = 0
    storage, views, _, _ = cache_to_device(mine)
    for r, L in enumerate(lens):
        pos = np.arange(L)
        slots = ref_cache.block_table[r].astype(np.int64)[pos // BS] * BS + pos % BS
        host.write_kv(torch.from_numpy(ref_cache.k_src[r]).cuda(), torch.from_numpy(ref_cache.v_src[r]).cuda(), views,
                      torch.from_numpy(slots).cuda())
    torch.cuda.synchronize()
    written = storage.cpu().numpy()
    back = orc.PagedInt8Cache(**{**mine.__dict__, "storage": written})
    for r, L in enumerate(lens):
        a, b = back.dense(r), ref_cache.dense(r)
        assert np.array_equal(a.k_int, b.k_int) and np.array_equal(a.v_int, b.v_int)
        assert np.array_equal(a.k_scale, b.k_scale) and np.array_equal(a.v_scale, b.v_scale)
    rng = np.random.default_rng(13)
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    ref = orc.ref_attention_paged(q, ref_cache, qsl, D ** -0.5)
    res = run_case(back, q, qsl, D ** -0.5, bq=4, num_splits=2)
    check_out(res["out"], ref.out, what="attention over the written cache")


def test_writer_refusals():
    lib = capi.load_library()
    a = capi.new_write_args()
    a.head_size, a.num_kv_heads, a.block_size, a.num_blocks, a.num_tokens = 96, 1, 16, 1, 1
    assert lib.write_kv(a) == capi.EINVAL and "head_size" in lib.last_error()
    a.head_size = 128
    assert lib.write_kv(a) == capi.EINVAL and "NULL" in lib.last_error()
    a.num_tokens = 0
    assert lib.write_kv(a) == capi.OK    # nothing to write
