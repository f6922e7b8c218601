"""Generates tests/golden/*.npz from the reference project's own oracle.

Run where the reference checkout is available (it cannot travel to a GPU box;
the committed .npz files can):

    REFERENCE=/path/to/pth-flash-attn python tests/golden/make_golden.py

What is recorded:

* writer.npz        - fp32 rows -> (int8, scale) from ``pth_testing.reference.quantize_rows``.
* cache_*.npz       - raw bytes of ``make_int8_cache`` caches built from explicit sources,
                      with their stream offsets/strides, block tables and lengths.
* attn_*.npz        - inputs (stored ints/scales per request, bf16 queries, query_start_loc,
                      scale, window, causal) and outputs (fp64 out, natural-log LSE, valid)
                      of ``ref_attention_dense``.
* split_*.npz       - per-split partials (fp32 ws_o, log2 ws_lse) and the combined output
                      from the reference's own C++ CPU path (``pth_ref_attention_host`` /
                      ``pth_ref_combine_host`` in oracle/_ref/libpth_ref_host.so, built by
                      oracle/Makefile).
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
# the reference checkout: $REFERENCE, else a directory `reference` next to this repository
REFERENCE = Path(os.environ.get("REFERENCE", Path(__file__).resolve().parents[3] / "reference"))
sys.path.insert(0, str(REFERENCE / "python"))

from pth_testing import ref_capi  # noqa: E402
from pth_testing.reference import (  # noqa: E402
    make_int8_cache,
    make_queries,
    quantize_rows,
    ref_attention_dense,
)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def save(name: str, **arrays) -> None:
    path = HERE / f"{name}.npz"
    np.savez_compressed(path, **arrays)
    print(f"{path.name}: {path.stat().st_size / 1024:.1f} KiB")


def gen_writer() -> None:
    g = torch.Generator().manual_seed(11)
    rows = [
        torch.tensor([127.0, 2.5, -2.5, 0.5, -0.5, 3.5, -126.5, 0.0]),  # exact ties, scale 1
        torch.zeros(8),  # all-zero row: scale on the floor
        torch.full((8,), 1.0e-5),  # below the floor
        torch.tensor([3.0, -3.0, 1.5, -1.5, 0.75, -0.75, 2.9999, -2.9999]),
    ]
    x_small = torch.stack(rows)
    x_rand = torch.randn(64, 128, generator=g) * torch.exp(torch.randn(64, 1, generator=g) * 2)
    qs, ss = quantize_rows(x_small)
    qr, sr = quantize_rows(x_rand)
    save("writer", x_small=x_small.numpy(), q_small=qs.numpy(), s_small=ss.numpy(),
         x_rand=x_rand.numpy(), q_rand=qr.numpy(), s_rand=sr.numpy())


def gen_cache(name: str, lens, Hkv, D, bs, layout, pad, off, seed) -> None:
    g = torch.Generator().manual_seed(seed)
    sources = [(torch.randn(L, Hkv, D, generator=g), torch.randn(L, Hkv, D, generator=g) * 3)
               for L in lens]
    c = make_int8_cache(lens, Hkv=Hkv, D=D, block_size=bs, layout=layout, pad_page_bytes=pad,
                        seed=seed, storage_offset_bytes=off, src_dtype=torch.float32,
                        sources=sources)
    base = c.storage.data_ptr()

    def geom(v):
        es = v.element_size()
        return np.asarray([v.data_ptr() - base] + [s * es for s in v.stride()[:3]], dtype=np.int64)

    arrays = dict(
        storage=c.storage.numpy().view(np.uint8).copy(),
        block_table=c.block_table.numpy(), seq_lens=c.seq_lens.numpy(),
        k_geom=geom(c.k_cache), v_geom=geom(c.v_cache), ks_geom=geom(c.k_scale),
        vs_geom=geom(c.v_scale),
        meta=np.asarray([Hkv, D, bs, pad, off, c.k_cache.shape[0], c.page_bytes], dtype=np.int64),
        layout=np.asarray(layout),
    )
    for r, (ks, vs) in enumerate(sources):
        arrays[f"k_src{r}"] = ks.numpy()
        arrays[f"v_src{r}"] = vs.numpy()
        d = c.dense(r)
        arrays[f"k_int{r}"] = d.k_int.numpy()
        arrays[f"k_scale{r}"] = d.k_scale.numpy()
        arrays[f"v_int{r}"] = d.v_int.numpy()
        arrays[f"v_scale{r}"] = d.v_scale.numpy()
    save(name, **arrays)


def gen_attn(name: str, lens, q_lens, Hq, Hkv, D, seed, window=0, causal=True, pad_rows=0,
             scale_mode="normal", use_normal_sources=True) -> None:
    g = torch.Generator().manual_seed(seed)
    if use_normal_sources:
        sources = [(torch.randn(L, Hkv, D, generator=g), torch.randn(L, Hkv, D, generator=g))
                   for L in lens]
        c = make_int8_cache(lens, Hkv=Hkv, D=D, block_size=16, seed=seed,
                            src_dtype=torch.float32, sources=sources)
    else:
        c = make_int8_cache(lens, Hkv=Hkv, D=D, block_size=16, seed=seed, scale_mode=scale_mode)
    q, qsl = make_queries(q_lens, Hq, D, seed=seed + 1)
    if pad_rows:
        q = torch.cat([q, torch.randn(pad_rows, Hq, D, generator=g).to(q.dtype)])
    scale = float(D) ** -0.5
    ref = ref_attention_dense(q, c.dense_all(), qsl, scale, window=window, causal=causal)
    arrays = dict(
        q_bits=bf16_bits(q), qsl=qsl.numpy(), seq_lens=c.seq_lens.numpy(),
        meta=np.asarray([Hq, Hkv, D, window, int(causal)], dtype=np.int64),
        softmax_scale=np.asarray(scale, dtype=np.float64),
        out=ref.out.numpy(), lse=ref.lse.numpy(), valid=ref.valid.numpy(),
    )
    for r in range(len(lens)):
        d = c.dense(r)
        arrays[f"k_int{r}"] = d.k_int.numpy()
        arrays[f"k_scale{r}"] = d.k_scale.numpy()
        arrays[f"v_int{r}"] = d.v_int.numpy()
        arrays[f"v_scale{r}"] = d.v_scale.numpy()
    save(name, **arrays)


def gen_split(name: str, lens, q_lens, Hq, Hkv, D, bq, S, seed, window=0, causal=True) -> None:
    lib_path = REPO / "oracle" / "_ref" / "libpth_ref_host.so"
    lib = ref_capi.RefLib(lib_path)
    g = torch.Generator().manual_seed(seed)
    sources = [(torch.randn(L, Hkv, D, generator=g), torch.randn(L, Hkv, D, generator=g))
               for L in lens]
    c = make_int8_cache(lens, Hkv=Hkv, D=D, block_size=16, seed=seed, src_dtype=torch.float32,
                        sources=sources)
    q, qsl = make_queries(q_lens, Hq, D, seed=seed + 1)
    T = q.shape[0]
    scale = float(D) ** -0.5
    ws_o = torch.full((S, T, Hq, D), float("nan"), dtype=torch.float32)
    ws_lse = torch.full((S, T, Hq), float("nan"), dtype=torch.float32)
    a = ref_capi.attn_args(c, q, qsl, None, softmax_scale=scale, bq=bq, num_splits=S,
                           ws_o=ws_o, ws_lse=ws_lse, window=window, causal=causal)
    rc = lib.attention(a, host=True)
    assert rc == 0, lib.last_error()
    out = torch.zeros(T, Hq, D, dtype=torch.float32)
    ca = ref_capi.combine_args(ws_o, ws_lse, out, qsl, len(lens), S)
    rc = lib.combine(ca, host=True)
    assert rc == 0, lib.last_error()
    # single-split output of the same library, fp32
    out1 = torch.zeros(T, Hq, D, dtype=torch.float32)
    a1 = ref_capi.attn_args(c, q, qsl, out1, softmax_scale=scale, bq=bq, num_splits=1,
                            window=window, causal=causal)
    rc = lib.attention(a1, host=True)
    assert rc == 0, lib.last_error()
    ref = ref_attention_dense(q, c.dense_all(), qsl, scale, window=window, causal=causal)
    arrays = dict(
        q_bits=bf16_bits(q), qsl=qsl.numpy(), seq_lens=c.seq_lens.numpy(),
        meta=np.asarray([Hq, Hkv, D, window, int(causal), bq, S], dtype=np.int64),
        softmax_scale=np.asarray(scale, dtype=np.float64),
        ws_o=ws_o.numpy(), ws_lse=ws_lse.numpy(), combined=out.numpy(), unsplit=out1.numpy(),
        out=ref.out.numpy(), lse=ref.lse.numpy(),
    )
    for r in range(len(lens)):
        d = c.dense(r)
        arrays[f"k_int{r}"] = d.k_int.numpy()
        arrays[f"k_scale{r}"] = d.k_scale.numpy()
        arrays[f"v_int{r}"] = d.v_int.numpy()
        arrays[f"v_scale{r}"] = d.v_scale.numpy()
    save(name, **arrays)


def main() -> None:
    gen_writer()
    gen_cache("cache_nhd", [1, 0, 19, 31], 2, 64, 16, "NHD", 0, 0, 7)
    gen_cache("cache_hnd_pad", [5, 40], 2, 64, 16, "HND", 72, 4, 8)
    gen_cache("cache_nhd_d128", [33], 3, 128, 16, "NHD", 8, 0, 9)
    # decode (1 token per request), GQA 4, D = 128
    gen_attn("attn_decode", [1, 37, 130, 300], [1, 1, 1, 1], 8, 2, 128, 21)
    # speculative verification: 4 causal draft tokens per request
    gen_attn("attn_verify4", [64, 129, 257], [4, 4, 4], 8, 2, 128, 22)
    # windowed drafter: 16 tokens, window 48, causal
    gen_attn("attn_window_causal", [200, 90], [16, 16], 8, 2, 128, 23, window=48)
    # non-causal with and without a window
    gen_attn("attn_window_noncausal", [150, 60], [8, 8], 8, 2, 128, 24, window=32, causal=False)
    gen_attn("attn_noncausal", [100], [6], 4, 1, 128, 25, causal=False)
    # prefill chunk over a prefix + an empty request + a decode + padding rows
    gen_attn("attn_mixed", [100, 0, 45, 40], [24, 0, 1, 40], 8, 2, 128, 26, pad_rows=3)
    # other head sizes / group sizes, the reference's wide-range data
    gen_attn("attn_d64_g6", [70, 33], [3, 1], 12, 2, 64, 27, use_normal_sources=False,
             scale_mode="mixed")
    gen_attn("attn_d256_g6", [50], [2], 12, 2, 256, 28, use_normal_sources=False)
    # the reference's C++ CPU path: partials of 3 splits + combine (64-token tiles)
    gen_split("split_cpp", [150, 70], [2, 1], 4, 2, 64, 2, 3, 31)


if __name__ == "__main__":
    main()
