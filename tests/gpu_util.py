"""GPU-side helpers of the parity tests: move an oracle cache to the device and
run the library on it through the C ABI."""
from __future__ import annotations

import numpy as np
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host

CANARY = 0xFF


def cache_to_device(c: orc.PagedInt8Cache, device="cuda"):
    """Copy the flat cache storage to the device; returns (storage tensor, CacheViews, bt, lens)."""
    storage = torch.from_numpy(c.storage).to(device)
    base = storage.data_ptr()

    def g(s: orc.StreamView):
        return (base + s.offset, s.stride_block, s.stride_slot, s.stride_head)

    views = host.CacheViews(g(c.k), g(c.v), g(c.ks), g(c.vs), c.num_blocks, c.block_size, c.Hkv, c.D)
    bt = torch.from_numpy(c.block_table).to(device)
    lens = torch.from_numpy(c.seq_lens).to(device)
    return storage, views, bt, lens


def q_to_device(q_f32: np.ndarray, dtype=torch.bfloat16, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(q_f32, dtype=np.float32)).to(device).to(dtype)


def run_case(c: orc.PagedInt8Cache, q_f32: np.ndarray, qsl, softmax_scale: float, *, bq: int,
             num_splits: int = 1, window: int = 0, causal: bool = True,
             kernel: int = capi.KERNEL_AUTO, flags: int = 0, out_dtype=torch.bfloat16, q_dtype=torch.bfloat16,
             pad_tokens: int = 0):
    """Run one launch; returns dict(out fp32 numpy, lse numpy, canaries intact flags, ws)."""
    dev = "cuda"
    storage, views, bt, lens = cache_to_device(c, dev)
    q = q_to_device(q_f32, q_dtype, dev)
    T, Hq, D = q.shape
    qsl_t = torch.tensor(list(qsl), dtype=torch.int32, device=dev)
    # canary rows around out: rows [T, T + 2) must keep their bytes
    esz = torch.empty((), dtype=out_dtype).element_size()
    out_buf = torch.full(((T + 2) * Hq * D * esz,), CANARY, dtype=torch.uint8, device=dev)
    out = out_buf[: T * Hq * D * esz].view(out_dtype).view(T, Hq, D)
    lse = torch.full((T, Hq), float("nan"), dtype=torch.float32, device=dev)
    ws_o = ws_lse = None
    if num_splits > 1:
        ws_o = torch.full((num_splits, T, Hq, D), float("nan"), dtype=torch.float32, device=dev)
        ws_lse = torch.full((num_splits, T, Hq), float("nan"), dtype=torch.float32, device=dev)
    host.attention_forward(q, out, views, bt, lens, qsl_t, bq=bq, num_splits=num_splits,
                           softmax_scale=softmax_scale, ws_o=ws_o, ws_lse=ws_lse, window=window,
                           causal=causal, lse_out=lse, kernel=kernel, flags=flags)
    torch.cuda.synchronize()
    tail = out_buf[T * Hq * D * esz:]
    res = dict(
        out=out.float().cpu().numpy(), lse=lse.cpu().numpy(),
        out_bytes=out_buf[: T * Hq * D * esz].cpu().numpy().reshape(T, -1),
        tail_intact=bool((tail == CANARY).all().item()),
        ws_o=None if ws_o is None else ws_o.cpu().numpy(),
        ws_lse=None if ws_lse is None else ws_lse.cpu().numpy(),
    )
    del storage
    return res
