"""Split-KV across GPUs on the device: the slices of every request (``sharding.context_shard``)
sit in separate caches, each is attended to on its own (causal only where the query positions
are), and one combine over the ranks' partials gives the result of the unsharded launch.

On one GPU the ranks run one after the other and the test stacks their partials itself; with two
or more GPUs visible the same path runs as NCCL ranks through
``sharding.context_parallel_attention`` (its all-gather is the only exchange)."""
import math
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import paged_int8_attention as orc
from pth_flash_attn_b200 import capi, host, sharding
from tests.helpers import check_lse, check_out

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent


def _case(seed, lens, qlens, Hq, Hkv, D):
    rng = np.random.default_rng(seed)
    k_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    v_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    return k_src, v_src, q, qsl


def _rank_cache(rank, world, lens, qlens, k_src, v_src, Hkv, D, block_size):
    mine = [sharding.context_shard(rank, world, L, ql) for L, ql in zip(lens, qlens)]
    src = [(k[s.begin:s.end], v[s.begin:s.end]) for s, k, v in zip(mine, k_src, v_src)]
    return orc.make_paged_cache([s.length for s in mine], Hkv, D, block_size, seed=40 + rank, sources=src), mine


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("D,Hq,Hkv,qlens", [(128, 8, 2, [1, 1, 1, 1]), (128, 8, 2, [4, 1, 2, 3]), (256, 12, 2, [1, 2, 1, 1])])
def test_ranks_one_after_the_other_on_one_gpu(world, D, Hq, Hkv, qlens):
    from tests.gpu_util import cache_to_device, q_to_device

    lens = [9000, 1300, 129, 7]
    k_src, v_src, q, qsl = _case(7 + world, lens, qlens, Hq, Hkv, D)
    T = int(qsl[-1])
    qd = q_to_device(q)
    qsl_t = torch.from_numpy(qsl).cuda()
    ws_o = torch.full((world, T, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
    ws_lse = torch.full((world, T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    keep = []
    for rank in range(world):
        c, mine = _rank_cache(rank, world, lens, qlens, k_src, v_src, Hkv, D, 16)
        storage, views, bt, lens_t = cache_to_device(c)
        keep.append(storage)
        S = 3 if rank % 2 else 1   # local pieces too, on some ranks
        lo = lw = None
        if S > 1:
            lo = torch.empty((S, T, Hq, D), dtype=torch.float32, device="cuda")
            lw = torch.empty((S, T, Hq), dtype=torch.float32, device="cuda")
        host.attention_forward(qd, ws_o[rank], views, bt, lens_t, qsl_t, bq=max(qlens), num_splits=S,
                               softmax_scale=D ** -0.5, ws_o=lo, ws_lse=lw, causal=mine[0].causal, lse_out=ws_lse[rank])
    ws_lse.mul_(1.0 / math.log(2.0))
    out = torch.full((T, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    host.combine_partials(ws_o, ws_lse, out, qsl_t, lse_out=lse)
    torch.cuda.synchronize()
    assert capi.load_library().device_status() == 0
    full = orc.make_paged_cache(lens, Hkv, D, 16, seed=99, sources=list(zip(k_src, v_src)))
    ref = orc.ref_attention_paged(q, full, qsl, D ** -0.5)
    check_out(out.float().cpu().numpy(), ref.out, what=f"{world} ranks")
    check_lse(lse.cpu().numpy(), ref.lse, what=f"{world} ranks")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, out_path):
    sys.path.insert(0, str(REPO))
    import torch.distributed as dist

    from tests.gpu_util import cache_to_device, q_to_device

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    D, Hq, Hkv = 128, 32, 8
    lens, qlens = [40000, 5000, 300], [1, 4, 2]
    k_src, v_src, q, qsl = _case(3, lens, qlens, Hq, Hkv, D)
    T = int(qsl[-1])
    c, _ = _rank_cache(rank, world, lens, qlens, k_src, v_src, Hkv, D, 16)
    storage, views, bt, lens_t = cache_to_device(c)
    qd, qsl_t = q_to_device(q), torch.from_numpy(qsl).cuda()
    out = torch.full((T, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((T, Hq), float("nan"), dtype=torch.float32, device="cuda")
    S = 4
    ws_o = torch.empty((S, T, Hq, D), dtype=torch.float32, device="cuda")
    ws_lse = torch.empty((S, T, Hq), dtype=torch.float32, device="cuda")
    sharding.context_parallel_attention(qd, out, views, bt, lens_t, qsl_t, rank=rank, world=world,
                                        softmax_scale=D ** -0.5, bq=4, num_splits=S, ws_o=ws_o, ws_lse=ws_lse,
                                        lse_out=lse)
    torch.cuda.synchronize()
    ok = capi.load_library().device_status() == 0
    full = orc.make_paged_cache(lens, Hkv, D, 16, seed=99, sources=list(zip(k_src, v_src)), keep_sources=False)
    ref = orc.ref_attention_paged(q, full, qsl, D ** -0.5)
    d = np.abs(out.float().cpu().numpy() - ref.out)
    dl = np.abs(lse.cpu().numpy() - ref.lse)
    np.save(f"{out_path}.{rank}.npy", np.array([d.max(), d.mean(), dl.max(), float(ok)]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_end_with_the_full_result(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    out = str(tmp_path / "err")
    mp.spawn(_nccl_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        mx, mean, dl, ok = np.load(f"{out}.{rank}.npy")
        assert ok == 1.0 and mx <= 2e-2 and mean <= 2e-3 and dl <= 1e-3, (rank, mx, mean, dl)
