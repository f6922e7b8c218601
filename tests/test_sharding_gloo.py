"""KV-head sharding over 2 ranks (gloo, CPU): each rank builds ITS OWN cache with its heads
only, runs the path on its head slice (here: the CPU oracle stands in for the device), and the
gathered head slices equal the unsharded result.  No collective touches the data path; the
gather below is the test's own check."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    sys.path.insert(0, str(REPO))
    from oracle import paged_int8_attention as orc
    from pth_flash_attn_b200 import planner, sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    Hq, Hkv, D = 8, 4, 128
    lens, qlens = [70, 33, 5], [2, 1, 2]
    rng = np.random.default_rng(3)  # replicated inputs
    k_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    v_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    sh = sharding.head_shard(rank, world, Hq, Hkv)
    # this rank's cache holds only its KV heads; block tables are its own
    src = [(k[:, sh.kv_begin:sh.kv_end], v[:, sh.kv_begin:sh.kv_end]) for k, v in zip(k_src, v_src)]
    cache = orc.make_paged_cache(lens, sh.num_kv_heads, D, 16, seed=10 + rank, sources=src)
    local = orc.ref_attention_paged(q[:, sh.q_begin:sh.q_end], cache, qsl, D ** -0.5)
    # the plan of a shard depends on its local head count only
    plan = planner.plan_launch(num_tokens=int(qsl[-1]), num_reqs=len(lens), max_query_len=2, G=Hq // Hkv,
                               Hkv=sh.num_kv_heads, D=D, num_sms=148, is_prefill=False, ws_token_splits=1 << 20)
    assert plan.Hq == sh.num_q_heads
    gathered = [torch.zeros(local.out.shape, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(local.out))
    if rank == 0:
        full_cache = orc.make_paged_cache(lens, Hkv, D, 16, seed=99, sources=list(zip(k_src, v_src)))
        full = orc.ref_attention_paged(q, full_cache, qsl, D ** -0.5)
        got = torch.cat(gathered, dim=1).numpy()
        np.save(out_path, np.abs(got - full.out).max())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_head_sharding(tmp_path):
    out = tmp_path / "err.npy"
    mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert float(np.load(out)) < 1e-12


def test_head_shard_ranges():
    from pth_flash_attn_b200 import sharding

    for world in (1, 2, 4, 8):
        shards = [sharding.head_shard(r, world, 64, 8) for r in range(world)]
        assert shards[0].kv_begin == 0 and shards[-1].kv_end == 8
        assert all(a.kv_end == b.kv_begin and a.q_end == b.q_begin for a, b in zip(shards, shards[1:]))
        assert all(s.num_q_heads == 8 * s.num_kv_heads for s in shards)
    with pytest.raises(ValueError):
        sharding.head_shard(0, 3, 64, 8)
    with pytest.raises(ValueError):
        sharding.head_shard(2, 2, 64, 8)
