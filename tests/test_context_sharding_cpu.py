"""Split-KV across GPUs, host logic (CPU): how a request's keys are sliced over the ranks, which
rank launches causal, and that the partials of the slices merge to the unsharded result.  In the
two-rank gloo run the CPU oracle stands in for each rank's device launch; the exchange is the
all-gather the GPU path uses."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pth_flash_attn_b200 import sharding

REPO = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("seq_len,q_len", [(131072, 1), (8192, 4), (1000, 16), (129, 1), (128, 128), (5, 2), (1, 1),
                                           (300, 300), (4096, 0), (0, 0)])
def test_slices_cover_the_keys_and_keep_the_query_positions_on_the_last_rank(world, seq_len, q_len):
    shards = [sharding.context_shard(r, world, seq_len, q_len) for r in range(world)]
    assert shards[0].begin == 0 and shards[-1].end == seq_len
    for a, b in zip(shards, shards[1:]):
        assert a.end == b.begin and a.begin <= a.end
        assert a.end % sharding.KV_TILE == 0          # boundaries fall between KV tiles
        assert a.end <= seq_len - q_len               # no query position before the last rank
    assert [s.causal for s in shards] == [False] * (world - 1) + [True]
    if seq_len >= 128 * world * 4 and q_len <= 128:   # long requests are spread evenly
        sizes = [s.length for s in shards]
        assert max(sizes) - min(sizes) <= 2 * sharding.KV_TILE


def test_bad_arguments_are_refused():
    with pytest.raises(ValueError):
        sharding.context_shard(2, 2, 100)
    with pytest.raises(ValueError):
        sharding.context_shard(0, 2, 10, q_len=11)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    sys.path.insert(0, str(REPO))
    from oracle import paged_int8_attention as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    Hq, Hkv, D = 8, 2, 64
    lens, qlens = [1000, 300, 129, 7], [4, 1, 2, 3]
    rng = np.random.default_rng(11)  # replicated inputs
    k_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    v_src = [rng.standard_normal((L, Hkv, D), dtype=np.float32) for L in lens]
    q = orc.round_to_bf16(rng.standard_normal((sum(qlens), Hq, D), dtype=np.float32))
    qsl = np.concatenate([[0], np.cumsum(qlens)])
    mine = [sharding.context_shard(rank, world, L, ql) for L, ql in zip(lens, qlens)]
    src = [(k[s.begin:s.end], v[s.begin:s.end]) for s, k, v in zip(mine, k_src, v_src)]
    cache = orc.make_paged_cache([s.length for s in mine], Hkv, D, 16, seed=20 + rank, sources=src)
    part = orc.ref_attention_paged(q, cache, qsl, D ** -0.5, causal=mine[0].causal)
    o = torch.from_numpy(np.ascontiguousarray(part.out))
    l2 = torch.from_numpy(np.ascontiguousarray(part.lse / np.log(2.0)))
    all_o = [torch.zeros_like(o) for _ in range(world)]
    all_l = [torch.zeros_like(l2) for _ in range(world)]
    dist.all_gather(all_o, o)
    dist.all_gather(all_l, l2)
    if rank == 0:
        merged, merged_l2 = orc.combine_partials(torch.stack(all_o).numpy(), torch.stack(all_l).numpy())
        full_cache = orc.make_paged_cache(lens, Hkv, D, 16, seed=99, sources=list(zip(k_src, v_src)))
        full = orc.ref_attention_paged(q, full_cache, qsl, D ** -0.5)
        np.save(out_path, np.array([np.abs(merged - full.out).max(),
                                    np.abs(orc.log2_to_ln(merged_l2) - full.lse).max()]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partials_of_the_slices_merge_to_the_unsharded_result(tmp_path, world):
    out = tmp_path / "err.npy"
    mp.spawn(_worker, args=(world, _free_port(), str(out)), nprocs=world, join=True)
    err = np.load(out)
    assert err[0] < 1e-9 and err[1] < 1e-9, err
