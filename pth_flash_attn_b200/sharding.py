"""KV-head sharding of the attention path across GPUs (no collective on the data path).

Rank g of N owns KV heads ``[g * Hkv / N, (g + 1) * Hkv / N)``, the query heads of those
groups, and its own paged cache holding only its heads (as a tensor-parallel engine allocates
it).  Block tables, sequence lengths and query_start_loc are replicated.  Attention of one KV
head never reads another head's cells, so the shards run independently and their outputs are
the head-slices of the unsharded output.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_begin: int
    kv_end: int
    q_begin: int
    q_end: int

    @property
    def num_kv_heads(self) -> int:
        return self.kv_end - self.kv_begin

    @property
    def num_q_heads(self) -> int:
        return self.q_end - self.q_begin


def head_shard(rank: int, world: int, num_q_heads: int, num_kv_heads: int) -> HeadShard:
    """The head ranges of ``rank``; whole GQA groups only."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} out of range for world size {world}")
    if num_kv_heads % world:
        raise ValueError(f"num_kv_heads={num_kv_heads} does not shard over {world} ranks")
    if num_q_heads % num_kv_heads:
        raise ValueError("num_q_heads must be a multiple of num_kv_heads")
    group = num_q_heads // num_kv_heads
    per = num_kv_heads // world
    kb, ke = rank * per, (rank + 1) * per
    return HeadShard(rank, world, kb, ke, kb * group, ke * group)
