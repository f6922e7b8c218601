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


# --------------------------------------------------------------------------
# Split-KV across GPUs: one long request whose keys do not fit (or do not pay) on one GPU
# --------------------------------------------------------------------------
KV_TILE = 128


@dataclass(frozen=True)
class ContextShard:
    """Keys ``[begin, end)`` of one request held by ``rank``; ``causal`` says how that rank
    must launch (only the rank that holds the query tokens' own positions masks by position)."""
    rank: int
    world: int
    begin: int
    end: int
    causal: bool

    @property
    def length(self) -> int:
        return self.end - self.begin


def context_shard(rank: int, world: int, seq_len: int, q_len: int = 1) -> ContextShard:
    """The slice of a request's keys that ``rank`` of ``world`` holds.

    Slices are contiguous runs of whole 128-key tiles in rank order, and every boundary lies at
    or below ``seq_len - q_len``: the query tokens' own positions are all in the LAST rank's
    slice.  A rank before the last then sees each of its keys from every query token (it
    launches non-causal over its local length), and the last rank launches causal over
    ``(local length, q_len)``, which places token ``i`` at local position ``local - q_len + i``,
    its global position minus the slice's begin.  Short requests leave leading ranks empty
    (their partial is the empty one: zero output, log-sum-exp -inf)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} out of range for world size {world}")
    if seq_len < 0 or q_len < 0 or q_len > max(seq_len, 0):
        raise ValueError("need 0 <= q_len <= seq_len")
    tiles = -(-seq_len // KV_TILE)
    cap = (seq_len - q_len) // KV_TILE * KV_TILE   # highest boundary that keeps the query positions together

    def boundary(g: int) -> int:
        if g <= 0:
            return 0
        if g >= world:
            return seq_len
        return min(g * tiles // world * KV_TILE, cap)

    return ContextShard(rank, world, boundary(rank), boundary(rank + 1), causal=rank == world - 1)


def context_parallel_attention(q, out, cache, block_table, local_seq_lens, query_start_loc, *, rank: int,
                               world: int, softmax_scale: float, bq: int, num_splits: int = 1, ws_o=None,
                               ws_lse=None, lse_out=None, group=None, partial_o=None, partial_lse=None,
                               gathered_o=None, gathered_lse=None):
    """Attention of requests whose KEYS are spread over ``world`` GPUs (:func:`context_shard`):
    this rank's cache holds its slice of every request (``local_seq_lens``), the queries are
    replicated, and every rank ends with the full result in ``out``.

    Per rank: one launch over the local slice into a normalised fp32 partial and its
    log-sum-exp (causal on the last rank only), one all-gather of the partials (the exchange
    step of this path: ``T * Hq * (D + 1) * 4`` bytes per rank), one combine over ``world``
    pieces - the rule that merges the pieces of a request inside one GPU.  No sliding window.
    The partial and gather buffers may be passed in (a serving engine allocates them once)."""
    import math

    import torch
    import torch.distributed as dist

    from . import host

    T, Hq, D = q.shape
    dev = q.device
    if partial_o is None:
        partial_o = torch.empty((T, Hq, D), dtype=torch.float32, device=dev)
    if partial_lse is None:
        partial_lse = torch.empty((T, Hq), dtype=torch.float32, device=dev)
    if gathered_o is None:
        gathered_o = torch.empty((world, T, Hq, D), dtype=torch.float32, device=dev)
    if gathered_lse is None:
        gathered_lse = torch.empty((world, T, Hq), dtype=torch.float32, device=dev)
    host.attention_forward(q, partial_o, cache, block_table, local_seq_lens, query_start_loc, bq=bq,
                           num_splits=num_splits, softmax_scale=softmax_scale, ws_o=ws_o, ws_lse=ws_lse,
                           causal=rank == world - 1, lse_out=partial_lse)
    partial_lse.mul_(1.0 / math.log(2.0))   # the pieces of a combine carry log2 units (-inf stays -inf)
    if world > 1:
        dist.all_gather_into_tensor(gathered_o, partial_o, group=group)
        dist.all_gather_into_tensor(gathered_lse, partial_lse, group=group)
    else:
        gathered_o.copy_(partial_o.unsqueeze(0))
        gathered_lse.copy_(partial_lse.unsqueeze(0))
    host.combine_partials(gathered_o, gathered_lse, out, query_start_loc, lse_out=lse_out)
