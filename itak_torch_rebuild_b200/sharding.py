"""KV-head sharding of the hot path across the GPUs of one box.

Each query head reads exactly one KV head (crates/attention/src/attention.rs:175-178), so the path splits by
KV head with no data-path exchange except one gather of the per-head outputs per layer.  Rank r of N owns KV
heads ``[r * Hkv / N, (r + 1) * Hkv / N)`` and the ``group`` query heads of each; where heads run out
(N > Hkv) whole sequences are split across ranks instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    kv_head_begin: int
    kv_heads: int        # KV heads resident on this rank
    q_head_begin: int
    q_heads: int         # query heads resident on this rank
    seq_begin: int
    seqs: int            # sequences resident on this rank


def plan(q_heads: int, kv_heads: int, n_seqs: int, rank: int, world: int) -> Shard:
    """The shard of (heads, sequences) that ``rank`` owns."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if q_heads % kv_heads != 0:
        raise ValueError(f"{q_heads} query heads do not divide evenly across {kv_heads} KV heads")
    group = q_heads // kv_heads
    if world <= kv_heads:
        if kv_heads % world != 0:
            raise ValueError(f"{kv_heads} KV heads do not shard evenly over {world} GPUs")
        per = kv_heads // world
        return Shard(rank, world, rank * per, per, rank * per * group, per * group, 0, n_seqs)
    # more GPUs than KV heads: one head per group of ranks, sequences split inside the group
    if world % kv_heads != 0:
        raise ValueError(f"{world} GPUs do not divide over {kv_heads} KV heads")
    ranks_per_head = world // kv_heads
    head, sub = divmod(rank, ranks_per_head)
    base, extra = divmod(n_seqs, ranks_per_head)
    begin = sub * base + min(sub, extra)
    count = base + (1 if sub < extra else 0)
    return Shard(rank, world, head, 1, head * group, group, begin, count)


def gathered_head_order(q_heads: int, kv_heads: int, world: int) -> List[int]:
    """Global query-head index of each row of an all-gather that concatenates rank shards in rank order
    (each shard laid out ``[q_heads_local]``).  With head sharding this is the identity."""
    order: List[int] = []
    for r in range(world):
        s = plan(q_heads, kv_heads, 1, r, world)
        order.extend(range(s.q_head_begin, s.q_head_begin + s.q_heads))
    return order
