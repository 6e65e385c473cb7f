"""Batch x head sharding of the log-linear attention operator across the GPUs of one node.

The operator is independent across (batch, head): the forward needs no communication, and the
backward needs one sum over ranks of dq / dk only when the heads of one q/k group end up on
different ranks (the reference sums dq, dk over the heads of a group, chunkwise.py:1583-1591).
`plan` shards the batch first and splits heads only when there are more ranks than batch items.
"""
from dataclasses import dataclass
from typing import List

import torch


@dataclass(frozen=True)
class Shard:
    b0: int
    b1: int
    h0: int
    h1: int
    qk_allreduce_group: int      # number of ranks that share this shard's (batch range, q/k groups); 1 = no collective


def plan(B: int, H: int, G: int, world: int) -> List[Shard]:
    """One shard per rank.  Requires world to divide B, or B to divide world with world // B dividing H."""
    if H % G != 0:
        raise ValueError("H must be a multiple of G")
    if world <= B:
        if B % world != 0:
            raise ValueError("world size must divide the batch")
        per = B // world
        return [Shard(r * per, (r + 1) * per, 0, H, 1) for r in range(world)]
    if world % B != 0:
        raise ValueError("batch must divide the world size")
    parts = world // B
    if H % parts != 0:
        raise ValueError("ranks per batch item must divide the number of heads")
    hp = H // parts
    heads_per_group = H // G
    out = []
    for r in range(world):
        b, j = divmod(r, parts)
        # ranks whose head range overlaps the same group(s) must add up their dq / dk
        share = max(1, heads_per_group // hp) if hp < heads_per_group else 1
        out.append(Shard(b, b + 1, j * hp, (j + 1) * hp, share))
    return out


def take(shard: Shard, q, k, v, g, l, H: int):
    """Slices of the operator inputs for one shard (q, k keep the groups that the shard's heads use)."""
    G = q.shape[2]
    hpg = H // G
    g0, g1 = shard.h0 // hpg, (shard.h1 - 1) // hpg + 1
    sb = slice(shard.b0, shard.b1)
    return (q[sb, :, g0:g1], k[sb, :, g0:g1], v[sb, :, shard.h0:shard.h1], g[sb, :, shard.h0:shard.h1],
            l[sb, :, shard.h0:shard.h1])


def reduce_qk_grads(dq: torch.Tensor, dk: torch.Tensor, shard: Shard, rank: int, group=None):
    """Sum dq / dk over the ranks that hold heads of the same q/k group (no-op when the group is whole)."""
    if shard.qk_allreduce_group <= 1:
        return dq, dk
    import torch.distributed as dist
    first = (rank // shard.qk_allreduce_group) * shard.qk_allreduce_group
    ranks = list(range(first, first + shard.qk_allreduce_group))
    sub = group if group is not None else dist.new_group(ranks)
    dist.all_reduce(dq, group=sub)
    dist.all_reduce(dk, group=sub)
    return dq, dk
