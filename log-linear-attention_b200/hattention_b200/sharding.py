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
    """One shard per rank.  Requires world to divide B, or B to divide world with world // B dividing H.
    When heads are split, a rank's head range must either consist of whole q/k groups (no collective) or lie
    inside one group that an aligned block of consecutive ranks shares (those ranks sum their dq / dk);
    a head range that straddles groups any other way is refused, because its dq / dk would silently miss
    the other ranks' contributions."""
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
    if hp >= heads_per_group:
        if hp % heads_per_group != 0:
            raise ValueError(f"{hp} heads per rank straddle q/k groups of {heads_per_group} heads")
        share = 1
    else:
        if heads_per_group % hp != 0:
            raise ValueError(f"q/k groups of {heads_per_group} heads cannot be split into ranks of {hp} heads")
        share = heads_per_group // hp
    out = []
    for r in range(world):
        b, j = divmod(r, parts)
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


_QK_GROUPS = {}      # (world size, ranks per q/k group) -> process groups, one per aligned block of ranks


def qk_groups(world: int, share: int):
    """Process groups over every aligned block of `share` consecutive ranks.  Collective: EVERY rank of the
    world must call it (torch.distributed.new_group has to be entered by all ranks, for all groups, in the
    same order), once; the result is cached for later calls."""
    import torch.distributed as dist
    key = (world, share)
    if key not in _QK_GROUPS:
        if world % share != 0:
            raise ValueError("ranks per q/k group must divide the world size")
        _QK_GROUPS[key] = [dist.new_group(list(range(first, first + share))) for first in range(0, world, share)]
    return _QK_GROUPS[key]


def reduce_qk_grads(dq: torch.Tensor, dk: torch.Tensor, shard: Shard, rank: int, group=None):
    """Sum dq / dk over the ranks that hold heads of the same q/k group (no-op when the group is whole).
    Without `group`, the subgroups are created on first use, which every rank of the world reaches together
    because the plan gives all ranks the same `qk_allreduce_group`."""
    if shard.qk_allreduce_group <= 1:
        return dq, dk
    import torch.distributed as dist
    if group is None:
        group = qk_groups(dist.get_world_size(), shard.qk_allreduce_group)[rank // shard.qk_allreduce_group]
    dist.all_reduce(dq, group=group)
    dist.all_reduce(dk, group=group)
    return dq, dk
