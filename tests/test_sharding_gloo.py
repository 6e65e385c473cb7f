"""Batch x head sharding on two CPU ranks (gloo): every rank computes its shard with the oracle,
the gathered output equals the unsharded result, and dq / dk need a sum over ranks exactly when
the heads of one q/k group are split."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hattention_b200 import sharding
from oracle import loglinear_oracle as orc


def test_plan_batch_first_then_heads():
    p = sharding.plan(8, 32, 1, 8)
    assert [(s.b0, s.b1, s.h0, s.h1) for s in p][:2] == [(0, 1, 0, 32), (1, 2, 0, 32)]
    assert all(s.qk_allreduce_group == 1 for s in p)
    p = sharding.plan(2, 32, 1, 8)            # config 3 on 8 GPUs: 4 ranks per batch item share one group
    assert (p[5].b0, p[5].h0, p[5].h1) == (1, 8, 16)
    assert all(s.qk_allreduce_group == 4 for s in p)
    p = sharding.plan(2, 32, 32, 8)           # one group per head: nothing to reduce
    assert all(s.qk_allreduce_group == 1 for s in p)
    with pytest.raises(ValueError):
        sharding.plan(3, 32, 1, 2)
    # head ranges that straddle q/k groups are refused (their dq / dk would miss other ranks' parts)
    with pytest.raises(ValueError):
        sharding.plan(1, 12, 2, 3)            # 4 heads per rank, groups of 6
    with pytest.raises(ValueError):
        sharding.plan(1, 12, 4, 3)            # 4 heads per rank, groups of 3
    p = sharding.plan(1, 12, 2, 2)            # 6 heads per rank = one whole group each
    assert all(s.qk_allreduce_group == 1 for s in p)
    p = sharding.plan(1, 12, 2, 6)            # 2 heads per rank, three ranks share a group
    assert all(s.qk_allreduce_group == 3 for s in p)


def _worker(rank, world, port, split_heads, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if world == 4:
        B, T, H, P, N, G, L = 2, 128, 4, 8, 8, 1, 8         # two batch items x two head halves: two subgroups of two ranks
    else:
        B, T, H, P, N, G, L = (1, 128, 4, 8, 8, 1, 8) if split_heads else (2, 128, 2, 8, 8, 1, 8)
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=3, dtype=torch.float64)
    do = torch.randn(B, T, H, P, generator=torch.Generator().manual_seed(4), dtype=torch.float64)
    g = g.double()
    o_full, grads_full = orc.mamba2_grads(q, k, v, g, l, do, fn=lambda *a: orc.mamba2_chunkwise(*a, chunk=16))
    shard = sharding.plan(B, H, G, world)[rank]
    qs, ks, vs, gs, ls = sharding.take(shard, q, k, v, g, l, H)
    dos = do[shard.b0:shard.b1, :, shard.h0:shard.h1]
    o_s, gr = orc.mamba2_grads(qs, ks, vs, gs, ls, dos, fn=lambda *a: orc.mamba2_chunkwise(*a, chunk=16))
    dq, dk = sharding.reduce_qk_grads(gr[0].clone(), gr[1].clone(), shard, rank)
    if world == 4:
        # a second step through the cached subgroups: both ranks of a subgroup hold the sum, so halves add up to it again
        dq, dk = sharding.reduce_qk_grads(dq / 2, dk / 2, shard, rank)
    ok = torch.allclose(o_s, o_full[shard.b0:shard.b1, :, shard.h0:shard.h1], atol=1e-12)
    ok &= torch.allclose(gr[2], grads_full[2][shard.b0:shard.b1, :, shard.h0:shard.h1], atol=1e-10)
    ok &= torch.allclose(dq, grads_full[0][shard.b0:shard.b1], atol=1e-10)
    ok &= torch.allclose(dk, grads_full[1][shard.b0:shard.b1], atol=1e-10)
    ok &= (shard.qk_allreduce_group == (2 if split_heads else 1))
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(int(flag.item()))
    dist.destroy_process_group()


@pytest.mark.parametrize("split_heads", [False, True])
def test_two_rank_gloo_sharding_matches_unsharded(split_heads):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29611 + (1 if split_heads else 0)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, split_heads, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1


def test_four_rank_gloo_two_subgroups():
    """World larger than the q/k group: two batch items, each split over two ranks by heads, so two disjoint
    subgroups of two ranks reduce dq / dk; the subgroups are created once, collectively, and reused."""
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 4, 29617, True, ret)) for r in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1
