"""Sequence-parallel mode on the CPU: the shard algebra against the oracle on the whole sequence (one
process, all shards), and the same through a gloo process group (all-gather forward, summed gradients
backward).  The in-shard operator is the oracle here; on a GPU it is the CUDA path
(tests/test_sequence_parallel_gpu.py)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hattention_b200 import sequence_parallel as sp
from oracle import loglinear_oracle as orc


def _local_op(q, k, v, g, l):
    return orc.mamba2_chunkwise(q, k, v, g, l, chunk=16)


def _inputs(B, T, H, P, N, G, L, seed):
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=seed, dtype=torch.float64)
    do = torch.randn(B, T, H, P, generator=torch.Generator().manual_seed(seed + 1), dtype=torch.float64)
    return q, k, v, g.double(), l, do


def test_cross_shard_levels_follow_the_fenwick_schedule():
    assert sp.cross_shard_levels(0, 8) == []
    assert sp.cross_shard_levels(1, 8) == [(1, [0])]
    assert sp.cross_shard_levels(2, 8) == [(2, [0, 1])]
    assert sp.cross_shard_levels(3, 8) == [(1, [2]), (2, [0, 1])]
    assert sp.cross_shard_levels(7, 8) == [(1, [6]), (2, [4, 5]), (3, [0, 1, 2, 3])]
    # every earlier shard is read exactly once, at level bit_length(r ^ r')
    for r in range(16):
        seen = {}
        for j, ranks in sp.cross_shard_levels(r, 16):
            for c in ranks:
                assert c not in seen
                seen[c] = j
        assert seen == {c: (r ^ c).bit_length() for c in range(r)}
    with pytest.raises(ValueError):
        sp.cross_shard_levels(0, 6)


@pytest.mark.parametrize("shards,G", [(2, 1), (4, 1), (4, 2), (8, 2)])
def test_emulated_shards_match_whole_sequence(shards, G):
    B, T, H, P, N, L = 2, 256, 2, 8, 8, 9
    q, k, v, g, l, do = _inputs(B, T, H, P, N, G, L, seed=11 + shards)
    want_o, want = orc.mamba2_grads(q, k, v, g, l, do, fn=_local_op)
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, l)]
    o = sp.hattention_sequence_parallel_emulated(*ins, shards=shards, local_op=_local_op)
    grads = torch.autograd.grad((o * do).sum(), ins)
    assert torch.allclose(o, want_o, atol=1e-11, rtol=1e-10)
    for a, w_, name in zip(grads, want, ("dq", "dk", "dv", "dg", "dl")):
        assert torch.allclose(a, w_, atol=1e-10, rtol=1e-9), name


def test_too_few_lambda_columns_is_rejected():
    B, T, H, P, N, G, L = 1, 128, 2, 8, 8, 1, 8
    q, k, v, g, l, _ = _inputs(B, T, H, P, N, G, L, seed=5)
    with pytest.raises(ValueError):
        sp.hattention_sequence_parallel_emulated(q, k, v, g, l[..., :7], shards=4, local_op=_local_op)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, T, H, P, N, G, L = 1, 64 * world, 2, 8, 8, 1, 9
    q, k, v, g, l, do = _inputs(B, T, H, P, N, G, L, seed=21)
    want_o, want = orc.mamba2_grads(q, k, v, g, l, do, fn=_local_op)
    Ts = T // world
    sl = slice(rank * Ts, (rank + 1) * Ts)
    ins = [x[:, sl].clone().requires_grad_(True) for x in (q, k, v, g, l)]
    o = sp.hattention_sequence_parallel(*ins, local_op=_local_op)
    grads = torch.autograd.grad((o * do[:, sl]).sum(), ins)
    ok = torch.allclose(o, want_o[:, sl], atol=1e-11, rtol=1e-10)
    for a, w_ in zip(grads, want):
        ok &= torch.allclose(a, w_[:, sl], atol=1e-10, rtol=1e-9)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(int(flag.item()))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_match_whole_sequence(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29640 + world, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1
