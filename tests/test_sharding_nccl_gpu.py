"""Head split over two GPUs with NCCL: each rank runs the CUDA forward + backward on its half of the heads of one
q/k group and the two ranks sum their dq / dk (`sharding.reduce_qk_grads` over a collectively created subgroup);
outputs and gradients equal the unsharded run.  Needs two GPUs; skipped otherwise."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hattention_b200 import HStruct, HType, hattention_kernel, sharding
    from oracle import loglinear_oracle as orc
    B, T, H, P, N, G, L = 1, 2048, 4, 64, 128, 1, 12
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=21)
    do = torch.randn(B, T, H, P, generator=torch.Generator().manual_seed(22))
    q, k, v, l, do = (x.bfloat16().to(dev) for x in (q, k, v, l, do))
    g = g.float().to(dev)

    def run(q_, k_, v_, g_, l_, do_):
        ins = [x.clone().requires_grad_(True) for x in (q_, k_, v_, g_, l_)]
        o = hattention_kernel(ins[0], ins[1], ins[2], None, ins[3], ins[4], None, False, 2, HType.WEAK, HStruct.MAMBA2)
        return o.detach(), torch.autograd.grad(o, ins, do_)

    o_full, gr_full = run(q, k, v, g, l, do)
    shard = sharding.plan(B, H, G, world)[rank]
    qs, ks, vs, gs, ls = sharding.take(shard, q, k, v, g, l, H)
    dos = do[shard.b0:shard.b1, :, shard.h0:shard.h1].contiguous()
    o_s, gr = run(qs.contiguous(), ks.contiguous(), vs.contiguous(), gs.contiguous(), ls.contiguous(), dos)
    dq, dk = sharding.reduce_qk_grads(gr[0].float(), gr[1].float(), shard, rank)
    torch.cuda.synchronize()
    ok = shard.qk_allreduce_group == 2
    ok &= torch.equal(o_s, o_full[shard.b0:shard.b1, :, shard.h0:shard.h1])
    ok &= torch.equal(gr[2], gr_full[2][shard.b0:shard.b1, :, shard.h0:shard.h1])
    for a, w_ in ((dq, gr_full[0]), (dk, gr_full[1])):
        w_ = w_.float()
        # each rank rounds its partial sum to bf16 before the all-reduce; the unsharded run rounds once
        ok &= bool(((a - w_).abs() <= 2e-2 * w_.abs() + 2e-3 * max(1.0, w_.abs().max().item())).all())
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(int(flag.item()))
    dist.destroy_process_group()


def test_head_split_over_two_gpus_with_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29631, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1
