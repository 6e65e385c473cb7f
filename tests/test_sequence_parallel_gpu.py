"""Sequence-parallel mode with the CUDA kernels as the in-shard operator, all shards on one device:
output and gradients against the unsharded CUDA operator on the whole sequence and against the fp64
oracle."""
import pytest
import torch

from oracle import loglinear_oracle as orc

pytestmark = pytest.mark.gpu


def _close(got, want, name, rtol=2e-2, atol=4e-3):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert torch.isfinite(got).all(), name
    tol = rtol * want.abs() + atol * max(1.0, want.abs().max().item())
    worst = ((got - want).abs() / tol).max().item()
    assert worst <= 1.0, f"{name}: worst err/tol = {worst:.3f}"


def _run(fn, tensors, do):
    ins = [x.clone().requires_grad_(True) for x in tensors]
    o = fn(*ins)
    grads = torch.autograd.grad(o, ins, do)
    torch.cuda.synchronize()
    return o, grads


@pytest.mark.parametrize("shards,T,G", [(2, 2048, 1), (4, 4096, 1), (8, 1024, 2)])
def test_emulated_shards_match_unsharded_kernels(shards, T, G):
    from hattention_b200 import sequence_parallel as sp
    dev = torch.device("cuda:0")
    B, H, P, N = 1, 4, 64, 128
    L = 7 + (T // 64 - 1).bit_length()
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=T + shards)
    do = torch.randn(B, T, H, P, generator=torch.Generator().manual_seed(2)).bfloat16().to(dev)
    tensors = [q.bfloat16().to(dev), k.bfloat16().to(dev), v.bfloat16().to(dev), g.float().to(dev), l.bfloat16().to(dev)]
    o_ref, g_ref = _run(sp._default_local_op, tensors, do)
    o_sp, g_sp = _run(lambda *a: sp.hattention_sequence_parallel_emulated(*a, shards=shards), tensors, do)
    _close(o_sp, o_ref, "o")
    for a, w_, name in zip(g_sp, g_ref, ("dq", "dk", "dv", "dg", "dl")):
        _close(a, w_, name)


def test_emulated_shards_match_oracle():
    from hattention_b200 import sequence_parallel as sp
    dev = torch.device("cuda:0")
    B, T, H, P, N, G, shards = 1, 512, 2, 64, 128, 1, 4
    L = 7 + (T // 64 - 1).bit_length()
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=9)
    q, k, v, l = (x.bfloat16().float() for x in (q, k, v, l))
    do = torch.randn(B, T, H, P, generator=torch.Generator().manual_seed(3)).bfloat16().float()
    want_o, want = orc.mamba2_grads(q.double(), k.double(), v.double(), g.double(), l.double(), do.double(),
                                    fn=orc.mamba2_chunkwise)
    tensors = [q.bfloat16().to(dev), k.bfloat16().to(dev), v.bfloat16().to(dev), g.float().to(dev), l.bfloat16().to(dev)]
    o_sp, g_sp = _run(lambda *a: sp.hattention_sequence_parallel_emulated(*a, shards=shards), tensors, do.bfloat16().to(dev))
    _close(o_sp, want_o, "o")
    for a, w_, name in zip(g_sp, want, ("dq", "dk", "dv", "dg", "dl")):
        _close(a, w_, name)
