"""Size-independent properties at the benchmark sizes, over the whole launch (oracle parity of head
subsets at the same sizes is in tests/test_baseline_configs_gpu.py): linearity in v, causality,
batch x head independence, and gradient identities that follow from the bilinear structure
o = A(q, k, g, lambda) v :
    sum(do * o) = sum(dv * v) = sum(dlambda * lambda)       (o is linear in v and in lambda)
Shapes: the headline Mamba-2 workload (B=2, T=16384, H=32, P=64, N=128, L=15), the forward-only
configuration (B=8, T=4096, H=24, L=13) and the Gated DeltaNet configuration (B=4, T=8192, H=16,
Dk=Dv=128, L=14)."""
import pytest
import torch

from oracle import loglinear_oracle as orc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _m2_inputs(B, T, H, L, seed):
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, 64, 128, 1, L, seed=seed)
    return [x.bfloat16().to(DEV) for x in (q, k, v)] + [g.float().to(DEV), l.bfloat16().to(DEV)]


def _fwd(q, k, v, g, l):
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_fwd
    return chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False)


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


@pytest.mark.parametrize("B,T,H,L", [(2, 16384, 32, 15), (8, 4096, 24, 13)])
def test_mamba2_forward_properties(B, T, H, L):
    q, k, v, g, l = _m2_inputs(B, T, H, L, seed=3)
    o, g_cum, _ = _fwd(q, k, v, g, l)
    assert torch.isfinite(o.float()).all()
    # in-chunk cumulative sum of g against torch
    want = torch.cumsum(g.view(B, T // 64, 64, H), dim=2).view(B, T, H)
    torch.testing.assert_close(g_cum, want, rtol=1e-5, atol=1e-5)
    # linearity in v (bf16 outputs: compare at bf16 resolution)
    v2 = torch.randn_like(v)
    o2, _, _ = _fwd(q, k, v2, g, l)
    o12, _, _ = _fwd(q, k, (v.float() + v2.float()).bfloat16(), g, l)
    assert _rel(o12.float(), o.float() + o2.float()) < 1e-2
    # causality: changing everything after t0 leaves the outputs before t0 bit-identical
    t0 = T // 2 + 64 * 3
    qc, kc, vc, gc, lc = (x.clone() for x in (q, k, v, g, l))
    for x in (qc, kc, vc, lc):
        x[:, t0:] = torch.randn_like(x[:, t0:])
    gc[:, t0:] = -torch.rand_like(gc[:, t0:])
    oc, _, _ = _fwd(qc, kc, vc, gc, lc)
    assert torch.equal(oc[:, :t0], o[:, :t0])
    # batch x head independence: the last batch element and the upper half of the heads on their own
    hs = H // 2
    op, _, _ = _fwd(q[-1:], k[-1:], v[-1:, :, hs:], g[-1:, :, hs:], l[-1:, :, hs:])
    assert torch.equal(op, o[-1:, :, hs:])


def test_mamba2_backward_identities_at_headline_size():
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd
    B, T, H, L = 2, 16384, 32, 15
    q, k, v, g, l = _m2_inputs(B, T, H, L, seed=4)
    do = torch.randn(B, T, H, 64, generator=torch.Generator().manual_seed(9)).bfloat16().to(DEV)
    o, g_cum, _ = _fwd(q, k, v, g, l)
    dq, dk, dv, dg, dl = chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64)
    for t in (dq, dk, dv, dg, dl):
        assert torch.isfinite(t.float()).all()
    s_o = (do.double() * o.double()).sum().item()
    s_v = (dv.double() * v.double()).sum().item()
    s_l = (dl.double() * l.double()).sum().item()
    scale = (do.double().abs() * o.double().abs()).sum().item()
    assert abs(s_o - s_v) < 2e-3 * scale
    assert abs(s_o - s_l) < 2e-3 * scale
    # q and k enter only through q.k^T: sum(dq * q) = sum(dk * k) (both equal the sum over pairs of dS * S)
    s_q = (dq.double() * q.double()).sum().item()
    s_k = (dk.double() * k.double()).sum().item()
    assert abs(s_q - s_k) < 2e-3 * max(abs(s_q), abs(s_k), 1e-3 * scale)


def test_gdn_properties_at_config_size():
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    B, T, H, D, L = 4, 8192, 16, 128, 14
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, D, D, L, seed=5)
    q, k, v, b, l = (x.bfloat16().to(DEV) for x in (q, k, v, b, l))
    g = g.float().to(DEV)
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, l, b)]
    o, _ = chunk_h_gated_delta_rule(*ins, use_qk_l2norm_in_kernel=True)
    do = torch.randn(B, T, H, D, generator=torch.Generator().manual_seed(1)).bfloat16().to(DEV)
    grads = torch.autograd.grad(o, ins, do)
    assert torch.isfinite(o.float()).all()
    for t in grads:
        assert torch.isfinite(t.float()).all()
    # o is linear in lambda: sum(do * o) = sum(dlambda * lambda)
    s_o = (do.double() * o.double()).sum().item()
    s_l = (grads[4].double() * l.double()).sum().item()
    scale = (do.double().abs() * o.double().abs()).sum().item()
    assert abs(s_o - s_l) < 3e-3 * scale
    # l2norm makes o invariant to the scale of q and k rows: the gradients are orthogonal to them
    for x, dx in ((q, grads[0]), (k, grads[1])):
        dots = (x.double() * dx.double()).sum(-1)
        assert dots.abs().max().item() < 2e-2 * (x.double().norm(dim=-1) * dx.double().norm(dim=-1)).max().item()
    # causality
    t0 = T // 2 + 64
    ins2 = [x.detach().clone() for x in ins]
    for i in (0, 1, 2, 4):
        ins2[i][:, t0:] = torch.randn_like(ins2[i][:, t0:])
    o2, _ = chunk_h_gated_delta_rule(*ins2, use_qk_l2norm_in_kernel=True)
    assert torch.equal(o2[:, :t0], o.detach()[:, :t0])
    # batch x head independence
    sub = [ins[0][-1:, :, 8:], ins[1][-1:, :, 8:], ins[2][-1:, :, 8:], ins[3][-1:, :, 8:], ins[4][-1:, :, 8:], ins[5][-1:, :, 8:]]
    o3, _ = chunk_h_gated_delta_rule(*[x.detach().contiguous() for x in sub], use_qk_l2norm_in_kernel=True)
    assert torch.equal(o3, o.detach()[-1:, :, 8:])


def test_mamba2_longest_sequence_identities():
    """T = 65536 (1024 chunks, 128 segments, seven segment levels: the shapes of the multi-GPU scaling
    configuration, one batch element and two heads of it): forward finite and causal, gradient identities."""
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd
    B, T, H, L = 1, 65536, 2, 17
    q, k, v, g, l = _m2_inputs(B, T, H, L, seed=6)
    do = torch.randn(B, T, H, 64, generator=torch.Generator().manual_seed(8)).bfloat16().to(DEV)
    o, g_cum, _ = _fwd(q, k, v, g, l)
    assert torch.isfinite(o.float()).all()
    t0 = 40000 - (40000 % 64)
    o_head, _, _ = _fwd(q[:, :t0], k[:, :t0], v[:, :t0], g[:, :t0], l[:, :t0])
    # the shorter call has fewer segment levels but the same buckets for every (target, source) pair
    assert _rel(o_head.float(), o[:, :t0].float()) < 5e-3
    dq, dk, dv, dg, dl = chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64)
    for t in (dq, dk, dv, dg, dl):
        assert torch.isfinite(t.float()).all()
    s_o = (do.double() * o.double()).sum().item()
    s_v = (dv.double() * v.double()).sum().item()
    s_l = (dl.double() * l.double()).sum().item()
    scale = (do.double().abs() * o.double().abs()).sum().item()
    assert abs(s_o - s_v) < 2e-3 * scale
    assert abs(s_o - s_l) < 2e-3 * scale
    # the same call on the warp-MMA kernels (seven segment levels take two level windows in the tensor-core
    # high-level backward and the eight-slot variant of the high-level forward)
    from hattention_b200 import _lib
    _lib.lib().llattn_testing_use_tensor_core_path(0)
    try:
        o_w, g_w, _ = _fwd(q, k, v, g, l)
        gr_w = chunkwise_bwd(q, k, v, g_w, l, do, False, 2, HType.WEAK, 64)
        torch.cuda.synchronize()
    finally:
        _lib.lib().llattn_testing_use_tensor_core_path(1)
    assert _rel(o.float(), o_w.float()) < 5e-3
    for a, b_, name in zip((dq, dk, dv, dg, dl), gr_w, ("dq", "dk", "dv", "dg", "dl")):
        assert _rel(a.float(), b_.float()) < 1e-2, name
