"""The `llattn::*` torch.library operators: registered, traceable with fake tensors (CPU), and on the GPU
identical to the Python drivers and clean under torch.library.opcheck."""
import pytest
import torch


def test_operators_are_registered_and_trace_with_fake_tensors():
    from torch._subclasses.fake_tensor import FakeTensorMode
    import hattention_b200.ops  # noqa: F401
    for name in ("mamba2_fwd", "mamba2_bwd", "gdn_fwd", "gdn_bwd", "l2norm_scale_fwd", "l2norm_scale_bwd"):
        assert hasattr(torch.ops.llattn, name)
    B, T, H, G, K, V, L = 2, 1024, 4, 1, 128, 64, 11
    with FakeTensorMode():
        q = torch.empty(B, T, G, K, dtype=torch.bfloat16)
        v = torch.empty(B, T, H, V, dtype=torch.bfloat16)
        g = torch.empty(B, T, H)
        l = torch.empty(B, T, H, L, dtype=torch.bfloat16)
        o, g_cum, ws = torch.ops.llattn.mamba2_fwd(q, q, v, g, l)
        assert o.shape == v.shape and o.dtype == torch.bfloat16 and g_cum.shape == g.shape and ws.dtype == torch.uint8
        assert ws.numel() >= 256
        dq, dk, dv, dg, dl = torch.ops.llattn.mamba2_bwd(q, q, v, g_cum, l, o, ws)
        assert dq.shape == q.shape and dv.shape == v.shape and dl.shape == l.shape and dl.dtype == torch.float32
        qh = torch.empty(B, T, H, K, dtype=torch.bfloat16)
        vh = torch.empty(B, T, H, 128, dtype=torch.bfloat16)
        beta = torch.empty(B, T, H, dtype=torch.bfloat16)
        g_cum, o, Aw, Au = torch.ops.llattn.gdn_fwd(qh, qh, vh, beta, g, l)
        assert o.shape == vh.shape and Aw.shape == (B, T, H, 64)
        grads = torch.ops.llattn.gdn_bwd(qh, qh, vh, beta, g_cum, l, Aw, Au, o)
        assert [t.shape for t in grads] == [qh.shape, qh.shape, vh.shape, beta.shape, g.shape, l.shape]
        assert torch.ops.llattn.l2norm_scale_fwd(qh, 0.5).shape == qh.shape


@pytest.mark.gpu
def test_operators_match_the_drivers_and_pass_opcheck():
    from hattention_b200 import ops  # noqa: F401
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd, chunkwise_fwd
    from oracle import loglinear_oracle as orc
    dev = torch.device("cuda:0")
    q, k, v, g, l = orc.make_mamba2_inputs(1, 1024, 2, 64, 128, 1, 11, seed=1)
    q, k, v, l = (x.bfloat16().to(dev) for x in (q, k, v, l))
    g = g.float().to(dev)
    do = torch.randn_like(v)
    o, g_cum, ws = torch.ops.llattn.mamba2_fwd(q, k, v, g, l)
    o2, g2, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False)
    assert torch.equal(o, o2) and torch.equal(g_cum, g2)
    got = torch.ops.llattn.mamba2_bwd(q, k, v, g_cum, l, do, ws)
    want = chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64)
    for a, b, name in zip(got, want, ("dq", "dk", "dv", "dg", "dl")):
        if name in ("dq", "dk", "dg"):  # fp32 reduce-adds (over heads / over kernels): order varies from run to run
            assert torch.allclose(a.float(), b.float(), rtol=2e-2, atol=1e-3), name
        else:
            assert torch.equal(a, b), name
    torch.library.opcheck(torch.ops.llattn.mamba2_fwd, (q, k, v, g, l), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.llattn.l2norm_scale_fwd, (torch.randn(4, 64, 2, 128, device=dev).bfloat16(), 0.5),
                          test_utils=("test_schema", "test_faketensor"))
