"""Parity of the CUDA log-linear Gated DeltaNet forward against the CPU oracle (token recurrence
with the delta-rule transition) and the reference-generated golden fixture.
Tolerance: |got - want| <= 2e-2 * |want| + 4e-3 * max(1, max|want|).  The absolute part is twice the
Mamba-2 one because the reference's own bf16 rounding points on this path (q * scale, lambda / scale,
the UT-transform inverses, w, u, the probability tile: hattention/kernel.py:20-29,
gated_delta_rule_apis.py:65-70, chunkwise_hgdn.py:649-700) already put an exact-arithmetic
evaluation of its formulas at 1.2x - 1.7x of the tighter bound against the fp64 recurrence
(tests/test_oracle_golden.py::test_gdn_reference_rounding_points_error_level pins that on the CPU)."""
import os

import numpy as np
import pytest
import torch

from oracle import loglinear_oracle as orc

pytestmark = pytest.mark.gpu


def assert_close(got, want, name, rtol=2e-2, atol=4e-3):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all(), name
    tol = rtol * want.abs() + atol * max(1.0, want.abs().max().item())
    err = (got - want).abs()
    worst = (err / tol).max().item()
    assert worst <= 1.0, f"{name}: worst err/tol = {worst:.3f}, max abs err {err.max().item():.3e}, max|want| {want.abs().max().item():.3e}"


def run_cuda(q, k, v, b, g, l):
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    dev = torch.device("cuda:0")
    o, st = chunk_h_gated_delta_rule(q.bfloat16().to(dev), k.bfloat16().to(dev), v.bfloat16().to(dev), g.float().to(dev),
                                     l.bfloat16().to(dev), b.bfloat16().to(dev), use_qk_l2norm_in_kernel=True)
    torch.cuda.synchronize()
    assert st is None
    return o


def test_golden_fixture_from_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "gdn_c64.npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    o = run_cuda(d["q"], d["k"], d["v"], d["b"], d["g"], d["l"])
    assert_close(o, d["o_chunk"], "o vs hgdn_minimal")
    assert_close(o, d["o_recurrent"], "o vs recurrence")


@pytest.mark.parametrize("B,T,H,Dk,Dv,L", [
    (1, 64, 2, 128, 64, 7),         # one chunk: UT transform and intra output only
    (1, 128, 2, 128, 128, 8),       # two chunks
    (2, 512, 2, 128, 128, 11),      # eight chunks, three levels
    (1, 704, 1, 128, 64, 11),       # 11 chunks (not a power of two)
    (1, 1024, 2, 128, 128, 14),     # 16 chunks, spare lambda levels
    (1, 16384, 1, 128, 64, 15),     # the longest supported sequence: 256 chunks, all eight inter-chunk levels
])
def test_forward_matches_recurrence(B, T, H, Dk, Dv, L):
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=T + Dv)
    q, k, v, b, l = (x.bfloat16().float() for x in (q, k, v, b, l))
    o = run_cuda(q, k, v, b, g, l)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q.double(), k.double(), scale)
    want, _ = orc.recurrent(qn, kn, v.double(), g.double(), l.double() / scale, b=b.double())
    assert_close(o, want, "o")


def run_cuda_grads(q, k, v, b, g, l, do):
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    dev = torch.device("cuda:0")
    ins = [x.to(dev).requires_grad_(True) for x in (q.bfloat16(), k.bfloat16(), v.bfloat16(), b.bfloat16(), g.float(), l.bfloat16())]
    o, _ = chunk_h_gated_delta_rule(ins[0], ins[1], ins[2], ins[4], ins[5], ins[3], use_qk_l2norm_in_kernel=True)
    grads = torch.autograd.grad((o.float() * do.to(dev).float()).sum(), ins)
    torch.cuda.synchronize()
    return o, grads


def test_gradients_match_reference_golden(golden_dir):
    """Gradients w.r.t. the raw q, k, v, beta, g, lambda from the CUDA backward against the reference's
    autograd through hgdn_minimal (fixture)."""
    z = np.load(os.path.join(golden_dir, "gdn_c64.npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    o, grads = run_cuda_grads(d["q"], d["k"], d["v"], d["b"], d["g"], d["l"], d["do"])
    assert_close(o, d["o_chunk"], "o")
    for got, key in zip(grads, ("dq", "dk", "dv", "db", "dg", "dl")):
        assert_close(got, d[key], key)


def test_gradients_match_oracle_multi_level():
    B, T, H, Dk, Dv, L = 1, 512, 2, 128, 64, 11
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=77)
    q, k, v, b, l = (x.bfloat16().float() for x in (q, k, v, b, l))
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(5)).bfloat16().float()
    scale = Dk ** -0.5
    o, grads = run_cuda_grads(q, k, v, b, g, l, do)
    # oracle: recurrence in fp64 with lambda / scale applied as the API does
    ins = [x.double().requires_grad_(True) for x in (q, k, v, b, g, l)]
    qn, kn = orc.gdn_layer_inputs(ins[0], ins[1], scale)
    want, _ = orc.recurrent(qn, kn, ins[2], ins[4], ins[5] / scale, b=ins[3])
    wg = torch.autograd.grad((want * do.double()).sum(), ins)
    assert_close(o, want, "o")
    for got, w_, key in zip(grads, wg, ("dq", "dk", "dv", "db", "dg", "dl")):
        assert_close(got, w_, key)


@pytest.mark.parametrize("Dk,Dv", [(128, 192), (64, 128)])
def test_wide_value_head_and_narrow_key_head_match_oracle(Dk, Dv):
    """Dv = 192: the host side runs a 128-column and a 64-column slice (the delta rule treats value columns
    independently).  Dk = 64: q and k are padded with zero features to the kernels' key width.  Output and every
    gradient against the fp64 recurrence."""
    B, T, H, L = 1, 256, 2, 9
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=Dv)
    q, k, v, b, l = (x.bfloat16().float() for x in (q, k, v, b, l))
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(6)).bfloat16().float()
    scale = Dk ** -0.5
    o, grads = run_cuda_grads(q, k, v, b, g, l, do)
    ins = [x.double().requires_grad_(True) for x in (q, k, v, b, g, l)]
    qn, kn = orc.gdn_layer_inputs(ins[0], ins[1], scale)
    want, _ = orc.recurrent(qn, kn, ins[2], ins[4], ins[5] / scale, b=ins[3])
    wg = torch.autograd.grad((want * do.double()).sum(), ins)
    assert_close(o, want, "o")
    for got, w_, key in zip(grads, wg, ("dq", "dk", "dv", "db", "dg", "dl")):
        assert_close(got, w_, key)


@pytest.mark.parametrize("B,T,H,Dv,L", [(1, 1408, 2, 128, 12), (2, 1024, 1, 64, 11)])
def test_backward_stages_match_whole_path_autograd(B, T, H, Dv, L):
    """Driver-level gradients (normalised q, k) from the CUDA backward, and from its level stage
    alone completed by a batched torch chunk-local stage, against autograd through the chunk-by-chunk torch restatement of the whole path; 22 chunks (not a power
    of two, five levels) with V = 128, and 16 chunks with V = 64."""
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    dev = torch.device("cuda:0")
    Dk = 128
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=T)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q, k, scale)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l / scale))
    g = g.float().to(dev)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(3)).bfloat16().to(dev)
    g_cum, o, Aw, Au, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False)
    got = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64)
    import gdn_torch_stages as gts
    staged = gts.chunkwise_bwd_staged(qn, kn, v, b, g_cum, l, Aw, Au, do)
    want = gts.chunkwise_bwd_autograd(qn, kn, v, b, g_cum, l, do)
    torch.cuda.synchronize()
    for a, w_, key in zip(staged, want, ("dq", "dk", "dv", "db", "dg", "dl")):
        rel = ((a.double() - w_.double()).norm() / w_.double().norm()).item()
        assert rel <= 5e-3, f"staged {key}: relative Frobenius error {rel:.2e}"
    # `want` is an fp32 evaluation with none of the bf16 rounding points of the kernels (chunk matrices,
    # level states and their adjoints are bf16 tensor-core operands), so the whole-tensor error must be at
    # bf16 rounding level and single elements get twice the absolute allowance of the other tests
    for a, w_, key in zip(got, want, ("dq", "dk", "dv", "db", "dg", "dl")):
        rel = ((a.double() - w_.double()).norm() / w_.double().norm()).item()
        assert rel <= 5e-3, f"{key}: relative Frobenius error {rel:.2e}"
        assert_close(a, w_, key, atol=8e-3)


@pytest.mark.parametrize("B,T,H,Dv,L", [(1, 1408, 2, 128, 12), (2, 1024, 1, 64, 11), (1, 64, 2, 128, 7)])
def test_backward_with_forward_states_kept(B, T, H, Dv, L):
    """The forward that leaves its chunk matrices and level states in the workspace returns the same
    output, and the backward that reads them returns the gradients of the recomputing backward (same
    kernels on the same bf16 values; only the order of the atomic adds into dl differs)."""
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    dev = torch.device("cuda:0")
    Dk = 128
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=T + 1)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q, k, scale)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l / scale))
    g = g.float().to(dev)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(4)).bfloat16().to(dev)
    g_cum, o, Aw, Au, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False)
    kept = []
    g_cum2, o2, Aw2, Au2, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
    assert len(kept) == 1
    for a, w_ in ((g_cum2, g_cum), (o2, o), (Aw2, Aw), (Au2, Au)):
        assert torch.equal(a, w_)
    want = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64)
    got = hg.chunkwise_bwd(qn, kn, v, b, g_cum2, l, Aw2, Au2, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])
    torch.cuda.synchronize()
    for a, w_, key in zip(got, want, ("dq", "dk", "dv", "db", "dg", "dl")):
        assert torch.isfinite(a).all(), key
        torch.testing.assert_close(a, w_, rtol=1e-4, atol=1e-5 * max(1.0, w_.abs().max().item()), msg=key)


def test_autograd_function_keeps_and_releases_forward_states():
    """hattention_kernel keeps the forward workspace on the autograd context and drops it in backward;
    with the switch off the gradients are the same."""
    from hattention_b200 import kernel as hk
    B, T, H, Dk, Dv, L = 1, 512, 2, 128, 64, 11
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=78)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(6))
    assert hk.KEEP_FORWARD_STATES
    _, kept_grads = run_cuda_grads(q, k, v, b, g, l, do)
    hk.KEEP_FORWARD_STATES = False
    try:
        _, plain_grads = run_cuda_grads(q, k, v, b, g, l, do)
    finally:
        hk.KEEP_FORWARD_STATES = True
    for a, w_, key in zip(kept_grads, plain_grads, ("dq", "dk", "dv", "db", "dg", "dl")):
        torch.testing.assert_close(a.float(), w_.float(), rtol=2e-2, atol=1e-2 * max(1.0, w_.float().abs().max().item()), msg=key)


@pytest.mark.parametrize("D", [64, 128, 256])
def test_l2norm_kernels(D):
    """l2norm forward (with the reference's two bf16 rounding points) and backward against torch."""
    from hattention_b200 import chunkwise_hgdn as hg
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(D)
    x = torch.randn(3, 37, 5, D, generator=gen).bfloat16().to(dev)
    dy = torch.randn(3, 37, 5, D, generator=gen).to(dev)
    scale = D ** -0.5
    y = hg.l2norm_fwd(x, scale)
    xf = x.float()
    rstd = torch.rsqrt((xf * xf).sum(-1, keepdim=True) + 1e-6)
    want = ((xf * rstd).bfloat16().float() * scale).bfloat16()
    # rsqrtf and the reduction order may move a value by one bf16 ulp
    assert ((y.float() - want.float()).abs() <= 2.0 ** -7 * want.float().abs() + 1e-30).all()
    assert (y == want).float().mean().item() > 0.98
    dx = hg.l2norm_bwd(x, dy, scale)
    xr = xf.clone().requires_grad_(True)
    yr = xr * torch.rsqrt((xr * xr).sum(-1, keepdim=True) + 1e-6) * scale
    (gx,) = torch.autograd.grad(yr, xr, dy)
    torch.testing.assert_close(dx.float(), gx, rtol=1e-2, atol=1e-2 * gx.abs().max().item())


@pytest.mark.parametrize("B,T,H,Dv,L", [(1, 1408, 2, 128, 12), (2, 1024, 1, 64, 11), (1, 8192, 1, 128, 14), (1, 192, 1, 64, 9),
                                         (1, 16384, 1, 128, 15), (1, 16320, 1, 64, 15), (1, 64, 2, 128, 7)])
def test_tensor_core_scans_match_warp_mma_scans(B, T, H, Dv, L):
    """The tcgen05 scans over chunks against the warp-MMA kernels on the same inputs: both keep fp32 master
    states and round the same operands to bf16 (level states, u - sum wd H), so outputs and gradients agree to
    accumulation-order level.  T = 8192 reaches all seven inter-chunk levels of the largest benchmark shape, T = 16384 the
    eighth (the longest supported sequence: every tensor-memory slot of the scans in use), 16320 = 255 chunks ends on the
    chunk with all eight levels live, T = 64 is a single chunk (no scan step at all)."""
    from hattention_b200 import _lib
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    dev = torch.device("cuda:0")
    Dk = 128
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=T + 9)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q, k, scale)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l / scale))
    g = g.float().to(dev)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(8)).bfloat16().to(dev)

    def run():
        g_cum, o, Aw, Au, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False)
        grads = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64)
        torch.cuda.synchronize()
        return (o,) + tuple(grads)

    got = run()
    _lib.lib().llattn_testing_use_tensor_core_path(0)
    try:
        want = run()
    finally:
        _lib.lib().llattn_testing_use_tensor_core_path(1)
    for a, w_, key in zip(got, want, ("o", "dq", "dk", "dv", "db", "dg", "dl")):
        assert torch.isfinite(a).all(), key
        rel = ((a.double() - w_.double()).norm() / w_.double().norm().clamp_min(1e-30)).item()
        assert rel <= 2e-3, f"{key}: relative Frobenius difference {rel:.2e}"
        assert_close(a.float(), w_.float(), key)       # single elements: this path's tolerance against the oracle


def test_repeated_calls_are_bit_identical():
    """Twenty forward + backward calls on the same inputs at 128 chunks (all seven inter-chunk levels): the output and every
    gradient must come out bit for bit the same (no kernel of this path accumulates with atomics).  The tcgen05 kernels hand tiles
    between a TMA producer, one MMA-issuing thread and eight element-wise warps through mbarriers; an ordering mistake there
    shows up as an occasional difference between repetitions rather than as a wrong result every time."""
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    dev = torch.device("cuda:0")
    B, T, H, Dk, Dv, L = 1, 8192, 4, 128, 128, 14
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=21)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q, k, scale)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l / scale))
    g = g.float().to(dev)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(9)).bfloat16().to(dev)
    first = None
    for rep in range(20):
        kept = []
        g_cum, o, Aw, Au, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
        dq, dk, dv, db, dg, dl = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])
        torch.cuda.synchronize()
        cur = dict(o=o, Aw=Aw, Au=Au, dq=dq, dk=dk, dv=dv, db=db, dg=dg, dl=dl)
        if first is None:
            first = {k_: x.clone() for k_, x in cur.items()}
            for k_, x in cur.items():
                assert torch.isfinite(x.float()).all(), k_
        else:
            for k_, x in cur.items():
                assert torch.equal(x, first[k_]), f"{k_} differs in repetition {rep}"


def test_kept_backward_writes_dv_in_bf16():
    """llattn_gdn_bwd_kept_bf16dv: dv written by the kernel in bf16 equals the fp32 dv of llattn_gdn_bwd_kept rounded to bf16,
    element for element, and the other gradients are bit-identical."""
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    dev = torch.device("cuda:0")
    B, T, H, Dk, Dv, L = 2, 1024, 3, 128, 128, 11
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=5)
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q, k, scale)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l / scale))
    g = g.float().to(dev)
    do = torch.randn(B, T, H, Dv, generator=torch.Generator().manual_seed(2)).bfloat16().to(dev)
    kept = []
    g_cum, o, Aw, Au, _ = hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
    ref = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])
    got = hg.chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0], dv_bf16=True)
    assert got[2].dtype == torch.bfloat16 and ref[2].dtype == torch.float32
    assert torch.equal(got[2], ref[2].to(torch.bfloat16))
    for i_ in (0, 1, 3, 4, 5):
        assert torch.equal(got[i_], ref[i_])
