"""Prefill hand-off and decode steps of the Mamba-2 structure against the CPU oracle's token
recurrence (whose level states and counts are pinned to the reference's `hattention_recurrent`
by the golden fixtures)."""
import pytest
import torch

from oracle import loglinear_oracle as orc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def assert_close(got, want, name, rtol=2e-2, atol=2e-3):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    tol = rtol * want.abs() + atol * max(1.0, want.abs().max().item())
    worst = ((got - want).abs() / tol).max().item()
    assert worst <= 1.0, f"{name}: worst err/tol = {worst:.3f}"


@pytest.mark.parametrize("T,N", [(200, 128), (64, 64), (333, 128), (1024, 128)])
def test_prefill_then_decode_matches_recurrence(T, N):
    from hattention_b200.base import HStruct, HType
    from hattention_b200.kernel import hattention_prefill, hattention_step
    B, H, P, G, L, NDEC = 2, 2, 64, 1, 12, 6
    q, k, v, g, l = orc.make_mamba2_inputs(B, T + NDEC, H, P, N, G, L, seed=T)
    q, k, v, l = (x.bfloat16().float() for x in (q, k, v, l))
    want_o, st = orc.recurrent(q[:, :T].double(), k[:, :T].double(), v[:, :T].double(), g[:, :T].double(), l[:, :T].double())
    dq, dk, dv, dl = (x.bfloat16().to(DEV) for x in (q, k, v, l))
    dg = g.float().to(DEV)
    o, hs = hattention_prefill(dq[:, :T], dk[:, :T], dv[:, :T], None, dg[:, :T], dl[:, :T], None, False, 2,
                               HType.WEAK, HStruct.MAMBA2, 64)
    torch.cuda.synchronize()
    assert_close(o, want_o, "prefill output")
    assert hs.counts == list(st.counts)
    assert hs.states.shape == (B, H, N, P, L) and hs.states.dtype == torch.float32
    assert_close(hs.states, torch.stack(st.states, dim=-1), "level states after prefill")
    # decode: continue token by token and compare with the recurrence over the whole sequence
    want_all, st2 = orc.recurrent(q.double(), k.double(), v.double(), g.double(), l.double())
    for t in range(T, T + NDEC):
        ot, hs = hattention_step(hs, dq[:, t], dk[:, t], dv[:, t], None, dg[:, t], dl[:, t], None, 2, HType.WEAK, HStruct.MAMBA2)
        assert_close(ot, want_all[:, t], f"decode step {t}")
    torch.cuda.synchronize()
    assert hs.counts == list(st2.counts)
    assert_close(hs.states, torch.stack(st2.states, dim=-1), "level states after decoding")


def test_decode_from_empty_state():
    """Stepping from an empty state reproduces the recurrence from its first token."""
    from hattention_b200.base import HStruct, HType
    from hattention_b200.kernel import HState, hattention_step
    B, H, P, N, G, L, T = 1, 4, 64, 128, 2, 8, 37
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=2)
    q, k, v, l = (x.bfloat16().float() for x in (q, k, v, l))
    want, st = orc.recurrent(q.double(), k.double(), v.double(), g.double(), l.double())
    hs = HState(2, HType.WEAK, HStruct.MAMBA2, (B, H, N, P, L), torch.float32, DEV)
    dq, dk, dv, dl = (x.bfloat16().to(DEV) for x in (q, k, v, l))
    dg = g.float().to(DEV)
    for t in range(T):
        ot, hs = hattention_step(hs, dq[:, t], dk[:, t], dv[:, t], None, dg[:, t], dl[:, t], None, 2, HType.WEAK, HStruct.MAMBA2)
        assert_close(ot, want[:, t], f"step {t}")
    assert hs.counts == list(st.counts)


def test_layer_api_prefill_states_then_layer_decode_step():
    """The calls the reference's mixer makes at inference (modeling_hattention.py:467-490, 342-362):
    hmamba_chunk_scan_combined(..., return_final_states=True) for the prompt, then hselective_state_update per
    token, against the oracle's recurrence on the prepared tensors; and return_final_states=False gives the same
    prompt outputs with no state."""
    from hattention_b200.base import HStruct, HType
    from hattention_b200.mamba_apis import hmamba_chunk_scan_combined, hselective_state_update
    from hattention_b200.recurrent import HState
    torch.manual_seed(1)
    B, T, H, P, N, L, NDEC = 2, 200, 2, 64, 128, 12, 4
    TT = T + NDEC
    x = torch.randn(B, TT, H, P).bfloat16()
    dt = (torch.randn(B, TT, H) - 2).bfloat16()
    A = -torch.exp(torch.rand(H) * 2.7)
    Bm = (torch.randn(B, TT, 1, N) / N ** 0.5).bfloat16()
    Cm = (torch.randn(B, TT, 1, N) / N ** 0.5).bfloat16()
    dl = torch.randn(B, TT, H, L).bfloat16()
    Lp = torch.ones(H, L)
    D = torch.randn(H)
    bias = torch.randn(H) * 0.1
    kw = dict(dt_softplus=True, lambda_mode="positive", lambda_level_max=L, lambda_level_base=2, lambda_htype=HType.WEAK,
              lambda_hstruct=HStruct.MAMBA2, lambda_level_fixed=True)
    d = lambda t: t.to(DEV)
    y, state = hmamba_chunk_scan_combined(d(x[:, :T]), d(dt[:, :T]), d(A), d(Bm[:, :T]), d(Cm[:, :T]), d(dl[:, :T]), d(Lp), 64,
                                          D=d(D), dt_bias=d(bias), return_final_states=True, **kw)
    assert isinstance(state, HState) and state.states.shape == (B, H, N, P, L) and sum(state.counts) == T
    y0, none = hmamba_chunk_scan_combined(d(x[:, :T - 8]), d(dt[:, :T - 8]), d(A), d(Bm[:, :T - 8]), d(Cm[:, :T - 8]),
                                          d(dl[:, :T - 8]), d(Lp), 64, D=d(D), dt_bias=d(bias), return_final_states=False, **kw)
    assert none is None
    # oracle on the prepared tensors
    dts = torch.nn.functional.softplus(dt.float() + bias[None, None])
    v = (x.float() * dts[..., None]).bfloat16().double()
    g = (A[None, None] * dts).double()
    lam = torch.nn.functional.softplus(Lp[None, None] * dl.float()).bfloat16().double()
    want, st = orc.recurrent(Cm.double(), Bm.double(), v, g, lam)
    want = want + x.double() * D[None, None, :, None].double()
    assert_close(y, want[:, :T], "prompt outputs with final states")
    assert_close(y0, want[:, :T - 8], "prompt outputs without final states")
    for t in range(T, TT):
        out, state = hselective_state_update(state, d(x[:, t]), d(dt[:, t]), d(A), d(Bm[:, t]), d(Cm[:, t]), d(dl[:, t]), d(Lp),
                                             D=d(D), dt_bias=d(bias), **kw)
        assert_close(out, want[:, t], f"layer decode step {t}")
    torch.cuda.synchronize()
    assert state.counts == list(st.counts)


@pytest.mark.parametrize("T,Dv", [(200, 64), (64, 128), (333, 128), (1024, 128), (40, 64)])
def test_gdn_prefill_then_decode_matches_recurrence(T, Dv):
    """Delta-rule structure through the layer API: prompt call with output_final_state=True (chunkwise kernels for the
    full chunks, level states exported before the last one, its tokens stepped), then one-token calls with the
    returned state, against the fp64 token recurrence on the prepared tensors."""
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    B, H, Dk, L, NDEC = 2, 2, 128, 12, 5
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T + NDEC, H, Dk, Dv, L, seed=T)
    q, k, v, b, l = (x.bfloat16().float() for x in (q, k, v, b, l))
    scale = Dk ** -0.5
    qn, kn = orc.gdn_layer_inputs(q.double(), k.double(), scale)
    want, st = orc.recurrent(qn, kn, v.double(), g.double(), l.double() / scale, b=b.double())
    d = lambda x: x.bfloat16().to(DEV)
    dq, dk, dv, db, dl = d(q), d(k), d(v), d(b), d(l)
    dg = g.float().to(DEV)
    o, hs = chunk_h_gated_delta_rule(dq[:, :T], dk[:, :T], dv[:, :T], dg[:, :T], dl[:, :T], db[:, :T],
                                     output_final_state=True, use_qk_l2norm_in_kernel=True)
    torch.cuda.synchronize()
    assert_close(o, want[:, :T], "prompt outputs", atol=4e-3)
    want_T, st_T = orc.recurrent(qn[:, :T], kn[:, :T], v.double()[:, :T], g.double()[:, :T], (l.double() / scale)[:, :T], b=b.double()[:, :T])
    assert hs.counts == list(st_T.counts)
    assert_close(hs.states, torch.stack(st_T.states, dim=-1), "level states after the prompt", atol=4e-3)
    for t in range(T, T + NDEC):
        ot, hs = chunk_h_gated_delta_rule(dq[:, t:t + 1], dk[:, t:t + 1], dv[:, t:t + 1], dg[:, t:t + 1], dl[:, t:t + 1],
                                          db[:, t:t + 1], initial_state=hs, output_final_state=True, use_qk_l2norm_in_kernel=True)
        assert_close(ot[:, 0], want[:, t], f"decode step {t}", atol=4e-3)
    torch.cuda.synchronize()
    assert hs.counts == list(st.counts)
    assert_close(hs.states, torch.stack(st.states, dim=-1), "level states after decoding", atol=4e-3)
