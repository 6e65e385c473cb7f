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
