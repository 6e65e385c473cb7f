"""CPU oracle for chunkwise log-linear attention (TEST INFRASTRUCTURE, not product code).

This module restates, in plain PyTorch on the CPU, the algorithms that the reference
project hattention uses to define log-linear attention.  It exists only so that the
CUDA kernels can be checked against it: nothing in the shipped package imports it, and
only the test-suite, the smoke check and the benchmark's CPU-baseline leg may call it.

Parity status: PINNED.  Every function here is compared (tests/test_oracle_golden.py)
against fixtures under tests/golden/ that were produced by importing the reference's own
PyTorch implementations (hattention/base.py, recurrent.py, hssd_minimal.py) and running
them on seeded inputs; tests/golden/make_golden.py is the generating script.

Notation (reference names):
    q, k : (B, T, G, K)   queries / keys, G groups shared by H // G heads each
    v    : (B, T, H, V)
    g    : (B, T, H)      per-token log decay (<= 0)
    l    : (B, T, H, L)   per-token, per-level weights (lambda)
    b    : (B, T, H)      delta-rule write strength beta (GDN only)
All functions are differentiable with torch.autograd unless stated otherwise.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# level arithmetic   (reference: hattention/base.py:29-46, 101-161)
# --------------------------------------------------------------------------------------
def ceil_log2(x: int) -> int:
    """ceil(log2(x)) for x >= 1, exact integer arithmetic (base.py:29-30 uses math.log)."""
    return (x - 1).bit_length()


def get_num_levels(length: int) -> int:
    """Number of Fenwick levels needed for `length` tokens (base.py:37-38, base 2)."""
    return ceil_log2(length) + 1


def level_index_recursive(t: int, s: int) -> int:
    """The reference's recursive definition of the bucket of source s for target t>s
    (base.py:41-46, `get_level_index_weak` with b=2)."""
    lg = t.bit_length() - 1
    top = 1 << lg
    if s < top:
        return lg + 1
    return level_index_recursive(t - top, s - top)


def level_index(t: int, s: int) -> int:
    """Closed form of the same bucket: bit_length(t XOR s); 0 on the diagonal."""
    return (t ^ s).bit_length()


def levels_matrix(length: int) -> np.ndarray:
    """(length, length) int64 table, levels[t, s] = bit_length(t ^ s) for s <= t and -1
    above the diagonal (base.py:101-161 with default=-1, clamp_min=None)."""
    idx = np.arange(length, dtype=np.int64)
    x = idx[:, None] ^ idx[None, :]
    lev = np.zeros_like(x)
    nz = x > 0
    lev[nz] = np.floor(np.log2(x[nz])).astype(np.int64) + 1
    lev[idx[:, None] < idx[None, :]] = -1
    return lev


def _expand_groups(x: torch.Tensor, H: int) -> torch.Tensor:
    """(B,T,G,K) -> (B,T,H,K); head h uses group h // (H // G) (chunkwise.py:1167-1172)."""
    G = x.shape[2]
    if G == H:
        return x
    return x.repeat_interleave(H // G, dim=2)


# --------------------------------------------------------------------------------------
# Mamba-2 structure (scalar decay)
# --------------------------------------------------------------------------------------
def mamba2_materialized(q, k, v, g, l) -> torch.Tensor:
    """O(T^2) definition: o_t = sum_{s<=t} l[t, level(t,s)] exp(sum_{r=s+1..t} g_r) (q_t.k_s) v_s.

    Follows `make_masked_H_matrix` + `hattention_materialized` (base.py:75-98, 334-349),
    with the product of decays written as exp of a cumulative-sum difference.
    """
    B, T, H, V = v.shape
    qh, kh = _expand_groups(q, H), _expand_groups(k, H)
    lev = torch.from_numpy(levels_matrix(T))                      # (T,T)
    tril = lev >= 0
    gc = torch.cumsum(g, dim=1)                                    # (B,T,H)
    diff = gc[:, :, None, :] - gc[:, None, :, :]                   # (B,t,s,H)
    diff = diff.masked_fill(~tril[None, :, :, None], float("-inf"))
    decay = torch.exp(diff)
    lam = torch.gather(
        l.permute(0, 2, 1, 3),                                     # (B,H,T,L)
        3, lev.clamp(min=0)[None, None].expand(B, H, T, T))        # (B,H,t,s)
    qk = torch.einsum("bthk,bshk->bhts", qh, kh)
    P = qk * lam * decay.permute(0, 3, 1, 2)
    return torch.einsum("bhts,bshv->bthv", P, v)


def mamba2_chunkwise(q, k, v, g, l, chunk: int = 64) -> torch.Tensor:
    """Chunkwise form, one sequential scan per inter-chunk level, as the reference's
    Triton driver organises it (chunkwise.py:1184-1273; kernels :110-280 and :488-647):

      intra : P[i,j] = (q_i.k_j) exp(G_i-G_j) l[t, bit_length(i^j)], j<=i ; o_c = P v_c
      level : for chunk c in order: readers (bit l of c set) add l[t,lh] exp(G_i) q_i.H ;
              H is zeroed after chunks with c % 2^(l+1) == 2^(l+1)-1, else decayed by
              exp(G_last) ; contributors (bit l clear) add k^T (v exp(G_last-G)).
    G is the inclusive cumulative sum of g inside each chunk (chunkwise.py:1175).
    """
    B, T, H, V = v.shape
    K = q.shape[-1]
    L = l.shape[-1]
    C = chunk
    assert T % C == 0
    NT = T // C
    qh = _expand_groups(q, H).reshape(B, NT, C, H, K)
    kh = _expand_groups(k, H).reshape(B, NT, C, H, K)
    vc = v.reshape(B, NT, C, H, V)
    lc = l.reshape(B, NT, C, H, L)
    Gc = torch.cumsum(g.reshape(B, NT, C, H), dim=2)
    lev = torch.from_numpy(levels_matrix(C))
    tril = lev >= 0
    diff = (Gc[:, :, :, None, :] - Gc[:, :, None, :, :]).masked_fill(~tril[None, None, :, :, None], float("-inf"))
    lam = torch.gather(lc.permute(0, 1, 3, 2, 4), 4,
                       lev.clamp(min=0)[None, None, None].expand(B, NT, H, C, C))   # (B,NT,H,i,j)
    P = torch.einsum("bcihk,bcjhk->bchij", qh, kh) * lam * torch.exp(diff).permute(0, 1, 4, 2, 3)
    o = torch.einsum("bchij,bcjhv->bcihv", P, vc)

    ell_h0 = get_num_levels(C)                 # first inter-chunk lambda column (chunkwise.py:1211)
    Lc = ceil_log2(NT) if NT > 1 else 0        # number of inter-chunk levels (chunkwise.py:1212)
    if ell_h0 + Lc > L:
        raise ValueError("not enough lambda levels")
    glast = Gc[:, :, -1, :]                    # (B,NT,H)
    kv = torch.einsum("bcjhk,bcjh,bcjhv->bchkv", kh, torch.exp(glast[:, :, None, :] - Gc), vc)
    outs = [o[:, c] for c in range(NT)]
    for ell in range(Lc):
        period = 1 << (ell + 1)
        Hs = torch.zeros(B, H, K, V, dtype=v.dtype)
        for c in range(NT):
            if (c >> ell) & 1:
                w = lc[:, c, :, :, ell_h0 + ell] * torch.exp(Gc[:, c])            # (B,C,H)
                outs[c] = outs[c] + torch.einsum("bihk,bhkv,bih->bihv", qh[:, c], Hs, w)
            if c % period == period - 1:
                Hs = torch.zeros_like(Hs)
            else:
                Hs = Hs * torch.exp(glast[:, c])[:, :, None, None]
            if not (c >> ell) & 1:
                Hs = Hs + kv[:, c]
    return torch.stack(outs, dim=1).reshape(B, T, H, V)


def mamba2_chunkwise_blocked(q, k, v, g, l, chunk: int = 64) -> torch.Tensor:
    """The same chunkwise function as `mamba2_chunkwise`, with every inter-chunk level evaluated
    for all chunks at once instead of by a scan over chunks, so that sequences of 16K-64K tokens
    finish in seconds.  It uses the closed form of the state a reader chunk sees
    (chunkwise.py:110-280: contributor chunks are the first half of the block of 2^(l+1) chunks
    that contains the reader, decayed by the chunk totals in between):

        H_l[c] = sum_{c' in [b, b + 2^l)} exp(GL[c-1] - GL[c']) KV_c',   b = (c >> (l+1)) << (l+1)

    with GL the running sum of the chunk totals of g.  Checked against `mamba2_chunkwise` and the
    reference-generated fixtures in tests/test_oracle_golden.py."""
    B, T, H, V = v.shape
    K = q.shape[-1]
    L = l.shape[-1]
    C = chunk
    assert T % C == 0
    NT = T // C
    qh = _expand_groups(q, H).reshape(B, NT, C, H, K)
    kh = _expand_groups(k, H).reshape(B, NT, C, H, K)
    vc = v.reshape(B, NT, C, H, V)
    lc = l.reshape(B, NT, C, H, L)
    Gc = torch.cumsum(g.reshape(B, NT, C, H), dim=2)
    lev = torch.from_numpy(levels_matrix(C))
    tril = lev >= 0
    diff = (Gc[:, :, :, None, :] - Gc[:, :, None, :, :]).masked_fill(~tril[None, None, :, :, None], float("-inf"))
    lam = torch.gather(lc.permute(0, 1, 3, 2, 4), 4,
                       lev.clamp(min=0)[None, None, None].expand(B, NT, H, C, C))
    P = torch.einsum("bcihk,bcjhk->bchij", qh, kh) * lam * torch.exp(diff).permute(0, 1, 4, 2, 3)
    o = torch.einsum("bchij,bcjhv->bcihv", P, vc)

    ell_h0 = get_num_levels(C)
    Lc = ceil_log2(NT) if NT > 1 else 0
    if ell_h0 + Lc > L:
        raise ValueError("not enough lambda levels")
    glast = Gc[:, :, -1, :]                                         # (B,NT,H)
    kv = torch.einsum("bcjhk,bcjh,bcjhv->bchkv", kh, torch.exp(glast[:, :, None, :] - Gc), vc)
    qs = qh * torch.exp(Gc)[..., None]                              # q_i exp(G_i)
    for ell in range(Lc):
        half = 1 << ell
        period = 2 * half
        nblk = -(-NT // period)
        pad = nblk * period - NT

        def blocks(x):
            if pad:
                x = torch.cat([x, x.new_zeros((B, pad) + tuple(x.shape[2:]))], dim=1)
            return x.reshape((B, nblk, period) + tuple(x.shape[2:]))

        GL = torch.cumsum(blocks(glast), dim=2)                     # running chunk totals inside each block
        mid = GL[:, :, half - 1:half]                               # total up to the last contributor
        F = torch.einsum("bjch,bjchkv->bjhkv", torch.exp(mid - GL[:, :, :half]), blocks(kv)[:, :, :half])
        dec = torch.exp(GL[:, :, half - 1:period - 1] - mid)        # reader m sees exp(GL[c-1] - GL[mid-1])
        w = blocks(lc[..., ell_h0 + ell])[:, :, half:] * dec[:, :, :, None, :]          # (B,nblk,half,C,H)
        add = torch.einsum("bjmihk,bjhkv,bjmih->bjmihv", blocks(qs)[:, :, half:], F, w)
        add = torch.cat([add.new_zeros(add.shape), add], dim=2).reshape(B, nblk * period, C, H, V)
        o = o + add[:, :NT]
    return o.reshape(B, T, H, V)


class FenwickState:
    """Out-of-place restatement of `HState` (recurrent.py:9-131): one (B,H,K,V) state and
    one token count per level; `cascade` merges level i into i+1 when it is full."""

    def __init__(self, B, H, K, V, L, dtype):
        self.states: List[torch.Tensor] = [torch.zeros(B, H, K, V, dtype=dtype) for _ in range(L)]
        self.counts = [0] * L

    def cascade(self):                         # recurrent.py:42-54
        for lev in range(len(self.states)):
            cap = 1 << lev
            if self.counts[lev] == cap:
                self.states[lev + 1] = self.states[lev + 1] + self.states[lev]
                self.counts[lev + 1] += self.counts[lev]
                self.states[lev] = torch.zeros_like(self.states[lev])
                self.counts[lev] = 0
            elif self.counts[lev] < cap:
                break
            else:
                raise ValueError("level over capacity")


def recurrent(q, k, v, g, l, b: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, FenwickState]:
    """Token-by-token O(log T)-state recurrence (recurrent.py:134-216).

    Per token: cascade; every level state is transformed by the gate (scalar exp(g) for
    Mamba-2, exp(g) (I - beta k k^T) applied from the left for GDN, recurrent.py:140-154);
    level 0 is set to k v^T (beta k v^T for GDN); output is q . sum_l l[t,l] S_l.
    """
    B, T, H, V = v.shape
    K = q.shape[-1]
    L = l.shape[-1]
    qh, kh = _expand_groups(q, H), _expand_groups(k, H)
    st = FenwickState(B, H, K, V, L, v.dtype)
    a = torch.exp(g)
    ys = []
    for t in range(T):
        st.cascade()
        kt, vt, at = kh[:, t], v[:, t], a[:, t]
        if b is None:
            st.states = [at[:, :, None, None] * s for s in st.states]
            value = torch.einsum("bhk,bhv->bhkv", kt, vt)
        else:
            bt = b[:, t]
            new = []
            for s in st.states:
                ks = torch.einsum("bhk,bhkv->bhv", kt, s)
                new.append(at[:, :, None, None] * (s - torch.einsum("bh,bhk,bhv->bhkv", bt, kt, ks)))
            st.states = new
            value = torch.einsum("bh,bhk,bhv->bhkv", bt, kt, vt)
        st.states[0] = value
        st.counts[0] += 1
        S = sum(l[:, t, :, i][:, :, None, None] * st.states[i] for i in range(L))
        ys.append(torch.einsum("bhk,bhkv->bhv", qh[:, t], S))
    return torch.stack(ys, dim=1), st


# --------------------------------------------------------------------------------------
# Gated DeltaNet structure (matrix-valued transition)
# --------------------------------------------------------------------------------------
def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Row L2 normalisation over the last dim as fla's l2norm_fwd computes it
    (x * rsqrt(sum(x^2) + eps); call sites hattention/kernel.py:20-29, 110-111)."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_materialized(q, k, v, b, g, l) -> torch.Tensor:
    """O(T^2) definition for the delta-rule structure (what `make_masked_H_tensor_dplr` +
    `hattention_materialized_dplr` state, base.py:258-331, 368-381): the write of source s,
    beta_s k_s v_s^T, is carried forward through every later transition
    exp(g_r) (I - beta_r k_r k_r^T), and target t reads it with weight l[t, level(t, s)].
    Cost O(T^2 K V); only meant for very small T.  q and k are used as given (the caller
    applies the l2norm / scale preparation)."""
    B, T, H, V = v.shape
    K = q.shape[-1]
    lev = levels_matrix(T)
    a = torch.exp(g)
    outs = []
    # S[s] : contribution of write s, propagated through later transitions
    contrib: List[torch.Tensor] = []
    for t in range(T):
        kt, bt, at = k[:, t], b[:, t], a[:, t]
        new = []
        for s_ in contrib:
            ks = torch.einsum("bhk,bhkv->bhv", kt, s_)
            new.append(at[:, :, None, None] * (s_ - torch.einsum("bh,bhk,bhv->bhkv", bt, kt, ks)))
        contrib = new
        contrib.append(torch.einsum("bh,bhk,bhv->bhkv", bt, kt, v[:, t]))
        S = sum(l[:, t, :, int(lev[t, s])][:, :, None, None] * contrib[s] for s in range(t + 1))
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
    return torch.stack(outs, dim=1)


def gdn_chunkwise(q, k, v, b, g, l, chunk: int = 64) -> torch.Tensor:
    """Chunkwise form of the delta-rule structure for normalised q, k (one per head), as the
    reference's driver organises it (chunkwise_hgdn.py:566-788 with the chunk matrices of
    fla_future/chunk_scaled_dot_kkt.py, solve_tril.py, wy_fast.py, chunk_delta_h.py):

      per chunk  Gam[i,j] = exp(G_i - G_j) [j <= i] ; A = strict_tril(beta_i k_i.k_j)
                 Aw = (I + A)^-1 ; Au = (I + A * Gam)^-1 ; w = Aw (beta k) ; u = Au (beta v)
                 kd = k exp(G_last - G) ; wd = w exp(G) ; qd = exp(G) (q - tril(q k^T) w)
      intra      o = ((tril(q k^T) Aw) * Gam * beta_j * l[t, bit_length(i^j)]) v
      level      readers (bit l of c set) add l[t,lh] qd.S ; then, unless c ends a period of the level
                 (state zeroed), S <- exp(G_last) S + kd^T ((bit clear ? u : 0) - wd S).

    All levels advance together through one loop over chunks.  Differentiable; evaluates in the
    dtype of its inputs on their device (fp64 on the CPU as the checker of the CUDA kernels).
    Checked against the reference-generated fixture and the token recurrence in
    tests/test_oracle_golden.py."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    L = l.shape[-1]
    C = chunk
    NT = T // C
    dev = q.device
    f = lambda x: x.reshape(B, NT, C, H, -1).permute(0, 3, 1, 2, 4)        # (B,H,NT,C,*)
    qc, kc, vc, lc = f(q), f(k), f(v), f(l)
    bc = b.reshape(B, NT, C, H).permute(0, 3, 1, 2)                         # (B,H,NT,C)
    G = torch.cumsum(g.reshape(B, NT, C, H).permute(0, 3, 1, 2), dim=-1)
    gl = G[..., -1]
    tril = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
    stril = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev), -1)
    Gam = torch.exp((G[..., :, None] - G[..., None, :]).masked_fill(~tril, float("-inf")))
    A = (bc[..., :, None] * (kc @ kc.transpose(-1, -2))).masked_fill(~stril, 0.0)
    eye = torch.eye(C, device=dev, dtype=q.dtype).expand(B, H, NT, C, C)
    Aw = torch.linalg.solve_triangular(eye + A, eye, upper=False)
    Au = torch.linalg.solve_triangular(eye + A * Gam, eye, upper=False)
    w = Aw @ (bc[..., None] * kc)
    u = Au @ (bc[..., None] * vc)
    kd = kc * torch.exp(gl[..., None] - G)[..., None]
    wd = w * torch.exp(G)[..., None]
    QK = (qc @ kc.transpose(-1, -2)).masked_fill(~tril, 0.0)
    qd = torch.exp(G)[..., None] * (qc - QK @ w)
    lev = torch.from_numpy(levels_matrix(C)).clamp(min=0).to(dev)
    lam = torch.gather(lc, 4, lev[None, None, None].expand(B, H, NT, C, C))
    o = ((QK @ Aw) * Gam * bc[..., None, :] * lam) @ vc                      # (B,H,NT,C,V)
    ell_h0 = get_num_levels(C)
    Lc = ceil_log2(NT) if NT > 1 else 0
    if ell_h0 + Lc > L:
        raise ValueError("not enough lambda levels")
    outs = [o[:, :, c] for c in range(NT)]
    if Lc > 0:
        lv = torch.arange(Lc, device=dev)
        S = torch.zeros(B, H, Lc, K, V, device=dev, dtype=q.dtype)
        for c in range(NT):
            bit = ((c >> lv) & 1).to(q.dtype)                                # (Lc,)
            reset = (((c + 1) % (2 << lv)) == 0).to(q.dtype)
            lam_c = lc[:, :, c, :, ell_h0:ell_h0 + Lc] * bit                  # (B,H,C,Lc)
            R = qd[:, :, c, None] @ S                                        # (B,H,Lc,C,V)
            outs[c] = outs[c] + (lam_c.permute(0, 1, 3, 2)[..., None] * R).sum(2)
            if c + 1 < NT:
                Z = wd[:, :, c, None] @ S
                Vh = u[:, :, c, None] * (1 - bit)[None, None, :, None, None] - Z
                S = (torch.exp(gl[:, :, c])[..., None, None, None] * S + kd[:, :, c, None].transpose(-1, -2) @ Vh) \
                    * (1 - reset)[None, None, :, None, None]
    o = torch.stack(outs, dim=2)                                             # (B,H,NT,C,V)
    return o.permute(0, 2, 3, 1, 4).reshape(B, T, H, V)


def gdn_chunkwise_grads(q, k, v, b, g, l, do, scale: float):
    """Gradients of sum(o * do) w.r.t. the RAW (q, k, v, b, g, l) of the GDN op through the
    l2norm / scale preparation and `gdn_chunkwise`, in float64 (l is the lambda the kernels see,
    i.e. already divided by scale)."""
    ins = [x.detach().double().requires_grad_(True) for x in (q, k, v, b, g, l)]
    qn, kn = gdn_layer_inputs(ins[0], ins[1], scale)
    o = gdn_chunkwise(qn, kn, ins[2], ins[3], ins[4], ins[5])
    grads = torch.autograd.grad((o * do.double()).sum(), ins)
    return o.detach(), grads


def gdn_layer_inputs(q, k, scale: float):
    """What the reference feeds its GDN kernels: q <- l2norm(q) * scale, k <- l2norm(k)
    (kernel.py:110-111)."""
    return l2norm(q) * scale, l2norm(k)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs with the value distributions of the benchmark configurations
# --------------------------------------------------------------------------------------
def make_mamba2_inputs(B, T, H, P, N, G, L, seed=0, dtype=torch.float32, a_lo=1.0, a_hi=16.0):
    """X~N(0,1); B,C~N(0,1)/sqrt(N); dt=softplus(N(0,1)-2); A=-exp(U(ln a_lo, ln a_hi)) per
    head; lambda=softplus(N(0,1)).  Returns kernel-level tensors (q=C, k=B, v=X*dt, g=A*dt, l)
    following hmamba_chunk_scan_combined's preparation (mamba_apis.py:352-372)."""
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(B, T, H, P, generator=gen)
    Bm = torch.randn(B, T, G, N, generator=gen) / math.sqrt(N)
    Cm = torch.randn(B, T, G, N, generator=gen) / math.sqrt(N)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen) - 2.0)
    A = -torch.exp(torch.rand(H, generator=gen) * (math.log(a_hi) - math.log(a_lo)) + math.log(a_lo))
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen))
    q, k = Cm.to(dtype), Bm.to(dtype)
    v = (X * dt[..., None]).to(dtype)
    g = (A[None, None, :] * dt).float()
    return q, k, v, g, lam.to(dtype)


def make_gdn_inputs(B, T, H, Dk, Dv, L, seed=0, dtype=torch.float32):
    """q,k~N(0,1) (L2-normalised by the op itself); v~N(0,1); beta=sigmoid(N(0,1));
    g=logsigmoid(N(0,1)+3); lambda=softplus(N(0,1))."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, Dk, generator=gen)
    k = torch.randn(B, T, H, Dk, generator=gen)
    v = torch.randn(B, T, H, Dv, generator=gen)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen) + 3.0)
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen))
    return q.to(dtype), k.to(dtype), v.to(dtype), beta.to(dtype), g.float(), lam.to(dtype)


def mamba2_grads(q, k, v, g, l, do, fn=mamba2_materialized):
    """Gradients of sum(o * do) w.r.t. (q, k, v, g, l) by autograd through `fn` in float64."""
    ins = [x.detach().double().requires_grad_(True) for x in (q, k, v, g, l)]
    o = fn(*ins)
    grads = torch.autograd.grad((o * do.double()).sum(), ins)
    return o.detach(), grads


def gdn_grads(q, k, v, b, g, l, do, scale: float):
    """Gradients of sum(o * do) w.r.t. the RAW (q, k, v, b, g, l) of the GDN op, through the
    l2norm/scale preparation and the recurrence, in float64."""
    ins = [x.detach().double().requires_grad_(True) for x in (q, k, v, b, g, l)]
    qn, kn = gdn_layer_inputs(ins[0], ins[1], scale)
    o, _ = recurrent(qn, kn, ins[2], ins[4], ins[5], b=ins[3])
    grads = torch.autograd.grad((o * do.double()).sum(), ins)
    return o.detach(), grads
