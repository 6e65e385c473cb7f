"""Test helpers for the Gated DeltaNet backward: a batched torch restatement of the chunk-local part of the
forward (differentiated by autograd), the CUDA level stage completed by it, and whole-path autograd
through the oracle's chunkwise form evaluated on the GPU.  Not product code."""
import torch

from hattention_b200 import _lib
from oracle import loglinear_oracle as orc

CHUNK = 64


def _levels_matrix(n: int, device) -> torch.Tensor:
    return torch.from_numpy(orc.levels_matrix(n)).clamp(min=0).to(device)


def gdn_prologue_torch(q, k, v, b, g, l):
    """Chunk-local part of the forward (everything before the scan over chunks) as batched fp32
    torch ops: returns qd, wd, kd, u, the intra-chunk output and the chunk totals of g, all
    (B,H,NT,C,*).  Differentiated by autograd in `chunkwise_bwd_staged`."""
    B, T, H, K = q.shape
    C = CHUNK
    NT = T // C
    dev = q.device
    f = lambda x: x.reshape(B, NT, C, H, -1).permute(0, 3, 1, 2, 4)
    qc, kc, vc, lc = f(q), f(k), f(v), f(l)
    bc = b.reshape(B, NT, C, H).permute(0, 3, 1, 2)
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
    lam = torch.gather(lc, 4, _levels_matrix(C, dev)[None, None, None].expand(B, H, NT, C, C))
    o = ((QK @ Aw) * Gam * bc[..., None, :] * lam) @ vc
    return qd, wd, kd, u, o, gl


def chunkwise_bwd_staged(q, k, v, b, g, l, Aw, Au, do):
    """Cross-check used by the test-suite: the CUDA level stage (`llattn_gdn_bwd_levels`) followed by
    autograd through the batched torch restatement of the chunk-local part."""
    B, T, H, K = q.shape
    V, L = v.shape[-1], l.shape[-1]
    lib = _lib.lib()
    NT = T // CHUNK
    with torch.cuda.device(q.device):
        q_, k_, v_, b_, l_, do_, Aw_, Au_ = (x.to(torch.bfloat16).contiguous() for x in (q, k, v, b, l, do, Aw, Au))
        gc_ = g.to(torch.float32).contiguous()
        d_qd = torch.empty(B, T, H, K, dtype=torch.float32, device=q.device)
        d_wd = torch.empty_like(d_qd)
        d_kd = torch.empty_like(d_qd)
        d_u = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=q.device)
        d_gl = torch.empty(B, NT, H, dtype=torch.float32, device=q.device)
        dl = torch.zeros(B, T, H, L, dtype=torch.float32, device=q.device)
        ws = torch.empty(lib.llattn_gdn_bwd_levels_workspace_bytes(B, T, H, K, V, L), dtype=torch.uint8, device=q.device)
        rc = lib.llattn_gdn_bwd_levels(q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), b_.data_ptr(), gc_.data_ptr(), l_.data_ptr(),
                                       Aw_.data_ptr(), Au_.data_ptr(), do_.data_ptr(), d_qd.data_ptr(), d_wd.data_ptr(),
                                       d_kd.data_ptr(), d_u.data_ptr(), d_gl.data_ptr(), dl.data_ptr(), ws.data_ptr(), ws.numel(),
                                       B, T, H, K, V, L, torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "llattn_gdn_bwd_levels")
        del ws
        graw = gc_.clone()
        gv = graw.view(B, NT, CHUNK, H)
        gv[:, :, 1:] = gv[:, :, 1:] - gc_.view(B, NT, CHUNK, H)[:, :, :-1]
        f = lambda x: x.reshape(B, NT, CHUNK, H, -1).permute(0, 3, 1, 2, 4).float()
        with torch.enable_grad():
            ins = [x.detach().float().requires_grad_(True) for x in (q_, k_, v_, b_, graw, l_)]
            outs = gdn_prologue_torch(*ins)
            grads = torch.autograd.grad(outs, ins, [f(d_qd), f(d_wd), f(d_kd), f(d_u), f(do_), d_gl.permute(0, 2, 1)])
        dq, dk, dv, db, dg, dl_low = grads
        return dq, dk, dv, db, dg, dl + dl_low


def chunkwise_bwd_autograd(q, k, v, b, g, l, do):
    """Whole-path autograd through the oracle's chunkwise form (fp32 on the GPU, a Python loop over chunks)."""
    B, T, H = g.shape
    graw = g.float().clone()
    gv = graw.view(B, T // CHUNK, CHUNK, H)
    gv[:, :, 1:] = gv[:, :, 1:] - g.float().view(B, T // CHUNK, CHUNK, H)[:, :, :-1]
    with torch.enable_grad():
        ins = [x.detach().float().requires_grad_(True) for x in (q, k, v, b, graw, l)]
        o = orc.gdn_chunkwise(*ins)
        grads = torch.autograd.grad(o, ins, do.float())
    return tuple(grads)


