"""Host drivers of the log-linear Gated DeltaNet chunkwise path, with the interface of the
reference's `hattention/chunkwise_hgdn.py` (`chunkwise_fwd` :566-578, `chunkwise_bwd` :799-817).

`chunkwise_fwd` takes q and k already L2-normalised (q also scaled), exactly like the reference
driver; `gdn_forward` / `gdn_backward` are what the autograd boundary calls and include the
l2norm / scale step that the reference's `HAttentionFunction` applies around the driver
(hattention/kernel.py:20-29, 100-120, 198-225).
"""
from typing import Optional, Tuple

import torch

from . import _lib
from .base import HType, ceil_log, get_num_levels

CHUNK = 64


def l2norm_fwd(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """bf16(bf16(x * rsqrt(sum(x^2) + 1e-6)) * scale) over the last dim (fla's l2norm_fwd followed by the
    reference's `* scale`, hattention/kernel.py:20-23), one CUDA pass."""
    if not x.is_cuda:
        raise RuntimeError("l2norm_fwd needs a CUDA tensor (there is no CPU path)")
    xb = x.to(torch.bfloat16).contiguous()
    y = torch.empty_like(xb)
    D = xb.shape[-1]
    with torch.cuda.device(x.device):
        rc = _lib.lib().llattn_l2norm_fwd(xb.data_ptr(), y.data_ptr(), xb.numel() // D, D, float(scale),
                                          torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "llattn_l2norm_fwd")
    return y


def l2norm_bwd(x: torch.Tensor, dy: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Gradient w.r.t. x of l2norm_fwd(x, scale) given dy (hattention/kernel.py:26-29), bf16."""
    if not x.is_cuda:
        raise RuntimeError("l2norm_bwd needs CUDA tensors (there is no CPU path)")
    xb = x.to(torch.bfloat16).contiguous()
    g = dy.to(torch.float32).contiguous()
    dx = torch.empty_like(xb)
    D = xb.shape[-1]
    with torch.cuda.device(x.device):
        rc = _lib.lib().llattn_l2norm_bwd(xb.data_ptr(), g.data_ptr(), dx.data_ptr(), xb.numel() // D, D, float(scale),
                                          torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "llattn_l2norm_bwd")
    return dx


def _check(q, k, v, b, g, l, head_first, level_base, htype, chunk_size):
    if head_first:
        raise NotImplementedError("head_first=True is not supported")
    if level_base != 2:
        raise NotImplementedError("level_base must be 2")
    if htype != HType.WEAK:
        raise NotImplementedError("only HType.WEAK is supported")
    if chunk_size != CHUNK:
        raise NotImplementedError("chunk_size must be 64")
    if not all(x.is_cuda for x in (q, k, v, b, g, l)):
        raise RuntimeError("log-linear attention kernels need CUDA tensors (there is no CPU path)")
    B, T, G, K = k.shape
    _, _, H, V = v.shape
    L = l.shape[-1]
    if q.shape != k.shape or b.shape != (B, T, H) or g.shape != (B, T, H) or l.shape[:3] != (B, T, H):
        raise ValueError("inconsistent shapes")
    if H % G != 0:
        raise ValueError(f"H={H} is not a multiple of G={G}")
    if K > 256:
        raise NotImplementedError("current kernel does not support head dimension larger than 256.")
    if T % CHUNK != 0:
        raise ValueError(f"T={T} and BT={CHUNK}")
    if get_num_levels(CHUNK, 2) + ceil_log(T // CHUNK, 2) > L:
        raise ValueError("not enough lambda levels for this length")
    return B, T, H, G, K, V, L


# Widest value head one kernel call takes.  The delta rule acts on every value column independently (the transition
# I - beta k k^T and the decay involve q, k, beta, g only), so a wider head (the reference's own model has Dv = 384,
# configs/flame/h_gated_deltanet_mid.json) is processed as slices of at most this many columns: outputs and dv are
# concatenated, the gradients of the shared inputs are summed.
V_SLICE = 128
V_MAX = 384


# Key width of the kernels.  Narrower q / k are padded with zero features: the products q k^T, k k^T, the transition and the
# level states' live rows are unchanged, the padded state rows stay zero, and the gradients of the padding are dropped.
K_CALL = 128


def _pad_k(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.pad(x, (0, K_CALL - x.shape[-1]))


def _v_slices(V: int):
    if V % 64 != 0 or V > V_MAX:
        raise ValueError(f"unsupported GDN shape (V must be a multiple of 64 up to {V_MAX}, got {V})")
    return [(s, min(s + V_SLICE, V)) for s in range(0, V, V_SLICE)]


def chunkwise_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: torch.Tensor,
    g: torch.Tensor,
    l: torch.Tensor,
    head_first: bool,
    level_base: int,
    htype: HType,
    chunk_size: int,
    output_final_state: bool,
    keep_workspace: Optional[list] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Returns (g_cum, o, Aw, Au, ht) like the reference driver (chunkwise_hgdn.py:566-788).
    With a list as `keep_workspace` the call's workspace (chunk matrices and every chunk's level states)
    is appended to it for `chunkwise_bwd(..., fwd_workspace=...)`, which then skips their recomputation.
    `output_final_state=True`: ht is (B,H,K,V,L) fp32 with the inter-chunk level states AS OF THE START OF THE LAST
    CHUNK (level 7 + j holds the block of 2^j chunks for each set bit j of NT - 1; levels 0..6 are zero); the prefill
    path steps the last chunk's tokens from there (the reference returns the states after the last chunk and
    rebuilds the levels inside it afterwards, kernel.py:378-466)."""
    B, T, H, G, K, V, L = _check(q, k, v, b, g, l, head_first, level_base, htype, chunk_size)
    if output_final_state and keep_workspace is not None:
        raise NotImplementedError("final states and a kept workspace in the same call")
    if V > V_SLICE:
        # slice by slice; nothing is kept for the backward (it recomputes, as the reference does)
        parts = [chunkwise_fwd(q, k, v[..., s:e], b, g, l, head_first, level_base, htype, chunk_size, output_final_state)
                 for s, e in _v_slices(V)]
        g_cum, _, Aw, Au, _ = parts[0]
        o = torch.cat([p_[1] for p_ in parts], dim=-1)
        ht = torch.cat([p_[4] for p_ in parts], dim=3) if output_final_state else None
        return g_cum, o, Aw, Au, ht
    if K < K_CALL:
        g_cum, o, Aw, Au, ht = chunkwise_fwd(_pad_k(q), _pad_k(k), v, b, g, l, head_first, level_base, htype, chunk_size,
                                             output_final_state, keep_workspace=keep_workspace)
        return g_cum, o, Aw, Au, (ht[:, :, :K].contiguous() if ht is not None else None)
    lib = _lib.lib()
    with torch.cuda.device(q.device):
        if G != H:   # one q/k per head, as the reference expands them (chunkwise_hgdn.py:613-620)
            q = q.repeat_interleave(H // G, dim=2)
            k = k.repeat_interleave(H // G, dim=2)
        q_, k_, v_, b_, l_ = (x.to(torch.bfloat16).contiguous() for x in (q, k, v, b, l))
        g_ = g.to(torch.float32).contiguous()
        o = torch.empty_like(v_)
        g_cum = torch.empty_like(g_)
        Aw = torch.empty(B, T, H, CHUNK, dtype=torch.bfloat16, device=q.device)
        Au = torch.empty_like(Aw)
        keep = keep_workspace is not None
        n = (lib.llattn_gdn_fwd_keep_workspace_bytes if keep else lib.llattn_gdn_fwd_workspace_bytes)(B, T, H, K, V, L)
        if n == 0:
            raise ValueError("unsupported GDN shape (K at most 128, V a multiple of 64, T <= 16384)")
        ws = torch.empty(n, dtype=torch.uint8, device=q.device)
        if keep:
            keep_workspace.append(ws)
        ht = None
        if output_final_state:
            ht = torch.empty(B, H, K, V, L, dtype=torch.float32, device=q.device)
            rc = lib.llattn_gdn_prefill(q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), b_.data_ptr(), g_.data_ptr(), l_.data_ptr(),
                                        o.data_ptr(), g_cum.data_ptr(), Aw.data_ptr(), Au.data_ptr(), ht.data_ptr(), ws.data_ptr(),
                                        ws.numel(), B, T, H, K, V, L, torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "llattn_gdn_prefill")
        else:
            rc = (lib.llattn_gdn_fwd_keep if keep else lib.llattn_gdn_fwd)(q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), b_.data_ptr(), g_.data_ptr(), l_.data_ptr(),
                                    o.data_ptr(), g_cum.data_ptr(), Aw.data_ptr(), Au.data_ptr(), ws.data_ptr(), ws.numel(),
                                    B, T, H, K, V, L, torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "llattn_gdn_fwd")
        if _lib.CHECK_STATUS:
            _lib.raise_on_status(ws, torch.cuda.current_stream().cuda_stream, "llattn_gdn_fwd")
    return g_cum, o, Aw, Au, ht


def chunkwise_bwd(q, k, v, b, g, l, Aw, Au, do, head_first, level_base, htype, chunk_size, fwd_workspace=None,
                  dv_bf16=False, **unused):
    """Gradients (dq, dk, dv, db, dg, dl), fp32, of the driver for normalised q, k (signature of
    chunkwise_hgdn.py:799-817; `g` is the in-chunk cumulative sum returned by chunkwise_fwd).  With `dv_bf16` and a kept
    forward workspace dv comes back in bf16 (what the autograd function hands on for bf16 v), written by the kernel itself.
    One C-ABI call: recomputation of the chunk matrices and level states (skipped when `fwd_workspace`
    is the workspace a `chunkwise_fwd(..., keep_workspace=[])` call on the same inputs left), reverse scan
    of the adjoint states, state-dependent gradients, chunk-local gradients."""
    B, T, H, G_, K, V, L = _check(q, k, v, b, g, l, head_first, level_base, htype, chunk_size)
    if G_ != H:
        raise NotImplementedError("GDN backward expects one q/k per head")
    if V > V_SLICE:
        if fwd_workspace is not None:
            raise ValueError("a kept forward workspace covers one value slice only")
        dq = dk = db = dg = dl = None
        dvs = []
        for s, e in _v_slices(V):
            pq, pk, pv, pb, pg, pl = chunkwise_bwd(q, k, v[..., s:e], b, g, l, Aw, Au, do[..., s:e], head_first, level_base,
                                                   htype, chunk_size)
            dvs.append(pv)
            if dq is None:
                dq, dk, db, dg, dl = pq, pk, pb, pg, pl
            else:
                dq += pq; dk += pk; db += pb; dg += pg; dl += pl
        return dq, dk, torch.cat(dvs, dim=-1), db, dg, dl
    if K < K_CALL:
        dq, dk, dv, db, dg, dl = chunkwise_bwd(_pad_k(q), _pad_k(k), v, b, g, l, Aw, Au, do, head_first, level_base, htype,
                                               chunk_size, fwd_workspace=fwd_workspace, dv_bf16=dv_bf16)
        return dq[..., :K].contiguous(), dk[..., :K].contiguous(), dv, db, dg, dl
    lib = _lib.lib()
    with torch.cuda.device(q.device):
        q_, k_, v_, b_, l_, do_, Aw_, Au_ = (x.to(torch.bfloat16).contiguous() for x in (q, k, v, b, l, do, Aw, Au))
        gc_ = g.to(torch.float32).contiguous()
        f32 = dict(dtype=torch.float32, device=q.device)
        dq, dk = torch.empty(B, T, H, K, **f32), torch.empty(B, T, H, K, **f32)
        kept = fwd_workspace is not None
        dv = torch.empty(B, T, H, V, dtype=torch.bfloat16 if (dv_bf16 and kept) else torch.float32, device=q.device)
        db, dg = torch.empty(B, T, H, **f32), torch.empty(B, T, H, **f32)
        dl = torch.empty(B, T, H, L, **f32)
        n = (lib.llattn_gdn_bwd_kept_workspace_bytes if kept else lib.llattn_gdn_bwd_workspace_bytes)(B, T, H, K, V, L)
        if n == 0:
            raise ValueError("unsupported GDN shape (K at most 128, V a multiple of 64, T <= 16384)")
        ws = torch.empty(n, dtype=torch.uint8, device=q.device)
        head = (q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), b_.data_ptr(), gc_.data_ptr(), l_.data_ptr(),
                Aw_.data_ptr(), Au_.data_ptr(), do_.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                db.data_ptr(), dg.data_ptr(), dl.data_ptr())
        tail = (ws.data_ptr(), ws.numel(), B, T, H, K, V, L, torch.cuda.current_stream().cuda_stream)
        if kept:
            fn = lib.llattn_gdn_bwd_kept_bf16dv if dv.dtype == torch.bfloat16 else lib.llattn_gdn_bwd_kept
            rc = fn(*head, fwd_workspace.data_ptr(), fwd_workspace.numel(), *tail)
        else:
            rc = lib.llattn_gdn_bwd(*head, *tail)
        _lib.check(rc, "llattn_gdn_bwd_kept" if kept else "llattn_gdn_bwd")
        if _lib.CHECK_STATUS:
            _lib.raise_on_status(ws, torch.cuda.current_stream().cuda_stream, "llattn_gdn_bwd")
    return dq, dk, dv, db, dg, dl


# Largest forward workspace (chunk matrices + level states, bytes) that gdn_forward keeps for the backward
# when asked to; above it the backward recomputes, which is the reference's memory behaviour.
KEEP_WORKSPACE_MAX_BYTES = 8 << 30


def gdn_forward(q, k, v, b, g, l, scale, head_first, level_base, htype, chunk_size, keep: Optional[list] = None):
    """l2norm(q) * scale, l2norm(k), then the driver (hattention/kernel.py:109-120).  With a list as
    `keep`, the normalised q, k and the driver's workspace are appended to it for gdn_backward."""
    qn = l2norm_fwd(q, scale)
    kn = l2norm_fwd(k)
    kept = None
    if keep is not None and q.shape[2] == v.shape[2]:
        B, T, H = v.shape[:3]
        n = _lib.lib().llattn_gdn_fwd_keep_workspace_bytes(B, T, H, q.shape[-1], v.shape[-1], l.shape[-1])
        if 0 < n <= KEEP_WORKSPACE_MAX_BYTES:
            kept = []
    g_cum, o, Aw, Au, _ = chunkwise_fwd(qn, kn, v, b, g, l, head_first, level_base, htype, chunk_size, False,
                                        keep_workspace=kept)
    if kept:
        keep.extend([qn, kn, kept[0]])
    return g_cum, o, Aw, Au


def gdn_backward(q, k, v, b, g_cum, l, Aw, Au, do, scale, head_first, level_base, htype, chunk_size, kept=None):
    """Backward of gdn_forward w.r.t. the raw q, k (through l2norm / scale), v, b, g, l
    (hattention/kernel.py:198-225).  `kept` is the list gdn_forward filled, or None / empty."""
    if kept:
        qn, kn, fwd_ws = kept
    else:
        qn = l2norm_fwd(q, scale)
        kn = l2norm_fwd(k)
        fwd_ws = None
    H = v.shape[2]
    G = k.shape[2]
    if G != H:
        raise NotImplementedError("GDN backward expects one q/k per head")
    dq, dk, dv, db, dg, dl = chunkwise_bwd(qn, kn, v, b, g_cum, l, Aw, Au, do, head_first, level_base, htype, chunk_size,
                                           fwd_workspace=fwd_ws, dv_bf16=(v.dtype == torch.bfloat16))
    dq = l2norm_bwd(q, dq, scale)
    dk = l2norm_bwd(k, dk)
    return dq, dk, dv, db, dg, dl
