"""Host drivers of the log-linear Mamba-2 chunkwise path, with the signatures of the
reference's `hattention/chunkwise.py` (`chunkwise_fwd` :1118-1129, `chunkwise_bwd` :1286-1299).

The work is done by libllattn.so; these functions validate arguments the way the reference
does, allocate outputs and scratch with torch, and launch on the current CUDA stream.
"""
from typing import Optional, Tuple

import torch

from . import _lib
from .base import HType, ceil_log, get_num_levels

CHUNK = 64


def _check(q, k, v, g, l, head_first, level_base, htype, chunk_size):
    if head_first:
        raise NotImplementedError("head_first=True is not supported")
    if level_base != 2:
        raise NotImplementedError("level_base must be 2")
    if htype != HType.WEAK:
        raise NotImplementedError("only HType.WEAK is supported")
    if chunk_size != CHUNK:
        raise NotImplementedError("chunk_size must be 64")
    if not (q.is_cuda and k.is_cuda and v.is_cuda and g.is_cuda and l.is_cuda):
        raise RuntimeError("log-linear attention kernels need CUDA tensors (there is no CPU path)")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        # the reference computes in the dtype it is given (hattention/kernel.py:127-135: fp32 inputs reach its
        # dots as fp32); these kernels take bf16 operands with fp32 accumulation only, and rounding other
        # dtypes silently would not be the same function
        raise NotImplementedError(f"q / k / v must be bfloat16 (got {q.dtype}, {k.dtype}, {v.dtype}): the kernels compute with "
                                  "bf16 operands and fp32 accumulation; the reference's fp32 mode is not implemented")
    B, T, G, K = k.shape
    _, _, H, V = v.shape
    L = l.shape[-1]
    if q.shape != k.shape or v.shape[:2] != (B, T) or g.shape != (B, T, H) or l.shape[:3] != (B, T, H):
        raise ValueError("inconsistent shapes")
    if H % G != 0:
        raise ValueError(f"H={H} is not a multiple of G={G}")
    if T % CHUNK != 0:
        raise ValueError(f"T={T} and BT={CHUNK}")
    for opt in (32, 64):
        if K % opt != 0:
            raise ValueError(f"K={K} and BK could be {opt}")
        if V % opt != 0:
            raise ValueError(f"V={V} and BV could be {opt}")
    if get_num_levels(CHUNK, 2) + ceil_log(T // CHUNK, 2) > L:
        raise ValueError("not enough lambda levels for this length")
    return B, T, H, G, K, V, L


def _as(x, dtype):
    return x.to(dtype).contiguous()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def chunkwise_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    l: torch.Tensor,
    head_first: bool,
    level_base: int,
    htype: HType,
    chunk_size: int,
    output_final_state: bool,
    keep_workspace: Optional[list] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Returns (o, in-chunk cumulative g, None) like the reference driver
    (chunkwise.py:1118-1275).  `keep_workspace` (not in the reference): a list that receives the
    call's scratch tensor, which `chunkwise_bwd(fwd_workspace=...)` can read the segment-level states
    from instead of recomputing them."""
    B, T, H, G, K, V, L = _check(q, k, v, g, l, head_first, level_base, htype, chunk_size)
    lib = _lib.lib()
    with torch.cuda.device(q.device):
        q_, k_, v_, l_ = (_as(x, torch.bfloat16) for x in (q, k, v, l))
        g_ = _as(g, torch.float32)
        o = torch.empty_like(v_)
        g_cum = torch.empty_like(g_)
        ws = _workspace(lib.llattn_mamba2_fwd_workspace_bytes(B, T, H, G, K, V, L), q.device)
        rc = lib.llattn_mamba2_fwd(q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), g_.data_ptr(), l_.data_ptr(),
                                   o.data_ptr(), g_cum.data_ptr(), ws.data_ptr(), ws.numel(),
                                   B, T, H, G, K, V, L, _stream())
        _lib.check(rc, "llattn_mamba2_fwd")
        if _lib.CHECK_STATUS:
            _lib.raise_on_status(ws, _stream(), "llattn_mamba2_fwd")
        if keep_workspace is not None:
            keep_workspace.append(ws)
        ht = final_states(k_, v_, g_, L) if output_final_state else None
    return o, g_cum, ht


def final_states(k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, L: int) -> torch.Tensor:
    """Level states (B,H,K,V,L) fp32 after the T tokens of k (B,T,G,K), v (B,T,H,V), g (B,T,H): what
    the reference's prefill assembles from `ht` of its state kernel and `postprocess_prefill_hstate_`
    (kernel.py:378-466, 521-557).  Every level is written (the reference's `ht` only carries the
    inter-chunk levels)."""
    lib = _lib.lib()
    B, T, G, K = k.shape
    H, V = v.shape[2], v.shape[3]
    with torch.cuda.device(k.device):
        k_, v_ = _as(k, torch.bfloat16), _as(v, torch.bfloat16)
        g_ = _as(g, torch.float32)
        st = torch.empty(B, H, K, V, L, dtype=torch.float32, device=k.device)
        rc = lib.llattn_mamba2_final_state(k_.data_ptr(), v_.data_ptr(), g_.data_ptr(), st.data_ptr(),
                                           B, T, H, G, K, V, L, _stream())
        _lib.check(rc, "llattn_mamba2_final_state")
    return st


def chunkwise_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    l: torch.Tensor,
    do: torch.Tensor,
    head_first: bool,
    level_base: int,
    htype: HType,
    chunk_size: int,
    fwd_workspace: Optional[torch.Tensor] = None,
):
    """`g` is the in-chunk cumulative sum returned by chunkwise_fwd (what the reference's
    autograd function saves, kernel.py:86,125).  Returns (dq, dk, dv, dg, dl) with dq, dk summed
    over the heads of each group and dg taken w.r.t. the raw g (chunkwise.py:1583-1597)."""
    B, T, H, G, K, V, L = _check(q, k, v, g, l, head_first, level_base, htype, chunk_size)
    lib = _lib.lib()
    with torch.cuda.device(q.device):
        q_, k_, v_, l_, do_ = (_as(x, torch.bfloat16) for x in (q, k, v, l, do))
        g_ = _as(g, torch.float32)
        dq = torch.empty_like(q_)
        dk = torch.empty_like(k_)
        dv = torch.empty_like(v_)
        dg = torch.empty_like(g_)
        dl = torch.empty(l_.shape, dtype=torch.float32, device=l_.device)
        ws = _workspace(lib.llattn_mamba2_bwd_workspace_bytes(B, T, H, G, K, V, L), q.device)
        fws = fwd_workspace if (fwd_workspace is not None and fwd_workspace.device == q.device) else None
        rc = lib.llattn_mamba2_bwd_saved(q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), g_.data_ptr(), l_.data_ptr(),
                                         do_.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(),
                                         dl.data_ptr(), ws.data_ptr(), ws.numel(),
                                         fws.data_ptr() if fws is not None else None, fws.numel() if fws is not None else 0,
                                         B, T, H, G, K, V, L, _stream())
        _lib.check(rc, "llattn_mamba2_bwd_saved")
        if _lib.CHECK_STATUS:
            _lib.raise_on_status(ws, _stream(), "llattn_mamba2_bwd_saved")
    return dq, dk, dv, dg, dl
