"""The kernels as `torch.library` operators (namespace `llattn`), for callers that want dispatcher-visible
ops: fake-tensor shape propagation (`torch.compile` tracing, `torch.export`), `torch.library.opcheck`.
Each operator calls the same C-ABI entry point as the Python drivers of this package; the drivers remain
the interface that mirrors the reference (`hattention/chunkwise.py`, `hattention/chunkwise_hgdn.py`,
`hattention/kernel.py:20-29`).

    llattn::mamba2_fwd(q, k, v, g, l)                        -> (o, g_cum, workspace)
    llattn::mamba2_bwd(q, k, v, g_cum, l, do, workspace)     -> (dq, dk, dv, dg, dl)
    llattn::gdn_fwd(q, k, v, beta, g, l)                     -> (g_cum, o, Aw, Au)
    llattn::gdn_bwd(q, k, v, beta, g_cum, l, Aw, Au, do)     -> (dq, dk, dv, dbeta, dg, dl)
    llattn::l2norm_scale_fwd(x, scale)                       -> y
    llattn::l2norm_scale_bwd(x, dy, scale)                   -> dx

`workspace` of mamba2_fwd is the call's scratch (uint8); handing it to mamba2_bwd lets the backward read the
segment-level states instead of recomputing them (pass an empty tensor to recompute).
"""
from typing import Tuple

import torch

from . import _lib
from .base import HType

_T = torch.Tensor


@torch.library.custom_op("llattn::mamba2_fwd", mutates_args=())
def mamba2_fwd(q: _T, k: _T, v: _T, g: _T, l: _T) -> Tuple[_T, _T, _T]:
    from .chunkwise import chunkwise_fwd
    kept = []
    o, g_cum, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
    return o, g_cum, kept[0]


@mamba2_fwd.register_fake
def _(q, k, v, g, l):
    B, T, G, K = k.shape
    H, V = v.shape[2], v.shape[3]
    n = _lib.lib().llattn_mamba2_fwd_workspace_bytes(B, T, H, G, K, V, l.shape[-1])
    return (torch.empty_like(v, dtype=torch.bfloat16), torch.empty_like(g, dtype=torch.float32),
            v.new_empty((max(int(n), 256),), dtype=torch.uint8))


@torch.library.custom_op("llattn::mamba2_bwd", mutates_args=())
def mamba2_bwd(q: _T, k: _T, v: _T, g_cum: _T, l: _T, do: _T, workspace: _T) -> Tuple[_T, _T, _T, _T, _T]:
    from .chunkwise import chunkwise_bwd
    return chunkwise_bwd(q, k, v, g_cum, l, do, False, 2, HType.WEAK, 64,
                         fwd_workspace=workspace if workspace.numel() > 0 else None)


@mamba2_bwd.register_fake
def _(q, k, v, g_cum, l, do, workspace):
    return (torch.empty_like(q, dtype=torch.bfloat16), torch.empty_like(k, dtype=torch.bfloat16),
            torch.empty_like(v, dtype=torch.bfloat16), torch.empty_like(g_cum, dtype=torch.float32),
            torch.empty_like(l, dtype=torch.float32))


@torch.library.custom_op("llattn::gdn_fwd", mutates_args=())
def gdn_fwd(q: _T, k: _T, v: _T, beta: _T, g: _T, l: _T) -> Tuple[_T, _T, _T, _T]:
    from .chunkwise_hgdn import chunkwise_fwd
    g_cum, o, Aw, Au, _ = chunkwise_fwd(q, k, v, beta, g, l, False, 2, HType.WEAK, 64, False)
    return g_cum, o, Aw, Au


@gdn_fwd.register_fake
def _(q, k, v, beta, g, l):
    B, T, H, _ = v.shape
    a = v.new_empty((B, T, H, 64), dtype=torch.bfloat16)
    return torch.empty_like(g, dtype=torch.float32), torch.empty_like(v, dtype=torch.bfloat16), a, torch.empty_like(a)


@torch.library.custom_op("llattn::gdn_bwd", mutates_args=())
def gdn_bwd(q: _T, k: _T, v: _T, beta: _T, g_cum: _T, l: _T, Aw: _T, Au: _T, do: _T) -> Tuple[_T, _T, _T, _T, _T, _T]:
    from .chunkwise_hgdn import chunkwise_bwd
    return chunkwise_bwd(q, k, v, beta, g_cum, l, Aw, Au, do, False, 2, HType.WEAK, 64)


@gdn_bwd.register_fake
def _(q, k, v, beta, g_cum, l, Aw, Au, do):
    f = torch.float32
    return (torch.empty_like(q, dtype=f), torch.empty_like(k, dtype=f), torch.empty_like(v, dtype=f),
            torch.empty_like(beta, dtype=f), torch.empty_like(g_cum, dtype=f), torch.empty_like(l, dtype=f))


@torch.library.custom_op("llattn::l2norm_scale_fwd", mutates_args=())
def l2norm_scale_fwd(x: _T, scale: float) -> _T:
    from .chunkwise_hgdn import l2norm_fwd
    return l2norm_fwd(x, scale)


@l2norm_scale_fwd.register_fake
def _(x, scale):
    return torch.empty_like(x, dtype=torch.bfloat16)


@torch.library.custom_op("llattn::l2norm_scale_bwd", mutates_args=())
def l2norm_scale_bwd(x: _T, dy: _T, scale: float) -> _T:
    from .chunkwise_hgdn import l2norm_bwd
    return l2norm_bwd(x, dy, scale)


@l2norm_scale_bwd.register_fake
def _(x, dy, scale):
    return torch.empty_like(x, dtype=torch.bfloat16)
