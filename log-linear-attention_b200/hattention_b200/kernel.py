"""Autograd boundary of log-linear attention, with the interface of the reference's
`hattention/kernel.py` (`HAttentionFunction` :32-244, `hattention_kernel` :338-374)."""
from typing import Optional, Tuple

import torch

from .base import HStruct, HType
from . import _lib
from .chunkwise import chunkwise_bwd, chunkwise_fwd, final_states
from .recurrent import HState  # noqa: F401  (re-exported: the reference imports it from both modules)


# Keep the forward call's scratch alive until the backward, which then skips its recomputation: the
# Mamba-2 segment-level states (about 0.2 GB at B=2, T=16384, H=32), and for Gated DeltaNet the chunk
# matrices and every chunk's level states (2.4 GB at B=4, T=8192, H=16, 128 x 128 heads; not kept above
# chunkwise_hgdn.KEEP_WORKSPACE_MAX_BYTES).  The reference keeps only the inputs (kernel.py:125); set to
# False for that memory behaviour.
KEEP_FORWARD_STATES = True


class HAttentionFunction(torch.autograd.Function):
    """Same argument list, validation and saved tensors as the reference's function
    (kernel.py:37-136); the chunkwise=False ("parallel") form is not provided."""

    @staticmethod
    def forward(ctx, q, k, v, b, g, l, scale, head_first, level_base, htype, hstruct, chunk_sizes, chunkwise,
                use_qk_l2norm_in_kernel):
        q, k, v, g, l = (x.contiguous() for x in (q, k, v, g, l))
        if hstruct == HStruct.MAMBA2 and chunkwise:
            if b is not None:
                raise ValueError
            if chunk_sizes[0] != chunk_sizes[1]:
                raise NotImplementedError
            if use_qk_l2norm_in_kernel:
                raise NotImplementedError
            if scale is not None:
                raise NotImplementedError
            kept = [] if KEEP_FORWARD_STATES else None
            o, g_cum, _ = chunkwise_fwd(q=q, k=k, v=v, g=g, l=l, head_first=head_first, level_base=level_base,
                                        htype=htype, chunk_size=chunk_sizes[0], output_final_state=False,
                                        keep_workspace=kept)
            ctx.fwd_workspace = kept[0] if kept else None
            Aw = Au = None
        elif hstruct == HStruct.GDELTA and chunkwise:
            from .chunkwise_hgdn import gdn_forward
            if b is None:
                raise ValueError
            if chunk_sizes[0] != chunk_sizes[1]:
                raise NotImplementedError
            if not use_qk_l2norm_in_kernel:
                raise NotImplementedError
            if scale is None:
                raise NotImplementedError
            kept = [] if KEEP_FORWARD_STATES and any(ctx.needs_input_grad[:6]) else None
            g_cum, o, Aw, Au = gdn_forward(q, k, v, b.contiguous(), g, l, scale, head_first, level_base, htype,
                                           chunk_sizes[0], keep=kept)
            ctx.fwd_workspace = kept if kept else None
        else:
            raise NotImplementedError
        ctx.save_for_backward(q, k, v, b, g_cum, l, Aw, Au)
        ctx.scale = scale
        ctx.dtype = g.dtype
        ctx.head_first = head_first
        ctx.level_base = level_base
        ctx.htype = htype
        ctx.hstruct = hstruct
        ctx.chunk_sizes = chunk_sizes
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, b, g_cum, l, Aw, Au = ctx.saved_tensors
        do = do.contiguous()
        if ctx.hstruct == HStruct.MAMBA2:
            dq, dk, dv, dg, dl = chunkwise_bwd(q=q, k=k, v=v, g=g_cum, l=l, do=do, head_first=ctx.head_first,
                                               level_base=ctx.level_base, htype=ctx.htype,
                                               chunk_size=ctx.chunk_sizes[0], fwd_workspace=ctx.fwd_workspace)
            ctx.fwd_workspace = None
            db = None
        else:
            from .chunkwise_hgdn import gdn_backward
            dq, dk, dv, db, dg, dl = gdn_backward(q, k, v, b, g_cum, l, Aw, Au, do, ctx.scale, ctx.head_first,
                                                  ctx.level_base, ctx.htype, ctx.chunk_sizes[0],
                                                  kept=ctx.fwd_workspace)
            ctx.fwd_workspace = None
        return (dq.to(q), dk.to(k), dv.to(v), db.to(b) if b is not None else None, dg.to(ctx.dtype), dl.to(l),
                None, None, None, None, None, None, None, None)


def hattention_kernel(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: Optional[torch.Tensor],
    g: torch.Tensor,
    l: torch.Tensor,
    scale: Optional[float],
    head_first: bool,
    level_base: int,
    htype: HType,
    hstruct: HStruct,
    chunk_sizes: Optional[Tuple[int, int]] = None,
    chunkwise: bool = True,
    use_qk_l2norm_in_kernel: bool = False,
) -> torch.Tensor:
    """o = log-linear attention(q, k, v, g, l[, b]) with gradients; see kernel.py:338-374."""
    if chunk_sizes is None:
        chunk_sizes = (64, 64)
    return HAttentionFunction.apply(q, k, v, b, g, l, scale, head_first, level_base, htype, hstruct, chunk_sizes,
                                    chunkwise, use_qk_l2norm_in_kernel)


@torch.no_grad()
def hattention_step(hstate: HState, q, k, v, b, g, l, scale, level_base, htype, hstruct,
                    use_qk_l2norm_in_kernel: bool = False):
    """One decoding step, signature of the reference's `hattention_step` (kernel.py:563-633):
    q, k (B,G,K), v (B,H,V), g (B,H), l (B,H,L)[, b (B,H)] -> (o (B,H,V), hstate).  One CUDA kernel per step for
    either structure (`llattn_mamba2_step`, `llattn_gdn_step`); for the delta-rule structure q and k are
    L2-normalised (q also scaled) first, as the reference does when `use_qk_l2norm_in_kernel` is set."""
    if not (q.ndim == 3 and k.ndim == 3 and v.ndim == 3 and g.ndim == 2 and l.ndim == 3
            and (b is None or b.ndim == 2) and g.dtype == hstate.dtype and q.dtype == k.dtype == v.dtype == l.dtype
            and hstate.base == level_base and hstate.htype == htype and hstate.hstruct == hstruct):
        raise TypeError
    if hstate.dtype != torch.float32:
        raise NotImplementedError("level states are kept in fp32")
    B, G, K = k.shape
    _, H, V = v.shape
    L = l.shape[-1]
    lib = _lib.lib()
    if hstruct == HStruct.MAMBA2:
        if b is not None:
            raise ValueError
        if use_qk_l2norm_in_kernel or scale is not None:
            raise NotImplementedError
    else:
        if b is None:
            raise ValueError
        if use_qk_l2norm_in_kernel:
            if scale is None:
                raise NotImplementedError
            from .chunkwise_hgdn import l2norm_fwd
            q, k = l2norm_fwd(q, scale), l2norm_fwd(k)
        elif scale is not None:
            raise NotImplementedError
        if G != H:
            q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    carry = hstate.cascade_counts()
    hstate.counts[0] += 1
    with torch.cuda.device(v.device):
        q_, k_, v_, l_ = (x.to(torch.bfloat16).contiguous() for x in (q, k, v, l))
        g_ = g.to(torch.float32).contiguous()
        o = torch.empty(B, H, V, dtype=torch.bfloat16, device=v.device)
        stream = torch.cuda.current_stream().cuda_stream
        if hstruct == HStruct.MAMBA2:
            rc = lib.llattn_mamba2_step(hstate.states.data_ptr(), q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), g_.data_ptr(),
                                        l_.data_ptr(), o.data_ptr(), B, H, G, K, V, L, carry, stream)
            _lib.check(rc, "llattn_mamba2_step")
        else:
            b_ = b.to(torch.bfloat16).contiguous()
            rc = lib.llattn_gdn_step(hstate.states.data_ptr(), q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), b_.data_ptr(),
                                     g_.data_ptr(), l_.data_ptr(), o.data_ptr(), B, H, K, V, L, carry, stream)
            _lib.check(rc, "llattn_gdn_step")
    return o.to(v.dtype), hstate


@torch.no_grad()
def hattention_prefill(q, k, v, b, g, l, scale, head_first, level_base, htype, hstruct,
                       chunk_size: Optional[int] = None, use_qk_l2norm_in_kernel: bool = False):
    """Outputs for a prompt and the level states to continue from, signature of the reference's
    `hattention_prefill` (kernel.py:469-560).  Mamba-2 structure: the largest multiple of the chunk size goes
    through the chunkwise kernels, its level states come from one kernel (`final_states`), the remaining tokens
    are stepped.  Delta-rule structure: the chunkwise kernels produce the outputs of the full chunks and the
    inter-chunk level states as of the start of the last full chunk; that chunk's tokens and the remaining ones
    are stepped through the decode kernel, which builds the levels inside the chunk."""
    if chunk_size is None:
        chunk_size = 64
    if head_first:
        raise NotImplementedError
    B, T, G, K = k.shape
    _, _, H, V = v.shape
    L = l.shape[-1]
    T0 = T - (T % chunk_size)
    o = torch.zeros_like(v)
    hstate = HState(base=level_base, htype=htype, hstruct=hstruct, shape=(B, H, K, V, L), dtype=torch.float32, device=g.device)
    if hstruct == HStruct.MAMBA2:
        if b is not None:
            raise ValueError
        if use_qk_l2norm_in_kernel or scale is not None:
            raise NotImplementedError
        if T0 != 0:
            o0, _, ht = chunkwise_fwd(q[:, :T0], k[:, :T0], v[:, :T0], g[:, :T0], l[:, :T0], head_first, level_base, htype,
                                      chunk_size, True)
            o[:, :T0] = o0.to(v.dtype)
            hstate.states = ht
            hstate.set_counts_after(T0)
        first_step = T0
    else:
        from .chunkwise_hgdn import chunkwise_fwd as chunkwise_fwd_hgdn, l2norm_fwd
        if b is None:
            raise ValueError
        if not use_qk_l2norm_in_kernel or scale is None:
            raise NotImplementedError
        first_step = 0
        if T0 != 0:
            qn, kn = l2norm_fwd(q[:, :T0], scale), l2norm_fwd(k[:, :T0])
            _, o0, _, _, ht = chunkwise_fwd_hgdn(qn, kn, v[:, :T0], b[:, :T0], g[:, :T0], l[:, :T0], head_first, level_base,
                                                 htype, chunk_size, True)
            o[:, :T0] = o0.to(v.dtype)
            hstate.states = ht
            first_step = T0 - chunk_size
            hstate.set_counts_before(first_step)
    for t in range(first_step, T):
        ot, hstate = hattention_step(hstate, q[:, t], k[:, t], v[:, t], b[:, t] if b is not None else None, g[:, t].float(),
                                     l[:, t], scale, level_base, htype, hstruct, use_qk_l2norm_in_kernel)
        if t >= T0:
            o[:, t] = ot
    return o, hstate
