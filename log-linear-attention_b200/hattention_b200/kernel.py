"""Autograd boundary of log-linear attention, with the interface of the reference's
`hattention/kernel.py` (`HAttentionFunction` :32-244, `hattention_kernel` :338-374)."""
from typing import Optional, Tuple

import torch

from .base import HStruct, HType
from .chunkwise import chunkwise_bwd, chunkwise_fwd


# Keep the Mamba-2 forward call's scratch (segment-level states, about 0.2 GB at B=2, T=16384, H=32)
# alive until the backward, which then skips their recomputation.  The reference keeps only the inputs
# (kernel.py:125); set to False for that memory behaviour.
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
            g_cum, o, Aw, Au = gdn_forward(q, k, v, b.contiguous(), g, l, scale, head_first, level_base, htype,
                                           chunk_sizes[0])
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
                                                  ctx.level_base, ctx.htype, ctx.chunk_sizes[0])
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
