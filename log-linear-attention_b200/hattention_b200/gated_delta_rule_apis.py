"""Layer-level log-linear Gated DeltaNet API with the signature of the reference's
`chunk_h_gated_delta_rule` (hattention/gated_delta_rule_apis.py:21-34)."""
import warnings
from typing import Optional

import torch

from .base import HStruct, HType
from .kernel import hattention_kernel, hattention_prefill, hattention_step

SCALE_LAMBDA = True


@torch.compiler.disable
def chunk_h_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    l: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state=None,
    output_final_state: bool = False,
    cu_seqlens: Optional[torch.LongTensor] = None,
    head_first: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
):
    """q,k (B,T,H,K), v (B,T,H,V), g (B,T,H) log decay, l (B,T,H,L), beta (B,T,H) -> (o, final_state).
    Same checks and dispatch as the reference (gated_delta_rule_apis.py:35-132): bf16 only, no varlen, l2norm
    in the kernel is mandatory, scale defaults to K^-1/2 and lambda is divided by it; training call without
    states, prompt call with `output_final_state=True` (-> `hattention_prefill`), and one-token call with an
    `initial_state` (-> `hattention_step`)."""
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16."
    assert len(beta.shape) == 3, "beta must be of shape [B, T, H] if head_first=False, or [B, H, T] otherwise."
    assert cu_seqlens is None
    assert use_qk_l2norm_in_kernel is True
    if head_first:
        raise DeprecationWarning("head_first is deprecated; use head_first=False")
    if q.shape[1] < q.shape[2]:
        warnings.warn(f"seq_len ({q.shape[1]}) < num_heads ({q.shape[2]}): inputs may be in head-first format")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if SCALE_LAMBDA:
        l = l / scale
    common = dict(scale=scale, level_base=2, htype=HType.WEAK, hstruct=HStruct.GDELTA,
                  use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel)
    if output_final_state is False:
        if initial_state is not None:
            raise NotImplementedError
        o = hattention_kernel(q=q, k=k, v=v, b=beta, g=g, l=l, head_first=False, **common)
        return o, None
    if initial_state is None:
        return hattention_prefill(q=q, k=k, v=v, b=beta, g=g, l=l, head_first=False, **common)
    if not (q.ndim == 4 and k.ndim == 4 and v.ndim == 4 and beta.ndim == 3 and g.ndim == 3 and l.ndim == 4
            and q.shape[1] == k.shape[1] == v.shape[1] == beta.shape[1] == g.shape[1] == l.shape[1] == 1):
        raise ValueError
    o, final_state = hattention_step(hstate=initial_state, q=q.squeeze(1), k=k.squeeze(1), v=v.squeeze(1), b=beta.squeeze(1),
                                     g=g.squeeze(1), l=l.squeeze(1), **common)
    return o.unsqueeze(1), final_state
