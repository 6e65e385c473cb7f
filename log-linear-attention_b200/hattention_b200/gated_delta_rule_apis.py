"""Layer-level log-linear Gated DeltaNet API with the signature of the reference's
`chunk_h_gated_delta_rule` (hattention/gated_delta_rule_apis.py:21-34)."""
import warnings
from typing import Optional

import torch

from .base import HStruct, HType
from .kernel import hattention_kernel

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
    """q,k (B,T,H,K), v (B,T,H,V), g (B,T,H) log decay, l (B,T,H,L), beta (B,T,H) -> (o, None).
    Same checks as the reference (gated_delta_rule_apis.py:35-70): bf16 only, no varlen, l2norm
    in the kernel is mandatory, scale defaults to K^-1/2 and lambda is divided by it."""
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
    if output_final_state or initial_state is not None:
        raise NotImplementedError("prefill / decode hand-off is not implemented")
    o = hattention_kernel(q=q, k=k, v=v, b=beta, g=g, l=l, scale=scale, head_first=False, level_base=2,
                          htype=HType.WEAK, hstruct=HStruct.GDELTA, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel)
    return o, None
