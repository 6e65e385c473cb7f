"""Layer-level log-linear Mamba-2 API with the signature of the reference's
`hmamba_chunk_scan_combined` (hattention/mamba_apis.py:263-404)."""
import warnings
from typing import Optional, Tuple

import torch

from .base import HStruct, HType
from .kernel import hattention_kernel


def compute_lambda(L: torch.Tensor, dl: torch.Tensor, lambda_mode: Optional[str]) -> torch.Tensor:
    """mamba_apis.py:70-85."""
    if lambda_mode == "positive":
        return torch.nn.functional.softplus(L * dl)
    if lambda_mode == "bounded":
        return torch.exp(-torch.exp(L) * torch.nn.functional.softplus(dl))
    if lambda_mode is None:
        return L * dl
    raise ValueError


def hmamba_chunk_scan_combined(
    x: torch.Tensor,
    dt: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    dl: torch.Tensor,
    L: torch.Tensor,
    chunk_size: int,
    D: Optional[torch.Tensor] = None,
    z: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    seq_idx: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    dt_softplus: bool = False,
    dt_limit: Tuple[float, float] = (0.0, float("inf")),
    return_final_states: bool = False,
    return_varlen_states: bool = False,
    lambda_mode: Optional[str] = None,
    lambda_level_max: Optional[int] = None,
    lambda_level_base: Optional[int] = None,
    lambda_htype: Optional[HType] = None,
    lambda_hstruct: Optional[HStruct] = None,
    lambda_level_fixed: Optional[bool] = None,
    lambda_level_module=None,
):
    """x (B,T,H,P), dt (B,T,H), A (H), B/C (B,T,G,N), dl (B,T,H,L), L (H,L) -> (y, None).

    Same preparation as the reference (mamba_apis.py:346-366): dt = softplus(dt + bias),
    v = x * dt, g = A * dt, lambda = compute_lambda(L, dl), then the kernel with q=C, k=B;
    y += D * x.  Unsupported options raise exactly where the reference raises.
    """
    if z is not None or initial_states is not None or seq_idx is not None or cu_seqlens is not None:
        raise NotImplementedError
    if dt_softplus is not True:
        raise NotImplementedError
    if tuple(dt_limit) != (0.0, float("inf")):
        raise NotImplementedError
    if return_varlen_states is not False:
        raise NotImplementedError
    if return_final_states:
        raise NotImplementedError("prefill hand-off (return_final_states=True) is not implemented")
    if B.shape != C.shape:
        raise ValueError("B and C must have the same shape")
    if lambda_level_max is None or lambda_level_base is None or lambda_htype is None or lambda_hstruct is None \
            or lambda_level_fixed is None:
        raise ValueError
    if not lambda_level_fixed:
        raise NotImplementedError("only fixed lambda levels are supported")
    if L.shape[-1] != lambda_level_max or dl.shape[-1] != lambda_level_max:
        raise ValueError
    if D is not None:
        if D.dim() != 1:
            raise ValueError
        D_residual = x * D[None, None, :, None]
    if dt_bias is not None:
        dt = dt + dt_bias[None, None, :]
    dt = torch.nn.functional.softplus(dt)
    x = x * dt[..., None]
    g = A[None, None, :] * dt
    lam = compute_lambda(L[None, None], dl, lambda_mode)
    y = hattention_kernel(q=C, k=B, v=x, b=None, g=g, l=lam, scale=None, head_first=False,
                          level_base=lambda_level_base, htype=lambda_htype, hstruct=lambda_hstruct)
    if D is not None:
        y = y + D_residual
    return y, None
