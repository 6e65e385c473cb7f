"""Layer-level log-linear Mamba-2 API with the signature of the reference's
`hmamba_chunk_scan_combined` (hattention/mamba_apis.py:263-404)."""
import warnings
from typing import Optional, Tuple

import torch

from . import _lib
from .base import HStruct, HType
from .chunkwise import chunkwise_bwd, chunkwise_fwd
from .kernel import KEEP_FORWARD_STATES, hattention_kernel, hattention_prefill, hattention_step
from .recurrent import HState

try:
    from torchtune.modules import RotaryPositionalEmbeddings
except ImportError:          # the reference tolerates a missing torchtune the same way (mamba_apis.py:26-29)
    RotaryPositionalEmbeddings = None

_LAMBDA_MODES = {"positive": 0, "bounded": 1, None: 2}
# bf16 CUDA activations take the fused element-wise kernels; False keeps the reference's sequence of
# torch ops around the kernel for every dtype (used by the tests as the cross-check)
FUSED_PREP = True


def _ptr(t):
    return t.data_ptr() if t is not None else None


class HMambaCombinedFunction(torch.autograd.Function):
    """The whole layer call for bf16 CUDA activations as one autograd node: fused element-wise
    preparation (one pass), the chunkwise kernels, the D residual; backward in the opposite order with
    one fused pass for every element-wise gradient (mamba_apis.py:346-366, 401-402 in the reference are
    separate torch ops, each differentiated by autograd)."""

    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, dl, Lp, D, dt_bias, lambda_mode, level_base, htype):
        lib = _lib.lib()
        Bsz, T, H, P = x.shape
        L = dl.shape[-1]
        rows = Bsz * T * H
        x_, dt_, dl_ = x.contiguous(), dt.contiguous(), dl.contiguous()
        A_, Lp_ = A.detach().float().contiguous(), Lp.detach().float().contiguous()
        D_ = D.detach().float().contiguous() if D is not None else None
        bias_ = dt_bias.detach().float().contiguous() if dt_bias is not None else None
        mode = _LAMBDA_MODES[lambda_mode]
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream().cuda_stream
            v = torch.empty_like(x_)
            g = torch.empty(Bsz, T, H, dtype=torch.float32, device=x.device)
            lam = torch.empty_like(dl_)
            rc = lib.llattn_mamba2_prep_fwd(x_.data_ptr(), dt_.data_ptr(), _ptr(bias_), A_.data_ptr(), dl_.data_ptr(), Lp_.data_ptr(),
                                            v.data_ptr(), g.data_ptr(), lam.data_ptr(), rows, H, P, L, mode, stream)
            _lib.check(rc, "llattn_mamba2_prep_fwd")
            kept = [] if KEEP_FORWARD_STATES else None
            o, g_cum, _ = chunkwise_fwd(q=Cm, k=Bm, v=v, g=g, l=lam, head_first=False, level_base=level_base, htype=htype,
                                        chunk_size=64, output_final_state=False, keep_workspace=kept)
            if D_ is not None:
                y_dtype = torch.promote_types(o.dtype, D.dtype)      # fp32 for an fp32 D, as x * D[...] + y gives
                y = torch.empty(o.shape, dtype=torch.float32 if y_dtype == torch.float32 else torch.bfloat16, device=o.device)
                rc = lib.llattn_mamba2_residual(o.data_ptr(), x_.data_ptr(), D_.data_ptr(), y.data_ptr(),
                                                1 if y.dtype == torch.float32 else 0, rows, H, P, stream)
                _lib.check(rc, "llattn_mamba2_residual")
            else:
                y = o
        ctx.save_for_backward(x_, dt_, A_, Bm, Cm, dl_, Lp_, D_, bias_, v, g_cum, lam)
        ctx.fwd_workspace = kept[0] if kept else None
        ctx.meta = (mode, level_base, htype, A.dtype, Lp.dtype, D.dtype if D is not None else None,
                    dt_bias.dtype if dt_bias is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_, dt_, A_, Bm, Cm, dl_, Lp_, D_, bias_, v, g_cum, lam = ctx.saved_tensors
        mode, level_base, htype, A_dt, L_dt, D_dt, b_dt = ctx.meta
        lib = _lib.lib()
        Bsz, T, H, P = x_.shape
        L = dl_.shape[-1]
        rows = Bsz * T * H
        dy = dy.to(torch.bfloat16).contiguous()
        dq, dk, dv, dg, dlam = chunkwise_bwd(q=Cm, k=Bm, v=v, g=g_cum, l=lam, do=dy, head_first=False, level_base=level_base,
                                             htype=htype, chunk_size=64, fwd_workspace=ctx.fwd_workspace)
        ctx.fwd_workspace = None
        with torch.cuda.device(x_.device):
            dx = torch.empty_like(x_)
            ddt = torch.empty_like(dt_)
            ddl = torch.empty_like(dl_)
            acc = torch.zeros(3 * H + H * L, dtype=torch.float32, device=x_.device)
            dA, dbias, dD, dLp = acc[:H], acc[H:2 * H], acc[2 * H:3 * H], acc[3 * H:].view(H, L)
            rc = lib.llattn_mamba2_prep_bwd(x_.data_ptr(), dt_.data_ptr(), _ptr(bias_), A_.data_ptr(), dl_.data_ptr(), Lp_.data_ptr(),
                                            _ptr(D_), dv.data_ptr(), dg.data_ptr(), dlam.data_ptr(), dy.data_ptr(),
                                            dx.data_ptr(), ddt.data_ptr(), ddl.data_ptr(), dA.data_ptr(), dbias.data_ptr(),
                                            dLp.data_ptr(), dD.data_ptr(), rows, H, P, L, mode, torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "llattn_mamba2_prep_bwd")
        return (dx, ddt, dA.to(A_dt), dk.to(Bm.dtype), dq.to(Cm.dtype), ddl, dLp.to(L_dt),
                dD.to(D_dt) if D_ is not None else None, dbias.to(b_dt) if bias_ is not None else None, None, None, None)


class LambdaLevelMLP(torch.nn.Module):
    """Per-level lambda inputs from `dim` features: a rotary position embedding whose position is the level
    index, then one linear unit, for each of the two operands (mamba_apis.py:32-67 in the reference).  Only the
    non-fixed lambda mode uses it; it needs torchtune's RotaryPositionalEmbeddings like the reference's."""

    def __init__(self, dim: int, max_num_levels: int, **kwargs) -> None:
        super().__init__()
        if RotaryPositionalEmbeddings is None:
            raise ImportError("LambdaLevelMLP needs torchtune (RotaryPositionalEmbeddings)")
        self.dim = dim
        self.max_num_levels = max_num_levels
        self.mlp0 = torch.nn.Linear(in_features=dim, out_features=1)
        self.mlp1 = torch.nn.Linear(in_features=dim, out_features=1)
        self.rope = RotaryPositionalEmbeddings(dim=dim, max_seq_len=max_num_levels)

    def forward(self, x0: torch.Tensor, x1: torch.Tensor, num_levels: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if x0.ndim != 4 or x1.ndim != 4:
            raise ValueError
        if num_levels > self.max_num_levels:
            raise ValueError
        y0s, y1s = [], []
        for level in range(num_levels):
            pos0 = torch.full((x0.shape[1],), level, dtype=torch.int32, device=x0.device)
            pos1 = torch.full((x1.shape[1],), level, dtype=torch.int32, device=x1.device)
            y0s.append(self.mlp0(self.rope(x0, input_pos=pos0)))
            y1s.append(self.mlp1(self.rope(x1, input_pos=pos1)))
        return torch.concat(y0s, dim=-1), torch.concat(y1s, dim=-1)


def compute_lambda_maybe_fixed(L: torch.Tensor, dl: torch.Tensor, lambda_mode: Optional[str], lambda_level_max: int,
                               lambda_level_fixed: bool, lambda_level_module) -> torch.Tensor:
    """mamba_apis.py:88-113: fixed levels use L and dl as they are; otherwise the level module expands
    `dim` features into `lambda_level_max` levels first."""
    if lambda_level_fixed:
        if not (L.ndim in (3, 4) and dl.ndim in (3, 4) and L.shape[-1] == lambda_level_max and dl.shape[-1] == lambda_level_max):
            raise ValueError
        return compute_lambda(L=L, dl=dl, lambda_mode=lambda_mode)
    if not (L.ndim in (3, 4) and dl.ndim in (3, 4) and L.shape[-1] == lambda_level_module.dim
            and dl.shape[-1] == lambda_level_module.dim):
        raise ValueError
    L_new, dl_new = lambda_level_module(L, dl, num_levels=lambda_level_max)
    return compute_lambda(L=L_new, dl=dl_new, lambda_mode=lambda_mode)


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
    if B.shape != C.shape:
        raise ValueError("B and C must have the same shape")
    if lambda_level_max is None or lambda_level_base is None or lambda_htype is None or lambda_hstruct is None \
            or lambda_level_fixed is None:
        raise ValueError
    if not lambda_level_fixed:
        raise NotImplementedError("only fixed lambda levels are supported")
    if L.shape[-1] != lambda_level_max or dl.shape[-1] != lambda_level_max:
        raise ValueError
    if D is not None and D.dim() != 1:
        raise ValueError
    if return_final_states:
        # inference: outputs for the prompt and the level states to decode from (mamba_apis.py:381-399)
        if D is not None:
            D_residual = x * D[None, None, :, None]
        if dt_bias is not None:
            dt = dt + dt_bias[None, None, :]
        dt = torch.nn.functional.softplus(dt.float())
        v = (x * dt[..., None]).to(C.dtype)
        lam = compute_lambda(L[None, None].to(dl.dtype), dl, lambda_mode)
        y, state = hattention_prefill(q=C, k=B, v=v, b=None, g=A[None, None, :].float() * dt, l=lam.to(C.dtype), scale=None,
                                      head_first=False, level_base=lambda_level_base, htype=lambda_htype,
                                      hstruct=lambda_hstruct)
        if D is not None:
            y = y + D_residual
        return y, state
    bf16_cuda = all(t.is_cuda and t.dtype == torch.bfloat16 for t in (x, dt, B, C, dl))
    if (FUSED_PREP and bf16_cuda and lambda_hstruct == HStruct.MAMBA2 and lambda_htype == HType.WEAK and lambda_level_base == 2
            and lambda_mode in _LAMBDA_MODES and x.shape[-1] % 8 == 0 and x.shape[-1] <= 256 and L.dim() == 2):
        y = HMambaCombinedFunction.apply(x, dt, A, B, C, dl, L, D, dt_bias, lambda_mode, lambda_level_base, lambda_htype)
        return y, None
    # other dtypes: the reference's own sequence of torch element-wise ops around the kernel
    if D is not None:
        D_residual = x * D[None, None, :, None]
    if dt_bias is not None:
        dt = dt + dt_bias[None, None, :]
    dt = torch.nn.functional.softplus(dt)
    x = (x * dt[..., None]).to(x.dtype)      # an fp32 dt must not promote the kernel's v operand (bf16 only)
    g = A[None, None, :] * dt
    lam = compute_lambda(L[None, None], dl, lambda_mode)
    y = hattention_kernel(q=C, k=B, v=x, b=None, g=g, l=lam, scale=None, head_first=False,
                          level_base=lambda_level_base, htype=lambda_htype, hstruct=lambda_hstruct)
    if D is not None:
        y = y + D_residual
    return y, None


def hselective_state_update(
    state: HState,
    x: torch.Tensor,
    dt: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    dl: torch.Tensor,
    L: torch.Tensor,
    D: Optional[torch.Tensor] = None,
    z: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    dt_softplus: bool = False,
    state_batch_indices: Optional[torch.Tensor] = None,
    lambda_mode: Optional[str] = None,
    lambda_level_max: Optional[int] = None,
    lambda_level_base: Optional[int] = None,
    lambda_htype: Optional[HType] = None,
    lambda_hstruct: Optional[HStruct] = None,
    lambda_level_fixed: Optional[bool] = None,
    lambda_level_module=None,
) -> Tuple[torch.Tensor, HState]:
    """One decode step of the layer: x (B,H,P), dt (B,H), A (H), B/C (B,G,N), dl (B,H,L), L (H,L) ->
    (out (B,H,P), state).  Signature, checks and preparation of the reference's function of this name
    (mamba_apis.py:407-566); the state update and read-out (its `step_state` / `step_output`) are one CUDA
    kernel here (`hattention_step`), which takes the log decay A*dt where the reference passes exp(A*dt)."""
    if state_batch_indices is not None:
        raise NotImplementedError
    if z is not None:
        raise NotImplementedError
    if x.dim() != 3 or dt.dim() != 2 or A.dim() != 1 or B.dim() != 3 or C.dim() != 3 or dl.dim() != 3 or L.dim() != 2:
        raise ValueError
    if D is not None and D.dim() != 1:
        raise ValueError
    if dt_bias is not None and dt_bias.dim() != 1:
        raise ValueError
    batch, nheads, headdim = x.shape
    _, ngroups, dstate = B.shape
    dlambda = L.shape[-1]
    if dt.shape != x.shape[:2] or A.shape != (nheads,) or nheads % ngroups != 0 or B.shape != (batch, ngroups, dstate) \
            or C.shape != B.shape or dl.shape != (batch, nheads, dlambda) or L.shape != (nheads, dlambda):
        raise ValueError
    if D is not None and D.shape != (nheads,):
        raise ValueError
    if lambda_level_max is None or lambda_level_base is None or lambda_htype is None or lambda_hstruct is None \
            or lambda_level_fixed is None:
        raise ValueError
    if D is not None:
        D_residual = x * D[None, :, None]
    if dt_bias is not None:
        if dt_bias.shape != (nheads,):
            raise ValueError
        dt = dt + dt_bias
    if dt_softplus:
        dt = torch.nn.functional.softplus(dt)
    g = (A[None, :].float() * dt.float())
    v = (x * dt[..., None]).to(C.dtype)
    lam = compute_lambda_maybe_fixed(L=L[None].to(dl.dtype), dl=dl, lambda_mode=lambda_mode, lambda_level_max=lambda_level_max,
                                     lambda_level_fixed=lambda_level_fixed, lambda_level_module=lambda_level_module)
    if not (C.dtype == B.dtype and state.base == lambda_level_base and state.htype == lambda_htype
            and state.hstruct == lambda_hstruct):
        raise TypeError
    out, state = hattention_step(state, q=C, k=B, v=v, b=None, g=g.to(state.dtype), l=lam.to(C.dtype), scale=None,
                                 level_base=lambda_level_base, htype=lambda_htype, hstruct=lambda_hstruct)
    if D is not None:
        out = out + D_residual
    return out, state


def _causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Depthwise causal convolution followed by SiLU on (B, D, T): what causal_conv1d_fn(..., activation="silu")
    computes (call site mamba_apis.py:213-220 in the reference).  Outside the log-linear attention path:
    a torch depthwise convolution."""
    width = weight.shape[-1]
    y = torch.nn.functional.conv1d(x, weight.unsqueeze(1).to(x.dtype), bias.to(x.dtype) if bias is not None else None,
                                   padding=width - 1, groups=x.shape[1])[..., : x.shape[-1]]
    return torch.nn.functional.silu(y)


def _gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm(y * silu(z)) * weight in fp32, returned in y's dtype (rmsnorm_fn with norm_before_gate=False,
    call site mamba_apis.py:251-258 in the reference)."""
    x = y.float() * torch.nn.functional.silu(z.float())
    out = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return out.to(z.dtype)


def hmamba_split_conv1d_scan_combined(
    zxbcdtdl: torch.Tensor,
    conv1d_weight: torch.Tensor,
    conv1d_bias: torch.Tensor,
    dt_bias: torch.Tensor,
    A: torch.Tensor,
    L: torch.Tensor,
    D: torch.Tensor,
    chunk_size: int,
    initial_states: Optional[torch.Tensor] = None,
    seq_idx: Optional[torch.Tensor] = None,
    dt_limit: Tuple[float, float] = (0.0, float("inf")),
    return_final_states: bool = False,
    activation: str = "silu",
    rmsnorm_weight: Optional[torch.Tensor] = None,
    rmsnorm_eps: float = 1e-6,
    outproj_weight: Optional[torch.Tensor] = None,
    outproj_bias: Optional[torch.Tensor] = None,
    headdim: Optional[int] = None,
    ngroups: int = 1,
    norm_before_gate: bool = True,
    lambda_mode: Optional[str] = None,
    lambda_level_max: Optional[int] = None,
    lambda_level_base: Optional[int] = None,
    lambda_htype: Optional[HType] = None,
    lambda_hstruct: Optional[HStruct] = None,
    lambda_level_fixed: Optional[bool] = None,
    lambda_level_module=None,
) -> torch.Tensor:
    """Signature, checks and data flow of the reference's function of this name (mamba_apis.py:116-262):
    split -> depthwise causal conv + SiLU on (x, B, C) -> hmamba_chunk_scan_combined -> gated RMSNorm ->
    output projection.  The convolution, the norm and the projection are torch ops here (the reference
    calls causal_conv1d / mamba_ssm kernels for the first two); the scan is this package's CUDA path."""
    if initial_states is not None or seq_idx is not None:
        raise NotImplementedError
    if tuple(dt_limit) != (0.0, float("inf")):
        raise NotImplementedError
    if return_final_states is not False:
        raise NotImplementedError
    if norm_before_gate is not False:
        raise NotImplementedError
    if rmsnorm_weight is None:
        raise NotImplementedError
    if activation not in ["silu", "swish"]:
        raise NotImplementedError
    if D.dim() != 1:
        raise ValueError
    if headdim is None:
        raise ValueError
    batch, seqlen, _ = zxbcdtdl.shape
    dlambda = L.shape[-1]
    nheads, = D.shape
    dim = nheads * headdim
    dstate = (zxbcdtdl.shape[-1] - 2 * dim - nheads - nheads * dlambda) // ngroups // 2
    if nheads % ngroups != 0:
        raise ValueError
    if zxbcdtdl.shape != (batch, seqlen, 2 * dim + 2 * ngroups * dstate + nheads + nheads * dlambda):
        raise ValueError
    if dt_bias.shape != (nheads,) or A.shape != (nheads,) or L.shape != (nheads, dlambda):
        raise ValueError
    z, xBC, dt, dl = torch.split(zxbcdtdl, [dim, dim + 2 * ngroups * dstate, nheads, nheads * dlambda], dim=-1)
    xBC = _causal_conv1d_silu(xBC.transpose(1, 2), conv1d_weight, conv1d_bias).transpose(1, 2)
    x, Bm, Cm = torch.split(xBC, [dim, ngroups * dstate, ngroups * dstate], dim=-1)
    y, _ = hmamba_chunk_scan_combined(
        x=x.reshape(batch, seqlen, nheads, headdim).contiguous(), dt=dt.contiguous(), A=A,
        B=Bm.reshape(batch, seqlen, ngroups, dstate).contiguous(), C=Cm.reshape(batch, seqlen, ngroups, dstate).contiguous(),
        dl=dl.reshape(batch, seqlen, nheads, dlambda).contiguous(), L=L, chunk_size=chunk_size, D=D, z=None, dt_bias=dt_bias,
        dt_softplus=True, seq_idx=None, cu_seqlens=None, dt_limit=dt_limit, return_final_states=False,
        return_varlen_states=False, lambda_mode=lambda_mode, lambda_level_max=lambda_level_max,
        lambda_level_base=lambda_level_base, lambda_htype=lambda_htype, lambda_hstruct=lambda_hstruct,
        lambda_level_fixed=lambda_level_fixed, lambda_level_module=lambda_level_module)
    y = _gated_rmsnorm(y.reshape(batch, seqlen, dim), z, rmsnorm_weight, rmsnorm_eps)
    return torch.nn.functional.linear(y, outproj_weight.to(y.dtype), outproj_bias.to(y.dtype) if outproj_bias is not None else None)
