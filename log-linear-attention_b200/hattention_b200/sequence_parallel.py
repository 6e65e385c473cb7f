"""Sequence-parallel log-linear Mamba-2 attention: one sequence split along T over the ranks of a group.

Rank r holds the r-th of R = 2^p equal shards of T_s = 2^n tokens.  Shards are aligned to their own
size, so for two tokens of one shard `bit_length(t ^ s)` is the same with global and with local indices:
the in-shard part of the output is the unsharded operator applied to the shard (the CUDA kernels, called
through `hattention_kernel`), reading lambda columns 0 .. n.  A token of shard r sees a token of an
earlier shard r' at level n + bit_length(r ^ r'), which depends on the shard indices only, so all that
has to cross between ranks is, per shard, its plain (single-level) final state

    F_r = sum_s exp(D_r - G_s) k_s (x) v_s   (B, H, K, V) fp32,     D_r = sum of g over the shard   (B, H)

with G the inclusive in-shard cumulative sum of g: one all-gather of K*V + 1 floats per (batch, head)
and rank in the forward and one reduce-scatter of the same size in the backward.  A reader shard merges,
for each of its set bits j-1, the states of the 2^(j-1) contributor shards of that level, decayed across
the shards in between, and adds  lambda[t, n + j] exp(G_t) q_t S_j  to its rows.  This is the Fenwick
schedule of the reference's per-level state scan (hattention/chunkwise.py:110-280, predicates :34-72)
applied to whole shards; the reference itself has no sequence-parallel mode (its kernels use the local
chunk index, chunkwise.py:179,236).

The cross-shard part is small (2 T_s K V flops per level and head, the cost of one level of the scan)
and is written with torch operations under autograd (library GEMMs on 16-bit operands, one per batch
item and q/k group); the in-shard part carries all the heavy work.
"""
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def _log2_exact(x: int, what: str) -> int:
    if x <= 0 or (x & (x - 1)) != 0:
        raise ValueError(f"{what} must be a power of two, got {x}")
    return x.bit_length() - 1


def cross_shard_levels(rank: int, world: int) -> List[Tuple[int, List[int]]]:
    """[(j, contributor ranks)] for the shard levels j = 1 .. log2(world) that shard `rank` reads:
    bit j-1 of rank set; contributors are the lower half of the aligned block of 2^j shards."""
    p = _log2_exact(world, "number of shards")
    out = []
    for j in range(1, p + 1):
        if (rank >> (j - 1)) & 1:
            base = (rank >> j) << j
            out.append((j, list(range(base, base + (1 << (j - 1))))))
    return out


def _compute_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.float64 if x.dtype == torch.float64 else torch.float32


def _product_dtype(x: torch.Tensor) -> torch.dtype:
    # operands of the shard-level products: the activations' own 16-bit type on the GPU (the kernels
    # also feed level states to the tensor cores in bf16), the compute dtype otherwise
    return x.dtype if x.dtype in (torch.bfloat16, torch.float16) else _compute_dtype(x)


def cumulative_decay(g: torch.Tensor) -> torch.Tensor:
    """Inclusive cumulative sum of g (B, T, H) along T in the compute dtype.  The scan runs along the
    innermost axis of a transposed copy (a scan along an outer axis is many times slower on the GPU)."""
    return torch.cumsum(g.to(_compute_dtype(g)).transpose(1, 2).contiguous(), dim=-1).transpose(1, 2)


def shard_summary(k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, gc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(B, H, K*V + 1): the shard's plain final state, flattened, followed by its total log-decay.
    The decay weights are folded into v, so that q/k groups are not expanded to heads: per (batch, group)
    the state of all its heads is one product k^T (K x T) by v' (T x heads*V)."""
    B, T, H = g.shape
    ct, pt = _compute_dtype(g), _product_dtype(k)
    G_, K, V = k.shape[2], k.shape[-1], v.shape[-1]
    hpg = H // G_
    gc = cumulative_decay(g) if gc is None else gc
    D = gc[:, -1]                                            # (B, H)
    # the (B, T, H) weights are rounded to the product dtype first: the passes over (B, T, H, V) tensors
    # then move 16-bit data only
    va = (v.to(pt) * torch.exp(D[:, None] - gc).to(pt)[..., None]).reshape(B, T, G_, hpg * V)
    F = torch.einsum("btgk,btgx->bgkx", k.to(pt), va)        # (B, G, K, hpg*V)
    F = F.reshape(B, G_, K, hpg, V).permute(0, 1, 3, 2, 4).reshape(B, H, K * V).to(ct)
    return torch.cat([F, D[..., None]], dim=-1)


def shard_cross_output(q: torch.Tensor, g: torch.Tensor, l: torch.Tensor, summaries: Sequence[torch.Tensor],
                       rank: int, K: int, V: int, gc: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Rows that shard `rank` receives from earlier shards, (B, T_s, H, V) in the product dtype, or None
    for a shard that reads nothing (rank 0).  `summaries[r]` is shard r's `shard_summary`."""
    world = len(summaries)
    B, T, H = g.shape
    n = _log2_exact(T, "tokens per shard")
    levels = cross_shard_levels(rank, world)
    if not levels:
        return None
    if l.shape[-1] < n + _log2_exact(world, "number of shards") + 1:
        raise ValueError("lambda has too few level columns for the whole sequence")
    ct, pt = _compute_dtype(g), _product_dtype(q)
    G_ = q.shape[2]
    hpg = H // G_
    qp = q.to(pt)
    eg = torch.exp(cumulative_decay(g) if gc is None else gc)   # decay from the shard's start to each row
    out = None
    for j, ranks in levels:
        S = None
        for r in ranks:
            F = summaries[r][..., : K * V].to(ct)
            between = sum(summaries[m][..., K * V].to(ct) for m in range(r + 1, rank)) if r + 1 < rank else None
            term = F if between is None else F * torch.exp(between)[..., None]
            S = term if S is None else S + term
        # (B, H, K*V) -> (B, G, K, hpg*V): one product per (batch, group) serves all heads of the group
        Sg = S.reshape(B, G_, hpg, K, V).permute(0, 1, 3, 2, 4).reshape(B, G_, K, hpg * V).to(pt)
        y = torch.einsum("btgk,bgkx->btgx", qp, Sg).reshape(B, T, H, V)
        part = y * (l[..., n + j].to(ct) * eg).to(pt)[..., None]
        out = part if out is None else out + part
    return out


class _AllGatherSummaries(torch.autograd.Function):
    """all-gather in the forward; in the backward every rank holds gradients for every shard's summary,
    which are summed over ranks and each rank keeps its own slot."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        x = x.contiguous()
        out = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(out, x, group=group)
        ctx.group = group
        ctx.rank = dist.get_rank(group)
        return torch.stack(out)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        if dist.get_backend(ctx.group) == "nccl":
            mine = torch.empty_like(grad[0])
            dist.reduce_scatter_tensor(mine, grad, group=ctx.group)
            return mine, None
        dist.all_reduce(grad, group=ctx.group)
        return grad[ctx.rank], None


def _default_local_op(q, k, v, g, l):
    from .base import HStruct, HType
    from .kernel import hattention_kernel
    return hattention_kernel(q, k, v, None, g, l, scale=None, head_first=False, level_base=2, htype=HType.WEAK,
                             hstruct=HStruct.MAMBA2)


def hattention_sequence_parallel(q, k, v, g, l, group=None, local_op: Optional[Callable] = None) -> torch.Tensor:
    """Output rows of this rank's shard.  q, k (B, T_s, G, K), v (B, T_s, H, V), g (B, T_s, H) fp32,
    l (B, T_s, H, L) with L >= log2(T_s) + log2(world) + 1 columns (the columns of the whole sequence).
    Differentiable; every rank of the group must call it, and call backward, the same number of times.
    `local_op(q, k, v, g, l) -> o` is the unsharded operator (default: the CUDA kernels)."""
    local_op = local_op or _default_local_op
    rank = dist.get_rank(group)
    K, V = q.shape[-1], v.shape[-1]
    o_local = local_op(q, k, v, g, l)
    gc = cumulative_decay(g)
    gathered = _AllGatherSummaries.apply(shard_summary(k, v, g, gc), group)
    cross = shard_cross_output(q, g, l, list(gathered.unbind(0)), rank, K, V, gc)
    if cross is None:
        # a rank that reads nothing still has to take part in the backward collective: keep the gathered
        # tensor in its graph with a zero weight
        return o_local + (gathered.sum() * 0).to(o_local.dtype)
    return o_local + cross.to(o_local.dtype)


def hattention_sequence_parallel_emulated(q, k, v, g, l, shards: int, local_op: Optional[Callable] = None) -> torch.Tensor:
    """The same computation for all shards in one process (no process group): splits the full-length
    inputs into `shards` pieces, runs every shard's part and concatenates.  For tests on one device."""
    local_op = local_op or _default_local_op
    T = g.shape[1]
    if T % shards != 0:
        raise ValueError("the number of shards must divide T")
    Ts = T // shards
    K, V = q.shape[-1], v.shape[-1]
    pieces = [tuple(x[:, r * Ts:(r + 1) * Ts] for x in (q, k, v, g, l)) for r in range(shards)]
    summaries = [shard_summary(p[1], p[2], p[3]) for p in pieces]
    outs = []
    for r, (qs, ks, vs, gs, ls) in enumerate(pieces):
        o_local = local_op(qs.contiguous(), ks.contiguous(), vs.contiguous(), gs.contiguous(), ls.contiguous())
        cross = shard_cross_output(qs, gs, ls, summaries, r, K, V)
        o = o_local if cross is None else o_local + cross.to(o_local.dtype)
        outs.append(o)
    return torch.cat(outs, dim=1)
