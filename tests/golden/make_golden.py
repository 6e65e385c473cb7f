"""Generate the golden fixtures in this directory by running the REFERENCE project's own
PyTorch implementations on seeded inputs.

Usage (needs a checkout of zian1117/log-linear-attention; CPU only):

    python tests/golden/make_golden.py /path/to/log-linear-attention

The reference package is imported without executing its __init__ (which needs mamba_ssm and
causal_conv1d): an empty package object is registered for `hattention` and the three pure
PyTorch modules are imported by name.  `make_levels_matrix` is rebound so that it builds the
level table for the requested length instead of a 16384^2 table in a Python double loop.

Fixtures written (float32 .npz; inputs are rounded through bfloat16 first for the *_c64 cases
so that a bf16 kernel sees exactly the same numbers):

    mamba2_c1.npz   B=1,T=256,H=2,P=16,N=16,G=1,L=9, chunk 16 : hssd_minimal_discrete,
                    hattention_recurrent, hattention_materialized, autograd grads
    mamba2_c64.npz  B=1,T=512,H=2,P=64,N=64,G=1,L=10, chunk 64 : same functions
    gdn_c1.npz      B=1,T=128,H=2,Dk=Dv=16,L=8, chunk 16 : hgdn_minimal, hattention_recurrent
                    (GDELTA), autograd grads through hgdn_minimal
    gdn_c64.npz     B=1,T=256,H=2,Dk=128,Dv=64,L=9, chunk 64 : same
    levels.npz      make_levels_matrix(256) and get_num_levels for several lengths
"""
import importlib
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import loglinear_oracle as orc  # input generators only


def import_reference(root):
    pkg = types.ModuleType("hattention")
    pkg.__path__ = [os.path.join(root, "hattention")]
    sys.modules["hattention"] = pkg
    base = importlib.import_module("hattention.base")
    rec = importlib.import_module("hattention.recurrent")
    hm = importlib.import_module("hattention.hssd_minimal")
    orig = base.make_levels_matrix

    def uncached(length, base, htype, dtype, device, default=-1, clamp_min=None, file_name=None, cached_length=None):
        return orig(length=length, base=base, htype=htype, dtype=dtype, device=device, default=default,
                    clamp_min=clamp_min, file_name=file_name, cached_length=None)

    base.make_levels_matrix = uncached
    hm.make_levels_matrix = uncached
    return base, rec, hm


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


def mamba2_case(base, rec, hm, name, B, T, H, P, N, G, L, chunk, round_bf16):
    q, k, v, g, l = orc.make_mamba2_inputs(B, T, H, P, N, G, L, seed=0)
    if round_bf16:
        q, k, v, l = map(bf16_round, (q, k, v, l))
    gen = torch.Generator().manual_seed(1)
    do = torch.randn(B, T, H, P, generator=gen)
    if round_bf16:
        do = bf16_round(do)
    W = base.HType.WEAK
    rep = H // G
    qh, kh = q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2)
    with torch.no_grad():
        o_rec, st = rec.hattention_recurrent(qh, kh, v, torch.exp(g), None, l, 2, W, base.HStruct.MAMBA2)
        o_mat, _ = base.hattention_materialized(qh, kh, v, torch.exp(g), l, 2, W)
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, l)]
    o_chk = hm.hssd_minimal_discrete(ins[2], ins[3], ins[1].repeat_interleave(rep, 2), ins[0].repeat_interleave(rep, 2),
                                     ins[4], 2, W, chunk)
    grads = torch.autograd.grad((o_chk * do).sum(), ins)
    np.savez_compressed(
        os.path.join(HERE, name), q=q, k=k, v=v, g=g, l=l, do=do,
        o_chunk=o_chk.detach(), o_recurrent=o_rec, o_materialized=o_mat,
        counts=st.counts.numpy(), dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dl=grads[4],
        chunk=np.int64(chunk))
    print(name, "max|chunk-rec|", (o_chk.detach() - o_rec).abs().max().item(),
          "max|chunk-mat|", (o_chk.detach() - o_mat).abs().max().item())


def gdn_case(base, rec, hm, name, B, T, H, Dk, Dv, L, chunk, round_bf16):
    q, k, v, beta, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=0)
    if round_bf16:
        q, k, v, beta, l = map(bf16_round, (q, k, v, beta, l))
    gen = torch.Generator().manual_seed(1)
    do = torch.randn(B, T, H, Dv, generator=gen)
    if round_bf16:
        do = bf16_round(do)
    scale = Dk ** -0.5
    W = base.HType.WEAK
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, beta, g, l)]
    # preparation of the layer API and the autograd boundary (gated_delta_rule_apis.py:65-70,
    # kernel.py:110-111): lambda / scale, q <- l2norm(q) * scale, k <- l2norm(k)
    qn = ins[0] * torch.rsqrt((ins[0] ** 2).sum(-1, keepdim=True) + 1e-6) * scale
    kn = ins[1] * torch.rsqrt((ins[1] ** 2).sum(-1, keepdim=True) + 1e-6)
    ls = ins[5] / scale
    o_chk = hm.hgdn_minimal(qn, kn, ins[2], ins[3], ins[4], ls, 2, W, chunk)
    grads = torch.autograd.grad((o_chk * do).sum(), ins)
    with torch.no_grad():
        o_rec, st = rec.hattention_recurrent(qn.detach(), kn.detach(), v, torch.exp(g), beta, ls.detach(), 2, W,
                                             base.HStruct.GDELTA)
    np.savez_compressed(
        os.path.join(HERE, name), q=q, k=k, v=v, b=beta, g=g, l=l, do=do, scale=np.float64(scale),
        o_chunk=o_chk.detach(), o_recurrent=o_rec, counts=st.counts.numpy(),
        dq=grads[0], dk=grads[1], dv=grads[2], db=grads[3], dg=grads[4], dl=grads[5], chunk=np.int64(chunk))
    print(name, "max|chunk-rec|", (o_chk.detach() - o_rec).abs().max().item())


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/log-linear-attention")
    root = sys.argv[1]
    base, rec, hm = import_reference(root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    W = base.HType.WEAK
    lev = base.make_levels_matrix(256, 2, W, torch.int64, torch.device("cpu"))
    lengths = np.array([1, 2, 3, 16, 64, 65, 256, 4096, 8192, 16384, 65536], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "levels.npz"), levels256=lev.numpy(), lengths=lengths,
                        num_levels=np.array([base.get_num_levels(int(x), 2) for x in lengths], dtype=np.int64))
    mamba2_case(base, rec, hm, "mamba2_c1.npz", 1, 256, 2, 16, 16, 1, 9, 16, False)
    mamba2_case(base, rec, hm, "mamba2_c64.npz", 1, 512, 2, 64, 64, 1, 10, 64, True)
    gdn_case(base, rec, hm, "gdn_c1.npz", 1, 128, 2, 16, 16, 8, 16, False)
    gdn_case(base, rec, hm, "gdn_c64.npz", 1, 256, 2, 128, 64, 9, 64, True)


if __name__ == "__main__":
    main()
