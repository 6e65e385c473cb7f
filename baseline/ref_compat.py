"""Import the reference's own Triton implementation (the copy made by baseline/make_ref.py) on the
library versions of this image.  Benchmark infrastructure: only bench.py's reference-Triton
measurement imports this module; the product package never does.

The reference was written against an older flash-linear-attention (`fla`) and pins no version.  The
shims below bridge the drift without touching the reference's kernels:

  1. `fla.ops.utils.op.safe_exp` no longer exists (imported at hattention/chunkwise.py:9,
     chunkwise_hgdn.py:11, fla_future/wy_fast.py:11, fla_future/chunk_scaled_dot_kkt.py:11).  Its
     meaning was exp(x) for x <= 0 and 0 otherwise; the same Triton function is defined here and
     placed into that module before the reference is imported.
  2. `hattention.base.make_levels_matrix` builds its T x T table with a Python double loop unless a
     cache file under a path of the authors' cluster exists (hattention/base.py:22-26, 101-161); for
     T = 16384 that loop would run for hours.  The function is rebound to one that fills the same
     int64 table (levels[t, s] = bit_length(t ^ s) for s <= t, `default` above the diagonal, optional
     clamp) with vectorised torch ops on the requested device; equality with the reference's loop is
     checked for T = 256 in tests/test_reference_compat.py.
The reference's pure-PyTorch forms (`hssd_minimal.py`, `recurrent.py`) import through the same two shims
and run on the CPU; bench.py times them as the reference arm on host cores.
"""
import functools
import importlib
import os
import sys

import torch

REF_ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def levels_matrix_closed_form(length, base, htype, dtype, device, default=-1, clamp_min=None, file_name=None,
                              cached_length=None):
    """Same table as hattention/base.py:101-161 for base 2 and the WEAK hierarchy."""
    if base != 2:
        raise NotImplementedError("closed form is for base 2")
    idx = torch.arange(length, device=device, dtype=torch.int64)
    x = idx[:, None] ^ idx[None, :]
    lev = torch.zeros_like(x)
    nz = x > 0
    # bit_length(x) = floor(log2(x)) + 1, exact in fp64 for x < 2^53
    lev[nz] = torch.floor(torch.log2(x[nz].double())).long() + 1
    lev = torch.where(idx[:, None] >= idx[None, :], lev, torch.full_like(lev, default))
    if clamp_min is not None:
        lev = torch.clamp(lev, min=clamp_min)
    return lev.to(dtype)


def _install_safe_exp():
    import triton
    import triton.language as tl
    import fla.ops.utils.op as op
    if hasattr(op, "safe_exp"):
        return

    @triton.jit
    def safe_exp(x):
        return tl.exp(tl.where(x <= 0, x, float("-inf")))

    op.safe_exp = safe_exp


def load_reference(triton_path: bool = True, torch_forms: bool = False):
    """Returns the reference's modules by name: `base`, plus `chunkwise` (the Triton drivers) and / or
    `hssd_minimal`, `recurrent` (the pure-PyTorch forms).  Raises with the first failing import."""
    if not os.path.isdir(os.path.join(REF_ROOT, "hattention")):
        raise RuntimeError("baseline/_ref/hattention is missing: run `python baseline/make_ref.py <reference checkout>`")
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    for name in [m for m in sys.modules if m == "hattention" or m.startswith("hattention.")]:
        del sys.modules[name]
    _install_safe_exp()
    base = importlib.import_module("hattention.base")
    cached = functools.lru_cache(maxsize=4)(levels_matrix_closed_form)
    base.make_levels_matrix = cached
    out = {"base": base}
    if triton_path:
        chunkwise = importlib.import_module("hattention.chunkwise")
        chunkwise.make_levels_matrix = cached
        out["chunkwise"] = chunkwise
    if torch_forms:
        hm = importlib.import_module("hattention.hssd_minimal")
        hm.make_levels_matrix = cached
        out["hssd_minimal"] = hm
        out["recurrent"] = importlib.import_module("hattention.recurrent")
    return out
