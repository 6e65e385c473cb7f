"""B200 (sm_100a) implementation of hattention's chunkwise log-linear attention.

Mirrors the module layout of the reference package for the one path it replaces:
`base` (level arithmetic, enums), `chunkwise` (Mamba-2 drivers), `chunkwise_hgdn` (Gated DeltaNet
drivers, l2norm), `kernel` (autograd boundary, prefill / decode step), `mamba_apis` and
`gated_delta_rule_apis` (layer-level APIs), `recurrent` (decode state), `sharding` (batch x head partition across GPUs).  The CUDA
kernels live in libllattn.so (C ABI, built from ../csrc) and are reached through ctypes; there is no CPU
or Triton fallback.
"""
from .base import HType, HStruct, get_num_levels  # noqa: F401
from .kernel import HState, hattention_kernel, hattention_prefill, hattention_step  # noqa: F401


def install_as_hattention():
    """Register this package's modules under the reference's names (`hattention.kernel`, ...)
    so that code written against the reference imports them unchanged."""
    import importlib
    import sys
    import types

    pkg = sys.modules.get("hattention")
    if pkg is None:
        pkg = types.ModuleType("hattention")
        pkg.__path__ = []
        sys.modules["hattention"] = pkg
    for name in ("base", "recurrent", "chunkwise", "kernel", "mamba_apis", "chunkwise_hgdn", "gated_delta_rule_apis"):
        try:
            mod = importlib.import_module(f"{__name__}.{name}")
        except ImportError:
            continue
        sys.modules[f"hattention.{name}"] = mod
        setattr(pkg, name, mod)
    return pkg
