"""llattn_mamba2_fwd_static: the forward entry point for callers that cannot allocate device
memory where the operator runs (no cudaMalloc allowed in their serving loop, or no torch / pool to
take a workspace from).  It keeps its segment scratch in a 16 MiB array inside the library.

Checked here, through the C ABI: two calls in a row (different inputs, so the second one runs on
top of the first one's leftovers in the shared array) each reproduce what the regular entry point
with a caller-provided workspace computes, and oversized problems are refused.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B, T, H, G, K, V, L, dev):
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, T, G, K, generator=gen) / K ** 0.5).bfloat16().to(dev)
    k = (torch.randn(B, T, G, K, generator=gen) / K ** 0.5).bfloat16().to(dev)
    v = torch.randn(B, T, H, V, generator=gen).bfloat16().to(dev)
    g = (-torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen) - 2)).float().to(dev)
    l = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen)).bfloat16().to(dev)
    return q, k, v, g, l


def test_static_scratch_forward_matches_workspace_forward_twice():
    from hattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    B, T, H, G, K, V, L = 1, 4096, 4, 1, 128, 64, 13      # 8 segments, 3 high levels -> scratch is used
    need = lib.llattn_mamba2_fwd_workspace_bytes(B, T, H, G, K, V, L)
    assert 0 < need <= lib.llattn_static_scratch_bytes()
    stream = torch.cuda.current_stream().cuda_stream
    for seed in (11, 12):
        q, k, v, g, l = _inputs(seed, B, T, H, G, K, V, L, dev)
        o_ref, gc_ref = torch.empty_like(v), torch.empty_like(g)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        rc = lib.llattn_mamba2_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), l.data_ptr(),
                                   o_ref.data_ptr(), gc_ref.data_ptr(), ws.data_ptr(), ws.numel(),
                                   B, T, H, G, K, V, L, stream)
        assert rc == 0
        o, gc = torch.zeros_like(v), torch.zeros_like(g)
        rc = lib.llattn_mamba2_fwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), l.data_ptr(),
                                          o.data_ptr(), gc.data_ptr(), B, T, H, G, K, V, L, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(o.float()).all()
        assert o_ref.float().abs().max() > 0
        # same kernels, same order of operations: the tolerance of the parity tests is ample
        err = (o.float() - o_ref.float()).abs()
        tol = 2e-2 * o_ref.float().abs() + 2e-3 * max(1.0, o_ref.float().abs().max().item())
        assert (err <= tol).all(), err.max().item()
        assert torch.allclose(gc, gc_ref, rtol=1e-6, atol=1e-7)


def test_static_scratch_rejects_oversized_problems():
    from hattention_b200 import _lib
    lib = _lib.lib()
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(256)      # non-null placeholders: the size check comes before any launch
    B, T, H, G, K, V, L = 2, 16384, 32, 1, 128, 64, 15
    assert lib.llattn_mamba2_fwd_workspace_bytes(B, T, H, G, K, V, L) > lib.llattn_static_scratch_bytes()
    rc = lib.llattn_mamba2_fwd_static(one, one, one, one, one, one, one, B, T, H, G, K, V, L, null)
    assert rc == -7
