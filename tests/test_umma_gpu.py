"""tcgen05 building blocks: shared-memory descriptors for the three operand-layout combinations,
the swizzled tile layout and the tensor-memory readback, checked against torch matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 10, 11, 12])
@pytest.mark.parametrize("N,kred", [(128, 128), (64, 128), (128, 64), (64, 64)])
def test_umma_tile_product(mode, N, kred):
    from hattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(mode * 10 + N + kred)
    issue_mode, mode = mode, mode % 10        # 10..12: the compile-time shaped issue loops of the kernels
    a_shape = (kred, 128) if mode == 2 else (128, kred)
    b_shape = (N, kred) if mode == 0 else (kred, N)
    A = torch.randn(a_shape, generator=gen).bfloat16().to(dev)
    B = torch.randn(b_shape, generator=gen).bfloat16().to(dev)
    D = torch.zeros(128, N, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.llattn_selftest_umma(A.data_ptr(), B.data_ptr(), D.data_ptr(), N, kred, issue_mode, err.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert err.item() == 0, "tensor core completion was not signalled"
    Af, Bf = A.float(), B.float()
    want = Af @ Bf.T if mode == 0 else (Af @ Bf if mode == 1 else Af.T @ Bf)
    assert torch.allclose(D, want, rtol=1e-3, atol=1e-2), (D - want).abs().max().item()


@pytest.mark.parametrize("mode,N,kred,bound", [
    (0, 128, 128, 72.0),    # K-major x K-major, N = 128: tensor-core bound, 64 cycles per K = 16 step
    (2, 128, 128, 72.0),    # MN-major x MN-major, N = 128
    (1, 64, 128, 64.0),     # N = 64: about 54 cycles per step (32 would be the arithmetic bound)
    (2, 64, 128, 64.0),
    (3, 32, 128, 64.0),     # Gated DeltaNet scans: one level (N = 32) from the 256-row transposed state tile
    (3, 64, 128, 64.0),     # two and four adjacent levels in one chain
    (3, 128, 128, 72.0),
    (4, 32, 64, 64.0),      # MN-major A (kd^T / qd^T), 64-token reduction
    (4, 96, 64, 64.0),
])
def test_mma_issue_rate(mode, N, kred, bound):
    """Cycles per tcgen05.mma (M = 128, K = 16) of the compile-time shaped issue loops that the kernels use,
    from back-to-back products with resident operands (difference between 64 and 8 repetitions, so the
    fixed issue-to-completion latency cancels).  Prints the figure; run with -s to see it."""
    from hattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    total = {}
    for reps in (8, 64):
        best = None
        for _ in range(3):
            rc = lib.llattn_selftest_umma_cycles(N, kred, mode, reps, 1, cyc.data_ptr(), err.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert err.item() == 0
            best = cyc.item() if best is None else min(best, cyc.item())
        total[reps] = best
    per_step = (total[64] - total[8]) / ((64 - 8) * (kred // 16))
    print(f"mode {mode} N={N} kred={kred}: {per_step:.1f} cycles per K=16 step; 8 repetitions take {total[8]} cycles")
    assert per_step <= bound


def test_wait_that_runs_out_sets_the_status_word():
    """A bounded wait that nothing completes: the kernel gives up after its poll limit, sets the status word and
    returns; the host reads the word through the C ABI and the context stays usable."""
    import ctypes
    from hattention_b200 import _lib
    DEV = torch.device("cuda:0")
    lib = _lib.lib()
    ws = torch.zeros(64, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    out = ctypes.c_int(-1)
    assert lib.llattn_workspace_status(ws.data_ptr(), ctypes.byref(out), stream) == 0 and out.value == 0
    before = lib.llattn_kernel_launches()
    assert lib.llattn_selftest_wait_timeout(2000, ws.data_ptr(), stream) == 0
    assert lib.llattn_kernel_launches() == before + 1
    assert lib.llattn_workspace_status(ws.data_ptr(), ctypes.byref(out), stream) == 0
    assert out.value == 1
    with pytest.raises(RuntimeError):
        _lib.raise_on_status(ws, stream, "self-test")
    # the device still answers
    assert torch.ones(4, device=DEV).sum().item() == 4.0


def test_phase_clock_stamps_of_one_pair():
    """Only in a library built with `make -C log-linear-attention_b200/csrc clean all EXTRA=-DLLATTN_STAMPS`: prints the
    clock64() stamps that three threads of one CTA take at fixed points of one chunk pair of the forward and the
    forward-order / reverse-order backward kernels (run with -s).  Skipped for the normal build."""
    import ctypes
    from hattention_b200 import _lib
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import chunkwise_bwd, chunkwise_fwd
    from oracle import loglinear_oracle as orc
    lib = _lib.lib()
    if not hasattr(lib, "llattn_debug_read_stamps"):
        pytest.skip("library built without -DLLATTN_STAMPS")
    dev = torch.device("cuda:0")
    q, k, v, g, l = orc.make_mamba2_inputs(1, 16384, 32, 64, 128, 1, 15, seed=0)
    q, k, v, l = (x.bfloat16().to(dev) for x in (q, k, v, l))
    g = g.float().to(dev)
    do = torch.randn_like(v)
    for _ in range(3):
        kept = []
        o, gc, _ = chunkwise_fwd(q, k, v, g, l, False, 2, HType.WEAK, 64, False, keep_workspace=kept)
        chunkwise_bwd(q, k, v, gc, l, do, False, 2, HType.WEAK, 64, fwd_workspace=kept[0])
    torch.cuda.synchronize()
    if hasattr(lib, "llattn_debug_read_stamps_seg"):
        # one CTA of the high-level backward kernel: entry, before / after the segment's cumulative decay, top of each pair,
        # end of the pairs, reader summaries written, reduce-adds complete, exit
        buf = (ctypes.c_longlong * 96)()
        f = lib.llattn_debug_read_stamps_seg
        f.argtypes = [ctypes.c_void_p]
        assert f(buf) == 0
        d = list(buf)[:16]
        print("high-level backward, one CTA", [x - d[0] if x else None for x in d])
    for name, fn in (("forward", "llattn_debug_read_stamps"), ("backward", "llattn_debug_read_stamps_bwd")):
        buf = (ctypes.c_longlong * 96)()
        f = getattr(lib, fn)
        f.argtypes = [ctypes.c_void_p]
        assert f(buf) == 0
        d = list(buf)
        for half, lo in (("forward-order / forward pass", 0), ("reverse-order pass", 16)):
            if not d[lo]:
                continue
            for s_, who in enumerate(("thread 0", "thread 200", "thread 96")):
                row = d[32 * s_ + lo: 32 * s_ + lo + 16]
                print(name, half, who, [x - d[lo] if x else None for x in row])


def test_phase_clock_stamps_of_one_gdn_scan_chunk():
    """Only in a library built with `make -C log-linear-attention_b200/csrc clean all EXTRA=-DLLATTN_STAMPS`: prints the
    clock64() stamps of one chunk (chunk 37 of CTA 5) of the Gated DeltaNet forward scan: an output thread, a staging
    thread and the MMA-issuing thread (run with -s).  Skipped for the normal build."""
    import ctypes
    from hattention_b200 import _lib
    from hattention_b200 import chunkwise_hgdn as hg
    from hattention_b200.base import HType
    from oracle import loglinear_oracle as orc
    lib = _lib.lib()
    if not hasattr(lib, "llattn_debug_read_stamps_gdn"):
        pytest.skip("library built without -DLLATTN_STAMPS")
    dev = torch.device("cuda:0")
    B, T, H, Dk, Dv, L = 4, 8192, 16, 128, 128, 14
    q, k, v, b, g, l = orc.make_gdn_inputs(B, T, H, Dk, Dv, L, seed=3)
    qn, kn = orc.gdn_layer_inputs(q, k, Dk ** -0.5)
    qn, kn, v, b, l = (x.bfloat16().to(dev) for x in (qn, kn, v, b, l))
    g = g.float().to(dev)
    for _ in range(3):
        hg.chunkwise_fwd(qn, kn, v, b, g, l, False, 2, HType.WEAK, 64, False)
    torch.cuda.synchronize()
    buf = (ctypes.c_longlong * 96)()
    f = lib.llattn_debug_read_stamps_gdn
    f.argtypes = [ctypes.c_void_p]
    assert f(buf) == 0
    d = list(buf)
    t0 = min(x for x in d if x)
    for s_, who in enumerate(("output thread 0", "staging thread 64", "MMA thread")):
        print(who, [x - t0 if x else None for x in d[32 * s_: 32 * s_ + 16]])
    # the chunk preparation kernel of the same forward: item 3 of CTA 5, threads 0 (lanes 0..63) and 64 (lanes 64..127);
    # the second half of each row holds the stamps inside the triangular inverses
    f = lib.llattn_debug_read_stamps_gdn_prep
    f.argtypes = [ctypes.c_void_p]
    assert f(buf) == 0
    d = list(buf)
    t0 = min(x for x in d if x)
    for s_, who in enumerate(("preparation, thread 0", "preparation, thread 64")):
        print(who, [x - t0 if x else None for x in d[32 * s_: 32 * s_ + 32]])


def test_phase_clock_stamps_of_the_gdn_backward_kernels():
    """Only in a library built with -DLLATTN_STAMPS (see above; LLATTN_LIB can name such a build): prints the clock64() stamps
    of one item of the level-gradient kernel (item 8 of CTA 5: per step, top / first batch complete / operands written for
    the element-wise threads 0 and 64, top / next first batch issued / operands ready / second batch issued for the MMA
    thread, then the stages of the result write-out) and of one CTA of the chunk-local gradient kernel (lane 0 of warps 0,
    7 and 2 after each barrier and between the products of the longer stages).  Run with -s."""
    import ctypes
    from hattention_b200 import _lib
    from hattention_b200.gated_delta_rule_apis import chunk_h_gated_delta_rule
    lib = _lib.lib()
    if not hasattr(lib, "llattn_debug_read_stamps_gdn_levels"):
        pytest.skip("library built without -DLLATTN_STAMPS")
    dev = torch.device("cuda:0")
    B, T, H, Dk, Dv, L = 4, 8192, 16, 128, 128, 14
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(B, T, H, Dk, generator=gen).bfloat16().to(dev)
    k = torch.randn(B, T, H, Dk, generator=gen).bfloat16().to(dev)
    v = torch.randn(B, T, H, Dv, generator=gen).bfloat16().to(dev)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen)).bfloat16().to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen) + 3.0).float().to(dev)
    lam = torch.nn.functional.softplus(torch.randn(B, T, H, L, generator=gen)).bfloat16().to(dev)
    do = torch.randn(B, T, H, Dv, generator=gen).bfloat16().to(dev)
    ins = [x.clone().requires_grad_(True) for x in (q, k, v, g, lam, beta)]
    for _ in range(3):
        o = chunk_h_gated_delta_rule(*ins, use_qk_l2norm_in_kernel=True)[0]
        torch.autograd.grad(o, ins, do)
    torch.cuda.synchronize()
    for fn, names in (("llattn_debug_read_stamps_gdn_levels", ("levels, thread 0 (q rows)", "levels, thread 64 (w rows)", "levels, MMA thread")),
                      ("llattn_debug_read_stamps_gdn_chunk", ("chunk-local, warp 0", "chunk-local, warp 7", "chunk-local, warp 2"))):
        buf = (ctypes.c_longlong * 96)()
        f = getattr(lib, fn)
        f.argtypes = [ctypes.c_void_p]
        assert f(buf) == 0
        d = list(buf)
        t0 = min(x for x in d if x)
        for s_, who in enumerate(names):
            print(who, [x - t0 if x else None for x in d[32 * s_: 32 * s_ + 32]])


def test_elementwise_phase_cycles():
    """Cycles of one element-wise phase in isolation (the fp32 block product of the triangular inverses: 256 threads, 72
    16-byte shared-memory loads and 256 FMAs per thread, one 256-thread barrier) as a function of the instruction footprint of
    the loop body around it (1 or 64 separate copies of the phase's code: 4 KB to 150 KB) and of features of the production
    kernels' environment (large dynamic shared memory, tensor memory held, a thread polling an mbarrier).  Prints the figures
    (run with -s).  Measured: 2.31 k cycles in every variant, the same as inside the preparation kernel: the phase is bound by
    shared-memory transactions (a 16-byte load costs four cycles per warp whatever the address pattern: 8 warps x 72 loads x
    4 = 2304), not by instruction fetch, polling warps or the allocation sizes."""
    import ctypes
    from hattention_b200 import _lib
    lib = _lib.lib()
    lib.llattn_selftest_ew_cycles.restype = ctypes.c_int
    lib.llattn_selftest_ew_cycles.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 3
    dev = torch.device("cuda:0")
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    sink = torch.zeros(384, dtype=torch.float32, device=dev)
    for spin, copies, env in ((0, 1, 0), (4, 1, 0), (0, 64, 0), (0, 1, 1), (0, 1, 2), (1, 1, 4), (2, 64, 7)):
        res = {}
        for reps in (4, 36):
            best = None
            for _ in range(3):
                assert lib.llattn_selftest_ew_cycles(reps, spin, copies, env, cyc.data_ptr(), sink.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream) == 0
                torch.cuda.synchronize()
                best = cyc.item() if best is None else min(best, cyc.item())
            res[reps] = best
        per = (res[36] - res[4]) / (32 * copies)
        print(f"polling warps {spin}, {copies:2d} copies of the code, environment bits {env}: {per:.0f} cycles per phase")
        assert 0 < per < 4000
