"""CPU-side checks of the C ABI: the library loads, exports every symbol that include/llattn.h
declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from hattention_b200 import _lib
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "llattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llattn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert "llattn_mamba2_fwd" in names and "llattn_mamba2_bwd" in names
    for n in names:
        assert hasattr(lib, n), n


def test_version_and_chunk(lib):
    assert lib.llattn_version() >= 2
    assert lib.llattn_chunk() == 64
    assert lib.llattn_kernel_launches() >= 0


def test_static_scratch_capacity_stated_in_the_header(lib):
    """include/llattn.h and INTEGRATION.md say: 1.125 MiB per (batch, head) at T = 4096, K = 128, V = 64, so the
    16 MiB array serves B*H <= 14 there."""
    cap = lib.llattn_static_scratch_bytes()
    assert cap == 16 << 20
    need = lambda bh: lib.llattn_mamba2_fwd_workspace_bytes(1, 4096, bh, 1, 128, 64, 13)
    assert abs((need(2) - need(1)) / 2 ** 20 - 1.125) < 1e-3
    assert need(14) <= cap < need(15)
    null = ctypes.c_void_p(0)
    # a size beyond the array is refused before anything touches a device or a pointer; so is a missing pointer
    dummy = ctypes.c_void_p(256)
    assert lib.llattn_mamba2_fwd_static(*([dummy] * 7), 1, 4096, 15, 1, 128, 64, 13, null) == -7
    assert lib.llattn_mamba2_fwd_static(*([null] * 7), 1, 4096, 14, 1, 128, 64, 13, null) == -6


def test_longest_supported_sequence(lib):
    """The scans over segments hold ten segment levels: T = 512 * 1024 is the longest sequence; longer ones are
    refused instead of reading levels that were never written."""
    assert lib.llattn_mamba2_fwd_workspace_bytes(1, 524288, 1, 1, 128, 64, 20) > 0
    assert lib.llattn_mamba2_fwd_workspace_bytes(1, 524288 + 512, 1, 1, 128, 64, 21) == 0
    null = ctypes.c_void_p(0)
    assert lib.llattn_mamba2_fwd(*([null] * 8), 0, 1, 1048576, 1, 1, 128, 64, 21, null) == -1


def test_bf16_only(lib):
    """fp32 q / k / v never reach a kernel: the Python driver refuses them (no fp32 mode; no CPU path either)."""
    import torch
    from hattention_b200.base import HType
    from hattention_b200.chunkwise import _check
    q = torch.zeros(1, 64, 1, 128)
    v = torch.zeros(1, 64, 2, 64)
    g = torch.zeros(1, 64, 2)
    l = torch.zeros(1, 64, 2, 7)
    with pytest.raises((NotImplementedError, RuntimeError)):
        _check(q, q, v, g, l, False, 2, HType.WEAK, 64)


def test_workspace_sizes(lib):
    # one segment (T <= 512): only the 256-byte status word
    assert lib.llattn_mamba2_fwd_workspace_bytes(1, 512, 2, 1, 128, 64, 10) == 256
    small = lib.llattn_mamba2_fwd_workspace_bytes(1, 1024, 2, 1, 128, 64, 11)
    big = lib.llattn_mamba2_fwd_workspace_bytes(2, 16384, 32, 1, 128, 64, 15)
    assert 0 < small < big
    assert lib.llattn_mamba2_bwd_workspace_bytes(2, 16384, 32, 1, 128, 64, 15) > big
    # rejected shapes size to zero
    assert lib.llattn_mamba2_fwd_workspace_bytes(1, 100, 2, 1, 128, 64, 10) == 0


@pytest.mark.parametrize("shape,code", [
    ((1, 100, 2, 1, 128, 64, 10), -2),     # T % 64
    ((1, 1024, 3, 2, 128, 64, 12), -4),    # H % G
    ((1, 1024, 2, 1, 96, 64, 12), -1),     # K
    ((1, 1024, 2, 1, 128, 32, 12), -1),    # V
    ((1, 1024, 2, 1, 128, 64, 10), -3),    # L < 7 + log2(16)
    ((1, 1024, 2, 1, 128, 64, 40), -1),    # L > 32
])
def test_bad_arguments_are_rejected_without_a_device(lib, shape, code):
    null = ctypes.c_void_p(0)
    rc = lib.llattn_mamba2_fwd(null, null, null, null, null, null, null, null, 0, *shape, null)
    assert rc == code
    rc = lib.llattn_mamba2_bwd(*([null] * 11), null, 0, *shape, null)
    assert rc == code


def test_null_pointers_are_rejected(lib):
    null = ctypes.c_void_p(0)
    assert lib.llattn_mamba2_fwd(null, null, null, null, null, null, null, null, 0, 1, 512, 2, 1, 128, 64, 10, null) == -6


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from hattention_b200 import HStruct, HType, hattention_kernel
    q = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16)
    v = torch.zeros(1, 64, 2, 64, dtype=torch.bfloat16)
    g = torch.zeros(1, 64, 2)
    l = torch.zeros(1, 64, 2, 7, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        hattention_kernel(q, q, v, None, g, l, None, False, 2, HType.WEAK, HStruct.MAMBA2)
    with pytest.raises(NotImplementedError):
        hattention_kernel(q, q, v, None, g, l, None, True, 2, HType.WEAK, HStruct.MAMBA2)
    with pytest.raises(ValueError):
        hattention_kernel(q, q, v, g, g, l, None, False, 2, HType.WEAK, HStruct.MAMBA2)


def test_gdn_entry_points_reject_bad_arguments(lib):
    null = ctypes.c_void_p(0)
    # K must be 128, V 64 or 128, at most eight inter-chunk levels
    assert lib.llattn_gdn_fwd_workspace_bytes(1, 1024, 2, 96, 64, 12) == 0
    assert lib.llattn_gdn_fwd_workspace_bytes(1, 1024, 2, 128, 256, 12) == 0
    assert lib.llattn_gdn_fwd_workspace_bytes(1, 32768, 2, 128, 64, 16) == 0
    fwd = lib.llattn_gdn_fwd_workspace_bytes(1, 1024, 2, 128, 128, 11)
    lev = lib.llattn_gdn_bwd_levels_workspace_bytes(1, 1024, 2, 128, 128, 11)
    bwd = lib.llattn_gdn_bwd_workspace_bytes(1, 1024, 2, 128, 128, 11)
    assert 0 < fwd < lev < bwd
    assert lib.llattn_gdn_fwd(*([null] * 10), null, 0, 1, 1000, 2, 128, 64, 11, null) == -2
    assert lib.llattn_gdn_fwd(*([null] * 10), null, 0, 1, 1024, 2, 128, 64, 10, null) == -3
    assert lib.llattn_gdn_fwd(*([null] * 10), null, 0, 1, 1024, 2, 128, 64, 11, null) == -6
    assert lib.llattn_gdn_bwd(*([null] * 15), null, 0, 1, 1024, 2, 64, 64, 11, null) == -1
    assert lib.llattn_gdn_bwd(*([null] * 15), null, 0, 1, 1024, 2, 128, 64, 11, null) == -6
    assert lib.llattn_gdn_bwd_levels(*([null] * 15), null, 0, 1, 1024, 2, 128, 64, 11, null) == -6
    # forward that keeps its intermediates / backward that reads them
    keep = lib.llattn_gdn_fwd_keep_workspace_bytes(1, 1024, 2, 128, 128, 11)
    bkept = lib.llattn_gdn_bwd_kept_workspace_bytes(1, 1024, 2, 128, 128, 11)
    assert keep > fwd and 0 < bkept < bwd and keep + bkept >= bwd
    assert lib.llattn_gdn_fwd_keep_workspace_bytes(1, 1024, 2, 96, 64, 12) == 0
    assert lib.llattn_gdn_fwd_keep(*([null] * 10), null, 0, 1, 1024, 2, 128, 64, 11, null) == -6
    assert lib.llattn_gdn_bwd_kept(*([null] * 15), null, 0, null, 0, 1, 1024, 2, 128, 64, 11, null) == -6
    assert lib.llattn_gdn_bwd_kept_bf16dv(*([null] * 15), null, 0, null, 0, 1, 1024, 2, 128, 64, 11, null) == -6


def test_elementwise_entry_points_reject_bad_arguments(lib):
    null = ctypes.c_void_p(0)
    assert lib.llattn_l2norm_fwd(null, null, 10, 128, 1.0, null) == -6
    assert lib.llattn_l2norm_fwd(null, null, 10, 100, 1.0, null) == -1          # D % 8
    assert lib.llattn_l2norm_bwd(null, null, null, 10, 512, 1.0, null) == -1     # D > 256
    assert lib.llattn_mamba2_prep_fwd(*([null] * 9), 64, 2, 64, 12, 7, null) == -1     # lambda mode
    assert lib.llattn_mamba2_prep_fwd(*([null] * 9), 63, 2, 64, 12, 0, null) == -1     # rows % H
    assert lib.llattn_mamba2_prep_fwd(*([null] * 9), 64, 2, 64, 12, 0, null) == -6
    assert lib.llattn_mamba2_prep_bwd(*([null] * 18), 64, 2, 60, 12, 0, null) == -1    # P % 8
    assert lib.llattn_mamba2_residual(null, null, null, null, 0, 64, 2, 64, null) == -6


def test_prefill_and_step_entry_points_reject_bad_arguments(lib):
    null = ctypes.c_void_p(0)
    assert lib.llattn_mamba2_final_state(null, null, null, null, 1, 1000, 2, 1, 128, 64, 8, null) == -3    # 1000 tokens need 11 levels
    assert lib.llattn_mamba2_final_state(null, null, null, null, 1, 1000, 2, 1, 128, 64, 11, null) == -6
    assert lib.llattn_mamba2_final_state(null, null, null, null, 1, 1000, 3, 2, 128, 64, 11, null) == -1
    assert lib.llattn_mamba2_step(*([null] * 7), 1, 2, 1, 128, 64, 11, 11, null) == -3                    # carry level out of range
    assert lib.llattn_mamba2_step(*([null] * 7), 1, 2, 1, 128, 48, 11, 0, null) == -1                     # 256 % V
    assert lib.llattn_mamba2_step(*([null] * 7), 1, 2, 1, 128, 64, 11, 0, null) == -6


def test_decode_state_counts_follow_the_cascade():
    """Host-side token counts of the decode state: after T tokens they are the binary decomposition of
    T - 1 plus the newest token, whether reached by stepping the cascade or set directly."""
    import torch
    from hattention_b200 import HState, HStruct, HType
    for T in (1, 2, 3, 64, 65, 200, 255, 256, 1000):
        hs = HState(2, HType.WEAK, HStruct.MAMBA2, (1, 1, 1, 1, 12), torch.float32, torch.device("cpu"))
        for _ in range(T):
            hs.cascade_counts()
            hs.counts[0] += 1
        ref = HState(2, HType.WEAK, HStruct.MAMBA2, (1, 1, 1, 1, 12), torch.float32, torch.device("cpu"))
        ref.set_counts_after(T)
        assert hs.counts == ref.counts, T
        assert sum(hs.counts) == T
