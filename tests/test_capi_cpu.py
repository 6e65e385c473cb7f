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
    assert lib.llattn_version() >= 1
    assert lib.llattn_chunk() == 64


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
