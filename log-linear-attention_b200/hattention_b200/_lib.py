"""ctypes binding of libllattn.so (declared in include/llattn.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# LLATTN_LIB names another build of the same library (for instance one compiled with -DLLATTN_STAMPS for the clock-stamp tests)
_LIB_PATH = os.environ.get("LLATTN_LIB") or os.path.join(_HERE, "libllattn.so")
_lib = None

ERRORS = {
    -1: "unsupported shape (K must be 64 or 128, V must be 64, L <= 32)",
    -2: "sequence length is not a multiple of the 64-token chunk",
    -3: "too few lambda levels for this sequence length",
    -4: "number of heads is not a multiple of the number of q/k groups",
    -5: "workspace missing, misaligned or too small",
    -6: "null pointer",
    -7: "problem needs more scratch than the built-in static array holds",
    -8: "the driver refused a TMA tensor map for these pointers",
}

_SHAPE = [ctypes.c_int] * 7
_P = ctypes.c_void_p


def lib():
    """Load the shared library once.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} not found: build it with `make -C log-linear-attention_b200/csrc` "
            "(or __graft_entry__.build()); this package has no CPU or Triton fallback")
    L = ctypes.CDLL(_LIB_PATH)
    L.llattn_version.restype = ctypes.c_int
    L.llattn_chunk.restype = ctypes.c_int
    L.llattn_mamba2_fwd_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_mamba2_fwd_workspace_bytes.argtypes = _SHAPE
    L.llattn_mamba2_bwd_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_mamba2_bwd_workspace_bytes.argtypes = _SHAPE
    L.llattn_mamba2_fwd.restype = ctypes.c_int
    L.llattn_mamba2_fwd.argtypes = [_P] * 7 + [_P, ctypes.c_size_t] + _SHAPE + [_P]
    L.llattn_static_scratch_bytes.restype = ctypes.c_size_t
    L.llattn_mamba2_fwd_static.restype = ctypes.c_int
    L.llattn_mamba2_fwd_static.argtypes = [_P] * 7 + _SHAPE + [_P]
    L.llattn_mamba2_bwd.restype = ctypes.c_int
    L.llattn_mamba2_bwd.argtypes = [_P] * 11 + [_P, ctypes.c_size_t] + _SHAPE + [_P]
    L.llattn_mamba2_bwd_saved.restype = ctypes.c_int
    L.llattn_mamba2_bwd_saved.argtypes = [_P] * 11 + [_P, ctypes.c_size_t, _P, ctypes.c_size_t] + _SHAPE + [_P]
    L.llattn_gdn_fwd_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_gdn_fwd_workspace_bytes.argtypes = [ctypes.c_int] * 6
    L.llattn_gdn_fwd.restype = ctypes.c_int
    L.llattn_gdn_fwd.argtypes = [_P] * 10 + [_P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_gdn_bwd_levels_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_gdn_bwd_levels_workspace_bytes.argtypes = [ctypes.c_int] * 6
    L.llattn_gdn_bwd_levels.restype = ctypes.c_int
    L.llattn_gdn_bwd_levels.argtypes = [_P] * 15 + [_P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_mamba2_prep_fwd.restype = ctypes.c_int
    L.llattn_mamba2_prep_fwd.argtypes = [_P] * 9 + [ctypes.c_long] + [ctypes.c_int] * 4 + [_P]
    L.llattn_mamba2_prep_bwd.restype = ctypes.c_int
    L.llattn_mamba2_prep_bwd.argtypes = [_P] * 18 + [ctypes.c_long] + [ctypes.c_int] * 4 + [_P]
    L.llattn_mamba2_residual.restype = ctypes.c_int
    L.llattn_mamba2_residual.argtypes = [_P] * 4 + [ctypes.c_int, ctypes.c_long, ctypes.c_int, ctypes.c_int, _P]
    L.llattn_mamba2_final_state.restype = ctypes.c_int
    L.llattn_mamba2_final_state.argtypes = [_P] * 4 + [ctypes.c_int] * 7 + [_P]
    L.llattn_mamba2_step.restype = ctypes.c_int
    L.llattn_mamba2_step.argtypes = [_P] * 7 + [ctypes.c_int] * 7 + [_P]
    L.llattn_gdn_prefill.restype = ctypes.c_int
    L.llattn_gdn_prefill.argtypes = [_P] * 11 + [_P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_gdn_step.restype = ctypes.c_int
    L.llattn_gdn_step.argtypes = [_P] * 8 + [ctypes.c_int] * 6 + [_P]
    L.llattn_l2norm_fwd.restype = ctypes.c_int
    L.llattn_l2norm_fwd.argtypes = [_P, _P, ctypes.c_long, ctypes.c_int, ctypes.c_float, _P]
    L.llattn_l2norm_bwd.restype = ctypes.c_int
    L.llattn_l2norm_bwd.argtypes = [_P, _P, _P, ctypes.c_long, ctypes.c_int, ctypes.c_float, _P]
    L.llattn_gdn_bwd_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_gdn_bwd_workspace_bytes.argtypes = [ctypes.c_int] * 6
    L.llattn_gdn_bwd.restype = ctypes.c_int
    L.llattn_gdn_bwd.argtypes = [_P] * 15 + [_P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_gdn_fwd_keep_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_gdn_fwd_keep_workspace_bytes.argtypes = [ctypes.c_int] * 6
    L.llattn_gdn_fwd_keep.restype = ctypes.c_int
    L.llattn_gdn_fwd_keep.argtypes = [_P] * 10 + [_P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_gdn_bwd_kept_workspace_bytes.restype = ctypes.c_size_t
    L.llattn_gdn_bwd_kept_workspace_bytes.argtypes = [ctypes.c_int] * 6
    L.llattn_gdn_bwd_kept.restype = ctypes.c_int
    L.llattn_gdn_bwd_kept.argtypes = [_P] * 15 + [_P, ctypes.c_size_t, _P, ctypes.c_size_t] + [ctypes.c_int] * 6 + [_P]
    L.llattn_gdn_bwd_kept_bf16dv.restype = ctypes.c_int
    L.llattn_gdn_bwd_kept_bf16dv.argtypes = L.llattn_gdn_bwd_kept.argtypes
    L.llattn_selftest_umma_cycles.restype = ctypes.c_int
    L.llattn_selftest_umma_cycles.argtypes = [ctypes.c_int] * 5 + [_P, _P, _P]
    L.llattn_testing_use_tensor_core_path.restype = None        # test-only symbol (csrc/llattn_testing.h)
    L.llattn_testing_use_tensor_core_path.argtypes = [ctypes.c_int]
    L.llattn_selftest_wait_timeout.restype = ctypes.c_int       # test-only symbol
    L.llattn_selftest_wait_timeout.argtypes = [ctypes.c_int, _P, _P]
    L.llattn_kernel_launches.restype = ctypes.c_ulonglong
    L.llattn_kernel_launches.argtypes = []
    L.llattn_workspace_status.restype = ctypes.c_int
    L.llattn_workspace_status.argtypes = [_P, _P, _P]
    L.llattn_static_scratch_status.restype = ctypes.c_int
    L.llattn_static_scratch_status.argtypes = [_P, _P]
    L.llattn_selftest_umma.restype = ctypes.c_int
    L.llattn_selftest_umma.argtypes = [_P, _P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, _P]
    _lib = L
    return L


# When set, every Mamba-2 driver call reads its workspace's status word after the launch (one stream
# synchronisation per call) and raises if a kernel gave up on a bounded wait.  Off by default: the
# drivers then never synchronise, like the reference's.  The test-suite, the smoke check and the
# benchmark switch it on or read the word themselves.
CHECK_STATUS = os.environ.get("LLATTN_CHECK_STATUS", "0") not in ("", "0")


def workspace_status(ws, stream) -> int:
    """Status word of a workspace tensor that a call on `stream` used (synchronises the stream)."""
    out = ctypes.c_int(-1)
    rc = lib().llattn_workspace_status(ws.data_ptr(), ctypes.byref(out), stream)
    check(rc, "llattn_workspace_status")
    return out.value


def raise_on_status(ws, stream, what: str):
    if workspace_status(ws, stream) != 0:
        raise RuntimeError(f"{what}: a kernel gave up on a bounded wait (status word set); the outputs are not valid")


def check(rc: int, what: str):
    if rc == 0:
        return
    if rc < 0:
        raise ValueError(f"{what}: {ERRORS.get(rc, rc)}")
    raise RuntimeError(f"{what}: CUDA error {rc}")
