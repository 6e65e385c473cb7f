"""The package as a drop-in for the reference's modules: after `install_as_hattention()` every name that the
reference's model files import from `hattention.*` for this path resolves, and the re-exported functions have
the reference's signatures.  The signature part reads the reference checkout and is skipped without it."""
import ast
import inspect
import os
import sys

import pytest

REF = "/root/reference/hattention"

# what modeling_hattention.py:45-52 and modeling_h_gated_deltanet.py:30-36 import for the hot path
NEEDED = {
    "hattention.base": ["HType", "HStruct", "get_num_levels"],
    "hattention.recurrent": ["HState"],
    "hattention.mamba_apis": ["LambdaLevelMLP", "hselective_state_update", "hmamba_chunk_scan_combined",
                              "hmamba_split_conv1d_scan_combined", "compute_lambda_maybe_fixed"],
    "hattention.gated_delta_rule_apis": ["chunk_h_gated_delta_rule"],
    "hattention.kernel": ["hattention_kernel", "hattention_prefill", "hattention_step", "HAttentionFunction"],
    "hattention.chunkwise": ["chunkwise_fwd", "chunkwise_bwd"],
    "hattention.chunkwise_hgdn": ["chunkwise_fwd", "chunkwise_bwd"],
}


@pytest.fixture()
def installed():
    saved = {k: v for k, v in sys.modules.items() if k == "hattention" or k.startswith("hattention.")}
    for k in saved:
        del sys.modules[k]
    import hattention_b200
    pkg = hattention_b200.install_as_hattention()
    yield pkg
    for k in [k for k in sys.modules if k == "hattention" or k.startswith("hattention.")]:
        del sys.modules[k]
    sys.modules.update(saved)


def test_names_the_model_files_import_resolve(installed):
    import importlib
    for mod, names in NEEDED.items():
        m = importlib.import_module(mod)
        for n in names:
            assert hasattr(m, n), f"{mod}.{n}"


def _reference_signature(path, func):
    """Argument names (and which have defaults) of a top-level function or class __init__ in a reference source
    file, read with `ast` so that the file's own imports (mamba_ssm, causal_conv1d) are not needed."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == func:
            a = node.args
            names = [x.arg for x in a.posonlyargs + a.args]
            return names, len(a.defaults)
    raise KeyError(func)


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference checkout not present")
@pytest.mark.parametrize("mod,func", [
    ("mamba_apis", "hmamba_chunk_scan_combined"), ("mamba_apis", "hmamba_split_conv1d_scan_combined"),
    ("mamba_apis", "hselective_state_update"), ("mamba_apis", "compute_lambda_maybe_fixed"), ("mamba_apis", "compute_lambda"),
    ("gated_delta_rule_apis", "chunk_h_gated_delta_rule"),
    ("kernel", "hattention_kernel"), ("kernel", "hattention_prefill"), ("kernel", "hattention_step"),
])
def test_signatures_match_the_reference(installed, mod, func):
    import importlib
    ours = getattr(importlib.import_module(f"hattention.{mod}"), func)
    want_names, want_defaults = _reference_signature(os.path.join(REF, f"{mod}.py"), func)
    sig = inspect.signature(ours)
    got_names = list(sig.parameters)
    assert got_names == want_names, (func, got_names, want_names)
    got_defaults = sum(1 for p in sig.parameters.values() if p.default is not inspect.Parameter.empty)
    assert got_defaults == want_defaults, func


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference checkout not present")
def test_driver_signatures_are_prefixes_of_ours(installed):
    """The inner drivers keep the reference's positional arguments; this package appends optional ones
    (keep_workspace / fwd_workspace) after them."""
    import importlib
    for mod, func in (("chunkwise", "chunkwise_fwd"), ("chunkwise_hgdn", "chunkwise_fwd")):
        ours = list(inspect.signature(getattr(importlib.import_module(f"hattention.{mod}"), func)).parameters)
        want, _ = _reference_signature(os.path.join(REF, f"{mod}.py"), func)
        assert ours[:len(want)] == want, (mod, func, ours, want)
    ours = list(inspect.signature(importlib.import_module("hattention.chunkwise").chunkwise_bwd).parameters)
    want, _ = _reference_signature(os.path.join(REF, "chunkwise.py"), "chunkwise_bwd")
    want = [w for w in want if w not in ("block_size_K", "block_size_V")]      # autotune parameters of the Triton host function
    assert ours[:len(want)] == want


def test_hstate_bookkeeping():
    import torch
    from hattention_b200 import HState, HStruct, HType
    a = HState(2, HType.WEAK, HStruct.MAMBA2, (1, 2, 4, 4, 9), torch.float32, torch.device("cpu"))
    b = HState(2, HType.WEAK, HStruct.MAMBA2, (1, 2, 4, 4, 9), torch.float32, torch.device("cpu"))
    b.states += 1.0
    b.set_counts_after(70)
    a.replace(b)
    assert a.states is b.states and a.counts == b.counts and sum(a.counts) == 70
    c = a.to(dtype=torch.float32)
    assert c.counts == a.counts and c.states is a.states
    a.reset_states()
    assert float(a.states.abs().sum()) == 0.0 and sum(a.counts) == 0
    with pytest.raises(ValueError):
        a.replace(HState(2, HType.WEAK, HStruct.MAMBA2, (1, 2, 4, 4, 8), torch.float32, torch.device("cpu")))


def test_gdn_value_heads_wider_than_one_kernel_call_are_sliced():
    """chunkwise_hgdn processes a value head wider than 128 columns as slices of at most 128: the slices tile the
    head exactly; widths that are not multiples of 64 or exceed 384 are refused."""
    from hattention_b200 import chunkwise_hgdn as m
    assert m._v_slices(192) == [(0, 128), (128, 192)]
    assert m._v_slices(256) == [(0, 128), (128, 256)]
    assert m._v_slices(384) == [(0, 128), (128, 256), (256, 384)]
    for bad in (96, 200, 448):
        with pytest.raises(ValueError):
            m._v_slices(bad)
    import torch
    x = torch.ones(1, 2, 1, 64)
    padded = m._pad_k(x)
    assert padded.shape == (1, 2, 1, m.K_CALL) and padded[..., 64:].abs().sum() == 0 and torch.equal(padded[..., :64], x)
