"""The import shims of baseline/ref_compat.py (benchmark infrastructure for the reference's own code): the closed-form
level table equals the reference's Python double loop, and the reference's PyTorch forms imported through the shims agree
with the oracle.  Skipped where the copy of the reference (baseline/make_ref.py) is absent."""
import importlib
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "hattention")),
                                reason="no copy of the reference (python baseline/make_ref.py <checkout>)")


def test_closed_form_level_table_equals_the_reference_loop():
    from baseline import ref_compat
    ref_compat.load_reference(triton_path=False, torch_forms=False)
    sys.modules.pop("hattention.base", None)
    base = importlib.import_module("hattention.base")          # fresh module: its own make_levels_matrix
    for clamp in (None, 0):
        want = base.make_levels_matrix(256, 2, base.HType.WEAK, torch.int64, torch.device("cpu"), clamp_min=clamp,
                                       cached_length=None)
        got = ref_compat.levels_matrix_closed_form(256, 2, base.HType.WEAK, torch.int64, torch.device("cpu"), clamp_min=clamp)
        assert torch.equal(got, want)


def test_reference_torch_forms_import_and_agree_with_the_oracle():
    from baseline import ref_compat
    from oracle import loglinear_oracle as orc
    m = ref_compat.load_reference(triton_path=False, torch_forms=True)
    hm, rec, base = m["hssd_minimal"], m["recurrent"], m["base"]
    q, k, v, g, l = orc.make_mamba2_inputs(1, 512, 2, 16, 32, 1, 10, seed=0)
    H = 2
    y = hm.hssd_minimal_discrete(v, g, k.expand(-1, -1, H, -1).contiguous(), q.expand(-1, -1, H, -1).contiguous(), l, 2,
                                 base.HType.WEAK, 64)
    assert torch.allclose(y, orc.mamba2_chunkwise(q, k, v, g, l), rtol=1e-4, atol=2e-5)
    y2, _ = rec.hattention_recurrent(q.expand(-1, -1, H, -1)[:, :96].contiguous(), k.expand(-1, -1, H, -1)[:, :96].contiguous(),
                                     v[:, :96], torch.exp(g[:, :96]), None, l[:, :96], 2, base.HType.WEAK, base.HStruct.MAMBA2)
    assert torch.allclose(y2, y[:, :96], rtol=1e-4, atol=2e-5)
