"""The reference's own caller of the scan, ``quick_ssm/layers.py``, executed unmodified against
this package (its ``from quick_ssm.scan_interface import scan`` resolves to our module).
Needs a checkout of the reference next to this repository (or $QUICK_SSM_REFERENCE_DIR); skipped otherwise."""
import importlib.util
import os
import sys
import types

import pytest
import torch

# the reference checkout: $QUICK_SSM_REFERENCE_DIR, or a directory named "reference" next to this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF_DIR = os.environ.get("QUICK_SSM_REFERENCE_DIR", os.path.join(os.path.dirname(_REPO), "reference"))
REF = os.path.join(_REF_DIR, "quick_ssm", "layers.py")
pytestmark = pytest.mark.skipif(not os.path.exists(REF), reason="reference tree not present")


def _load_reference_layers():
    import quick_ssm_b200.scan_interface as ours
    pkg = types.ModuleType("quick_ssm")
    pkg.__path__ = []
    saved = {k: sys.modules.get(k) for k in ("quick_ssm", "quick_ssm.scan_interface")}
    sys.modules["quick_ssm"] = pkg
    sys.modules["quick_ssm.scan_interface"] = ours
    try:
        spec = importlib.util.spec_from_file_location("quick_ssm_reference_layers", REF)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mod


def test_reference_layer_runs_on_our_scan_and_matches_our_mirror():
    ref_layers = _load_reference_layers()
    from quick_ssm_b200.layers import SSM
    torch.manual_seed(0)
    theirs = ref_layers.SSM(hidden_size=16, state_size_mult=4.0, compute_dtype=torch.float32)
    ours = SSM(hidden_size=16, state_size_mult=4.0, compute_dtype=torch.float32)
    ours.load_state_dict(theirs.state_dict())
    x = torch.randn(2, 24, 16)
    kw = dict(block_l=128, checkpoint=True, tile_b=1, tile_d=512, scan_out_dtype=torch.float32, backend="torch")
    x1 = x.clone().requires_grad_()
    x2 = x.clone().requires_grad_()
    y1 = theirs(x1, **kw)
    y2 = ours(x2, **kw)
    assert torch.allclose(y1, y2, rtol=1e-6, atol=1e-6)
    y1.sum().backward()
    y2.sum().backward()
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-5, atol=1e-6)
    # without an explicit backend the reference layer reaches the CUDA kernels; on CPU that raises
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        theirs(x)
