"""This library against the reference's own Triton kernels on the same GPU and inputs.

The reference package is installed unmodified under the git-ignored ``baseline/_ref`` (``python -m pip install
--no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the reference without its assets folder>``);
where it is absent the tests skip.  Shapes and distributions are those of the reference's own tests
(test_forwards.py:108-114, test_backwards.py:120-125, test_scan_interface.py:7-31)."""
import importlib
import os
import sys

import pytest
import torch

from quick_ssm_b200 import _lib, scan
from quick_ssm_b200.synth import make_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _reference_scan():
    if not os.path.isdir(os.path.join(REF, "quick_ssm")):
        pytest.skip("the reference package is not installed under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    return importlib.import_module("quick_ssm.scan_interface").scan


@pytest.mark.parametrize("shape,block_l", [((2, 512, 8), 128), ((2, 2048, 8), 256), ((2, 32, 4), 16), ((1, 50, 2), 16),
                                           ((3, 300, 72), 64)], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else f"blk{v}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
def test_forward_and_gradients_match_the_reference_triton_path(shape, block_l, dtype):
    ref_scan = _reference_scan()
    inp = make_inputs(*shape, dtype=dtype, seed=13).to("cuda")
    res = []
    for fn in (lambda *t: ref_scan(*t, block_l=block_l, checkpoint=True, backend="triton"),
               lambda *t: scan(*t, block_l=block_l, checkpoint=True)):
        leaves = [t.detach().clone().requires_grad_() for t in inp.tensors()]
        y = fn(*leaves)
        y.backward(inp.dy)
        res.append([y.detach()] + [t.grad for t in leaves])
    _lib.check_device_status(synchronize=True)
    # both sides accumulate in fp32 and round once per stored value; the reference's own kernel tests allow
    # rtol 1e-3 / atol 1e-5 in fp32 (test_forwards.py:85)
    tol = dict(rtol=1e-3, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
    for name, u, v in zip(("y", "dx", "da", "db", "dc"), *res):
        assert torch.allclose(v.float(), u.float(), **tol), (name, float((v.float() - u.float()).abs().max()))


def test_kernel_level_entry_points_match_the_reference_drivers():
    """block_scan_forward_3d -> (cumulative prod a, h), block_scan_backward_3d -> four fp32 gradients and the
    forward-only driver, reference (triton_forwards.py:134-172, triton_backwards.py:168-209,
    forward_only.py:423-540) against the shims of this package with the same arguments."""
    _reference_scan()
    ref_f = importlib.import_module("quick_ssm.triton_forwards")
    ref_b = importlib.import_module("quick_ssm.triton_backwards")
    ref_o = importlib.import_module("quick_ssm.forward_only")
    from quick_ssm_b200 import forward_only as our_o
    from quick_ssm_b200 import triton_backwards as our_b
    from quick_ssm_b200 import triton_forwards as our_f
    inp = make_inputs(2, 1024, 8, dtype=torch.float32, seed=19).to("cuda")
    x, a, b, c = inp.tensors()
    ra, rh = ref_f.block_scan_forward_3d(x, a, b, 256)
    oa, oh = our_f.block_scan_forward_3d(x, a, b, 256)
    assert torch.allclose(oh, rh, rtol=1e-3, atol=1e-5)
    assert torch.allclose(oa, ra, rtol=1e-3, atol=1e-30)   # cumulative products fall towards zero: relative only
    rg = ref_b.block_scan_backward_3d(a, b, c, x, rh, inp.dy, 256)
    og = our_b.block_scan_backward_3d(a, b, c, x, oh, inp.dy, 256)
    for name, u, v in zip(("dx", "da", "db", "dc"), rg, og):
        assert torch.allclose(v, u, rtol=1e-3, atol=2e-5), name
    h_ref = ref_o.block_scan_forward_3d(x, a, b, 256)
    h_our = our_o.block_scan_forward_3d(x, a, b, 256)
    assert torch.allclose(h_our, h_ref, rtol=1e-3, atol=1e-5)
    _lib.check_device_status(synchronize=True)
