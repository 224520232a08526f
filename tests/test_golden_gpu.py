"""The CUDA path against the committed fixtures that were generated from the reference itself."""
import glob
import os

import numpy as np
import pytest
import torch

from quick_ssm_b200 import _lib, scan
from quick_ssm_b200.forward_only import block_scan_forward_3d as forward_only_h
from quick_ssm_b200.triton_backwards import block_scan_backward_3d
from quick_ssm_b200.triton_forwards import block_scan_forward_3d
from tolerances import assert_close_f32, assert_close_half

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return {k: torch.from_numpy(v) for k, v in np.load(os.path.join(GOLD, name + ".npz")).items()}


@pytest.mark.parametrize("name", ["fwd_2x512x8_seed42", "fwd_1x4x1_seed3", "fwd_1x1024x1_seed4"])
def test_forward_fixtures(name):
    g = _load(name)
    _, h = block_scan_forward_3d(g["x"].cuda(), g["a"].cuda(), g["b"].cuda(), BLOCK_L=128)
    assert torch.allclose(h.cpu(), g["h"], rtol=1e-3, atol=1e-5)      # test_forwards.py:85
    h2 = forward_only_h(g["x"].cuda(), g["a"].cuda(), g["b"].cuda())
    assert torch.allclose(h2.cpu(), g["h"], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("name", ["bwd_2x2048x8_seed0", "bwd_1x1024x1_seed0", "iface_2x32x4_seed0"])
def test_backward_fixtures(name):
    g = _load(name)
    cu = {k: v.cuda() for k, v in g.items()}
    grads = block_scan_backward_3d(cu["a"], cu["b"], cu["c"], cu["x"], cu["h"], cu["dy"])
    for k, got in zip(("dx", "da", "db", "dc"), grads):
        assert torch.allclose(got.cpu(), g[k], rtol=1e-3, atol=1e-5), k  # test_backwards.py:91
    x, a, b, c = (cu[k].clone().requires_grad_() for k in ("x", "a", "b", "c"))
    y = scan(x, a, b, c, block_l=16, checkpoint=True)
    (y * cu["dy"]).sum().backward()
    assert torch.allclose(y.detach().cpu(), g["y"], rtol=1e-3, atol=1e-5)
    for k, t in zip(("dx", "da", "db", "dc"), (x, a, b, c)):
        assert torch.allclose(t.grad.cpu(), g[k], rtol=1e-3, atol=1e-4), k  # test_scan_interface.py:31


@pytest.mark.parametrize("name", ["full_1x50x2", "full_1x7x1", "full_2x64x3", "full_2x17x40",
                                  "cfg0_4x2048x16_ch0_7_15"])
def test_full_fixtures_against_float64(name):
    g = _load(name)
    x, a, b, c = (g[k].cuda().requires_grad_() for k in ("x", "a", "b", "c"))
    for ckpt in (True, False):
        for t in (x, a, b, c):
            t.grad = None
        y = scan(x, a, b, c, checkpoint=ckpt)
        y.backward(g["dy"].cuda())
        assert_close_f32(y, g["y64"], "y")
        for k, t in zip(("dx", "da", "db", "dc"), (x, a, b, c)):
            assert_close_f32(t.grad, g[k + "64"], k)
    _lib.check_device_status(synchronize=True)


@pytest.mark.parametrize("name,dtype", [("half_bf16_2x128x8", torch.bfloat16), ("half_fp16_2x128x8", torch.float16)])
def test_half_fixtures(name, dtype):
    g = _load(name)
    x, a, b, c = (g[k].to(dtype).cuda() for k in ("x", "a", "b", "c"))
    y = scan(x, a, b, c)
    assert y.dtype == dtype
    assert_close_half(y, g["y"], "y")
    h = forward_only_h(x, a, b)
    assert_close_half(h, g["h"], "h")
