"""RMS normalisation: the CPU oracle against fixtures made from the reference's ``RMSNorm`` module
(CPU tests), and the CUDA kernels against the oracle, the fixtures and the torch layer (GPU tests).

Tolerances: fp32 storage against the float64 oracle on the same inputs, max|err| <= 1e-5 * max|ref|
and allclose(rtol=1e-3, atol=1e-5); fp16/bf16 storage against the fp32 oracle, allclose(rtol=2e-2,
atol=1e-3).  dw is a sum over all rows: its error is measured against max|dw|."""
import os

import numpy as np
import pytest
import torch

from oracle import norm_oracle as no
from tolerances import assert_close_f32, assert_close_half

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = ["rmsnorm_f64_3x5x36", "rmsnorm_f32_2x7x128", "rmsnorm_f32_4x1032"]
gpu = pytest.mark.gpu


def _load(name):
    return dict(np.load(os.path.join(GOLD, name + ".npz")))


@pytest.mark.parametrize("name", FIXTURES)
def test_oracle_matches_the_reference_module(name):
    g = _load(name)
    eps = float(g["eps"])
    y, _ = no.rmsnorm_forward(g["x"], g["w"], eps)
    dx, dw = no.rmsnorm_backward(g["x"], g["w"], g["dy"], eps)
    tol = 1e-12 if g["x"].dtype == np.float64 else 2e-6  # fp32 fixtures carry fp32 rounding
    for got, ref in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"])):
        assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_oracle_backward_is_the_derivative_of_its_forward():
    rng = np.random.default_rng(3)
    x, w, dy = rng.standard_normal((4, 12)), rng.standard_normal(12), rng.standard_normal((4, 12))
    dx, dw = no.rmsnorm_backward(x, w, dy, 1e-5)
    h = 1e-6
    for idx in [(0, 0), (2, 7), (3, 11)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += h
        xm[idx] -= h
        num = ((no.rmsnorm_forward(xp, w, 1e-5)[0] - no.rmsnorm_forward(xm, w, 1e-5)[0]) * dy).sum() / (2 * h)
        assert abs(num - dx[idx]) <= 1e-6 * max(1.0, abs(dx[idx]))
    wp, wm = w.copy(), w.copy()
    wp[5] += h
    wm[5] -= h
    num = ((no.rmsnorm_forward(x, wp, 1e-5)[0] - no.rmsnorm_forward(x, wm, 1e-5)[0]) * dy).sum() / (2 * h)
    assert abs(num - dw[5]) <= 1e-6 * max(1.0, abs(dw[5]))


def test_composed_path_and_layer_match_the_oracle_on_cpu():
    """The torch composition used for row lengths the kernels do not take, and the mirrored layer on
    CPU tensors, follow the same formula as the oracle (float64)."""
    from quick_ssm_b200.layers import RMSNorm, RMSNormFused
    from quick_ssm_b200.norm import _composed, rms_norm
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 5, 30, generator=g, dtype=torch.float64, requires_grad=True)
    w = (torch.randn(30, generator=g, dtype=torch.float64) * 0.3 + 1.0).requires_grad_()
    dy = torch.randn(3, 5, 30, generator=g, dtype=torch.float64)
    y = _composed(x, w, 1e-5)
    y.backward(dy)
    ry, _ = no.rmsnorm_forward(x.detach().numpy(), w.detach().numpy(), 1e-5)
    rdx, rdw = no.rmsnorm_backward(x.detach().numpy(), w.detach().numpy(), dy.numpy(), 1e-5)
    assert np.abs(y.detach().numpy() - ry).max() <= 1e-12
    assert np.abs(x.grad.numpy() - rdx).max() <= 1e-12 and np.abs(w.grad.numpy() - rdw).max() <= 1e-11
    for cls in (RMSNorm, RMSNormFused):  # CPU tensors: both modules are the torch formula
        m = cls(30, dtype=torch.float64)
        with torch.no_grad():
            m.weight.copy_(w)
        assert np.abs(m(x.detach()).detach().numpy() - ry).max() <= 1e-12
    with pytest.raises(RuntimeError):
        rms_norm(x.detach().float(), w.detach().float(), 1e-5)  # the kernel entry point has no CPU path


# ------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------
def _run(x, w, dy, eps):
    from quick_ssm_b200.norm import rms_norm
    xg = x.cuda().requires_grad_()
    wg = w.cuda().requires_grad_()
    y = rms_norm(xg, wg, eps)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    return y.detach(), xg.grad, wg.grad


@gpu
@pytest.mark.parametrize("name", FIXTURES[1:])
def test_kernels_match_the_reference_fixtures(name):
    g = {k: torch.from_numpy(np.asarray(v)) for k, v in _load(name).items()}
    y, dx, dw = _run(g["x"], g["w"], g["dy"], float(g["eps"]))
    assert_close_f32(y, g["y"], "y")
    assert_close_f32(dx, g["dx"], "dx")
    assert_close_f32(dw, g["dw"], "dw")


@gpu
@pytest.mark.parametrize("shape", [(1, 4), (3, 128), (5, 7, 132), (64, 1024), (37, 2048), (9, 2052), (6, 4096),
                                   (5, 4100), (3, 8192), (2000, 256)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
def test_kernels_match_the_oracle(shape, dtype):
    """Row lengths on both sides of every register-chunk boundary, rows longer than the register
    paths take (read twice), more rows than warps, a single row."""
    g = torch.Generator().manual_seed(hash(shape) % 1000)
    x = torch.randn(*shape, generator=g).to(dtype)
    dy = torch.randn(*shape, generator=g).to(dtype)
    w = torch.randn(shape[-1], generator=g) * 0.5 + 1.0
    y, dx, dw = _run(x, w, dy, 1e-5)
    ref_t = np.float64 if dtype == torch.float32 else np.float32
    ry, _ = no.rmsnorm_forward(x.float().numpy(), w.numpy(), 1e-5, dtype=ref_t)
    rdx, rdw = no.rmsnorm_backward(x.float().numpy(), w.numpy(), dy.float().numpy(), 1e-5, dtype=ref_t)
    if dtype == torch.float32:
        assert_close_f32(y, ry, "y")
        assert_close_f32(dx, rdx, "dx")
        assert np.abs(dw.cpu().numpy() - rdw).max() <= 1e-5 * np.abs(rdw).max() + 1e-5
    else:
        assert_close_half(y, ry, "y")
        assert_close_half(dx, rdx, "dx")
        assert np.abs(dw.cpu().numpy() - rdw).max() <= 1e-3 * max(1.0, np.abs(rdw).max())


@gpu
def test_dw_is_deterministic_and_rows_are_independent():
    g = torch.Generator().manual_seed(5)
    x, dy, w = torch.randn(3000, 512, generator=g), torch.randn(3000, 512, generator=g), torch.randn(512, generator=g)
    a = _run(x, w, dy, 1e-5)
    b = _run(x, w, dy, 1e-5)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    sub = _run(x[100:200], w, dy[100:200], 1e-5)
    assert torch.equal(sub[0], a[0][100:200]) and torch.equal(sub[1], a[1][100:200])


@gpu
def test_unsupported_shapes_are_composed_on_the_device_and_cpu_raises():
    from quick_ssm_b200.norm import rms_norm
    x = torch.randn(4, 7, 30).cuda().requires_grad_()  # 30 % 4 != 0
    w = torch.ones(30).cuda()
    y = rms_norm(x, w, 1e-5)
    ry, _ = no.rmsnorm_forward(x.detach().cpu().numpy(), w.cpu().numpy(), 1e-5)
    assert_close_f32(y, ry, "y")
    with pytest.raises(RuntimeError):
        rms_norm(torch.randn(2, 8), torch.ones(8), 1e-5)


@gpu
def test_fused_norm_layer_matches_the_torch_layer():
    from quick_ssm_b200.layers import RMSNorm, RMSNormFused
    torch.manual_seed(0)
    ref = RMSNorm(1024).cuda().double()
    with torch.no_grad():
        ref.weight.copy_(torch.randn(1024).double() * 0.3 + 1.0)
    fused = RMSNormFused(1024).cuda()
    fused.load_state_dict({k: v.float() for k, v in ref.state_dict().items()})
    x = torch.randn(4, 96, 1024, device="cuda")
    dy = torch.randn_like(x)
    xr = x.double().requires_grad_()
    ref(xr).backward(dy.double())
    xf = x.clone().requires_grad_()
    y = fused(xf)
    y.backward(dy)
    assert_close_f32(y, ref(xr).detach(), "y")
    assert_close_f32(xf.grad, xr.grad, "dx")
    assert_close_f32(fused.weight.grad, ref.weight.grad, "dw")
