"""Parity tolerances, written once.

fp32 storage: against a float64 sequential loop on the same stored inputs,
    max|got - ref| <= 1e-5 * max|ref|   and   allclose(rtol=1e-3, atol=1e-5)
  (the second line is the tolerance of the reference's own kernel tests,
  test_forwards.py:29-30,85 and test_backwards.py:31-32,91).
fp16 / bf16 storage: against the fp32 sequential loop on the same stored inputs,
    allclose(rtol=2e-2, atol=1e-3).
"""
import numpy as np
import torch

F32_NORM = 1e-5
F32_RTOL, F32_ATOL = 1e-3, 1e-5
HALF_RTOL, HALF_ATOL = 2e-2, 1e-3


def _as64(t):
    if isinstance(t, torch.Tensor):
        t = t.detach().float().cpu().numpy() if t.dtype != torch.float64 else t.detach().cpu().numpy()
    return np.asarray(t, dtype=np.float64)


def assert_close_f32(got, ref64, name=""):
    g, r = _as64(got), _as64(ref64)
    assert g.shape == r.shape, f"{name}: shape {g.shape} vs {r.shape}"
    if g.size == 0:
        return
    assert np.isfinite(g).all(), f"{name}: non-finite values"
    scale = np.abs(r).max()
    err = np.abs(g - r).max()
    assert err <= F32_NORM * max(scale, 1e-30), f"{name}: max err {err:.3e} vs scale {scale:.3e}"
    assert np.allclose(g, r, rtol=F32_RTOL, atol=F32_ATOL), f"{name}: allclose(rtol=1e-3, atol=1e-5) failed"


def assert_close_half(got, ref32, name="", scale_atol=1.0):
    g, r = _as64(got), _as64(ref32)
    assert g.shape == r.shape, f"{name}: shape {g.shape} vs {r.shape}"
    if g.size == 0:
        return
    assert np.isfinite(g).all(), f"{name}: non-finite values"
    bad = np.abs(g - r) > HALF_ATOL * scale_atol + HALF_RTOL * np.abs(r)
    assert not bad.any(), (f"{name}: {bad.sum()} of {bad.size} outside rtol=2e-2/atol=1e-3; "
                           f"worst abs err {np.abs(g - r).max():.3e}")
