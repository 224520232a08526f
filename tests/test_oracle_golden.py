"""The CPU oracle against fixtures generated from the reference implementation itself
(tests/golden/make_golden.py imports the reference's naive_baseline and stores its outputs).
fp32 and fp64 results must match bit for bit; this is what pins the oracle."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import naive_torch
from oracle import scan_oracle as so

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return dict(np.load(os.path.join(GOLD, name + ".npz")))


def test_fixture_set_is_complete():
    names = {os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz"))}
    assert {"fwd_2x512x8_seed42", "fwd_1x4x1_seed3", "fwd_1x1024x1_seed4", "bwd_2x2048x8_seed0",
            "bwd_1x1024x1_seed0", "iface_2x32x4_seed0", "cfg0_4x2048x16_ch0_7_15"} <= names


@pytest.mark.parametrize("name", ["fwd_2x512x8_seed42", "fwd_1x4x1_seed3", "fwd_1x1024x1_seed4"])
def test_forward_bit_exact_fp32(name):
    g = _load(name)
    h, _, h_last = so.scan_forward(g["x"], g["a"], g["b"], dtype=np.float32)
    assert np.array_equal(h, g["h"])
    assert np.array_equal(h_last, g["h"][:, -1])
    # float64 blockwise restatement agrees with the sequential float64 loop
    h64, _, _ = so.scan_forward(g["x"], g["a"], g["b"], dtype=np.float64)
    for blk in (8, 128, 256):
        hb = so.scan_forward_blockwise(g["x"], g["a"], g["b"], blk)
        assert np.abs(hb - h64).max() <= 1e-12 * max(1.0, np.abs(h64).max())


@pytest.mark.parametrize("name", ["bwd_2x2048x8_seed0", "bwd_1x1024x1_seed0", "iface_2x32x4_seed0"])
def test_backward_bit_exact_fp32(name):
    g = _load(name)
    h, y, _ = so.scan_forward(g["x"], g["a"], g["b"], g["c"], dtype=np.float32)
    assert np.array_equal(h, g["h"]) and np.array_equal(y, g["y"])
    grads = so.scan_backward(g["x"], g["a"], g["b"], g["c"], g["dy"], dtype=np.float32)[:4]
    for k, got in zip(("dx", "da", "db", "dc"), grads):
        assert np.array_equal(got, g[k + "_loop"]), k          # the reference's explicit backward loop
        assert np.allclose(got, g[k], rtol=1e-3, atol=1e-5), k  # autograd through its forward


@pytest.mark.parametrize("name", ["full_1x50x2", "full_1x7x1", "full_2x64x3", "full_2x17x40",
                                  "cfg0_4x2048x16_ch0_7_15"])
def test_full_bit_exact_fp32_and_fp64(name):
    g = _load(name)
    for dt, sfx in ((np.float32, ""), (np.float64, "64")):
        h, y, _ = so.scan_forward(g["x"], g["a"], g["b"], g["c"], dtype=dt)
        grads = so.scan_backward(g["x"], g["a"], g["b"], g["c"], g["dy"], dtype=dt)[:4]
        assert np.array_equal(h, g["h" + sfx]) and np.array_equal(y, g["y" + sfx])
        for k, got in zip(("dx", "da", "db", "dc"), grads):
            assert np.array_equal(got, g[k + sfx]), (k, sfx)


@pytest.mark.parametrize("name,dtype", [("half_bf16_2x128x8", torch.bfloat16), ("half_fp16_2x128x8", torch.float16)])
def test_half_inputs_follow_reference_rounding(name, dtype):
    """Reference on 16-bit inputs: fp32 accumulate, h rounded to the dtype, y = c*h in the dtype."""
    g = _load(name)
    h32, _, _ = so.scan_forward(g["x"], g["a"], g["b"], dtype=np.float32)
    h_r = torch.from_numpy(h32).to(dtype)
    assert np.array_equal(h_r.float().numpy(), g["h"])
    y_r = (torch.from_numpy(g["c"]).to(dtype) * h_r)
    assert np.array_equal(y_r.float().numpy(), g["y"])
    # a single rounding of the fp32 product (what the CUDA kernels do) stays within the 16-bit tolerance
    _, y32, _ = so.scan_forward(g["x"], g["a"], g["b"], g["c"], dtype=np.float32)
    assert np.allclose(y32, g["y"], rtol=2e-2, atol=1e-3)


def test_seeded_forms_compose():
    """h_in / g_in extensions: two halves chained equal the whole (float64, exact up to rounding)."""
    rng = np.random.default_rng(0)
    B, L, D = 2, 40, 5
    x, b, dy = (rng.standard_normal((B, L, D)) for _ in range(3))
    a = rng.uniform(0.9, 1.0, (B, L, D))
    c = rng.uniform(0.0, 1.0, (B, L, D))
    h, y, h_last = so.scan_forward(x, a, b, c)
    gx = so.scan_backward(x, a, b, c, dy)
    lo, hi = slice(0, 17), slice(17, L)
    h1, y1, mid = so.scan_forward(x[:, lo], a[:, lo], b[:, lo], c[:, lo])
    h2, y2, end = so.scan_forward(x[:, hi], a[:, hi], b[:, hi], c[:, hi], h_in=mid)
    assert np.allclose(np.concatenate([y1, y2], 1), y, rtol=1e-13, atol=1e-13) and np.allclose(end, h_last)
    g2 = so.scan_backward(x[:, hi], a[:, hi], b[:, hi], c[:, hi], dy[:, hi], h_in=mid)
    g1 = so.scan_backward(x[:, lo], a[:, lo], b[:, lo], c[:, lo], dy[:, lo], g_in=g2[4])
    for k in range(4):
        assert np.allclose(np.concatenate([g1[k], g2[k]], 1), gx[k], rtol=1e-12, atol=1e-12)


def test_torch_restatement_matches_c_oracle():
    g = _load("full_2x64x3")
    t = {k: torch.from_numpy(v) for k, v in g.items()}
    h, y = naive_torch.forward_y(t["x"], t["a"], t["b"], t["c"])
    assert torch.equal(h, t["h"]) and torch.equal(y, t["y"])
    for got, k in zip(naive_torch.backward(t["x"], t["a"], t["b"], t["c"], t["dy"]), ("dx", "da", "db", "dc")):
        assert torch.equal(got, t[k])
