"""Host-side logic that needs no GPU: argument handling of the scan interface, the explicit
torch backend, the layer that calls the scan, the status-word check."""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from quick_ssm_b200 import SSM, RMSNorm, _lib, scan, scan_interface
from quick_ssm_b200.synth import CONFIGS, make_config, make_inputs


def test_chunk_ranges_matches_reference_semantics():
    cr = scan_interface._chunk_ranges
    assert cr(10, None) == [(0, 10)]
    assert cr(10, 0) == [(0, 10)] and cr(10, -3) == [(0, 10)] and cr(10, 10) == [(0, 10)] and cr(10, 99) == [(0, 10)]
    assert cr(10, 4) == [(0, 4), (4, 8), (8, 10)]
    assert cr(0, 4) == [(0, 0)]


def test_compute_dtype_and_layout_decisions():
    x16 = torch.zeros(2, 8, 16, dtype=torch.bfloat16)
    x32 = torch.zeros(2, 8, 16)
    assert scan_interface._compute_dtype(x16, x16) == torch.bfloat16
    assert scan_interface._compute_dtype(x16, x32) == torch.float32
    assert scan_interface._compute_dtype(x32.double()) == torch.float32
    assert scan_interface._kernel_out_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert scan_interface._kernel_out_dtype(torch.bfloat16, torch.float16) == torch.float32
    assert scan_interface._kernel_out_dtype(torch.float16, torch.float16) == torch.float16
    # channel shard view keeps its row pitch and is addressed in place
    view = x16[:, :, 4:12]
    assert _lib.layout_ok(view) and not view.is_contiguous()
    out = scan_interface._prepare_inputs(view, view, view, view)
    assert out[0].data_ptr() == view.data_ptr()
    # D not innermost: copied
    tr = x16.transpose(1, 2)
    assert not _lib.layout_ok(tr)
    out = scan_interface._prepare_inputs(tr, tr, tr, tr)
    assert out[0].is_contiguous()
    # differing layouts among the four inputs: copied to a common one
    out = scan_interface._prepare_inputs(view, x16[:, :, :8].contiguous(), view, view)
    assert all(t.is_contiguous() for t in out)
    # expanded (stride 0) upstream gradient is not addressable
    assert not _lib.layout_ok(torch.zeros(1, 1, 16).expand(2, 8, 16))


def test_backend_selection_never_falls_back_to_cpu():
    x = torch.zeros(1, 4, 4)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        scan(x, x, x, x)                      # auto == the CUDA kernels
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        scan(x, x, x, x, backend="triton")
    with pytest.raises(ValueError, match="Unsupported backend"):
        scan(x, x, x, x, backend="jax")
    assert scan(x, x, x, x, backend="torch").shape == x.shape


def test_explicit_torch_backend_matches_oracle_with_autograd():
    inp = make_inputs(2, 32, 4, dtype=torch.float32, seed=0)
    x, a, b, c = (t.clone().requires_grad_() for t in inp.tensors())
    y = scan(x, a, b, c, block_l=16, checkpoint=True, backend="torch")
    (y * inp.dy).sum().backward()
    _, y_ref, _ = so.scan_forward(inp.x, inp.a, inp.b, inp.c, dtype=np.float64)
    g_ref = so.scan_backward(inp.x, inp.a, inp.b, inp.c, inp.dy, dtype=np.float64)
    assert np.allclose(y.detach().numpy(), y_ref, rtol=1e-3, atol=1e-4)
    for got, ref in zip((x.grad, a.grad, b.grad, c.grad), g_ref):
        assert np.allclose(got.numpy(), ref, rtol=1e-3, atol=1e-4)   # test_scan_interface.py:31
    # out_dtype and 16-bit inputs
    y16 = scan(inp.x.bfloat16(), inp.a.bfloat16(), inp.b.bfloat16(), inp.c.bfloat16(), backend="torch",
               out_dtype=torch.float32)
    assert y16.dtype == torch.float32


def test_layer_runs_on_cpu_with_torch_backend():
    torch.manual_seed(0)
    layer = SSM(hidden_size=16, state_size_mult=4.0, compute_dtype=torch.float32)
    assert layer.state_size_dim == 64
    x = torch.randn(2, 12, 16, requires_grad=True)
    y = layer(x, backend="torch", block_l=128, tile_b=1, tile_d=512, scan_out_dtype=torch.float32)
    assert y.shape == x.shape
    y.pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())
    n = RMSNorm(16)
    z = n(x)
    assert torch.allclose(z.pow(2).mean(-1), torch.ones(2, 12), atol=1e-3)


def test_status_word_raises_once_and_clears():
    import ctypes
    w = torch.zeros(1, dtype=torch.int32)
    _lib._status_words[99] = (w, w.data_ptr(), ctypes.c_int.from_address(w.data_ptr()))
    try:
        w[0] = 10001
        with pytest.raises(RuntimeError, match="expired"):
            _lib.check_device_status()
        assert int(w[0]) == 0
        _lib.check_device_status()
    finally:
        del _lib._status_words[99]


def test_synthetic_configs():
    assert set(CONFIGS) == {"cfg0", "cfg1", "cfg2", "cfg3_scan", "cfg4"}
    inp = make_config("cfg0")
    assert inp.x.shape == (4, 2048, 16) and inp.x.dtype == torch.float32
    assert float(inp.a.min()) >= 0.9 and float(inp.a.max()) <= 1.0
    assert float(inp.c.min()) > 0 and float(inp.c.max()) < 1
    again = make_config("cfg0")
    assert torch.equal(inp.x, again.x) and torch.equal(inp.dy, again.dy)
    other = make_config("cfg0", rank=1)
    assert not torch.equal(inp.x, other.x)
    nu = make_inputs(1, 4096, 8, dtype=torch.float16, decay="near_unit", seed=0)
    assert float(nu.a.float().min()) >= 0.89 and float(nu.a.float().max()) <= 1.0
