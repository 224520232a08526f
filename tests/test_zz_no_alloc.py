"""Forward scan with the library's built-in scratch (``qssm_scan_fwd_static_ws``).

Some callers cannot allocate device memory around the call (a plugin inside a host runtime whose
pool owns the device heap, a service that may not allocate after start-up, a latency-critical
loop that cannot take cudaMalloc's device-wide synchronisation), so this entry point keeps the
segment aggregates in a fixed array inside the library instead of a caller-provided workspace.
The test calls it through the C ABI and checks it against ``qssm_scan_fwd`` fed a workspace
from the caller and against the CPU oracle, twice in a row with different inputs: the second
call starts from whatever the first left in the shared array and must not be affected by it.
A third case lets the library choose (``n_seg=0``) on a long, narrow shape, where the single-pass
kernels keep their ticket counter and chunk descriptors in the same array.

The file sorts last so that a run that stops at the first failure has already run everything
else; it passes on its own in a fresh process as well as after the other tests.
"""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from quick_ssm_b200 import _lib
from quick_ssm_b200.synth import make_inputs
from tolerances import assert_close_f32, assert_close_half

pytestmark = pytest.mark.gpu


def _both(inp, n_seg):
    x, a, b, c = inp.tensors()
    B, L, D = x.shape
    nt = (L + _lib.tile_rows() - 1) // _lib.tile_rows()
    out = {}
    for name, fn in (("caller_ws", _lib.scan_fwd), ("static_ws", _lib.scan_fwd_static_ws)):
        y = torch.empty_like(x)
        tile_h = torch.empty((B, nt, D), dtype=torch.float32, device=x.device)
        h_last = torch.empty((B, D), dtype=torch.float32, device=x.device)
        fn(x, a, b, c, y, tile_h=tile_h, h_last=h_last, n_seg=n_seg)
        out[name] = (y, tile_h, h_last)
    _lib.check_device_status(synchronize=True)
    return out


def _oracle(inp, dtype):
    """y, the state before every 16th step, and the final state, from the sequential CPU loop."""
    acc = np.float64 if dtype == torch.float32 else np.float32
    f = [t.float().cpu() for t in inp.tensors()]
    h, y, h_last = so.scan_forward(*f, dtype=acc)
    before = np.concatenate([np.zeros_like(h[:, :1]), h[:, :-1]], axis=1)
    return y, before[:, ::_lib.tile_rows()], h_last


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_static_scratch_matches_caller_workspace_twice(dtype):
    rtol, atol = (1e-3, 1e-5) if dtype == torch.float32 else (2e-2, 1e-3)
    check = assert_close_f32 if dtype == torch.float32 else assert_close_half
    cases = [((2, 2048, 96), 4, 21), ((3, 1500, 40), 7, 22), ((1, 6000, 64), 0, 23)]
    for call, (shape, n_seg, seed) in enumerate(cases):
        inp = make_inputs(*shape, dtype=dtype, seed=seed).to("cuda")
        res = _both(inp, n_seg)
        for got, want, ref, name in zip(res["static_ws"], res["caller_ws"], _oracle(inp, dtype),
                                        ("y", "tile_h", "h_last")):
            assert torch.isfinite(got.float()).all(), f"call {call}: {name} not finite"
            assert torch.allclose(got.float(), want.float(), rtol=rtol, atol=atol), f"call {call}: {name}"
            if name == "y":
                check(got, ref, f"call {call}: {name} against the oracle")
            else:  # fp32 states computed from 16-bit inputs: fp32 arithmetic on both sides
                assert np.allclose(got.cpu().numpy(), ref, rtol=1e-3, atol=1e-4), f"call {call}: {name} vs oracle"


def test_static_scratch_refuses_the_reuse_form():
    """``n_seg < 0`` means "aggregates already in the workspace"; nothing can have put them into the
    built-in array, so the entry point refuses instead of scanning from stale seeds."""
    x = torch.zeros(1, 2048, 64, dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="bad shape"):
        _lib.scan_fwd_static_ws(x, x, x, x, torch.empty_like(x), n_seg=-4)


def test_static_scratch_rejects_oversized_request():
    # 3 * B * n_seg * D * 4 bytes = 3 * 4 * 64 * 2048 * 4 = 6 MiB > the 4 MiB built-in array
    x = torch.zeros(4, 64 * 256, 2048, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    with pytest.raises(RuntimeError, match="built-in maximum"):
        _lib.scan_fwd_static_ws(x, x, x, x, y, n_seg=64)
    # the same request with a caller workspace is fine
    _lib.scan_fwd(x, x, x, x, y, n_seg=64)
    torch.cuda.synchronize()
