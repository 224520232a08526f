"""Scan with the SSM layer's gate activations fused into the kernels.

``layers.SSM`` (reference: quick_ssm/layers.py:76-104) turns five projection outputs into the four
scan inputs with element-wise kernels - two sigmoids, a SiLU times a product, four casts - and
autograd runs their backward kernels as well.  Around a memory-bound scan those kernels move several
times the scan's own bytes.  ``gated_scan`` takes the five projection outputs directly:

    a = sigmoid(pa)    x = px    c = silu(pc1) * pc2    b = sigmoid(pd)    y = scan(x, a, b, c)

with every gate rounded to ``gate_dtype`` exactly where the layer casts to its compute dtype, and
returns gradients with respect to the projection outputs.  When the tensors cannot be handed to the
fused kernels (layout the copy engine cannot address, unsupported dtype pair) the same result is
composed from torch element-wise ops and ``scan`` - still on the GPU, never on the CPU.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from .scan_interface import _addressable, _n_tiles, scan


def _composed(pa, px, pc1, pc2, pd, gate_dtype, out_dtype):
    a = torch.sigmoid(pa).to(gate_dtype)
    x = px.to(gate_dtype)
    c = (F.silu(pc1) * pc2).to(gate_dtype)
    b = torch.sigmoid(pd).to(gate_dtype)
    return scan(x=x, a=a, b=b, c=c, out_dtype=out_dtype)


def _fusable(ts, gate_dtype, out_dtype) -> bool:
    t0 = ts[0]
    if t0.device.type != "cuda" or any(t.dtype != t0.dtype or t.stride() != t0.stride() for t in ts[1:]):
        return False
    if not _lib.layout_ok(t0) or t0.numel() == 0:
        return False
    if t0.dtype == torch.float32:
        return out_dtype == torch.float32 and gate_dtype in (torch.float32, torch.bfloat16, torch.float16)
    if t0.dtype in (torch.bfloat16, torch.float16):
        return gate_dtype == t0.dtype and out_dtype in (t0.dtype, torch.float32)
    return False


class _GatedScanFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pa, px, pc1, pc2, pd, gate_dtype, out_dtype):
        B, L, D = pa.shape
        y = torch.empty((B, L, D), dtype=out_dtype, device=pa.device)
        needs_grad = any(ctx.needs_input_grad[:5])
        tile_h = torch.empty((B, _n_tiles(L), D), dtype=torch.float32, device=pa.device) if needs_grad else None
        _lib.gated_scan_fwd(pa, px, pc1, pc2, pd, y, gate_dtype, tile_h=tile_h)
        if needs_grad:
            ctx.save_for_backward(pa, px, pc1, pc2, pd, tile_h)
        ctx.gate_dtype = gate_dtype
        return y

    @staticmethod
    def backward(ctx, grad_output):
        pa, px, pc1, pc2, pd, tile_h = ctx.saved_tensors
        dy = _addressable(grad_output)
        grads = [torch.empty(pa.shape, dtype=pa.dtype, device=pa.device) for _ in range(5)]
        _lib.gated_scan_bwd(pa, px, pc1, pc2, pd, dy, tile_h, grads, ctx.gate_dtype)
        return (*grads, None, None)


def gated_scan(pa: torch.Tensor, px: torch.Tensor, pc1: torch.Tensor, pc2: torch.Tensor, pd: torch.Tensor, *,
               gate_dtype: Optional[torch.dtype] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = c*h`` with ``h(t) = a h(t-1) + b x`` and the gates computed from projection outputs
    ``[B, L, D]`` as described in the module docstring.  ``gate_dtype`` defaults to the input dtype,
    ``out_dtype`` to float32 for float32 inputs and to the input dtype otherwise."""
    ts = (pa, px, pc1, pc2, pd)
    if any(t.shape != pa.shape for t in ts) or pa.dim() != 3:
        raise ValueError("the five projection outputs must share one shape [B, L, D].")
    if pa.device.type != "cuda":
        raise RuntimeError("gated_scan requires CUDA tensors.")
    gate_dtype = gate_dtype or pa.dtype
    out_dtype = out_dtype or pa.dtype
    if _fusable(ts, gate_dtype, out_dtype):
        try:
            return _GatedScanFunction.apply(pa, px, pc1, pc2, pd, gate_dtype, out_dtype)
        except _lib.Unsupported:
            pass
    return _composed(pa, px, pc1, pc2, pd, gate_dtype, out_dtype)
