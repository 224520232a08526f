"""RMS normalisation of the layer input as one kernel per direction.

``rms_norm(x, weight, eps)`` computes what ``layers.RMSNorm`` computes
(reference: quick_ssm/layers.py:9-17), ``x * weight / sqrt(mean(x^2, -1) + eps)``, through
``qssm_rmsnorm_fwd`` / ``qssm_rmsnorm_bwd``: the forward reads x and writes y, the backward reads x
and dy and writes dx; dw is summed in a fixed order (no atomics).  Shapes the kernels cannot take
(last axis not a multiple of 4, unaligned views) are composed from torch operations on the same
device; CPU tensors raise.
"""
from __future__ import annotations

import torch

from . import _lib


def _composed(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    norm = torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * (weight / norm)


class _RMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        xc = x.contiguous()
        w32 = weight.detach().float().contiguous()
        y = torch.empty_like(xc)
        rows = xc.numel() // xc.shape[-1] if xc.shape[-1] else 0
        rstd = torch.empty(rows, dtype=torch.float32, device=xc.device)
        _lib.rmsnorm_fwd(xc, w32, y, rstd, eps)
        ctx.save_for_backward(xc, w32, rstd)
        ctx.w_dtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w32, rstd = ctx.saved_tensors
        dyc = dy.contiguous()
        if dyc.dtype != xc.dtype:
            dyc = dyc.to(xc.dtype)
        dx = torch.empty_like(xc)
        dw = torch.empty_like(w32)
        _lib.rmsnorm_bwd(xc, w32, dyc, rstd, dx, dw)
        return dx, dw.to(ctx.w_dtype), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if x.device.type != "cuda":
        raise RuntimeError("rms_norm needs CUDA tensors; there is no CPU path")
    if weight.shape != x.shape[-1:]:
        raise ValueError("weight must have the size of the last axis of x")
    H = x.shape[-1]
    if H % 4 != 0 or x.numel() == 0 or x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return _composed(x, weight, eps)
    return _RMSNormFunction.apply(x, weight, eps)
