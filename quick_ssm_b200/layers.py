"""Caller of the scan: the gated SSM block and its RMS norm, with the constructor and forward
signatures of the reference's ``quick_ssm/layers.py`` (``RMSNorm`` :9-17, ``SSM`` :20-107) so
that the reference's training and example scripts run against this package unchanged.  The
projections stay in torch (cuBLAS GEMMs); only the scan goes through the CUDA library."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .scan_interface import scan


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5, dtype=torch.float32, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rms = torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return x * (self.weight / rms)


class RMSNormFused(RMSNorm):
    """``RMSNorm`` through the normalisation kernels (``norm.rms_norm``): same parameter, same
    result up to fp32 rounding, one kernel per direction instead of torch's element-wise chain."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.device.type != "cuda":
            return super().forward(x)
        from .norm import rms_norm
        return rms_norm(x, self.weight, self.eps)


class SSM(nn.Module):
    """Pre-norm, five input projections (decay, input, two halves of a SwiGLU output gate, input
    gate), the scan over the state dimension, output projection, residual."""

    def __init__(self, hidden_size: int, state_size_mult: float = 1.0, eps: float = 1e-5,
                 dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None,
                 compute_dtype: torch.dtype = torch.float16, use_residual: bool = True, use_norm: bool = True):
        super().__init__()
        self.hidden_size = hidden_size
        self.state_size_dim = int(hidden_size * state_size_mult)
        self.compute_dtype = compute_dtype
        self.use_residual = use_residual
        self.use_norm = use_norm
        kw = dict(device=device, dtype=dtype)
        n = self.state_size_dim
        self.A_proj = nn.Linear(hidden_size, n, bias=True, **kw)
        self.B_proj = nn.Linear(hidden_size, n, bias=False, **kw)
        self.C_proj_a = nn.Linear(hidden_size, n, bias=False, **kw)
        self.C_proj_b = nn.Linear(hidden_size, n, bias=False, **kw)
        self.D_proj = nn.Linear(hidden_size, n, bias=False, **kw)
        self.out_proj = nn.Linear(n, hidden_size, bias=True, **kw)
        self.pre_norm = RMSNorm(hidden_size, eps=eps, dtype=dtype, device=device) if use_norm else nn.Identity()

    def forward(self, x: torch.Tensor, *, block_l: int = 256, checkpoint: bool = True,
                tile_b: Optional[int] = None, tile_d: Optional[int] = None, backend: str = "auto",
                scan_out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        skip = x if self.use_residual else 0
        u = self.pre_norm(x) if self.use_norm else x
        cd = self.compute_dtype
        decay = torch.sigmoid(self.A_proj(u)).to(cd)
        drive = self.B_proj(u).to(cd)
        out_gate = (F.silu(self.C_proj_a(u)) * self.C_proj_b(u)).to(cd)
        in_gate = torch.sigmoid(self.D_proj(u)).to(cd)
        if scan_out_dtype is None:
            scan_out_dtype = self.out_proj.weight.dtype
        h = scan(x=drive, a=decay, b=in_gate, c=out_gate, block_l=block_l, checkpoint=checkpoint,
                 tile_b=tile_b, tile_d=tile_d, out_dtype=scan_out_dtype, backend=backend)
        return self.out_proj(h.to(self.out_proj.weight.dtype)) + skip


class SSMFused(SSM):
    """``SSM`` with the gate activations fused into the scan kernels (``gated.gated_scan``) and the
    pre-norm done by the normalisation kernels (``norm.rms_norm``): same parameters, same arguments,
    same result up to the rounding of the activations; the element-wise kernels around the
    projections, and their backward, disappear."""

    def forward(self, x: torch.Tensor, *, block_l: int = 256, checkpoint: bool = True,
                tile_b: Optional[int] = None, tile_d: Optional[int] = None, backend: str = "auto",
                scan_out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if backend == "torch" or x.device.type != "cuda" or not checkpoint:
            return super().forward(x, block_l=block_l, checkpoint=checkpoint, tile_b=tile_b, tile_d=tile_d,
                                   backend=backend, scan_out_dtype=scan_out_dtype)
        from .gated import gated_scan
        skip = x if self.use_residual else 0
        if self.use_norm:  # the normalisation kernels on the layer's own weight
            from .norm import rms_norm
            u = rms_norm(x, self.pre_norm.weight, self.pre_norm.eps)
        else:
            u = x
        if scan_out_dtype is None:
            scan_out_dtype = self.out_proj.weight.dtype
        h = gated_scan(self.A_proj(u), self.B_proj(u), self.C_proj_a(u), self.C_proj_b(u), self.D_proj(u),
                       gate_dtype=self.compute_dtype, out_dtype=scan_out_dtype)
        return self.out_proj(h.to(self.out_proj.weight.dtype)) + skip


__all__ = ["SSM", "SSMFused", "RMSNorm", "RMSNormFused"]
