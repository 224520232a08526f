"""Kernel-level forward entry point with the reference's name and signature
(``block_scan_forward_3d``, triton_forwards.py:134-172), served by the CUDA library."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib
from . import scan_interface


def block_scan_forward_3d(x, a, b, BLOCK_L=256) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(out_a, out_x)``, both fp32 ``[B, L, D]``: the running product of ``a`` and the
    hidden state ``h``.  ``BLOCK_L`` is accepted and has no effect on the result.

    ``out_a`` is produced by the same kernel: with ``b*x = 0`` and a unit start state the
    recurrence reduces to ``h(t) = a(t) h(t-1)``, the cumulative product.
    """
    for t in (x, a, b):
        assert t.dim() == 3, "All inputs should be [B, L, D]."
        assert t.device.type == "cuda", "Inputs must be on CUDA device."
    B, L, D = x.shape
    if L == 0:
        return torch.empty_like(a), torch.empty_like(x)
    xs, as_, bs = (t.contiguous().float() for t in (x, a, b))
    out_x = torch.empty_like(xs)
    _lib.scan_fwd(xs, as_, bs, None, out_x, n_seg=scan_interface.DEFAULT_SEGMENTS)
    zeros = torch.zeros_like(xs)
    ones = torch.ones((B, D), dtype=torch.float32, device=xs.device)
    out_a = torch.empty_like(xs)
    _lib.scan_fwd(zeros, as_, zeros, None, out_a, h_in=ones, n_seg=scan_interface.DEFAULT_SEGMENTS)
    return out_a, out_x
