"""Kernel-level backward entry point with the reference's name and signature
(``block_scan_backward_3d``, triton_backwards.py:168-209), served by the CUDA library."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib
from . import scan_interface


def block_scan_backward_3d(a, b, c, x, h, grad_y, BLOCK_L=256) -> Tuple[torch.Tensor, ...]:
    """Gradients ``(dx, da, db, dc)`` in fp32 given the hidden states ``h`` of the forward.
    ``BLOCK_L`` is accepted and has no effect on the result."""
    for t in (a, b, c, x, h, grad_y):
        assert t.dim() == 3, "All inputs should be [B, L, D]."
        assert t.device.type == "cuda", "Inputs must be on CUDA device."
    B, L, D = x.shape
    if L == 0:
        return torch.empty_like(x), torch.empty_like(a), torch.empty_like(b), torch.empty_like(c)
    as_, bs, cs, xs, hs, gy = (t.detach().contiguous().float() for t in (a, b, c, x, h, grad_y))
    dx, da, db, dc = (torch.empty_like(xs) for _ in range(4))
    _lib.scan_bwd(xs, as_, bs, cs, gy, dx, da, db, dc, h_saved=hs, n_seg=scan_interface.DEFAULT_SEGMENTS)
    return dx, da, db, dc
