"""Inference forward returning the hidden state only, with the reference's name and signature
(``block_scan_forward_3d``, forward_only.py:423-540), served by the CUDA library."""
from __future__ import annotations

import torch

from . import _lib
from . import scan_interface
from .scan_interface import _prepare_inputs


def block_scan_forward_3d(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, BLOCK_L: int = 256,
                          use_naive_if_small: bool = True) -> torch.Tensor:
    """``h`` of shape ``[B, L, D]`` in the dtype of ``x``.

    Any ``L >= 0`` is accepted (the reference needs a power-of-two block count).  ``BLOCK_L`` and
    ``use_naive_if_small`` are accepted and have no effect: short sequences run the same kernel.
    """
    assert x.is_cuda and a.is_cuda and b.is_cuda, "Input tensors must be on a CUDA device."
    assert x.shape == a.shape == b.shape, f"Input shapes must match: x={x.shape}, a={a.shape}, b={b.shape}"
    assert x.dim() == 3, "Input tensors must be 3D (B, L, D)."
    xs, as_, bs, _ = _prepare_inputs(x, a, b, None)
    h = torch.empty(x.shape, dtype=xs.dtype, device=x.device)
    if x.numel() > 0:
        _lib.scan_fwd(xs, as_, bs, None, h, n_seg=scan_interface.DEFAULT_SEGMENTS)
    return h if h.dtype == x.dtype else h.to(x.dtype)
