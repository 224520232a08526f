"""Stateful forward scan: feed a sequence in pieces and carry the hidden state between calls.

The recurrence needs nothing from the past except ``h`` at the last step, so inference over a
stream (or token-by-token decoding) is a chain of ordinary forward scans, each seeded with the
state the previous one left (``h_in`` / ``h_last`` of the C ABI).  The reference lists a fast
inference mode as future work; its block scan has no way to pass a state in.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .scan_interface import _kernel_out_dtype, _prepare_inputs


class ScanState:
    """Hidden state ``h`` after the last step seen, ``[B, D]`` fp32 on the device."""

    def __init__(self, h: torch.Tensor):
        if h.dim() != 2 or h.dtype != torch.float32:
            raise ValueError("state must be a [B, D] float32 tensor")
        self.h = h

    @classmethod
    def zeros(cls, batch: int, channels: int, device="cuda") -> "ScanState":
        return cls(torch.zeros((batch, channels), dtype=torch.float32, device=device))

    def clone(self) -> "ScanState":
        return ScanState(self.h.clone())


@torch.no_grad()
def scan_chunk(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor],
               state: Optional[ScanState] = None, *, out_dtype: Optional[torch.dtype] = None
               ) -> Tuple[torch.Tensor, ScanState]:
    """Forward scan over one piece ``[B, L_piece, D]`` of a longer sequence.

    Returns ``(y, new_state)`` with ``y = c*h`` (or ``h`` itself when ``c`` is None).  Passing the
    returned state to the next call continues the same recurrence; the concatenated outputs equal
    one scan over the concatenated inputs up to fp32 rounding of the carried state.
    """
    if x.dim() != 3 or x.shape != a.shape or x.shape != b.shape or (c is not None and c.shape != x.shape):
        raise ValueError("x, a, b, c must share the same shape [B, L, D].")
    B, L, D = x.shape
    if state is not None and tuple(state.h.shape) != (B, D):
        raise ValueError(f"state is {tuple(state.h.shape)}, expected {(B, D)}")
    xs, as_, bs, cs = _prepare_inputs(x, a, b, c)
    out_dtype = out_dtype or x.dtype
    k_out = _kernel_out_dtype(xs.dtype, out_dtype)
    y = torch.empty((B, L, D), dtype=k_out, device=x.device)
    h_last = torch.empty((B, D), dtype=torch.float32, device=x.device)
    _lib.scan_fwd(xs, as_, bs, cs, y, h_in=None if state is None else state.h, h_last=h_last)
    return (y if k_out == out_dtype else y.to(out_dtype)), ScanState(h_last)
