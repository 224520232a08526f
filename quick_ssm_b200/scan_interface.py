"""Public scan interface: same names, arguments and error behaviour as the reference's
``quick_ssm/scan_interface.py`` (``scan`` :169-213, ``_TritonScanFunction`` :49-158,
``_chunk_ranges`` :36-46), with the body replaced by the sm_100a kernels behind the C ABI.

    h(t) = a(t) * h(t-1) + b(t) * x(t)        y(t) = c(t) * h(t)        all tensors [B, L, D]

What changed behind the unchanged signature
  * ``backend="auto"`` and ``"triton"`` both mean the CUDA library (the name "triton" is kept
    so existing callers keep working) and raise on CPU tensors: nothing ever falls back to a
    CPU implementation on its own.  ``backend="torch"`` must be asked for by name; it runs a
    plain sequential torch loop that exists for CPU-side tests of callers such as
    ``layers.SSM``, as in the reference (:161-166, :210-211).
  * ``block_l``, ``tile_b`` and ``tile_d`` are accepted and validated but have no effect: the
    kernels keep the carry in registers and need no B*L*D scratch that tiling would bound.
  * ``checkpoint=True`` keeps only the state at every 16th step (fp32, 1/16 of a tensor) and
    rebuilds ``h`` inside the backward kernel; ``checkpoint=False`` stores ``h`` in fp32 in the
    forward and reads it in the backward, as the reference does (:86, :136).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib

Tensor = torch.Tensor

# Number of parallel time segments the kernels use: 0 = let the library decide.  Results are
# the same for every value up to fp32 rounding; tests set it to exercise the segmented path.
DEFAULT_SEGMENTS = 0


def _chunk_ranges(total: int, tile: Optional[int]) -> List[Tuple[int, int]]:
    """Half-open ranges covering ``[0, total)`` in steps of ``tile`` (one range if no tile)."""
    if tile is None or tile <= 0 or tile >= total:
        return [(0, total)]
    return [(lo, min(lo + tile, total)) for lo in range(0, total, tile)]


def _compute_dtype(*ts: Tensor) -> torch.dtype:
    """Storage dtype the kernel runs on: the common 16-bit dtype, else fp32."""
    dts = {t.dtype for t in ts}
    if len(dts) == 1:
        (dt,) = dts
        if dt in (torch.float16, torch.bfloat16, torch.float32):
            return dt
    return torch.float32


def _prepare_inputs(x: Tensor, a: Tensor, b: Tensor, c: Optional[Tensor]):
    """Bring the inputs to one dtype and one addressable layout, copying only when needed."""
    ts = [t for t in (x, a, b, c) if t is not None]
    dt = _compute_dtype(*ts)
    ts = [t if t.dtype == dt else t.to(dt) for t in ts]
    if not (all(_lib.layout_ok(t) for t in ts) and _lib.same_layout(*ts)):
        ts = [t.contiguous() for t in ts]
    if c is None:
        ts.append(None)
    return ts


def _kernel_out_dtype(in_dtype: torch.dtype, out_dtype: torch.dtype) -> torch.dtype:
    return out_dtype if out_dtype in (in_dtype, torch.float32) else torch.float32


def _addressable(t: Tensor) -> Tensor:
    return t if _lib.layout_ok(t) else t.contiguous()


def _n_tiles(L: int) -> int:
    rows = _lib.tile_rows()
    return (L + rows - 1) // rows


class _TritonScanFunction(torch.autograd.Function):
    """Autograd wrapper of the CUDA scan.  Keeps the reference's class name and its nine
    positional inputs / nine-entry gradient tuple (scan_interface.py:49-158)."""

    @staticmethod
    def forward(ctx, x: Tensor, a: Tensor, b: Tensor, c: Tensor, block_l: int, checkpoint: bool,
                tile_b: Optional[int], tile_d: Optional[int], out_dtype: torch.dtype) -> Tensor:
        if x.shape != a.shape or x.shape != b.shape or x.shape != c.shape:
            raise ValueError("x, a, b, c must share the same shape [B, L, D].")
        if x.device.type != "cuda":
            raise RuntimeError("Triton backend requires CUDA tensors.")
        if x.dim() != 3:
            raise ValueError("x, a, b, c must be 3-D tensors [B, L, D].")

        ctx.block_l = int(block_l)
        ctx.checkpoint = bool(checkpoint)
        ctx.tile_b = tile_b
        ctx.tile_d = tile_d
        ctx.out_dtype = out_dtype
        ctx.in_dtypes = (x.dtype, a.dtype, b.dtype, c.dtype)

        B, L, D = x.shape
        xs, as_, bs, cs = _prepare_inputs(x, a, b, c)
        k_out = _kernel_out_dtype(xs.dtype, out_dtype)
        y = torch.empty((B, L, D), dtype=k_out, device=x.device)

        needs_grad = any(ctx.needs_input_grad[:4])
        tile_h = h_saved = None
        if needs_grad and ctx.checkpoint:
            tile_h = torch.empty((B, _n_tiles(L), D), dtype=torch.float32, device=x.device)
        elif needs_grad:
            h_saved = torch.empty((B, L, D), dtype=torch.float32, device=x.device)

        _lib.scan_fwd(xs, as_, bs, cs, y, h_saved=h_saved, tile_h=tile_h, n_seg=DEFAULT_SEGMENTS)

        ctx.k_out = k_out
        ctx.has_tile_h = tile_h is not None
        if needs_grad:
            ctx.save_for_backward(xs, as_, bs, cs, tile_h if tile_h is not None else h_saved)
        ctx.h_saved = h_saved
        return y if k_out == out_dtype else y.to(out_dtype)

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        xs, as_, bs, cs, hstate = ctx.saved_tensors
        dy = grad_output if grad_output.dtype == ctx.k_out else grad_output.to(ctx.k_out)
        dy = _addressable(dy)
        dx, da, db, dc = (torch.empty(xs.shape, dtype=xs.dtype, device=xs.device) for _ in range(4))
        if ctx.has_tile_h:
            _lib.scan_bwd(xs, as_, bs, cs, dy, dx, da, db, dc, tile_h=hstate, n_seg=DEFAULT_SEGMENTS)
        else:
            _lib.scan_bwd(xs, as_, bs, cs, dy, dx, da, db, dc, h_saved=hstate, n_seg=DEFAULT_SEGMENTS)
        dtx, dta, dtb, dtc = ctx.in_dtypes
        return (dx.to(dtx), da.to(dta), db.to(dtb), dc.to(dtc), None, None, None, None, None)


def _torch_scan(x: Tensor, a: Tensor, b: Tensor, c: Tensor, out_dtype: torch.dtype) -> Tensor:
    """Sequential torch loop for CPU-side tests of callers (reference: scan_interface.py:161-166,
    naive_baseline.py:12-40).  fp32 accumulation for 16-bit inputs, ``h`` rounded to the input
    dtype before the output gate, differentiable through plain autograd."""
    acc = torch.float32 if x.dtype in (torch.float16, torch.bfloat16) else x.dtype
    xs, as_, bs = x.to(acc), a.to(acc), b.to(acc)
    B, L, D = x.shape
    state = torch.zeros((B, D), dtype=acc, device=x.device)
    steps = []
    for t in range(L):
        state = as_[:, t] * state + bs[:, t] * xs[:, t]
        steps.append(state)
    h = torch.stack(steps, dim=1) if steps else torch.zeros((B, 0, D), dtype=acc, device=x.device)
    return (c * h.to(x.dtype)).to(out_dtype)


def scan(x: Tensor, a: Tensor, b: Tensor, c: Tensor, *, block_l: int = 256, checkpoint: bool = True,
         tile_b: Optional[int] = None, tile_d: Optional[int] = None, backend: str = "auto",
         out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """Gated linear scan ``y = c * h`` with ``h(t) = a(t) h(t-1) + b(t) x(t)``.

    Args:
        x, a, b, c: tensors of shape ``[B, L, D]``.
        block_l, tile_b, tile_d: accepted for compatibility; the result does not depend on them.
        checkpoint: ``True`` rebuilds ``h`` in the backward kernel, ``False`` stores it in fp32.
        backend: ``"auto"`` or ``"triton"`` (the CUDA kernels; CPU tensors raise) or
            ``"torch"`` (sequential torch loop, only when named explicitly).
        out_dtype: dtype of the result; defaults to ``x.dtype``.
    """
    out_dtype = out_dtype or x.dtype
    chosen = "triton" if backend == "auto" else backend
    if chosen == "triton":
        return _TritonScanFunction.apply(x, a, b, c, block_l, checkpoint, tile_b, tile_d, out_dtype)
    if chosen == "torch":
        return _torch_scan(x, a, b, c, out_dtype)
    raise ValueError(f"Unsupported backend '{backend}'. Use 'auto', 'triton', or 'torch'.")


__all__ = ["scan"]
