"""Sequence-sharded scan: each rank holds a contiguous range of time steps of the same
``[B, L, D]`` problem (rank r owns steps ``[r*L/G, (r+1)*L/G)``).

The recurrence is linear, so a shard is summarised by two numbers per channel,
``(A, H) = (prod a, end state from a zero start)``: for any incoming state ``h_in`` its end state is
``A*h_in + H``.  Forward: every rank computes its aggregate (one read of x, a, b), the ranks
all-gather them (``2*B*D`` floats per rank - a latency-bound exchange), each rank folds the
aggregates of the ranks before it into its ``h_in`` and runs the normal scan seeded with it.
Backward mirrors this with ``(P, Q) = (prod a, a(t0)*dh(t0) from a zero carry)`` folded over the
ranks after it.  The reference has no multi-GPU code; the combine is its block-carry combine
(triton_forwards.py:26-30) applied across ranks instead of across blocks.

Batch or channel sharding needs none of this: those recurrences are independent, every rank
simply calls ``scan`` on its own shard.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from .scan_interface import _addressable, _kernel_out_dtype, _n_tiles, _prepare_inputs


class CudaShardOps:
    """The five device operations of a sequence shard, through the C ABI.

    When the local shard is itself cut into time segments, the aggregate pass leaves the
    per-segment aggregates in a workspace that the scan call right after it reuses, so the
    tensors the carry depends on are read once for both purposes."""

    def __init__(self):
        self._ws_fwd = None  # (workspace, segments) left by aggregate_fwd for the next forward
        self._ws_bwd = None

    @staticmethod
    def _segments(t):
        B, L, D = t.shape
        k = _lib.auto_segments(B, L, D, t.dtype)
        ws = torch.empty(3 * B * k * D * 4, dtype=torch.uint8, device=t.device) if k > 1 else None
        return k, ws

    def aggregate_fwd(self, x, a, b):
        B, L, D = x.shape
        A = torch.empty((B, D), dtype=torch.float32, device=x.device)
        H = torch.empty_like(A)
        k, ws = self._segments(x)
        _lib.aggregate_fwd(x, a, b, A, H, n_seg=k, ws=ws)
        self._ws_fwd = (ws, k) if k > 1 else None
        return A, H

    def aggregate_bwd(self, a, c, dy):
        B, L, D = a.shape
        P = torch.empty((B, D), dtype=torch.float32, device=a.device)
        Q = torch.empty_like(P)
        k, ws = self._segments(a)
        _lib.aggregate_bwd(a, c, dy, P, Q, n_seg=k, ws=ws)
        self._ws_bwd = (ws, k) if k > 1 else None
        return P, Q

    def fold(self, A, H, upto: int, reverse: bool):
        return _lib.carry_fold(A, H, upto, reverse=reverse)

    def forward(self, x, a, b, c, y, tile_h, h_in):
        if self._ws_fwd is not None:
            ws, k = self._ws_fwd
            self._ws_fwd = None
            _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h, h_in=h_in, n_seg=-k, ws=ws)
        else:
            _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h, h_in=h_in)

    def backward(self, x, a, b, c, dy, tile_h, g_in, grads):
        if self._ws_bwd is not None:
            ws, k = self._ws_bwd
            self._ws_bwd = None
            _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h, g_in=g_in, n_seg=-k, ws=ws)
        else:
            _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h, g_in=g_in)


def _gather(pair, group):
    """All-gather a (first, second) pair of [B, D] fp32 tensors -> two [G, B, D] stacks."""
    packed = torch.stack(pair).contiguous()
    world = dist.get_world_size(group)
    parts = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(parts, packed, group=group)
    full = torch.stack(parts)  # [G, 2, B, D]
    return full[:, 0].contiguous(), full[:, 1].contiguous()


def shard_forward(ops, group, xs, as_, bs, cs, k_out, keep_boundaries: bool):
    """Forward of one sequence shard (no autograd): returns ``(y, tile_h or None)``."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, L, D = xs.shape
    if rank == world - 1:  # nobody comes after the last shard: identity aggregate, no read
        A = torch.ones((B, D), dtype=torch.float32, device=xs.device)
        H = torch.zeros_like(A)
    else:
        A, H = ops.aggregate_fwd(xs, as_, bs)
    A_all, H_all = _gather((A, H), group)
    h_in = ops.fold(A_all, H_all, rank, False)
    y = torch.empty((B, L, D), dtype=k_out, device=xs.device)
    tile_h = torch.empty((B, _n_tiles(L), D), dtype=torch.float32, device=xs.device) if keep_boundaries else None
    ops.forward(xs, as_, bs, cs, y, tile_h, h_in)
    return y, tile_h


def shard_backward(ops, group, xs, as_, bs, cs, dy, tile_h):
    """Backward of one sequence shard (no autograd): returns ``[dx, da, db, dc]`` in the input dtype."""
    rank = dist.get_rank(group)
    B, L, D = xs.shape
    if rank == 0:  # nobody comes before the first shard
        P = torch.ones((B, D), dtype=torch.float32, device=xs.device)
        Q = torch.zeros_like(P)
    else:
        P, Q = ops.aggregate_bwd(as_, cs, dy)
    P_all, Q_all = _gather((P, Q), group)
    g_in = ops.fold(P_all, Q_all, rank, True)
    grads = [torch.empty(xs.shape, dtype=xs.dtype, device=xs.device) for _ in range(4)]
    ops.backward(xs, as_, bs, cs, dy, tile_h, g_in, grads)
    return grads


class _SequenceShardedScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, b, c, group, out_dtype, ops):
        in_dtypes = (x.dtype, a.dtype, b.dtype, c.dtype)
        xs, as_, bs, cs = _prepare_inputs(x, a, b, c)
        k_out = _kernel_out_dtype(xs.dtype, out_dtype)
        needs_grad = any(ctx.needs_input_grad[:4])
        y, tile_h = shard_forward(ops, group, xs, as_, bs, cs, k_out, needs_grad)
        if needs_grad:
            ctx.save_for_backward(xs, as_, bs, cs, tile_h)
        ctx.group, ctx.ops, ctx.k_out, ctx.in_dtypes = group, ops, k_out, in_dtypes
        return y if k_out == out_dtype else y.to(out_dtype)

    @staticmethod
    def backward(ctx, grad_output):
        xs, as_, bs, cs, tile_h = ctx.saved_tensors
        dy = _addressable(grad_output if grad_output.dtype == ctx.k_out else grad_output.to(ctx.k_out))
        grads = shard_backward(ctx.ops, ctx.group, xs, as_, bs, cs, dy, tile_h)
        return tuple(g.to(dt) for g, dt in zip(grads, ctx.in_dtypes)) + (None, None, None)


def scan_sequence_sharded(x, a, b, c, *, group: Optional[dist.ProcessGroup] = None,
                          out_dtype: Optional[torch.dtype] = None, _ops=None) -> torch.Tensor:
    """``scan`` for tensors whose time axis is split across the ranks of ``group`` in rank order.

    Every rank passes its own ``[B, L_local, D]`` shard and gets the matching shard of ``y``;
    gradients flow to the local shards.  One all-gather of ``2*B*D`` floats per rank in each
    direction is the only communication.
    """
    if x.shape != a.shape or x.shape != b.shape or x.shape != c.shape:
        raise ValueError("x, a, b, c must share the same shape [B, L, D].")
    if not dist.is_initialized():
        raise RuntimeError("scan_sequence_sharded needs an initialised torch.distributed process group")
    ops = _ops if _ops is not None else CudaShardOps()
    return _SequenceShardedScan.apply(x, a, b, c, group, out_dtype or x.dtype, ops)


def channel_shard(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's channel range of a ``[B, L, D]`` tensor as a view (no copy, no communication)."""
    D = t.shape[2]
    per = (D + world - 1) // world
    return t[:, :, rank * per:min(D, (rank + 1) * per)]
