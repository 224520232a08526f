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

    def __init__(self, peer: Optional["PeerCarryExchange"] = None):
        self.peer = peer     # carry exchange through peer memory instead of an all-gather (optional)
        self._ws_fwd = None  # (workspace, segments) left by aggregate_fwd for the next forward
        self._ws_bwd = None
        self._ws_cache = {}

    def _segments(self, t, which):
        B, L, D = t.shape
        k = _lib.auto_segments(B, L, D, t.dtype)
        if k <= 1:
            return k, None
        key = (which, t.device, B, k, D)
        ws = self._ws_cache.get(key)
        if ws is None:
            ws = torch.empty(3 * B * k * D * 4, dtype=torch.uint8, device=t.device)
            self._ws_cache[key] = ws
        return k, ws

    def aggregate_fwd(self, x, a, b, A, H):
        """(A, H) [B, D] fp32 views receive (prod a, end state from a zero start)."""
        k, ws = self._segments(x, "f")
        _lib.aggregate_fwd(x, a, b, A, H, n_seg=k, ws=ws)
        self._ws_fwd = (ws, k) if k > 1 else None

    def aggregate_bwd(self, a, c, dy, P, Q):
        """(P, Q) [B, D] fp32 views receive (prod a, a(t0)*dh(t0) from a zero carry)."""
        k, ws = self._segments(a, "b")
        _lib.aggregate_bwd(a, c, dy, P, Q, n_seg=k, ws=ws)
        self._ws_bwd = (ws, k) if k > 1 else None

    def fold(self, A, H, upto: int, reverse: bool):
        """A, H: [G, B, D] views (any stride between ranks) of the gathered aggregates."""
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


class TorchComm:
    """The one collective a sequence shard needs, over a ``torch.distributed`` process group."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_gather(self, full: torch.Tensor, send: torch.Tensor) -> None:
        """``full[r] = send of rank r`` for every rank r; ordered on the calling stream."""
        dist.all_gather_into_tensor(full.view(-1, *send.shape[1:]), send, group=self.group)


def _as_comm(group):
    return group if hasattr(group, "all_gather") else TorchComm(group)


class Exchange:
    """The carry exchange of one direction: a ``[2, B, D]`` send buffer the aggregate kernel writes
    into, one all-gather into a ``[G, 2, B, D]`` buffer, and views of that buffer for the fold - no
    packing, stacking or copies around the collective.  Buffers are kept per (direction, device,
    B, D, communicator) and reused from call to call: every user is ordered on the calling stream
    (the collective makes that stream wait for it)."""

    _cache = {}

    def __init__(self, comm, which: str, B: int, D: int, device):
        self.comm = comm
        key = (which, str(device), B, D, comm.world, id(getattr(comm, "group", comm)))
        bufs = Exchange._cache.get(key)
        if bufs is None:
            send = torch.empty((2, B, D), dtype=torch.float32, device=device)
            full = torch.empty((comm.world, 2, B, D), dtype=torch.float32, device=device)
            bufs = Exchange._cache[key] = (send, full)
        self.send, self.full = bufs

    def set_identity(self):
        self.send[0].fill_(1.0)
        self.send[1].zero_()

    def gather(self):
        """Returns the ``[G, B, D]`` views (first, second) of every rank's pair."""
        self.comm.all_gather(self.full, self.send)
        return self.full[:, 0], self.full[:, 1]


class PeerCarryExchange:
    """Carry exchange of sequence shards through peer memory instead of an all-gather.

    Every rank allocates an inbox (aggregate pairs of all ranks, four slots, and their flags) from
    torch's symmetric memory: a ``cuMemCreate`` allocation whose handle the ranks of ``group`` (all
    on one node) exchange and map with access for their OWN device, so a kernel on this rank's GPU
    may store into any rank's inbox over NVLink.  ``carry_in`` then is two small kernels on the calling stream: ``qssm_carry_push`` stores this rank's pair into
    every inbox and raises its flag there; ``qssm_carry_wait_fold`` waits - bounded - for every
    rank's pair and folds those it depends on in rank order, the same arithmetic as
    ``qssm_carry_fold`` on gathered pairs, so results are bit-identical to the all-gather path.
    No collective, no host synchronisation, no multicast, no bulk copies on peer memory.  All ranks
    must call ``carry_in`` the same number of times per direction.
    """

    def __init__(self, group, n_chan: int, device, wait_ms: int = 2000):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all it needs
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks")
        self.n_chan, self.wait_ms = int(n_chan), int(wait_ms)
        self.device = torch.device(device)
        nbytes = _lib.peer_inbox_bytes(self.world, self.n_chan)
        self.inbox = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.inbox.zero_()
        self._handle = symm_mem.rendezvous(self.inbox, group)
        self.inbox_ptrs = [int(p) for p in self._handle.buffer_ptrs]
        if self.inbox_ptrs[self.rank] != self.inbox.data_ptr():
            raise RuntimeError("symmetric memory: the local buffer is not at its own mapping")
        self.counters = torch.zeros(max(self.world, 32), dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # every inbox is zeroed and mapped before the first push
        self.epoch = [0, 0]  # per direction

    def carry_in(self, first: torch.Tensor, second: torch.Tensor, reverse: bool) -> torch.Tensor:
        d = 1 if reverse else 0
        self.epoch[d] += 1
        epoch = self.epoch[d]
        slot = 2 * d + (epoch & 1)
        carry = torch.empty_like(first)
        _lib.carry_push(first, second, self.inbox_ptrs, self.counters, self.rank, slot, epoch)
        _lib.carry_wait_fold(self.inbox_ptrs[self.rank], self.n_chan, self.rank, self.world, slot, epoch, reverse,
                             carry, wait_ms=self.wait_ms)
        return carry


def _carry_in(ops, comm, ex: "Exchange", reverse: bool):
    """State entering this rank's shard: through the peer exchange when the ops carry one, else one
    all-gather and a fold."""
    peer = getattr(ops, "peer", None)
    if peer is not None:
        return peer.carry_in(ex.send[0], ex.send[1], reverse)
    first_all, second_all = ex.gather()
    return ops.fold(first_all, second_all, comm.rank, reverse)


def forward_aggregate(ops, comm, xs, as_, bs) -> Exchange:
    """First half of a shard's forward: its aggregate, written into the send buffer of the exchange."""
    B, L, D = xs.shape
    ex = Exchange(comm, "f", B, D, xs.device)
    # Nobody folds the last shard's aggregate, but that rank computes it all the same: the pass leaves the
    # per-segment aggregates its own seeded scan reuses, and with identical work on every rank nobody waits
    # at the exchange for a rank that started late.  (Skipping it was measured slower: the rank idles while
    # the others aggregate and then scans without the segment aggregates.)  A lone rank has nobody to wait for.
    if comm.world == 1:
        ex.set_identity()
    else:
        ops.aggregate_fwd(xs, as_, bs, ex.send[0], ex.send[1])
    return ex


def forward_finish(ops, comm, ex: Exchange, xs, as_, bs, cs, y, tile_h, mark=lambda: None):
    """Second half: all-gather, fold the shards before this one into ``h_in``, seeded scan."""
    h_in = _carry_in(ops, comm, ex, False)
    mark()
    ops.forward(xs, as_, bs, cs, y, tile_h, h_in)


def backward_aggregate(ops, comm, as_, cs, dy) -> Exchange:
    B, L, D = as_.shape
    ex = Exchange(comm, "b", B, D, as_.device)
    if comm.world == 1:  # see forward_aggregate: the first shard's aggregate is computed too
        ex.set_identity()
    else:
        ops.aggregate_bwd(as_, cs, dy, ex.send[0], ex.send[1])
    return ex


def backward_finish(ops, comm, ex: Exchange, xs, as_, bs, cs, dy, tile_h, grads, mark=lambda: None):
    g_in = _carry_in(ops, comm, ex, True)
    mark()
    ops.backward(xs, as_, bs, cs, dy, tile_h, g_in, grads)


def shard_forward(ops, group, xs, as_, bs, cs, k_out, keep_boundaries: bool, *, y=None, tile_h=None, marks=None):
    """Forward of one sequence shard (no autograd): returns ``(y, tile_h or None)``.

    ``group``: a process group (or None for the default one), or any object with ``rank``,
    ``world`` and ``all_gather(full, send)``.  ``y`` / ``tile_h`` may be passed in preallocated.
    ``marks``, if a list, receives four CUDA events on the calling stream: start, aggregate done,
    exchange and fold done, scan done."""
    comm = _as_comm(group)
    B, L, D = xs.shape
    mark = (lambda: marks.append(_event(xs.device))) if marks is not None else (lambda: None)
    mark()
    ex = forward_aggregate(ops, comm, xs, as_, bs)
    mark()
    if y is None:
        y = torch.empty((B, L, D), dtype=k_out, device=xs.device)
    if keep_boundaries and tile_h is None:
        tile_h = torch.empty((B, _n_tiles(L), D), dtype=torch.float32, device=xs.device)
    forward_finish(ops, comm, ex, xs, as_, bs, cs, y, tile_h if keep_boundaries else None, mark)
    mark()
    return y, (tile_h if keep_boundaries else None)


def shard_backward(ops, group, xs, as_, bs, cs, dy, tile_h, *, grads=None, marks=None):
    """Backward of one sequence shard (no autograd): returns ``[dx, da, db, dc]`` in the input dtype."""
    comm = _as_comm(group)
    mark = (lambda: marks.append(_event(xs.device))) if marks is not None else (lambda: None)
    mark()
    ex = backward_aggregate(ops, comm, as_, cs, dy)
    mark()
    if grads is None:
        grads = [torch.empty(xs.shape, dtype=xs.dtype, device=xs.device) for _ in range(4)]
    backward_finish(ops, comm, ex, xs, as_, bs, cs, dy, tile_h, grads, mark)
    mark()
    return grads


def _event(device):
    ev = torch.cuda.Event(enable_timing=True)
    ev.record(torch.cuda.current_stream(device))
    return ev


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
