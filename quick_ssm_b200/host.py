"""Scan on HOST buffers: pinned host memory in, pinned host memory out.

The kernels work on device memory.  A caller whose tensors live in host memory (a data
loader, an offloaded activation store, another runtime calling through the C ABI) pays for
the PCIe transfers; this module overlaps them with the kernels by cutting the batch axis into
slices and running three streams (host->device copies, kernels, device->host copies) over a
small ring of device buffers.  Channels and batch entries are independent recurrences, so
slicing the batch changes no value.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import _lib

_IN = ("x", "a", "b", "c", "dy")
_OUT = ("y", "dx", "da", "db", "dc")


def alloc_pinned(B: int, L: int, D: int, dtype: torch.dtype, out_dtype: Optional[torch.dtype] = None
                 ) -> Dict[str, torch.Tensor]:
    """Pinned host buffers for one forward+backward: inputs x, a, b, c, dy and results y, dx, da, db, dc."""
    out_dtype = out_dtype or dtype
    bufs = {}
    for name in _IN + _OUT:
        dt = out_dtype if name in ("dy", "y") else dtype
        bufs[name] = torch.empty((B, L, D), dtype=dt).pin_memory()
    return bufs


class HostScan:
    """Forward + backward scan over pinned host buffers, pipelined over batch slices."""

    def __init__(self, B: int, L: int, D: int, dtype: torch.dtype, out_dtype: Optional[torch.dtype] = None,
                 device="cuda", batch_slice: Optional[int] = None, ring: int = 3):
        self.B, self.L, self.D = B, L, D
        self.dtype, self.out_dtype = dtype, out_dtype or dtype
        self.device = torch.device(device)
        self.bs = batch_slice or max(1, B // 8)
        self.ring = ring
        nt = (L + _lib.tile_rows() - 1) // _lib.tile_rows()
        self.sets = []
        for _ in range(ring):
            s = {}
            for name in _IN + _OUT:
                dt = self.out_dtype if name in ("dy", "y") else dtype
                s[name] = torch.empty((self.bs, L, D), dtype=dt, device=self.device)
            s["tile_h"] = torch.empty((self.bs, nt, D), dtype=torch.float32, device=self.device)
            self.sets.append(s)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_k = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.kernel_launches = 0
        # last users of every device buffer set, kept across calls so that consecutive calls overlap
        self._drained = [None] * ring   # D2H of the slice that last used a set
        self._computed = [None] * ring  # kernels of the slice that last used a set
        self._next = 0

    @property
    def h2d_bytes(self) -> int:
        n = self.B * self.L * self.D
        return n * (4 * torch.empty((), dtype=self.dtype).element_size()
                    + torch.empty((), dtype=self.out_dtype).element_size())

    @property
    def d2h_bytes(self) -> int:
        return self.h2d_bytes  # y in out_dtype + four gradients in the input dtype

    def run(self, host: Dict[str, torch.Tensor], compute: bool = True) -> torch.cuda.Event:
        """Enqueue one forward+backward over ``host`` (see ``alloc_pinned``) and return the event that
        marks its last device->host copy.  The call does not wait: the caller synchronises on the
        event (or the device) before reading the results.  The input buffers must stay unchanged
        until then; consecutive calls overlap their transfers.

        ``compute=False`` runs the same copies without the kernels - the transfer-only time the
        pipeline cannot beat, for benchmarks."""
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)  # whatever produced the host-visible inputs on this stream
        drained, computed = self._drained, self._computed
        last = None
        for lo in range(0, self.B, self.bs):
            hi = min(lo + self.bs, self.B)
            n = hi - lo
            k = self._next
            self._next = (k + 1) % self.ring
            dev = self.sets[k]
            with torch.cuda.stream(self.s_in):
                if computed[k] is not None:
                    self.s_in.wait_event(computed[k])  # inputs of this set are no longer being read
                for name in _IN:
                    dev[name][:n].copy_(host[name][lo:hi], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(loaded)
                if drained[k] is not None:
                    self.s_k.wait_event(drained[k])  # results of this set have left the device
                v = {name: t[:n] for name, t in dev.items()}
                if compute:
                    _lib.scan_fwd(v["x"], v["a"], v["b"], v["c"], v["y"], tile_h=v["tile_h"])
                    _lib.scan_bwd(v["x"], v["a"], v["b"], v["c"], v["dy"], v["dx"], v["da"], v["db"], v["dc"],
                                  tile_h=v["tile_h"])
                    self.kernel_launches += 2
                done = torch.cuda.Event()
                done.record(self.s_k)
                computed[k] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for name in _OUT:
                    host[name][lo:hi].copy_(dev[name][:n], non_blocking=True)
                out = torch.cuda.Event()
                out.record(self.s_out)
                drained[k] = out
                last = out
        return last
