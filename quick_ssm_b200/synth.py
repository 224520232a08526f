"""Seeded synthetic inputs for the gated linear scan.

The reference uses no dataset: its tests and demos draw ``x ~ N(0,1)``,
``a = U(0,1)*0.1 + 0.9``, ``b = N(0,1)*0.1`` (test_forwards.py:51-53,
test_scan_interface.py:10-13) and an output gate through a sigmoid.  The
benchmark configurations reuse those distributions, plus a near-unit decay
``a = 1 - 10^U(-4,-1)`` that stresses carry precision on very long sequences.

Every tensor is drawn in fp32 from its own generator (seed + fixed offset) and
then rounded to the storage dtype, so a CPU oracle and a GPU kernel can be fed
bit-identical stored values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_OFFSETS = {"x": 0, "a": 1, "b": 2, "c": 3, "dy": 4}


@dataclass
class ScanInputs:
    x: torch.Tensor
    a: torch.Tensor
    b: torch.Tensor
    c: torch.Tensor
    dy: Optional[torch.Tensor]

    def tensors(self):
        return self.x, self.a, self.b, self.c

    def to(self, device):
        return ScanInputs(*(None if t is None else t.to(device) for t in
                            (self.x, self.a, self.b, self.c, self.dy)))


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def make_inputs(B: int, L: int, D: int, *, dtype: torch.dtype = torch.float32,
                out_dtype: Optional[torch.dtype] = None, device="cpu", seed: int = 0,
                decay: str = "default", with_dy: bool = True, rank: int = 0) -> ScanInputs:
    """Draw one set of scan inputs of shape ``[B, L, D]``.

    decay="default":   a = U(0,1)*0.1 + 0.9
    decay="near_unit": a = 1 - 10^U(-4,-1)
    ``rank`` offsets every seed by 100*rank so shards of a multi-GPU run differ.
    """
    device = torch.device(device)
    shape = (B, L, D)
    base = int(seed) + 100 * int(rank)

    def normal(name):
        return torch.randn(shape, generator=_gen(device, base + _OFFSETS[name]),
                           device=device, dtype=torch.float32)

    def uniform(name):
        return torch.rand(shape, generator=_gen(device, base + _OFFSETS[name]),
                          device=device, dtype=torch.float32)

    x = normal("x")
    if decay == "default":
        a = uniform("a").mul_(0.1).add_(0.9)
    elif decay == "near_unit":
        a = 1.0 - torch.pow(10.0, uniform("a").mul_(3.0).sub_(4.0))
    else:
        raise ValueError(f"unknown decay '{decay}'")
    b = normal("b").mul_(0.1)
    c = torch.sigmoid(normal("c"))
    dy = normal("dy").to(out_dtype or dtype) if with_dy else None
    return ScanInputs(x.to(dtype), a.to(dtype), b.to(dtype), c.to(dtype), dy)


# The five benchmark configurations, as (shape, storage dtype, decay) records.
CONFIGS = {
    "cfg0": dict(B=4, L=2048, D=16, dtype=torch.float32, decay="default"),
    "cfg1": dict(B=8, L=8192, D=4096, dtype=torch.bfloat16, decay="default"),
    "cfg2": dict(B=1, L=1 << 20, D=2048, dtype=torch.float16, decay="near_unit"),
    "cfg3_scan": dict(B=16, L=4096, D=4096, dtype=torch.bfloat16, out_dtype=torch.float32,
                      decay="default"),
    "cfg4": dict(B=64, L=4096, D=8192, dtype=torch.float16, decay="default"),
}


def make_config(name: str, *, device="cpu", seed: int = 0, rank: int = 0, **override) -> ScanInputs:
    kw = dict(CONFIGS[name])
    kw.update(override)
    return make_inputs(device=device, seed=seed, rank=rank, **kw)
