"""Sequential torch restatement of the gated linear scan (test infrastructure only).

Same arithmetic and dtype rules as the reference's CPU path
(quick_ssm/naive_baseline.py): the forward accumulates in fp32 when the inputs
are fp16/bf16 and otherwise in the input dtype (:29), returns ``h`` rounded to
the input dtype (:40); the backward recomputes ``h`` (:96) and carries the
upstream term in the input dtype (:99-101).  Unlike the reference the time loop
is vectorised over the batch, which changes no value.
"""
from __future__ import annotations

import torch


def forward_h(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    acc = torch.float32 if x.dtype in (torch.float16, torch.bfloat16) else x.dtype
    xs, as_, bs = x.to(acc), a.to(acc), b.to(acc)
    B, L, D = x.shape
    out = torch.empty((B, L, D), dtype=acc, device=x.device)
    state = torch.zeros((B, D), dtype=acc, device=x.device)
    for t in range(L):
        state = as_[:, t] * state + bs[:, t] * xs[:, t]
        out[:, t] = state
    return out.to(x.dtype)


def forward_y(x, a, b, c):
    h = forward_h(x, a, b)
    return h, c * h


def backward(x, a, b, c, dy):
    B, L, D = x.shape
    h = forward_h(x, a, b)
    carry = torch.zeros((B, D), dtype=x.dtype, device=x.device)
    dx, da, db, dc = (torch.zeros_like(v) for v in (x, a, b, c))
    zero = torch.zeros((B, D), dtype=x.dtype, device=x.device)
    for t in range(L - 1, -1, -1):
        total = dy[:, t] * c[:, t] + carry
        dc[:, t] = dy[:, t] * h[:, t]
        db[:, t] = total * x[:, t]
        da[:, t] = total * (h[:, t - 1] if t > 0 else zero)
        dx[:, t] = total * b[:, t]
        carry = total * a[:, t]
    return dx, da, db, dc
