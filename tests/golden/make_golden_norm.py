"""Generates the RMS-norm fixtures of this folder from the REFERENCE module.

    PYTHONPATH=/path/to/quick_ssm python tests/golden/make_golden_norm.py

Imports ``quick_ssm.layers.RMSNorm`` (layers.py:9-17), runs it on small seeded inputs in fp64 and
fp32 and stores inputs, output and the autograd gradients for loss = sum(y * dy).
"""
import os

import numpy as np
import torch

from quick_ssm.layers import RMSNorm  # the reference

HERE = os.path.dirname(os.path.abspath(__file__))


def case(name, shape, dtype, seed, eps):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g, dtype=dtype).requires_grad_()
    dy = torch.randn(*shape, generator=g, dtype=dtype)
    m = RMSNorm(shape[-1], eps=eps, dtype=dtype)
    with torch.no_grad():
        m.weight.copy_(torch.randn(shape[-1], generator=g, dtype=dtype) * 0.5 + 1.0)
    y = m(x)
    (y * dy).sum().backward()
    np.savez(os.path.join(HERE, name + ".npz"), x=x.detach().numpy(), w=m.weight.detach().numpy(), dy=dy.numpy(),
             y=y.detach().numpy(), dx=x.grad.numpy(), dw=m.weight.grad.numpy(), eps=np.float64(eps))
    print(name, shape, dtype)


if __name__ == "__main__":
    case("rmsnorm_f64_3x5x36", (3, 5, 36), torch.float64, 0, 1e-5)
    case("rmsnorm_f32_2x7x128", (2, 7, 128), torch.float32, 1, 1e-5)
    case("rmsnorm_f32_4x1032", (4, 1032), torch.float32, 2, 1e-6)
