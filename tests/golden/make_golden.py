"""Generates the golden fixtures of this folder from the REFERENCE implementation.

Run in a checkout where the reference project (samblouir/quick_ssm) is importable:

    PYTHONPATH=/path/to/quick_ssm python tests/golden/make_golden.py

It imports the reference's ``quick_ssm.naive_baseline`` (the sequential CPU implementation the
reference's own tests use as ground truth) and stores inputs and outputs of small cases as
``.npz`` files.  The cases follow the reference's tests: shapes, seeds and distributions of
test_forwards.py:23-90,108-114, test_backwards.py:26-116,120-125 and test_scan_interface.py:7-31,
plus odd shapes and the CPU benchmark configuration (B=4, L=2048, D=16; three channels kept).
The fixtures travel with the repository; the reference does not.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from quick_ssm.naive_baseline import naive_backward_3d, naive_forward_3d, naive_full_3d  # the reference

from quick_ssm_b200.synth import make_inputs


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach()
            v = v.float().numpy() if v.dtype in (torch.float16, torch.bfloat16) else v.numpy()
        out[k] = v
    np.savez(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def forward_case(name, shape, seed):
    """test_forwards.py: torch.manual_seed, x=randn, a=rand*0.1+0.9, b=randn*0.1; h from the naive loop."""
    torch.manual_seed(seed)
    x = torch.randn(*shape)
    a = torch.rand(*shape) * 0.1 + 0.9
    b = torch.randn(*shape) * 0.1
    save(name, x=x, a=a, b=b, h=naive_forward_3d(x, a, b))


def backward_case(name, shape, seed):
    """test_backwards.py: c ~ N(0,1); gradients by autograd through naive_full_3d with loss sum(y*dy)."""
    torch.manual_seed(seed)
    x = torch.randn(*shape, requires_grad=True)
    a = (torch.rand(*shape) * 0.1 + 0.9).requires_grad_()
    b = torch.randn(*shape, requires_grad=True)
    c = torch.randn(*shape, requires_grad=True)
    dy = torch.randn(*shape)
    h, y = naive_full_3d(x, a, b, c)
    (y * dy).sum().backward()
    loop = naive_backward_3d(x.detach(), a.detach(), b.detach(), c.detach(), dy)
    save(name, x=x, a=a, b=b, c=c, dy=dy, h=h, y=y, dx=x.grad, da=a.grad, db=b.grad, dc=c.grad,
         dx_loop=loop[0], da_loop=loop[1], db_loop=loop[2], dc_loop=loop[3])


def full_case(name, inp, keep=None, f64=True):
    x, a, b, c, dy = inp.x, inp.a, inp.b, inp.c, inp.dy
    h, y = naive_full_3d(x, a, b, c)
    g = naive_backward_3d(x, a, b, c, dy)
    arrays = dict(x=x, a=a, b=b, c=c, dy=dy, h=h, y=y, dx=g[0], da=g[1], db=g[2], dc=g[3])
    if f64:
        xd, ad, bd, cd, dyd = (t.double() for t in (x, a, b, c, dy))
        h64, y64 = naive_full_3d(xd, ad, bd, cd)
        g64 = naive_backward_3d(xd, ad, bd, cd, dyd)
        arrays.update(h64=h64, y64=y64, dx64=g64[0], da64=g64[1], db64=g64[2], dc64=g64[3])
    if keep is not None:
        arrays = {k: v[:, :, keep] for k, v in arrays.items()}
        arrays["channels"] = np.asarray(keep)
    save(name, **arrays)


def half_case(name, shape, dtype, seed):
    """The reference's scan on 16-bit inputs: fp32 accumulation, h rounded to the input dtype, y = c*h
    in the input dtype (naive_baseline.py:29,40,62)."""
    inp = make_inputs(*shape, dtype=dtype, seed=seed)
    h, y = naive_full_3d(inp.x, inp.a, inp.b, inp.c)
    save(name, x=inp.x, a=inp.a, b=inp.b, c=inp.c, h=h, y=y)


if __name__ == "__main__":
    forward_case("fwd_2x512x8_seed42", (2, 512, 8), 42)
    forward_case("fwd_1x4x1_seed3", (1, 4, 1), 3)
    forward_case("fwd_1x1024x1_seed4", (1, 1024, 1), 4)
    backward_case("bwd_2x2048x8_seed0", (2, 2048, 8), 0)
    backward_case("bwd_1x1024x1_seed0", (1, 1024, 1), 0)
    backward_case("iface_2x32x4_seed0", (2, 32, 4), 0)
    for shape in [(1, 50, 2), (1, 7, 1), (2, 64, 3), (2, 17, 40)]:
        full_case("full_%dx%dx%d" % shape, make_inputs(*shape, dtype=torch.float32, seed=11))
    full_case("cfg0_4x2048x16_ch0_7_15", make_inputs(4, 2048, 16, dtype=torch.float32, seed=0), keep=[0, 7, 15])
    half_case("half_bf16_2x128x8", (2, 128, 8), torch.bfloat16, 5)
    half_case("half_fp16_2x128x8", (2, 128, 8), torch.float16, 5)
