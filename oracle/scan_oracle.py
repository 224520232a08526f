"""ctypes front end of the CPU oracle (``scan_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Importers are the test-suite, the smoke run and the
CPU-baseline / reference legs of the benchmark.  The CUDA product path never
imports this module.

The C file restates the sequential loops of the reference's
``quick_ssm/naive_baseline.py`` (``naive_forward_3d`` :12-40, ``naive_full_3d``
:43-64, ``naive_backward_3d`` :67-137).  This wrapper only moves numpy/torch
buffers in and out; all arithmetic happens in C.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "scan_oracle.c")
_SO = os.path.join(_HERE, "libscan_oracle.so")

_lib = None


def build(force: bool = False) -> str:
    """Compile ``scan_oracle.c`` with gcc (OpenMP, no FMA contraction)."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
           "-o", _SO, _SRC]
    subprocess.check_call(cmd)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def _np(t, dtype) -> np.ndarray:
    """Any array-like (torch CPU tensor of any float dtype, numpy) -> contiguous numpy of dtype."""
    if t is None:
        return None
    if hasattr(t, "detach"):
        t = t.detach().cpu()
        if str(t.dtype) in ("torch.bfloat16", "torch.float16"):
            t = t.float()
        t = t.numpy()
    return np.ascontiguousarray(t, dtype=dtype)


def _ptr(arr: Optional[np.ndarray]):
    return None if arr is None else arr.ctypes.data_as(ctypes.c_void_p)


def _suffix(dtype) -> str:
    return {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[np.dtype(dtype)]


def scan_forward(x, a, b, c=None, *, dtype=np.float64, h_in=None
                 ) -> Tuple[np.ndarray, Optional[np.ndarray], np.ndarray]:
    """Sequential forward. Returns ``(h, y or None, h_last[B,D])`` in ``dtype``."""
    x, a, b, c, h_in = (_np(v, dtype) for v in (x, a, b, c, h_in))
    B, L, D = x.shape
    h = np.empty_like(x)
    y = np.empty_like(x) if c is not None else None
    h_last = np.empty((B, D), dtype=dtype)
    fn = getattr(lib(), "oracle_scan_fwd_" + _suffix(dtype))
    fn(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(h_in), _ptr(h), _ptr(y), _ptr(h_last),
       ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(D))
    return h, y, h_last


def scan_backward(x, a, b, c, dy, *, dtype=np.float64, h=None, h_in=None, g_in=None):
    """Sequential backward for the loss ``sum(y*dy)``.

    ``h`` defaults to a recompute with the same accumulation width, as the
    reference does (naive_baseline.py:96).  Returns ``(dx, da, db, dc, g_first)``
    where ``g_first[B,D] = a(0)*dh(0)`` is the carry a sequence shard hands to
    the shard before it.
    """
    x, a, b, c, dy, h, h_in, g_in = (_np(v, dtype) for v in (x, a, b, c, dy, h, h_in, g_in))
    B, L, D = x.shape
    if h is None:
        h, _, _ = scan_forward(x, a, b, None, dtype=dtype, h_in=h_in)
    dx, da, db, dc = (np.empty_like(x) for _ in range(4))
    g_first = np.empty((B, D), dtype=dtype)
    fn = getattr(lib(), "oracle_scan_bwd_" + _suffix(dtype))
    fn(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(h), _ptr(h_in), _ptr(dy), _ptr(g_in),
       _ptr(dx), _ptr(da), _ptr(db), _ptr(dc), _ptr(g_first),
       ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(D))
    return dx, da, db, dc, g_first


def scan_forward_backward_inplace(x, a, b, c, dy, h_scratch, y, dx, da, db, dc) -> None:
    """Timed leg of the CPU baseline: all buffers preallocated numpy arrays of one dtype."""
    B, L, D = x.shape
    fn = getattr(lib(), "oracle_scan_fwd_bwd_" + _suffix(x.dtype))
    fn(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(dy), _ptr(h_scratch), _ptr(y),
       _ptr(dx), _ptr(da), _ptr(db), _ptr(dc),
       ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(D))


def scan_forward_blockwise(x, a, b, block_l: int = 256) -> np.ndarray:
    """Blockwise (local scan, carry scan, fix-up) float64 forward; returns h."""
    x, a, b = (_np(v, np.float64) for v in (x, a, b))
    B, L, D = x.shape
    h = np.empty_like(x)
    lib().oracle_scan_fwd_blockwise_f64(_ptr(x), _ptr(a), _ptr(b), _ptr(h),
                                        ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(D),
                                        ctypes.c_int64(block_l))
    return h
