"""Build recipe for the C-ABI library (``libqssm.so``): one nvcc call, sm_100a only.

Run ``python -m quick_ssm_b200.build`` (add ``--force`` to rebuild, ``-v`` for ptxas
resource usage).  The library links the CUDA runtime statically and resolves the one driver
entry point it needs at run time, so it loads on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(_PKG, "csrc", "qssm.cu")
HEADER = os.path.join(os.path.dirname(_PKG), "include", "qssm.h")
LIB = os.path.join(_PKG, "libqssm.so")


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    csrc = os.path.dirname(SRC)
    return [os.path.join(csrc, f) for f in sorted(os.listdir(csrc)) if f.endswith((".cu", ".cuh"))] + [HEADER]


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > built for p in _sources())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-o", LIB, SRC]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    extra = os.environ.get("QSSM_NVCC_FLAGS")  # e.g. -DQSSM_RESIDENT_SWEEP for measurement builds
    if extra:
        cmd[1:1] = extra.split()
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
