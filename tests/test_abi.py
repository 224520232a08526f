"""The C-ABI library loads without a GPU and exports exactly what include/qssm.h declares.
Only argument validation is exercised here (it returns before any CUDA call)."""
import ctypes
import os
import re

import pytest

from quick_ssm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "qssm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(qssm_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert {"qssm_scan_fwd", "qssm_scan_bwd", "qssm_scan_aggregate_fwd", "qssm_scan_aggregate_bwd",
            "qssm_carry_fold", "qssm_workspace_bytes", "qssm_status_string", "qssm_version"} <= names
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in qssm.h but not exported"
    assert names == set(_lib.SIGNATURES), "ctypes signatures and header disagree"


def test_version_and_strings():
    lib = _lib.load()
    assert lib.qssm_version() >= 100
    assert _lib.tile_rows() == 16
    assert _lib.status_string(0) == "ok"
    assert "tile_h" in _lib.status_string(-5)
    assert "expired" in _lib.status_string(10001)


def test_argument_validation_without_gpu():
    lib = _lib.load()
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    args_tail = lambda B, L, D, din, dout: (None, 0, B, L, D, L * D, D, L * D, D, din, dout, 0, None, None)
    fwd = lambda *t: lib.qssm_scan_fwd(one, one, one, one, one, None, None, None, None, *t)
    assert fwd(*args_tail(-1, 4, 4, 0, 0)) == -2          # QSSM_E_SHAPE
    assert fwd(*args_tail(1, 4, 4, 7, 0)) == -3           # QSSM_E_DTYPE
    assert fwd(*args_tail(1, 4, 4, 0, 2)) == -3           # fp32 in, bf16 out: unsupported pair
    assert fwd(*args_tail(1, 0, 4, 0, 0)) == 0            # empty: nothing to do
    assert lib.qssm_scan_fwd(None, one, one, one, one, None, None, None, None, *args_tail(1, 4, 4, 0, 0)) == -1
    assert lib.qssm_scan_fwd(one, one, one, one, one, None, None, None, None,
                             None, 0, 1, 4, 8, 32, 4, 32, 8, 0, 0, 0, None, None) == -4  # row stride < D
    # backward without h source
    assert lib.qssm_scan_bwd(one, one, one, one, one, None, None, None, None, None, one, one, one, one,
                             None, 0, 1, 4, 4, 16, 4, 16, 4, 0, 0, 0, None, None) == -5
    # forced segments without workspace
    assert lib.qssm_scan_fwd(one, one, one, one, one, None, None, None, None,
                             None, 0, 1, 4096, 4, 16384, 4, 16384, 4, 0, 0, 4, None, None) == -6
    # built-in scratch: 3*4*64*2048*4 bytes > 4 MiB
    assert lib.qssm_scan_fwd_static_ws(one, one, one, one, one, None, None, None, None,
                                       4, 16384, 2048, 16384 * 2048, 2048, 16384 * 2048, 2048,
                                       2, 2, 64, None, None) == -8
    # built-in scratch: "aggregates already in ws" cannot be true of the library's own array
    assert lib.qssm_scan_fwd_static_ws(one, one, one, one, one, None, None, None, None,
                                       1, 4096, 64, 4096 * 64, 64, 4096 * 64, 64, 0, 0, -4, None, None) == -2


def test_tuning_knobs_by_name():
    lib = _lib.load()
    assert lib.qssm_tune_set(b"CHUNK_ROWS", 64) == 0
    assert lib.qssm_tune_set(b"QSSM_CHUNK_ROWS", 128) == 0   # the environment spelling is accepted too
    assert lib.qssm_tune_set(b"NO_SUCH_KNOB", 1) == -2
    assert lib.qssm_tune_set(None, 1) == -1
    lib.qssm_tune_reset()
    with pytest.raises(KeyError):
        _lib.tune_set("nope", 1)


def test_workspace_and_segment_policy():
    lib = _lib.load()
    # plenty of chains: no segmentation, no scratch
    assert lib.qssm_auto_segments(8, 8192, 4096, 2) == 1
    assert lib.qssm_workspace_bytes(8, 8192, 4096, 2) == 0
    # long sequence, few channels: segmented
    n = lib.qssm_auto_segments(1, 1 << 20, 2048, 1)
    assert n > 1
    # scratch covers both ways of running it: segment aggregates, or the chunk descriptors of the single-pass kernel
    assert lib.qssm_workspace_bytes(1, 1 << 20, 2048, 1) >= 3 * 1 * n * 2048 * 4
    # short sequences are never cut below 256 rows per segment
    assert lib.qssm_auto_segments(1, 300, 32, 0) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libqssm.so"))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
