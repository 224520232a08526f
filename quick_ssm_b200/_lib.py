"""ctypes binding of ``libqssm.so`` (the C ABI declared in ``include/qssm.h``).

Only device pointers, sizes, strides, dtype codes and the current CUDA stream cross this
boundary; torch is used for memory and streams, never for the arithmetic.  There is no CPU
or eager fallback: if the library is missing, or a tensor is not on a CUDA device, the calls
raise.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional, Tuple

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libqssm.so")

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_c_i64, _c_int, _c_vp, _c_sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/qssm.h declaration by declaration
SIGNATURES = {
    "qssm_version": (_c_int, []),
    "qssm_status_string": (ctypes.c_char_p, [_c_int]),
    "qssm_tune_set": (_c_int, [ctypes.c_char_p, _c_int]),
    "qssm_tune_reset": (None, []),
    "qssm_tile_rows": (_c_int, []),
    "qssm_workspace_bytes": (_c_sz, [_c_i64, _c_i64, _c_i64, _c_int]),
    "qssm_auto_segments": (_c_int, [_c_i64, _c_i64, _c_i64, _c_int]),
    "qssm_scan_fwd": (_c_int, [_c_vp] * 5 + [_c_vp] * 4 + [_c_vp, _c_sz] + [_c_i64] * 3 + [_c_i64] * 4
                      + [_c_int] * 3 + [_c_vp, _c_vp]),
    "qssm_scan_fwd_static_ws": (_c_int, [_c_vp] * 5 + [_c_vp] * 4 + [_c_i64] * 3 + [_c_i64] * 4 + [_c_int] * 3
                                + [_c_vp, _c_vp]),
    "qssm_scan_bwd": (_c_int, [_c_vp] * 5 + [_c_vp] * 5 + [_c_vp] * 4 + [_c_vp, _c_sz] + [_c_i64] * 3
                      + [_c_i64] * 4 + [_c_int] * 3 + [_c_vp, _c_vp]),
    "qssm_gated_scan_fwd": (_c_int, [_c_vp] * 6 + [_c_vp] * 3 + [_c_i64] * 3 + [_c_i64] * 4 + [_c_int] * 3
                            + [_c_vp, _c_vp]),
    "qssm_gated_scan_bwd": (_c_int, [_c_vp] * 6 + [_c_vp] * 3 + [_c_vp] * 5 + [_c_i64] * 3 + [_c_i64] * 4
                            + [_c_int] * 3 + [_c_vp, _c_vp]),
    "qssm_scan_aggregate_fwd": (_c_int, [_c_vp] * 3 + [_c_vp] * 2 + [_c_vp, _c_sz] + [_c_i64] * 3 + [_c_i64] * 2
                                + [_c_int] * 2 + [_c_vp, _c_vp]),
    "qssm_scan_aggregate_bwd": (_c_int, [_c_vp] * 3 + [_c_vp] * 2 + [_c_vp, _c_sz] + [_c_i64] * 3 + [_c_i64] * 4
                                + [_c_int] * 3 + [_c_vp, _c_vp]),
    "qssm_carry_fold": (_c_int, [_c_vp, _c_vp, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_vp, _c_vp, _c_vp]),
    "qssm_peer_inbox_bytes": (_c_sz, [_c_int, _c_i64]),
    "qssm_peer_flags_offset": (_c_sz, [_c_int, _c_i64]),
    "qssm_carry_push": (_c_int, [_c_vp, _c_vp, _c_i64, _c_vp, _c_vp] + [_c_int] * 4 + [_c_vp]),
    "qssm_carry_wait_fold": (_c_int, [_c_vp, _c_i64] + [_c_int] * 5 + [_c_vp, _c_vp, _c_int, _c_vp, _c_vp]),
    "qssm_rmsnorm_workspace_bytes": (_c_sz, [_c_i64]),
    "qssm_rmsnorm_fwd": (_c_int, [_c_vp] * 4 + [_c_i64] * 4 + [ctypes.c_float, _c_int, _c_vp]),
    "qssm_rmsnorm_bwd": (_c_int, [_c_vp] * 6 + [_c_vp, _c_sz] + [_c_i64] * 5 + [_c_int, _c_vp]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise ImportError(
                        f"{LIB_PATH} is missing: build it with `python -m quick_ssm_b200.build` "
                        "(nvcc, sm_100a). There is no fallback implementation.")
                lib = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = lib
    return _lib


def tune_set(name: str, value: int) -> None:
    """Set one launch-shape knob of the library (measurement scripts and tests only)."""
    if load().qssm_tune_set(name.encode(), int(value)) != 0:
        raise KeyError(f"unknown qssm tuning knob '{name}'")


def tune_reset() -> None:
    """Put every knob back to its start-up value (the QSSM_<NAME> environment variables, read once)."""
    load().qssm_tune_reset()


def status_string(code: int) -> str:
    return load().qssm_status_string(int(code)).decode()


def tile_rows() -> int:
    return int(load().qssm_tile_rows())


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported storage dtype {dt}; use float32, float16 or bfloat16") from None


# ---------------------------------------------------------------------------------------------
# device status word: pinned host memory the kernels can write, read by the host without a sync
# ---------------------------------------------------------------------------------------------
_status_words = {}   # device index -> (pinned tensor, its address, a ctypes view of the int)


_status_lock = threading.Lock()


def _status_entry(index: int):
    e = _status_words.get(index)
    if e is None:
        with _status_lock:  # two host threads may make their first call at the same time
            e = _status_words.get(index)
            if e is None:
                w = torch.zeros(1, dtype=torch.int32).pin_memory()
                e = _status_words[index] = (w, w.data_ptr(), ctypes.c_int.from_address(w.data_ptr()))
    return e


def _status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return _status_entry(index)[0]


def _raise_status(entry) -> None:
    code = entry[2].value
    entry[2].value = 0
    raise RuntimeError(f"qssm device error {code}: {status_string(code)}")


def check_device_status(device: Optional[torch.device] = None, synchronize: bool = False) -> None:
    """Raise if a kernel launched earlier reported a device-side error (e.g. an expired wait)."""
    if synchronize:
        torch.cuda.synchronize(device)
    if device is None:
        entries = list(_status_words.values())
    else:
        device = torch.device(device)
        entries = [_status_entry(device.index if device.index is not None else torch.cuda.current_device())]
    for e in entries:
        if e[2].value != 0:
            _raise_status(e)


def _rc(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}: {status_string(code)}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _on_device:
    """``with _on_device(dev)``: make ``dev`` current for the call; free when it already is."""

    __slots__ = ("index", "prev")

    def __init__(self, device: torch.device):
        self.index = device.index

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.index is None or cur == self.index:
            self.prev = None
        else:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def _begin(dev: torch.device):
    """Per-call prologue: surface an earlier device-side error, return the status word's address."""
    if _lib is None:
        load()
    e = _status_entry(dev.index if dev.index is not None else torch.cuda.current_device())
    if e[2].value != 0:
        _raise_status(e)
    return e[1]


def _require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        d = t.device
        if d.type != "cuda":
            raise RuntimeError("the qssm kernels need CUDA tensors; there is no CPU path")
        if dev is None:
            dev = d
        elif d != dev:
            raise RuntimeError("all tensors must live on the same CUDA device")
    return dev


def _blds(t: torch.Tensor) -> Tuple[int, int]:
    """(stride_b, stride_l) in elements of a [B, L, D] tensor whose D stride is 1."""
    return int(t.stride(0)), int(t.stride(1))


def layout_ok(t: torch.Tensor) -> bool:
    """Can the kernels address this [B, L, D] view in place?"""
    B, L, D = t.shape
    if B * L * D == 0:
        return True
    return (D == 1 or t.stride(2) == 1) and (L == 1 or t.stride(1) >= D) and (B == 1 or t.stride(0) >= D)


def same_layout(*ts: torch.Tensor) -> bool:
    s0 = ts[0].stride()
    return all(t.stride() == s0 for t in ts[1:])


_ws_bytes = {}   # (B, L, D, dtype code) -> bytes the library wants when it picks the segments itself


def workspace(B: int, L: int, D: int, code: int, n_seg: int, device) -> Optional[torch.Tensor]:
    if n_seg and n_seg > 1:
        nbytes = 3 * B * n_seg * D * 4
    else:
        key = (B, L, D, code)
        nbytes = _ws_bytes.get(key)
        if nbytes is None:
            if len(_ws_bytes) > 4096:
                _ws_bytes.clear()
            nbytes = _ws_bytes[key] = int(load().qssm_workspace_bytes(B, L, D, code))
    if nbytes == 0:
        return None
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


# ---------------------------------------------------------------------------------------------
# thin call wrappers (arguments already validated / laid out by the caller)
# ---------------------------------------------------------------------------------------------
def scan_fwd(x, a, b, c, y, *, h_saved=None, tile_h=None, h_in=None, h_last=None, n_seg: int = 0, ws=None) -> None:
    """``n_seg`` < 0 with ``ws`` from ``aggregate_fwd``: reuse the segment aggregates already in ``ws``."""
    dev = _require_cuda(x, a, b, c, y, h_saved, tile_h, h_in, h_last, ws)
    B, L, D = x.shape
    status = _begin(dev)
    with _on_device(dev):
        code_in, code_out = _DTYPE_CODE.get(x.dtype), _DTYPE_CODE.get(y.dtype)
        if code_in is None or code_out is None:
            dtype_code(x.dtype), dtype_code(y.dtype)
        if ws is None:
            ws = workspace(B, L, D, code_in, abs(n_seg), dev)
        rc = _lib.qssm_scan_fwd(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(y), _ptr(h_saved), _ptr(tile_h),
                                _ptr(h_in), _ptr(h_last), _ptr(ws), 0 if ws is None else ws.numel(),
                                B, L, D, x.stride(0), x.stride(1), y.stride(0), y.stride(1), code_in, code_out,
                                n_seg, status, _stream(dev))
    if rc != 0:
        _rc(rc, "qssm_scan_fwd")


def scan_fwd_static_ws(x, a, b, c, y, *, h_saved=None, tile_h=None, h_in=None, h_last=None, n_seg: int = 0) -> None:
    """Forward scan whose segment scratch is the library's built-in device array: this wrapper and
    the C entry point allocate no device memory (for callers that cannot allocate around the call,
    e.g. inside a runtime whose pool owns the device heap, or under a no-allocation-after-start-up
    rule).  Raises when the
    shape needs more scratch than the built-in array holds.  Calls that may overlap on one GPU
    must be ordered by the caller, since they share that array."""
    dev = _require_cuda(x, a, b, c, y, h_saved, tile_h, h_in, h_last)
    B, L, D = x.shape
    check_device_status(dev)
    with torch.cuda.device(dev):
        sb, sl = _blds(x)
        ob, ol = _blds(y)
        rc = load().qssm_scan_fwd_static_ws(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(y), _ptr(h_saved),
                                            _ptr(tile_h), _ptr(h_in), _ptr(h_last), B, L, D, sb, sl, ob, ol,
                                            dtype_code(x.dtype), dtype_code(y.dtype), int(n_seg),
                                            _status_word(dev).data_ptr(), _stream(dev))
    _rc(rc, "qssm_scan_fwd_static_ws")


def scan_bwd(x, a, b, c, dy, dx, da, db, dc, *, h_saved=None, tile_h=None, h_in=None, g_in=None, g_first=None,
             n_seg: int = 0, ws=None) -> None:
    """``n_seg`` < 0 with ``ws`` from ``aggregate_bwd``: reuse the segment aggregates already in ``ws``."""
    dev = _require_cuda(x, a, b, c, dy, dx, da, db, dc, h_saved, tile_h, h_in, g_in, g_first, ws)
    B, L, D = x.shape
    status = _begin(dev)
    with _on_device(dev):
        code_in, code_out = _DTYPE_CODE.get(x.dtype), _DTYPE_CODE.get(dy.dtype)
        if code_in is None or code_out is None:
            dtype_code(x.dtype), dtype_code(dy.dtype)
        if ws is None:
            ws = workspace(B, L, D, code_in, abs(n_seg), dev)
        rc = _lib.qssm_scan_bwd(_ptr(x), _ptr(a), _ptr(b), _ptr(c), _ptr(dy), _ptr(h_saved), _ptr(tile_h),
                                _ptr(h_in), _ptr(g_in), _ptr(g_first), _ptr(dx), _ptr(da), _ptr(db), _ptr(dc),
                                _ptr(ws), 0 if ws is None else ws.numel(), B, L, D, x.stride(0), x.stride(1),
                                dy.stride(0), dy.stride(1), code_in, code_out, n_seg, status, _stream(dev))
    if rc != 0:
        _rc(rc, "qssm_scan_bwd")


class Unsupported(RuntimeError):
    """The fused-gate kernels cannot take these tensors (layout or dtype combination)."""


def gated_scan_fwd(pa, px, pc1, pc2, pd, y, gate_dtype, *, tile_h=None, h_in=None, h_last=None) -> None:
    dev = _require_cuda(pa, px, pc1, pc2, pd, y, tile_h, h_in, h_last)
    B, L, D = pa.shape
    check_device_status(dev)
    with torch.cuda.device(dev):
        sb, sl = _blds(pa)
        ob, ol = _blds(y)
        rc = load().qssm_gated_scan_fwd(_ptr(pa), _ptr(px), _ptr(pc1), _ptr(pc2), _ptr(pd), _ptr(y), _ptr(tile_h),
                                        _ptr(h_in), _ptr(h_last), B, L, D, sb, sl, ob, ol, dtype_code(pa.dtype),
                                        dtype_code(gate_dtype), dtype_code(y.dtype),
                                        _status_word(dev).data_ptr(), _stream(dev))
    if rc in (-3, -4):
        raise Unsupported(status_string(rc))
    _rc(rc, "qssm_gated_scan_fwd")


def gated_scan_bwd(pa, px, pc1, pc2, pd, dy, tile_h, grads, gate_dtype, *, g_in=None, g_first=None) -> None:
    dev = _require_cuda(pa, px, pc1, pc2, pd, dy, tile_h, *grads)
    B, L, D = pa.shape
    check_device_status(dev)
    with torch.cuda.device(dev):
        sb, sl = _blds(pa)
        gb, gl = _blds(dy)
        rc = load().qssm_gated_scan_bwd(_ptr(pa), _ptr(px), _ptr(pc1), _ptr(pc2), _ptr(pd), _ptr(dy), _ptr(tile_h),
                                        _ptr(g_in), _ptr(g_first), *[_ptr(t) for t in grads], B, L, D, sb, sl, gb, gl,
                                        dtype_code(pa.dtype), dtype_code(gate_dtype), dtype_code(dy.dtype),
                                        _status_word(dev).data_ptr(), _stream(dev))
    if rc in (-3, -4):
        raise Unsupported(status_string(rc))
    _rc(rc, "qssm_gated_scan_bwd")


def auto_segments(B: int, L: int, D: int, dtype: torch.dtype) -> int:
    return int(load().qssm_auto_segments(B, L, D, dtype_code(dtype)))


def aggregate_fwd(x, a, b, A, H, *, n_seg: int = 0, ws=None) -> None:
    dev = _require_cuda(x, a, b, A, H, ws)
    B, L, D = x.shape
    check_device_status(dev)
    with torch.cuda.device(dev):
        code = dtype_code(x.dtype)
        if ws is None:
            ws = workspace(B, L, D, code, n_seg, dev)
        sb, sl = _blds(x)
        rc = load().qssm_scan_aggregate_fwd(_ptr(x), _ptr(a), _ptr(b), _ptr(A), _ptr(H), _ptr(ws),
                                            0 if ws is None else ws.numel(), B, L, D, sb, sl, code, int(n_seg),
                                            _status_word(dev).data_ptr(), _stream(dev))
    _rc(rc, "qssm_scan_aggregate_fwd")


def aggregate_bwd(a, c, dy, P, Q, *, n_seg: int = 0, ws=None) -> None:
    dev = _require_cuda(a, c, dy, P, Q, ws)
    B, L, D = a.shape
    check_device_status(dev)
    with torch.cuda.device(dev):
        code, code_dy = dtype_code(a.dtype), dtype_code(dy.dtype)
        if ws is None:
            ws = workspace(B, L, D, code, n_seg, dev)
        sb, sl = _blds(a)
        gb, gl = _blds(dy)
        rc = load().qssm_scan_aggregate_bwd(_ptr(a), _ptr(c), _ptr(dy), _ptr(P), _ptr(Q), _ptr(ws),
                                            0 if ws is None else ws.numel(), B, L, D, sb, sl, gb, gl, code, code_dy,
                                            int(n_seg), _status_word(dev).data_ptr(), _stream(dev))
    _rc(rc, "qssm_scan_aggregate_bwd")


def carry_fold(A, H, upto: int, *, reverse: bool, seed=None) -> torch.Tensor:
    """A, H: [n, ...] fp32 contiguous stacks of aggregates; returns the carry entering slot ``upto``."""
    dev = _require_cuda(A, H, seed)
    n = A.shape[0]
    n_chan = A[0].numel() if n > 0 else (seed.numel() if seed is not None else 0)
    out = torch.empty(A.shape[1:], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = load().qssm_carry_fold(_ptr(A), _ptr(H), n, int(A.stride(0)) if n > 0 else n_chan, n_chan, int(upto),
                                    1 if reverse else 0, _ptr(seed), _ptr(out), _stream(dev))
    _rc(rc, "qssm_carry_fold")
    return out


def _rows(t: torch.Tensor) -> Tuple[int, int, int]:
    """(rows, H, row pitch in elements) of a tensor whose last axis is contiguous and whose leading
    axes collapse into one row index."""
    H = t.shape[-1]
    if t.dim() == 1:
        return 1, H, H
    if t.stride(-1) != 1 and H > 1:
        raise Unsupported("last axis must be contiguous")
    flat = t.reshape(-1, H) if t.is_contiguous() else None
    if flat is None:
        if t.dim() != 2:
            raise Unsupported("leading axes do not collapse into rows")
        return t.shape[0], H, t.stride(0)
    return flat.shape[0], H, H


def rmsnorm_fwd(x, w, y, rstd, eps: float) -> None:
    """y = x * w / sqrt(mean(x^2, -1) + eps); rstd [rows] fp32 receives 1/sqrt(...) (or None)."""
    dev = _require_cuda(x, w, y, rstd)
    rows, H, xs = _rows(x)
    _, _, ys = _rows(y)
    with torch.cuda.device(dev):
        rc = load().qssm_rmsnorm_fwd(_ptr(x), _ptr(w), _ptr(y), _ptr(rstd), rows, H, xs, ys, float(eps),
                                     dtype_code(x.dtype), _stream(dev))
    if rc in (-3, -4):
        raise Unsupported(status_string(rc))
    _rc(rc, "qssm_rmsnorm_fwd")


def rmsnorm_bwd(x, w, dy, rstd, dx, dw) -> None:
    dev = _require_cuda(x, w, dy, rstd, dx, dw)
    rows, H, xs = _rows(x)
    _, _, gs = _rows(dy)
    _, _, ds = _rows(dx)
    with torch.cuda.device(dev):
        nbytes = int(load().qssm_rmsnorm_workspace_bytes(H))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        rc = load().qssm_rmsnorm_bwd(_ptr(x), _ptr(w), _ptr(dy), _ptr(rstd), _ptr(dx), _ptr(dw), _ptr(ws), nbytes,
                                     rows, H, xs, gs, ds, dtype_code(x.dtype), _stream(dev))
    if rc in (-3, -4):
        raise Unsupported(status_string(rc))
    _rc(rc, "qssm_rmsnorm_bwd")


MAX_PEERS, PEER_SLOTS = 16, 4


def peer_inbox_bytes(world: int, n_chan: int) -> int:
    return int(load().qssm_peer_inbox_bytes(int(world), int(n_chan)))


def carry_push(first, second, inbox_ptrs, counters, rank: int, slot: int, epoch: int) -> None:
    """Store this rank's aggregate pair into slot ``slot`` of every rank's inbox (device pointers as
    ints, own rank included) and publish ``epoch`` in this rank's flag there."""
    dev = _require_cuda(first, second, counters)
    world = len(inbox_ptrs)
    arr_t = ctypes.c_void_p * world
    with _on_device(dev):
        rc = load().qssm_carry_push(_ptr(first), _ptr(second), first.numel(), arr_t(*inbox_ptrs), _ptr(counters),
                                    rank, world, slot, epoch, _stream(dev))
    _rc(rc, "qssm_carry_push")


def carry_wait_fold(inbox_ptr: int, n_chan: int, rank: int, world: int, slot: int, epoch: int, reverse: bool,
                    carry, seed=None, wait_ms: int = 2000) -> None:
    """Wait (bounded) until every rank's pair of this call has arrived in the local inbox, then fold
    the pairs of the ranks this one depends on."""
    dev = _require_cuda(carry, seed)
    status = _begin(dev)
    with _on_device(dev):
        rc = load().qssm_carry_wait_fold(inbox_ptr, n_chan, rank, world, slot, epoch, 1 if reverse else 0,
                                         _ptr(seed), _ptr(carry), int(wait_ms), status, _stream(dev))
    _rc(rc, "qssm_carry_wait_fold")
