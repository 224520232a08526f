"""Benchmark of the gated linear scan, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one forward (y = c*h, keeping the 1/16 boundary states) plus one backward (four
gradients, h rebuilt in-kernel) over one batch of seeded synthetic inputs of the single-GPU
benchmark configuration: B=8, L=8192, D=4096, bf16 storage, fp32 accumulation, checkpoint=True.
Metric: Gelem/s = B*L*D / (t_fwd + t_bwd) / 1e9, whole job (all ranks).

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank scans its own
batch/channel shard of an N-times larger problem: the recurrences are independent, so there is
no collective on the data path (weak scaling).  Time is taken on the device with CUDA events,
max over ranks.

The same line carries, outside the headline value:
  forward_only   the two inference forms on the same workload: y under no_grad (5 tensor passes)
                 and h only (forward_only, 4 passes);
  api            the same step through the Python API, scan(...) + .backward() (autograd, allocations);
  host_call_us   host time of one qssm_scan_fwd + qssm_scan_bwd call pair on a tiny shape;
  gpu_reference  optional third column: the reference's own Triton path (unmodified, installed under the
                 git-ignored baseline/_ref) on the same GPU and inputs, a B=1 slice of the workload: its time, this
                 library's time on the same slice, and the element-wise agreement of the two;
  seq_sharded    the long-sequence configuration (B=1, L=2^20, D=2048, fp16, decay close to one) with
                 the TIME axis split over the N ranks: per rank one aggregate pass, one NCCL all-gather
                 of 2*B*D floats, a fold and a seeded scan, forward and backward; at N=1 the single-pass
                 kernels.  One 64-channel strip of the result is checked against the CPU oracle outside
                 the timed region.

--impl reference times the CPU implementation of the same path (the sequential-loop oracle,
all host threads) on a bounded sample of the same workload and prints the same JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fwd+bwd scan Gelem/s (B*L*D)"
UNIT = "Gelem/s"
CFG = dict(B=8, L=8192, D=4096)
WORKLOAD = "cfg1: scan fwd+bwd, B=8 L=8192 D=4096, bf16 storage / fp32 accumulate, checkpoint=True"

CFG2 = dict(B=1, L=1 << 20, D=2048)
HOST_CPUS = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)

# DRAM bytes (read + write) of one backward launch come from an ncu capture of the same kernel on a
# shorter sequence (same chains, same residency); the capture's figures and the commit it was taken
# at live in this file, which the ncu summary beside it quotes too.  Traffic grows in proportion to L.
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "scan_bwd_tile4_cfg1_traffic.json")


def _ncu_traffic(L: int):
    try:
        with open(TRAFFIC_FILE) as f:
            t = json.load(f)
        return (float(t["dram_bytes_read"]) + float(t["dram_bytes_write"])) * (L / float(t["L"])), t.get("commit")
    except Exception:
        return None, None


def _peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Reads SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# CPU legs (the oracle is the thing timed here, never on the product path)
# ---------------------------------------------------------------------------------------------
def _cpu_sample_inputs(sample_b: int):
    import numpy as np
    import torch
    from quick_ssm_b200.synth import make_inputs
    inp = make_inputs(sample_b, CFG["L"], CFG["D"], dtype=torch.bfloat16, seed=0)
    arrs = [t.float().numpy() for t in (inp.x, inp.a, inp.b, inp.c, inp.dy)]
    outs = [np.empty_like(arrs[0]) for _ in range(6)]  # h scratch, y, dx, da, db, dc
    return arrs, outs


def cpu_baseline(budget_s: float = 12.0, sample_b: int = 1):
    """Sequential-loop oracle (C, OpenMP over channels) on a batch slice of the workload."""
    from oracle import scan_oracle as so
    so.set_num_threads(HOST_CPUS)  # every host core, whatever OMP_NUM_THREADS the launcher set
    arrs, outs = _cpu_sample_inputs(sample_b)
    x, a, b, c, dy = arrs
    n = x.size
    so.scan_forward_backward_inplace(x, a, b, c, dy, *outs)  # warm-up, page in
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        so.scan_forward_backward_inplace(x, a, b, c, dy, *outs)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": n / best / 1e9, "unit": UNIT, "cores": so.num_threads(), "kind": "port",
            "sample": f"batch slice B={sample_b} of the workload ({n} elements, bf16 values held as fp32), "
                      f"best of {len(times)} passes of {best * 1e3:.1f} ms",
            "host_cpus": os.cpu_count()}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import scan_oracle as so
    so.set_num_threads(HOST_CPUS)  # torch.distributed.run exports OMP_NUM_THREADS=1: do not inherit it
    sample_b = 1
    arrs, outs = _cpu_sample_inputs(sample_b)
    x, a, b, c, dy = arrs
    n = x.size
    for _ in range(max(1, args.warmup)):
        so.scan_forward_backward_inplace(x, a, b, c, dy, *outs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        so.scan_forward_backward_inplace(x, a, b, c, dy, *outs)
    dt = (time.perf_counter() - t0) / args.steps
    value = n / dt / 1e9
    sample = (f"each step = fwd+bwd over a batch slice B={sample_b} of the workload ({n} elements); "
              "per-element throughput is independent of B (recurrences are independent)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": so.num_threads(), "kind": "port",
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm: pieces measured next to the headline step
# ---------------------------------------------------------------------------------------------
def _timed_ms(torch, fn, steps, sync, warmup=3):
    """Mean device time of `steps` back-to-back calls (CUDA events on the launching stream)."""
    for _ in range(warmup):
        fn()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    return e0.elapsed_time(e1) / steps


def measure_forward_only(torch, _lib, x, a, b, c, y, steps, sync, peak):
    """Inference forms of the forward on the headline workload (reference: scan() under no_grad,
    scan_interface.py:169-213, and forward_only.block_scan_forward_3d, forward_only.py:423-540)."""
    n, es = x.numel(), x.element_size()
    out = {}
    for name, cc, passes in (("y_no_grad", c, 5), ("h_only", None, 4)):
        ms = _timed_ms(torch, lambda: _lib.scan_fwd(x, a, b, cc, y), steps, sync)
        gbs = n * passes * es / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "algorithmic_bytes": n * passes * es, "achieved": gbs, "unit": "GB/s",
                     "frac": gbs / peak, "gelems": n / (ms * 1e-3) / 1e9}
    return out


def measure_api(torch, x, a, b, c, dy, steps, sync):
    """The same step through the public Python API: scan(...) then .backward() (autograd graph, output
    and gradient allocations from the caching allocator on every step)."""
    from quick_ssm_b200 import scan
    leaves = [t.detach().requires_grad_() for t in (x, a, b, c)]

    def step():
        for t in leaves:
            t.grad = None
        scan(*leaves, block_l=256, checkpoint=True).backward(dy)

    ms = _timed_ms(torch, step, steps, sync)
    for t in leaves:
        t.grad = None
    return {"ms_per_step": ms, "gelems": x.numel() / (ms * 1e-3) / 1e9, "steps": steps,
            "path": "quick_ssm_b200.scan(x, a, b, c, block_l=256, checkpoint=True) + y.backward(dy)"}


def measure_host_call(torch, _lib, dev, calls=1000):
    """Host time of one forward + backward call pair through the binding on the copy-task shape of the
    reference's training demo (copy_train.py:35-38: B=32, L=16, state 1024), and its device time."""
    B, L, D = 32, 16, 1024
    t = [torch.randn(B, L, D, device=dev, dtype=torch.bfloat16) for _ in range(5)]
    y = torch.empty_like(t[0])
    th = torch.empty((B, 1, D), dtype=torch.float32, device=dev)
    g = [torch.empty_like(t[0]) for _ in range(4)]

    def pair():
        _lib.scan_fwd(t[0], t[1], t[2], t[3], y, tile_h=th)
        _lib.scan_bwd(t[0], t[1], t[2], t[3], t[4], *g, tile_h=th)

    def time_loop(fn):
        for _ in range(20):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(calls):
            fn()
        host_us = (time.perf_counter() - t0) / calls * 1e6
        e1.record()
        torch.cuda.synchronize(dev)
        return host_us, e0.elapsed_time(e1) / calls * 1e3

    binding_us, device_us = time_loop(pair)

    # the same two calls straight through the C ABI with the arguments converted once
    lib = _lib.load()
    p = [v.data_ptr() for v in t]
    status = _lib._status_word(dev).data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    sb, sl = L * D, D
    args_f = (p[0], p[1], p[2], p[3], y.data_ptr(), None, th.data_ptr(), None, None, None, 0, B, L, D, sb, sl, sb, sl,
              _lib.BF16, _lib.BF16, 0, status, stream)
    args_b = (p[0], p[1], p[2], p[3], p[4], None, th.data_ptr(), None, None, None, *[v.data_ptr() for v in g], None, 0,
              B, L, D, sb, sl, sb, sl, _lib.BF16, _lib.BF16, 0, status, stream)

    def pair_c():
        lib.qssm_scan_fwd(*args_f)
        lib.qssm_scan_bwd(*args_b)

    c_abi_us, _ = time_loop(pair_c)
    return {"host_us_per_fwd_bwd_pair": binding_us, "c_abi_host_us_per_pair": c_abi_us,
            "device_us_per_pair": device_us, "shape": [B, L, D], "calls": calls,
            "note": "host_us: through quick_ssm_b200._lib (argument checks, current stream, ctypes); c_abi: "
                    "ctypes straight into qssm_scan_fwd + qssm_scan_bwd with prepared arguments; device_us: the "
                    "same loop's device time per pair (two launches)"}


def _strip_check(np, strips, ref_fn):
    """|got - ref| <= 1e-3 * max(1, max|ref|) + 2e-2 * |ref| per tensor (16-bit storage against the
    fp32 sequential loop; gradients of a 2^20-step chain with decay close to one reach hundreds, so the
    absolute floor scales with the tensor's magnitude)."""
    refs = ref_fn()
    report, ok = {}, True
    for name in ("y", "dx", "da", "db", "dc"):
        g, r = strips[name].astype(np.float64), refs[name].astype(np.float64)
        scale = max(1.0, float(np.abs(r).max()))
        bad = np.abs(g - r) > 1e-3 * scale + 2e-2 * np.abs(r)
        report[name] = {"max_abs_err": float(np.abs(g - r).max()), "max_abs_ref": float(np.abs(r).max()),
                        "outside": int(bad.sum())}
        ok = ok and not bad.any() and bool(np.isfinite(g).all())
    return ok, report


def measure_seq_sharded(torch, dist, _lib, dev, rank, world, steps, sync, peak):
    """The long-sequence configuration with the time axis split over the ranks (see the module
    docstring).  Returns the dict for the JSON line on rank 0, None elsewhere."""
    import numpy as np
    from quick_ssm_b200 import sharded
    from quick_ssm_b200.synth import make_inputs

    B, L, D = CFG2["B"], CFG2["L"], CFG2["D"]
    Ls = L // world
    dtype, es = torch.float16, 2
    inp = make_inputs(B, Ls, D, dtype=dtype, device=dev, seed=0, rank=rank, decay="near_unit")
    x, a, b, c = inp.tensors()
    dy = inp.dy
    y = torch.empty_like(x)
    tile_h = torch.empty((B, (Ls + _lib.tile_rows() - 1) // _lib.tile_rows(), D), dtype=torch.float32, device=dev)
    grads = [torch.empty_like(x) for _ in range(4)]

    def timed(ops, comm):
        """Per-rank table [total, fwd, bwd, 3 forward phases, 3 backward phases] in ms per step."""
        if world == 1:
            def fwd(marks=None):
                _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h)

            def bwd(marks=None):
                _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h)
        else:
            def fwd(marks=None):
                sharded.shard_forward(ops, comm, x, a, b, c, dtype, True, y=y, tile_h=tile_h, marks=marks)

            def bwd(marks=None):
                sharded.shard_backward(ops, comm, x, a, b, c, dy, tile_h, grads=grads, marks=marks)

        for _ in range(3):
            fwd()
            bwd()
        sync()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1)]
        marks_f, marks_b = [], []
        ev[0].record()
        for k in range(steps):
            fwd(marks_f if world > 1 else None)
            ev[2 * k + 1].record()
            bwd(marks_b if world > 1 else None)
            ev[2 * k + 2].record()
        sync()
        _lib.check_device_status(dev)
        total_ms = ev[0].elapsed_time(ev[-1]) / steps
        fwd_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(steps)) / steps
        bwd_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(steps)) / steps

        def phases(marks):  # mean ms of (aggregate, exchange + fold, seeded scan)
            if not marks:
                return [0.0, 0.0, 0.0]
            k = len(marks) // 4
            return [sum(marks[4 * i + j].elapsed_time(marks[4 * i + j + 1]) for i in range(k)) / k for j in range(3)]

        mine = torch.tensor([total_ms, fwd_ms, bwd_ms] + phases(marks_f) + phases(marks_b), device=dev,
                            dtype=torch.float64)
        if world > 1:
            allr = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
            return torch.stack(allr).cpu()
        return mine.cpu()[None]

    comm = sharded.TorchComm(None) if world > 1 else None
    # the same step with the carries pushed into the peers' inboxes instead of the all-gather: timed
    # first, so that the results checked below are those of the all-gather path
    peer_table, peer_note = None, None
    if world > 1 and not os.environ.get("QSSM_BENCH_NO_PEER"):
        try:
            peer = sharded.PeerCarryExchange(None, B * D, dev)
            peer_table = timed(sharded.CudaShardOps(peer=peer), comm)
        except Exception as e:  # symmetric memory unavailable on this box: the all-gather path stands alone
            peer_note = f"{type(e).__name__}: {e}"[:200]
    table = timed(sharded.CudaShardOps() if world > 1 else None, comm)

    # ---- one 64-channel strip, whole sequence, against the oracle (outside the timed region) ----
    d0 = (D // 2 // 64) * 64
    got = {"y": y, "dx": grads[0], "da": grads[1], "db": grads[2], "dc": grads[3]}
    ins = {"x": x, "a": a, "b": b, "c": c, "dy": dy}
    local = {k: v[:, :, d0:d0 + 64].contiguous() for k, v in {**got, **ins}.items()}
    if world > 1:
        whole = {}
        for k, v in local.items():
            parts = [torch.empty_like(v) for _ in range(world)] if rank == 0 else None
            dist.gather(v, parts, dst=0)
            if rank == 0:
                whole[k] = torch.cat(parts, dim=1)
    else:
        whole = local
    if rank != 0:
        return None
    from oracle import scan_oracle as so  # the checker, never the thing measured
    host = {k: v.float().cpu().numpy() for k, v in whole.items()}

    def ref_fn():
        _, y_ref, _ = so.scan_forward(host["x"], host["a"], host["b"], host["c"], dtype=np.float32)
        g = so.scan_backward(host["x"], host["a"], host["b"], host["c"], host["dy"], dtype=np.float32)
        return {"y": y_ref, "dx": g[0], "da": g[1], "db": g[2], "dc": g[3]}

    ok, report = _strip_check(np, host, ref_fn)
    n_total = B * L * D
    t_max = float(table[:, 0].max())
    gelems = n_total / (t_max * 1e-3) / 1e9
    gbs14 = n_total * 14 * es / (t_max * 1e-3) / 1e9
    gbs20 = n_total * 20 * es / (t_max * 1e-3) / 1e9
    out = {
        "workload": "cfg2: B=1 L=2^20 D=2048 fp16, decay 1-10^U(-4,-1), fwd+bwd, checkpoint=True, "
                    + ("single-pass kernels on one GPU" if world == 1 else f"time axis split over {world} ranks"),
        "value": gelems, "unit": UNIT, "ms_per_step": t_max, "steps": steps, "scaling": "strong",
        "fwd_ms_per_rank": [float(v) for v in table[:, 1]], "bwd_ms_per_rank": [float(v) for v in table[:, 2]],
        "frac_of_14s_bytes": gbs14 / (world * peak),
        "frac_of_20s_bytes": (gbs20 if world > 1 else gbs14) / (world * peak),
        "bytes_note": "a shard reads the tensors its carry depends on twice (aggregate pass + scan): 20 tensor "
                      "passes instead of 14 when the time axis is split; one GPU needs 14",
        "parity": {"strip": [d0, d0 + 64], "rows": L, "ok": ok, "tensors": report,
                   "rule": "|got-ref| <= 1e-3*max(1,max|ref|) + 2e-2*|ref| against the fp32 sequential loop"},
    }
    if world > 1:
        names = ("aggregate_ms", "allgather_fold_ms", "scan_ms")
        out["fwd_phases_per_rank"] = {n: [float(v) for v in table[:, 3 + j]] for j, n in enumerate(names)}
        out["bwd_phases_per_rank"] = {n: [float(v) for v in table[:, 6 + j]] for j, n in enumerate(names)}
        out["collective"] = "one NCCL all_gather_into_tensor of 2*B*D fp32 per rank and direction (16 KB per rank)"
        if peer_table is not None:
            tp = float(peer_table[:, 0].max())
            out["peer_exchange"] = {
                "what": "same step, carries stored into every rank's inbox through peer memory (plain stores over "
                        "NVLink + flag, bounded-wait fold) instead of the all-gather",
                "value": n_total / (tp * 1e-3) / 1e9, "ms_per_step": tp,
                "frac_of_20s_bytes": n_total * 20 * es / (tp * 1e-3) / 1e9 / (world * peak),
                "fwd_exchange_fold_ms_per_rank": [float(v) for v in peer_table[:, 4]],
                "bwd_exchange_fold_ms_per_rank": [float(v) for v in peer_table[:, 7]]}
        elif peer_note is not None:
            out["peer_exchange"] = {"unavailable": peer_note}
        out["gpu_launches_per_step"] = "fwd: aggregate + segment carry + fold + scan; bwd: the same"
    return out


def _bind_to_gpu_cpus(local: int):
    """Run this rank on the CPUs NVML lists as local to its GPU, so that the pinned host buffers of
    the end-to-end leg are first touched on that NUMA node.  A process setting; nothing on the GPU."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + j for i, w in enumerate(words) for j in range(64) if (int(w) >> j) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from quick_ssm_b200 import _lib
    from quick_ssm_b200.host import HostScan, alloc_pinned
    from quick_ssm_b200.synth import make_inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path exists for the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    gpu_local_cpus = _bind_to_gpu_cpus(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, L, D = CFG["B"], args.seq_len or CFG["L"], CFG["D"]
    dtype = torch.bfloat16
    n_elem = B * L * D
    es = 2
    inp = make_inputs(B, L, D, dtype=dtype, device=dev, seed=0, rank=rank)
    x, a, b, c = inp.tensors()
    dy = inp.dy
    y = torch.empty_like(x)
    nt = (L + _lib.tile_rows() - 1) // _lib.tile_rows()
    tile_h = torch.empty((B, nt, D), dtype=torch.float32, device=dev)
    grads = [torch.empty_like(x) for _ in range(4)]

    def step():
        _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h)
        _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        t_begin.record()
        for k in range(K):
            ev[k][0].record()
            _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h)
            ev[k][1].record()
            _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h)
            ev[k][2].record()
        t_end.record()
        barrier()
    _lib.check_device_status(dev)
    total_ms = t_begin.elapsed_time(t_end)
    fwd_all = sorted(e[0].elapsed_time(e[1]) for e in ev)
    bwd_all = sorted(e[1].elapsed_time(e[2]) for e in ev)
    fwd_ms = sum(fwd_all) / K
    bwd_ms = sum(bwd_all) / K

    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"note": "profiling run, not a bench line", "L": L, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through host buffers (pinned host memory in and out, every step) ----
    e2e_steps = max(3, min(K, 8))
    host = alloc_pinned(B, L, D, dtype)
    for name, t in zip(("x", "a", "b", "c", "dy"), (x, a, b, c, dy)):
        host[name].copy_(t)
    pipe = HostScan(B, L, D, dtype, device=dev)
    pipe.run(host)
    barrier()
    launches0 = pipe.kernel_launches
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        done = pipe.run(host)
    torch.cuda.current_stream(dev).wait_event(done)  # the last device->host copy is inside the timed region
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    e2e_launches = pipe.kernel_launches - launches0
    # the host results of the last step must agree with the device-resident results (same kernels on
    # batch slices; a slice may take the chunked single-pass kernels, whose carries round differently)
    def _close(u, v):
        return torch.allclose(u.float(), v.float(), rtol=2e-2, atol=1e-3)
    same = _close(host["dx"][-1].to(dev), grads[0][-1]) and _close(host["y"][0].to(dev), y[0])
    if not same:
        raise SystemExit("e2e host-buffer path disagrees with the device-resident path")
    # the same copies without the kernels: the time the transfers alone take (not part of any bench value)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        done = pipe.run(host, compute=False)
    torch.cuda.current_stream(dev).wait_event(done)
    e1.record()
    barrier()
    copy_only_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- measured next to the headline: inference forwards, the Python API, host cost per call ----
    extra_steps = max(5, min(K, 20))
    peak, peak_kind = _peak_hbm()
    fwd_only = api = host_call = None
    if rank == 0:
        fwd_only = measure_forward_only(torch, _lib, x, a, b, c, y, extra_steps, lambda: torch.cuda.synchronize(dev), peak)
        api = measure_api(torch, x, a, b, c, dy, extra_steps, lambda: torch.cuda.synchronize(dev))
        host_call = measure_host_call(torch, _lib, dev)
    barrier()

    # ---- optional third column: the reference's own Triton kernels on this GPU (rank 0, when installed) ----
    gpu_reference = None
    if rank == 0 and not args.no_ref_triton:
        try:
            import bench_configs
            gpu_reference = bench_configs.ref_triton_compare(steps=3, warmup=1, L=L, local_rank=local)
        except Exception as e:  # never let the optional column break the bench line
            gpu_reference = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    barrier()

    # ---- the long-sequence configuration, time axis split over the ranks ----
    h2d_bytes, d2h_bytes = pipe.h2d_bytes, pipe.d2h_bytes
    del pipe, host, grads, y, tile_h, inp, x, a, b, c, dy
    torch.cuda.empty_cache()
    seq = None
    if not args.no_seq:
        seq = measure_seq_sharded(torch, dist, _lib, dev, rank, world, max(3, min(K, 10)), barrier, peak)

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms, fwd_ms, bwd_ms, copy_only_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, fwd_ms, bwd_ms, copy_only_ms = (float(v) for v in t.tolist())

    if rank == 0:
        ms_per_step = total_ms / K
        value = world * n_elem / (ms_per_step * 1e-3) / 1e9
        traffic, traffic_commit = _ncu_traffic(L)
        bwd_bytes = n_elem * 9 * es
        fwd_bytes = n_elem * 5 * es
        bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9
        step_gbs = n_elem * 14 * es / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "B": B, "L": L, "D": D, "accumulate": "fp32", "checkpoint": True,
                       "per_rank": "every rank scans its own B x L x D shard (no data-path collective)",
                       "l2": "no flush needed: each step streams 7.5 GB of distinct tensors, far above the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": "scan_bwd_tile4_kernel", "achieved": bwd_gbs, "peak": peak,
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "unit": "GB/s",
                         "frac": bwd_gbs / peak, "traffic": traffic,
                         "traffic_source": f"profiles/{os.path.basename(TRAFFIC_FILE)} (ncu capture at commit "
                                           f"{traffic_commit}, scaled by L)",
                         "algorithmic_bytes": bwd_bytes, "ms": bwd_ms,
                         "ms_min_median_max": [bwd_all[0], bwd_all[K // 2], bwd_all[-1]],
                         "fwd": {"kernel": "scan_fwd_kernel", "achieved": fwd_gbs, "frac": fwd_gbs / peak,
                                 "algorithmic_bytes": fwd_bytes, "ms": fwd_ms,
                                 "ms_min_median_max": [fwd_all[0], fwd_all[K // 2], fwd_all[-1]]},
                         "step": {"achieved": step_gbs, "frac": step_gbs / peak,
                                  "roofline_gelems": peak / (14 * es)}},
            "e2e": {"value": world * n_elem / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "transfers_alone_ms_per_step": copy_only_ms,
                    "cpus_local_to_gpu": gpu_local_cpus,
                    "path": "quick_ssm_b200.host.HostScan: pinned host buffers -> H2D -> qssm_scan_fwd/bwd -> D2H"},
            "gpu_launches": 2 * K * world,
            "gpu_launches_e2e": e2e_launches * world,
            "clocks": clocks.summary(),
            "forward_only": fwd_only, "api": api, "host_call": host_call, "seq_sharded": seq,
            "gpu_reference": gpu_reference,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="profiling aid: device-resident loop only, no bench line")
    ap.add_argument("--no-seq", action="store_true", help="skip the sequence-sharded long-sequence leg")
    ap.add_argument("--no-ref-triton", action="store_true", help="skip the reference's Triton kernels on this GPU")
    ap.add_argument("--seq-len", type=int, default=0, help="profiling aid: shorter L (same chains, less memory)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
