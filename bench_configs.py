"""Timing of the scan on the benchmark configurations other than the headline one.

    python bench_configs.py --config cfg4 [--no-checkpoint]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_configs.py --config cfg2 --shard seq      # time axis split over N GPUs
        bench_configs.py --config cfg4 --shard batch    # batch split over N GPUs

Configurations (seeded synthetic inputs, see ``synth.CONFIGS``):
  cfg1       B=8  L=8192  D=4096 bf16                     (the headline; bench.py reports it)
  cfg2       B=1  L=2^20  D=2048 fp16, decay close to one  (long sequence; --shard seq)
  cfg3_scan  B=16 L=4096  D=4096 bf16 gates, fp32 y / dy   (the scan inside a 12-layer SSM stack)
  cfg4       B=64 L=4096  D=8192 fp16                     (throughput sweep; --shard batch)
  cfg3_stack 12 x layers.SSM (hidden 1024, state 4096, fp32 parameters, bf16 gates), B=16, L=4096,
             MSE loss to a random target: whole forward+backward step, with the time spent inside
             the scan kernels taken separately from CUDA events around every scan call
  cfg3_gates the same scan shape with the layer's gate activations: fused kernels vs torch gates + scan
  cfg3_norm  the layer's pre-norm: the RMS-norm kernels vs torch's element-wise chain, and the kernels alone
  strips     launch-shape sweep: D=2048, 2^27 elements, B = 1..32 (32..1024 strips of 64 channels), --dtype fp32|bf16|fp16;
             one JSON line per batch size with forward / backward ms and the fraction of the copy peak
  ref_triton the reference's own Triton path (installed unmodified under the git-ignored baseline/_ref) on the
             same GPU and inputs, a batch slice of cfg1: timing and element-wise agreement with this library
With --shard the TOTAL problem is fixed and split over the ranks (strong scaling); the reported
throughput is total elements over the slowest rank's device time.  One JSON line per run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from quick_ssm_b200 import _lib
from quick_ssm_b200.sharded import CudaShardOps, shard_backward, shard_forward
from quick_ssm_b200.synth import CONFIGS, make_inputs


def _median_ms(fn, steps, warmup, sync):
    """Mean device time of `steps` back-to-back calls (CUDA events on the launching stream)."""
    for _ in range(max(3, warmup)):
        fn()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    return e0.elapsed_time(e1) / steps


def run_gates(args):
    """The scan of configuration 3 together with the layer's gate activations: fused kernels
    (`gated_scan`) against torch element-wise gates followed by `scan`, forward + backward through
    autograd, for fp32 projection outputs (fp32 parameters, the reference's setting) and bf16 ones."""
    from quick_ssm_b200.gated import _composed, gated_scan

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, D = 16, args.seq_len or 4096, 4096
    out = {"config": "cfg3_gates", "shape": [B, L, D], "gate_dtype": "bfloat16", "scan_out_dtype": "float32"}
    for name, dtype in (("fp32_projections", torch.float32), ("bf16_projections", torch.bfloat16)):
        torch.manual_seed(0)
        pre = [torch.randn(B, L, D, device=dev, dtype=dtype) for _ in range(5)]
        dy = torch.randn(B, L, D, device=dev)

        def step(fn):
            leaves = [t.detach().requires_grad_() for t in pre]
            fn(leaves).backward(dy)

        fused = _median_ms(lambda: step(lambda l: gated_scan(*l, gate_dtype=torch.bfloat16, out_dtype=torch.float32)),
                           args.steps, args.warmup, torch.cuda.synchronize)
        composed = _median_ms(lambda: step(lambda l: _composed(*l, torch.bfloat16, torch.float32)),
                              args.steps, args.warmup, torch.cuda.synchronize)
        s = pre[0].element_size()
        out[name] = {"fused_ms": round(fused, 3), "torch_gates_plus_scan_ms": round(composed, 3),
                     "speedup": round(composed / fused, 2),
                     "fused_gelems": B * L * D / (fused * 1e-3) / 1e9,
                     "fused_algorithmic_bytes_per_elem": 5 * s + 4 + 10 * s + 4}
        del pre, dy
        torch.cuda.empty_cache()
    _lib.check_device_status(dev)
    print(json.dumps(out), flush=True)


def run_norm(args):
    """The pre-norm of configuration 3 (rows = 16 x 4096, hidden 1024): the normalisation kernels against
    torch's element-wise chain, forward + backward through autograd, fp32 and bf16 activations."""
    from quick_ssm_b200.norm import _composed, rms_norm

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, H = 16, args.seq_len or 4096, 1024
    out = {"config": "cfg3_norm", "shape": [B, L, H]}
    for name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        g = torch.Generator(device=dev).manual_seed(0)
        x = torch.randn(B, L, H, device=dev, generator=g).to(dt).requires_grad_()
        dy = torch.randn(B, L, H, device=dev, generator=g).to(dt)
        w = (torch.randn(H, device=dev, generator=g) * 0.3 + 1.0).requires_grad_()

        def step(fn):
            x.grad = None
            w.grad = None
            fn(x, w, 1e-5).backward(dy)

        fused = _median_ms(lambda: step(rms_norm), args.steps, args.warmup, torch.cuda.synchronize)
        composed = _median_ms(lambda: step(_composed), args.steps, args.warmup, torch.cuda.synchronize)
        s = x.element_size()
        # the kernels alone, through the C ABI on preallocated tensors (no autograd, no allocations)
        xd, w32 = x.detach(), w.detach().float()
        y, dx, dw = torch.empty_like(xd), torch.empty_like(xd), torch.empty_like(w32)
        rstd = torch.empty(B * L, dtype=torch.float32, device=dev)
        k_fwd = _median_ms(lambda: _lib.rmsnorm_fwd(xd, w32, y, rstd, 1e-5), args.steps, args.warmup,
                           torch.cuda.synchronize)
        k_bwd = _median_ms(lambda: _lib.rmsnorm_bwd(xd, w32, dy, rstd, dx, dw), args.steps, args.warmup,
                           torch.cuda.synchronize)
        n = B * L * H
        out[name] = {"fused_ms": round(fused, 4), "torch_ms": round(composed, 4), "speedup": round(composed / fused, 2),
                     "fused_gbs_of_5s_bytes": n * 5 * s / (fused * 1e-3) / 1e9,
                     "kernel_fwd_ms": round(k_fwd, 4), "kernel_fwd_gbs_of_2s_bytes": n * 2 * s / (k_fwd * 1e-3) / 1e9,
                     "kernel_bwd_ms": round(k_bwd, 4), "kernel_bwd_gbs_of_3s_bytes": n * 3 * s / (k_bwd * 1e-3) / 1e9}
    print(json.dumps(out), flush=True)


def run_strips(args):
    """Forward + backward on a fixed element count while the number of 64-channel strips (batch x D/64) goes from
    far fewer than the SMs to several per SM: shows which launch shape the library picks for each count."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[args.dtype]
    D = 2048
    peak = _copy_peak_gbs()
    for B in ((args.batch,) if args.batch else (1, 2, 3, 4, 5, 6, 8, 10, 12, 16, 32)):
        L = args.seq_len or ((1 << 27) // (B * D)) // 256 * 256
        inp = make_inputs(B, L, D, dtype=dtype, device=dev, seed=0)
        x, a, b, c = inp.tensors()
        y = torch.empty_like(x)
        tile_h = torch.empty((B, L // _lib.tile_rows(), D), dtype=torch.float32, device=dev)
        grads = [torch.empty_like(x) for _ in range(4)]
        f = _median_ms(lambda: _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h), args.steps, args.warmup, torch.cuda.synchronize)
        g = _median_ms(lambda: _lib.scan_bwd(x, a, b, c, inp.dy, *grads, tile_h=tile_h), args.steps, args.warmup,
                       torch.cuda.synchronize)
        _lib.check_device_status(synchronize=True)
        n, s = B * L * D, x.element_size()
        print(json.dumps({"config": "strips", "dtype": args.dtype, "B": B, "L": L, "D": D, "strips": B * D // 64,
                          "fwd_ms": round(f, 4), "bwd_ms": round(g, 4),
                          "fwd_gbs": round(n * 5 * s / f / 1e6, 1), "bwd_gbs": round(n * 9 * s / g / 1e6, 1),
                          "frac_of_copy_peak": round(n * 14 * s / (f + g) / 1e6 / peak, 3)}), flush=True)
        del inp, x, a, b, c, y, tile_h, grads
        torch.cuda.empty_cache()


def _copy_peak_gbs() -> float:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0  # an earlier measurement on the same pool


def run_ref_triton(args):
    print(json.dumps(ref_triton_compare(args.steps, args.warmup, args.seq_len or 8192)), flush=True)


def ref_triton_compare(steps: int, warmup: int, L: int = 8192, local_rank: int = 0) -> dict:
    """The reference's own Triton path (`quick_ssm.scan_interface.scan`, backend "triton", installed unmodified
    under baseline/_ref) on the same B200 and the same inputs as this library: a batch slice of configuration 1
    (B=1, L=8192, D=4096, bf16; the reference needs about 7 GiB of fp32 scratch per batch entry pair, so the slice
    keeps it small), forward + backward through autograd, plus the results of both compared element by element.
    Optional third column next to the CPU baseline: a GPU-over-GPU ratio on identical hardware."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    out = {"config": "ref_triton"}
    if not os.path.isdir(os.path.join(ref_dir, "quick_ssm")):
        out["unavailable"] = "baseline/_ref/quick_ssm is not installed on this machine"
        return out
    sys.path.insert(0, ref_dir)
    import importlib
    ref_iface = importlib.import_module("quick_ssm.scan_interface")
    from quick_ssm_b200 import scan as our_scan

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, D = 1, 4096
    inp = make_inputs(B, L, D, dtype=torch.bfloat16, device=dev, seed=0)
    out["shape"] = [B, L, D]
    results = {}
    for name, fn in (("ours", lambda *t: our_scan(*t, block_l=256, checkpoint=True)),
                     ("reference_triton", lambda *t: ref_iface.scan(*t, block_l=256, checkpoint=True, backend="triton"))):
        leaves = [t.detach().clone().requires_grad_() for t in inp.tensors()]

        def step():
            for t in leaves:
                t.grad = None
            y = fn(*leaves)
            y.backward(inp.dy)
            return y

        y = step()   # first call: the reference compiles one kernel specialisation per shape here
        torch.cuda.synchronize()
        ms = _median_ms(step, steps, warmup, torch.cuda.synchronize)
        results[name] = [y.detach()] + [t.grad.detach().clone() for t in leaves]
        out[name] = {"fwd_bwd_ms": round(ms, 4), "gelems": B * L * D / (ms * 1e-3) / 1e9,
                     "peak_mem_gib": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)}
        torch.cuda.reset_peak_memory_stats(dev)
    out["speedup_over_reference_triton"] = out["reference_triton"]["fwd_bwd_ms"] / out["ours"]["fwd_bwd_ms"]
    agree = {}
    for k, u, v in zip(("y", "dx", "da", "db", "dc"), results["ours"], results["reference_triton"]):
        d = (u.float() - v.float()).abs()
        bad = d > 1e-3 * max(1.0, float(v.float().abs().max())) + 2e-2 * v.float().abs()
        agree[k] = {"max_abs_diff": float(d.max()), "max_abs_ref": float(v.float().abs().max()), "outside": int(bad.sum())}
    out["agreement_with_reference_triton"] = agree
    out["all_within_tolerance"] = all(v["outside"] == 0 for v in agree.values())
    return out


def run_stack(args):
    """Configuration 3: the scan inside a 12-layer SSM stack (projections stay torch GEMMs)."""
    from quick_ssm_b200 import scan_interface
    from quick_ssm_b200.gated import _GatedScanFunction
    from quick_ssm_b200.layers import SSM, SSMFused

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    layers, hidden, B, L = 12, 1024, 16, 4096
    Layer = SSMFused if args.fused else SSM
    stack = torch.nn.ModuleList([Layer(hidden_size=hidden, state_size_mult=4.0, dtype=torch.float32,
                                     compute_dtype=torch.bfloat16, device=dev) for _ in range(layers)])
    x = torch.randn(B, L, hidden, device=dev)
    target = torch.randn(B, L, hidden, device=dev)

    # CUDA events around every scan forward and backward
    events = []
    fn = _GatedScanFunction if args.fused else scan_interface._TritonScanFunction
    orig_fwd, orig_bwd = fn.forward, fn.backward

    def timed(orig, kind):
        def wrapper(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(*a, **k)
            e1.record()
            events.append((kind, e0, e1))
            return out
        return staticmethod(wrapper)

    fn.forward, fn.backward = timed(orig_fwd, "fwd"), timed(orig_bwd, "bwd")
    try:
        def step():
            h = x
            for layer in stack:
                h = layer(h, block_l=256, checkpoint=True)
            loss = torch.nn.functional.mse_loss(h, target)
            loss.backward()
            return loss

        for _ in range(args.warmup):
            step()
            stack.zero_grad(set_to_none=True)
        torch.cuda.synchronize()
        events.clear()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = step()
            stack.zero_grad(set_to_none=True)
        e1.record()
        torch.cuda.synchronize()
    finally:
        fn.forward, fn.backward = orig_fwd, orig_bwd
    _lib.check_device_status(dev)
    step_ms = e0.elapsed_time(e1) / args.steps
    scan_fwd_ms = sum(a.elapsed_time(b) for k, a, b in events if k == "fwd") / args.steps
    scan_bwd_ms = sum(a.elapsed_time(b) for k, a, b in events if k == "bwd") / args.steps
    n = B * L * 4096
    print(json.dumps({
        "config": "cfg3_stack", "fused_gates": bool(args.fused), "layers": layers, "hidden": hidden, "state_dim": 4096, "B": B, "L": L,
        "compute_dtype": "bfloat16", "scan_out_dtype": "float32", "loss": float(loss.detach()),
        "step_ms": round(step_ms, 3), "scan_fwd_ms_per_step": round(scan_fwd_ms, 3),
        "scan_bwd_ms_per_step": round(scan_bwd_ms, 3),
        "scan_share_of_step": round((scan_fwd_ms + scan_bwd_ms) / step_ms, 4),
        "scan_gelems_fwd_bwd": layers * n / ((scan_fwd_ms + scan_bwd_ms) * 1e-3) / 1e9,
        "scan_calls_per_step": len(events) // args.steps,
        "note": "scan times include the autograd wrapper (output allocation, dtype casts), 12 layers per step",
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="cfg4", choices=sorted(CONFIGS) + ["cfg3_stack", "cfg3_gates", "cfg3_norm", "strips", "ref_triton"])
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"], help="strips: storage type")
    ap.add_argument("--batch", type=int, default=0, help="strips: one batch size instead of the sweep (with --seq-len: a small case for a profiler)")
    ap.add_argument("--shard", default="none", choices=["none", "batch", "seq"])
    ap.add_argument("--no-checkpoint", action="store_true", help="store fp32 h in the forward instead of recomputing")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--segments", type=int, default=0, help="time segments per GPU (0 = automatic)")
    ap.add_argument("--fused", action="store_true", help="cfg3_stack: SSMFused layers (gates inside the scan kernels)")
    ap.add_argument("--seq-len", type=int, default=0, help="override L (a small case of the same kernels for a profiler)")
    args = ap.parse_args()
    if args.config == "cfg3_stack":
        return run_stack(args)
    if args.config == "cfg3_gates":
        return run_gates(args)
    if args.config == "cfg3_norm":
        return run_norm(args)
    if args.config == "strips":
        return run_strips(args)
    if args.config == "ref_triton":
        return run_ref_triton(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = dict(CONFIGS[args.config])
    B, L, D = cfg["B"], args.seq_len or cfg["L"], cfg["D"]
    total = B * L * D
    if args.shard == "batch":
        assert B % world == 0, "batch must divide over the ranks"
        B //= world
    elif args.shard == "seq":
        assert L % world == 0, "sequence must divide over the ranks"
        L //= world
    dtype, out_dtype = cfg["dtype"], cfg.get("out_dtype", cfg["dtype"])
    inp = make_inputs(B, L, D, dtype=dtype, out_dtype=out_dtype, device=dev, seed=0, decay=cfg["decay"], rank=rank)
    x, a, b, c = inp.tensors()
    dy = inp.dy
    s, so = x.element_size(), dy.element_size()
    ckpt = not args.no_checkpoint

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    res = {}
    if args.shard == "seq" and world > 1:
        ops = CudaShardOps()
        holder = {}

        def fwd():
            holder["y"], holder["tile_h"] = shard_forward(ops, None, x, a, b, c, out_dtype, True)

        def bwd():
            holder["grads"] = shard_backward(ops, None, x, a, b, c, dy, holder["tile_h"])

        res["fwd_ms"] = _median_ms(fwd, args.steps, args.warmup, sync)
        res["bwd_ms"] = _median_ms(bwd, args.steps, args.warmup, sync)
    else:
        y = torch.empty((B, L, D), dtype=out_dtype, device=dev)
        nt = (L + _lib.tile_rows() - 1) // _lib.tile_rows()
        tile_h = torch.empty((B, nt, D), dtype=torch.float32, device=dev) if ckpt else None
        h_saved = None if ckpt else torch.empty((B, L, D), dtype=torch.float32, device=dev)
        grads = [torch.empty_like(x) for _ in range(4)]
        n_seg = args.segments
        res["fwd_ms"] = _median_ms(lambda: _lib.scan_fwd(x, a, b, c, y, tile_h=tile_h, h_saved=h_saved, n_seg=n_seg),
                                   args.steps, args.warmup, sync)
        res["bwd_ms"] = _median_ms(lambda: _lib.scan_bwd(x, a, b, c, dy, *grads, tile_h=tile_h, h_saved=h_saved,
                                                         n_seg=n_seg), args.steps, args.warmup, sync)
        res["fwd_inference_ms"] = _median_ms(lambda: _lib.scan_fwd(x, a, b, c, y, n_seg=n_seg),
                                             args.steps, args.warmup, sync)
        hbuf = grads[0]
        res["forward_only_h_ms"] = _median_ms(lambda: _lib.scan_fwd(x, a, b, None, hbuf, n_seg=n_seg),
                                              args.steps, args.warmup, sync)
    _lib.check_device_status(dev)

    keys = sorted(res)
    t = torch.tensor([res[k] for k in keys], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = dict(zip(keys, (float(v) for v in t.tolist())))

    if rank == 0:
        peak = _copy_peak_gbs()
        extra = 0 if ckpt else 4
        bytes_fwd = 4 * s + so + extra
        bytes_bwd = 8 * s + so + extra
        step_ms = res["fwd_ms"] + res["bwd_ms"]
        n_seg_auto = int(_lib.load().qssm_auto_segments(B, L, D, _lib.dtype_code(dtype)))
        line = {
            "config": args.config, "shard": args.shard, "n_gpus": world, "checkpoint": ckpt,
            "per_rank_shape": [B, L, D], "dtype": str(dtype).replace("torch.", ""),
            "out_dtype": str(out_dtype).replace("torch.", ""),
            "segments_per_gpu": args.segments or n_seg_auto,
            "gelems_fwd_bwd": total / (step_ms * 1e-3) / 1e9,
            "algorithmic_bytes_per_elem": {"fwd": bytes_fwd, "bwd": bytes_bwd},
            "gbs_fwd": total * bytes_fwd / (res["fwd_ms"] * 1e-3) / 1e9,
            "gbs_bwd": total * bytes_bwd / (res["bwd_ms"] * 1e-3) / 1e9,
            "frac_of_measured_hbm_peak": total * (bytes_fwd + bytes_bwd) / (step_ms * 1e-3) / 1e9 / (peak * world),
            "peak_gbs_per_gpu": peak,
            **{k: round(v, 4) for k, v in res.items()},
        }
        if "fwd_inference_ms" in res:
            line["gbs_fwd_inference"] = total * (4 * s + so) / (res["fwd_inference_ms"] * 1e-3) / 1e9
            line["gbs_forward_only_h"] = total * 4 * s / (res["forward_only_h_ms"] * 1e-3) / 1e9
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
