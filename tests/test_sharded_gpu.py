"""Sequence shards on ONE GPU: the device side of the sharded scan (``CudaShardOps``: aggregate with
its segment workspace, the fold over the gathered aggregates read in place, the seeded scan that
reuses the workspace) run for G = 2, 3, 4, 8 shards one after the other on the same device and
checked against the CPU oracle over the whole sequence.  The collective is replaced by a stand-in
that hands every "rank" the stacked aggregates, so no process group is needed; the NCCL path
itself is covered by the multi-GPU test and by the gloo tests on CPU."""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from quick_ssm_b200 import _lib
from quick_ssm_b200 import sharded
from quick_ssm_b200.synth import make_inputs
from tolerances import assert_close_f32, assert_close_half

pytestmark = pytest.mark.gpu
DEV = "cuda"


class BoardComm:
    """Rank ``rank`` of ``world`` in-process shards; ``all_gather`` copies the board the test has
    filled with every rank's send buffer."""

    def __init__(self, rank, world):
        self.rank, self.world = rank, world
        self.board = None

    def all_gather(self, full, send):
        assert torch.equal(self.board[self.rank], send), "a rank's own entry must be what it sent"
        full.copy_(self.board)


def _bounds(L, G, ragged):
    if not ragged:
        per = L // G
        return [(r * per, (r + 1) * per if r < G - 1 else L) for r in range(G)]
    cuts = [0] + sorted(int(L * f) for f in np.linspace(0.13, 0.91, G - 1)) + [L]
    return list(zip(cuts[:-1], cuts[1:]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16_near_unit"])
@pytest.mark.parametrize("G,ragged", [(2, False), (3, True), (4, False), (8, False)], ids=["G2", "G3_ragged", "G4", "G8"])
def test_in_process_shards_match_the_oracle(dtype, G, ragged):
    B, L, D = 2, 8192, 96
    inp = make_inputs(B, L, D, dtype=dtype, seed=7, decay="near_unit")
    dev = inp.to(DEV)
    bounds = _bounds(L, G, ragged)
    shards = [[t[:, lo:hi] for t in (dev.x, dev.a, dev.b, dev.c, dev.dy)] for lo, hi in bounds]
    comms = [BoardComm(r, G) for r in range(G)]
    ops = [sharded.CudaShardOps() for _ in range(G)]
    # the shards are long and narrow enough that the library cuts each of them into time segments,
    # so the aggregate call leaves per-segment aggregates that the seeded scan reuses
    assert _lib.auto_segments(B, bounds[0][1] - bounds[0][0], D, dtype) > 1

    # forward: every rank's aggregate, the "all-gather", then fold + seeded scan per rank
    exs = [sharded.forward_aggregate(ops[r], comms[r], *shards[r][:3]) for r in range(G)]
    board = torch.stack([ex.send for ex in exs])
    ys, tile_hs = [], []
    for r in range(G):
        comms[r].board = board
        x, a, b, c, dy = shards[r]
        y = torch.empty_like(x)
        th = torch.empty((B, (x.shape[1] + 15) // 16, D), dtype=torch.float32, device=DEV)
        sharded.forward_finish(ops[r], comms[r], exs[r], x, a, b, c, y, th)
        assert ops[r]._ws_fwd is None, "the segment workspace must have been consumed by the scan"
        ys.append(y)
        tile_hs.append(th)

    # backward
    exs = [sharded.backward_aggregate(ops[r], comms[r], shards[r][1], shards[r][3], shards[r][4]) for r in range(G)]
    board = torch.stack([ex.send for ex in exs])
    grads = []
    for r in range(G):
        comms[r].board = board
        x, a, b, c, dy = shards[r]
        g = [torch.empty_like(x) for _ in range(4)]
        sharded.backward_finish(ops[r], comms[r], exs[r], x, a, b, c, dy, tile_hs[r], g)
        grads.append(g)
    _lib.check_device_status(synchronize=True)

    acc = np.float64 if dtype == torch.float32 else np.float32
    f = [t.float() for t in (inp.x, inp.a, inp.b, inp.c, inp.dy)]
    _, y_ref, _ = so.scan_forward(*f[:4], dtype=acc)
    g_ref = so.scan_backward(*f, dtype=acc)[:4]
    check = assert_close_f32 if dtype == torch.float32 else assert_close_half
    check(torch.cat(ys, dim=1), y_ref, f"y (G={G})")
    for i, name in enumerate(("dx", "da", "db", "dc")):
        got = torch.cat([g[i] for g in grads], dim=1)
        if dtype == torch.float32:
            assert_close_f32(got, g_ref[i], f"{name} (G={G})")
        else:
            # near-unit decay over 8192 steps: gradients reach tens, the absolute floor scales with them
            assert_close_half(got, g_ref[i], f"{name} (G={G})", scale_atol=max(1.0, float(np.abs(g_ref[i]).max())))


def test_fold_reads_the_gathered_buffer_in_place():
    """``carry_fold`` on strided ``[G, B, D]`` views of a ``[G, 2, B, D]`` buffer equals the fold of
    contiguous copies, forward and reverse, for every rank."""
    G, B, D = 5, 3, 70
    torch.manual_seed(0)
    full = torch.rand(G, 2, B, D, device=DEV) * 0.2 + 0.85
    A, H = full[:, 0], full[:, 1]
    assert not A.is_contiguous()
    for upto in range(G):
        for reverse in (False, True):
            got = _lib.carry_fold(A, H, upto, reverse=reverse)
            want = _lib.carry_fold(A.contiguous(), H.contiguous(), upto, reverse=reverse)
            assert torch.equal(got, want)
            run = np.zeros((B, D))
            ks = range(G - 1, upto, -1) if reverse else range(0, upto)
            for k in ks:
                run = A[k].double().cpu().numpy() * run + H[k].double().cpu().numpy()
            assert np.allclose(got.cpu().numpy(), run, rtol=1e-5, atol=1e-6)


def test_full_size_long_sequence_in_eight_shards():
    """The long-sequence benchmark configuration (B=1, L=2^20, D=2048, fp16, decay close to one) at full size,
    cut into eight shards run one after the other on this GPU: the sharded result must agree with the unsharded
    one everywhere (same kernels' arithmetic, different carries' rounding) and with the oracle on whole strips."""
    from quick_ssm_b200.synth import make_config
    inp = make_config("cfg2", device=DEV)
    x, a, b, c = inp.tensors()
    dy = inp.dy
    B, L, D = x.shape
    G = 8
    bounds = _bounds(L, G, False)
    shards = [[t[:, lo:hi] for t in (x, a, b, c, dy)] for lo, hi in bounds]
    comms = [BoardComm(r, G) for r in range(G)]
    ops = [sharded.CudaShardOps() for _ in range(G)]
    y = torch.empty_like(x)
    tile_h = torch.empty((B, L // 16, D), dtype=torch.float32, device=DEV)
    grads = [torch.empty_like(x) for _ in range(4)]
    exs = [sharded.forward_aggregate(ops[r], comms[r], *shards[r][:3]) for r in range(G)]
    board = torch.stack([ex.send for ex in exs])
    for r, (lo, hi) in enumerate(bounds):
        comms[r].board = board
        sharded.forward_finish(ops[r], comms[r], exs[r], *shards[r][:4], y[:, lo:hi], tile_h[:, lo // 16:hi // 16])
    exs = [sharded.backward_aggregate(ops[r], comms[r], shards[r][1], shards[r][3], shards[r][4]) for r in range(G)]
    board = torch.stack([ex.send for ex in exs])
    for r, (lo, hi) in enumerate(bounds):
        comms[r].board = board
        sharded.backward_finish(ops[r], comms[r], exs[r], *shards[r], tile_h[:, lo // 16:hi // 16],
                                [g[:, lo:hi] for g in grads])
    _lib.check_device_status(synchronize=True)

    # oracle on three 64-channel strips over all 2^20 steps
    for d0 in (0, 1024, D - 64):
        sl = (slice(None), slice(None), slice(d0, d0 + 64))
        f = [t[sl].float().cpu() for t in (x, a, b, c, dy)]
        _, y_ref, _ = so.scan_forward(*f[:4], dtype=np.float32)
        g_ref = so.scan_backward(*f, dtype=np.float32)[:4]
        assert_close_half(y[sl], y_ref, f"y[{d0}]")
        for name, g, r in zip(("dx", "da", "db", "dc"), grads, g_ref):
            assert_close_half(g[sl], r, f"{name}[{d0}]", scale_atol=max(1.0, float(np.abs(r).max())))

    # the unsharded scan (single-pass kernels) on the same tensors: element-wise agreement over everything
    y1 = torch.empty_like(x)
    g1 = [torch.empty_like(x) for _ in range(4)]
    _lib.scan_fwd(x, a, b, c, y1, tile_h=tile_h)
    _lib.scan_bwd(x, a, b, c, dy, *g1, tile_h=tile_h)
    _lib.check_device_status(synchronize=True)
    chunk = 1 << 27
    for got, ref, name in zip([y] + grads, [y1] + g1, ("y", "dx", "da", "db", "dc")):
        scale = max(1.0, float(ref.float().abs().max()))
        fg, fr = got.reshape(-1), ref.reshape(-1)
        for lo in range(0, fg.numel(), chunk):
            u, v = fg[lo:lo + chunk].float(), fr[lo:lo + chunk].float()
            assert bool(((u - v).abs() <= 1e-3 * scale + 2e-2 * v.abs()).all()), name
