"""GPU parity tests: the CUDA scan (through the C ABI) against the CPU oracle on identical
seeded inputs.  Shapes, distributions and tolerances follow the reference's own tests
(test_forwards.py:23-90,108-114; test_backwards.py:26-116,120-125; test_scan_interface.py:7-31)."""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from quick_ssm_b200 import _lib, scan_interface
from quick_ssm_b200.scan_interface import scan
from quick_ssm_b200.synth import make_inputs
from tolerances import assert_close_f32, assert_close_half

pytestmark = pytest.mark.gpu

DEV = "cuda"

SHAPES = [
    (2, 512, 8),     # test_forwards.py __main__ case 1
    (1, 4, 1),       # tiny, D = 1 (guarded path)
    (1, 1024, 1),    # one channel, long
    (2, 2048, 8),    # test_backwards.py __main__ case 1
    (2, 32, 4),      # test_scan_interface.py
    (1, 50, 2),      # L not a multiple of the tile, guarded path
    (1, 7, 1),
    (2, 64, 3),
    (1, 1, 5),       # single step
    (1, 16, 32),     # exactly one tile
    (2, 17, 40),     # one row into the second tile; partial second column strip (fp32)
    (3, 100, 72),    # partial strips for both element sizes
    (2, 333, 130),
    (4, 2048, 16),   # benchmark configuration 0
]


def _oracle(inp, dtype):
    x, a, b, c, dy = (t.float().cpu() for t in (inp.x, inp.a, inp.b, inp.c, inp.dy))
    h, y, _ = so.scan_forward(x, a, b, c, dtype=dtype)
    dx, da, db, dc, _ = so.scan_backward(x, a, b, c, dy, dtype=dtype)
    return dict(h=h, y=y, dx=dx, da=da, db=db, dc=dc)


def _run_scan(inp, checkpoint=True, out_dtype=None, **kw):
    x, a, b, c = (t.to(DEV).requires_grad_() for t in inp.tensors())
    y = scan(x, a, b, c, checkpoint=checkpoint, out_dtype=out_dtype, **kw)
    y.backward(inp.dy.to(DEV))
    _lib.check_device_status(synchronize=True)
    return dict(y=y, dx=x.grad, da=a.grad, db=b.grad, dc=c.grad)


def _check(got, ref, dtype):
    for k in ("y", "dx", "da", "db", "dc"):
        if dtype == torch.float32:
            assert_close_f32(got[k], ref[k], k)
        else:
            assert_close_half(got[k], ref[k], k)


@pytest.fixture(params=[0, 3], ids=["seg_auto", "seg3"])
def segments(request):
    old = scan_interface.DEFAULT_SEGMENTS
    scan_interface.DEFAULT_SEGMENTS = request.param
    yield request.param
    scan_interface.DEFAULT_SEGMENTS = old


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("checkpoint", [True, False], ids=["ckpt", "saved_h"])
def test_fp32_matches_float64_loop(shape, checkpoint, segments):
    inp = make_inputs(*shape, dtype=torch.float32, seed=11)
    ref = _oracle(inp, np.float64)
    got = _run_scan(inp, checkpoint=checkpoint)
    _check(got, ref, torch.float32)


@pytest.mark.parametrize("shape", [(2, 512, 8), (1, 50, 2), (3, 100, 72), (2, 333, 130), (2, 128, 256),
                                   (2, 100, 330), (1, 45, 520), (3, 17, 1024)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("checkpoint", [True, False], ids=["ckpt", "saved_h"])
def test_half_matches_fp32_loop(shape, dtype, checkpoint, segments):
    inp = make_inputs(*shape, dtype=dtype, seed=5)
    ref = _oracle(inp, np.float32)
    got = _run_scan(inp, checkpoint=checkpoint)
    assert got["y"].dtype == dtype and got["dx"].dtype == dtype
    _check(got, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_half_inputs_fp32_output(dtype, segments):
    """layers.SSM asks for an fp32 result from 16-bit gates (layers.py:90-104)."""
    inp = make_inputs(2, 200, 136, dtype=dtype, out_dtype=torch.float32, seed=9)
    ref = _oracle(inp, np.float32)
    got = _run_scan(inp, out_dtype=torch.float32)
    assert got["y"].dtype == torch.float32 and got["da"].dtype == dtype
    assert_close_f32(got["y"], _oracle(inp, np.float64)["y"], "y")
    for k in ("dx", "da", "db", "dc"):
        assert_close_half(got[k], ref[k], k)


def test_invariant_to_block_and_tiles():
    inp = make_inputs(3, 300, 48, dtype=torch.float32, seed=2)
    base = _run_scan(inp)
    other = _run_scan(inp, block_l=16, tile_b=1, tile_d=16)
    for k in base:
        assert torch.equal(base[k], other[k]), k


def test_segment_counts_agree():
    inp = make_inputs(2, 1000, 40, dtype=torch.float32, seed=4)
    ref = _oracle(inp, np.float64)
    old = scan_interface.DEFAULT_SEGMENTS
    try:
        for n in (1, 2, 5, 16, 63):
            scan_interface.DEFAULT_SEGMENTS = n
            _check(_run_scan(inp), ref, torch.float32)
    finally:
        scan_interface.DEFAULT_SEGMENTS = old


def test_no_grad_and_partial_grads():
    inp = make_inputs(2, 70, 24, dtype=torch.float32, seed=8).to(DEV)
    with torch.no_grad():
        y0 = scan(*inp.tensors())
    x = inp.x.clone().requires_grad_()
    y1 = scan(x, inp.a, inp.b, inp.c)
    y1.backward(inp.dy)
    assert torch.equal(y0, y1)
    ref = _oracle(inp, np.float64)
    assert_close_f32(x.grad, ref["dx"], "dx")


def test_noncontiguous_views_and_mixed_dtypes():
    big = make_inputs(2, 96, 192, dtype=torch.bfloat16, seed=3).to(DEV)
    sl = slice(64, 192)  # channel shard: same row pitch, fewer channels
    views = [t[:, :, sl] for t in big.tensors()]
    y = scan(*views)
    y_ref = scan(*[v.contiguous() for v in views])
    assert torch.equal(y, y_ref)
    # transposed storage (D not innermost) and a mixed-dtype call are made addressable by copying
    xt = big.x.transpose(1, 2).contiguous().transpose(1, 2)
    assert torch.equal(scan(xt, big.a, big.b, big.c), scan(big.x, big.a, big.b, big.c))
    y_mixed = scan(big.x.float(), big.a, big.b, big.c)
    assert y_mixed.dtype == torch.float32
    inp32 = [t.float() for t in big.tensors()]
    assert torch.allclose(y_mixed, scan(*inp32))


def test_shape_and_backend_errors():
    x = torch.zeros(2, 8, 4, device=DEV)
    with pytest.raises(ValueError):
        scan(x, x[:, :4], x, x)
    with pytest.raises(ValueError):
        scan(x, x, x, x, backend="cudnn")
    with pytest.raises(RuntimeError):
        scan(x.cpu(), x.cpu(), x.cpu(), x.cpu(), backend="triton")


def test_empty_inputs():
    for shape in [(2, 0, 4), (0, 8, 4), (2, 8, 0)]:
        x = torch.zeros(shape, device=DEV, requires_grad=True)
        y = scan(x, x, x, x)
        assert y.shape == torch.Size(shape)
        y.sum().backward()
        assert x.grad.shape == torch.Size(shape)


def test_known_answer_geometric_decay():
    """Impulse response with a constant gate g: h(t) = g^t (forward_only.py:548-629, with a
    gate that keeps the expected value well above the underflow that makes the reference's
    own check degenerate)."""
    from quick_ssm_b200.forward_only import block_scan_forward_3d
    L, g = 1 << 16, 0.9999
    x = torch.zeros(1, L, 8, device=DEV)
    x[:, 0] = 1.0
    a = torch.full_like(x, g)
    b = torch.ones_like(x)
    h = block_scan_forward_3d(x, a, b)
    g32 = float(np.float32(g))
    expect = g32 ** np.arange(L, dtype=np.float64)
    got = h[0, :, 3].double().cpu().numpy()
    assert np.abs(got / expect - 1).max() < 1e-5 * 50  # 65535 fp32 roundings of a running product
    assert abs(got[-1] / expect[-1] - 1) < 5e-4


def test_seeded_halves_equal_whole():
    """Two sequence shards run one after the other reproduce the unsharded scan."""
    inp = make_inputs(2, 256, 40, dtype=torch.float32, seed=6).to(DEV)
    x, a, b, c = inp.tensors()
    B, L, D = x.shape
    whole = torch.empty_like(x)
    h_last = torch.empty(B, D, device=DEV)
    _lib.scan_fwd(x, a, b, c, whole, h_last=h_last)
    half = L // 2
    lo, hi = slice(0, half), slice(half, L)
    y = torch.empty_like(x)
    mid = torch.empty(B, D, device=DEV)
    end = torch.empty(B, D, device=DEV)
    _lib.scan_fwd(x[:, lo], a[:, lo], b[:, lo], c[:, lo], y[:, lo], h_last=mid)
    _lib.scan_fwd(x[:, hi], a[:, hi], b[:, hi], c[:, hi], y[:, hi], h_in=mid, h_last=end)
    torch.cuda.synchronize()
    assert torch.allclose(y, whole, rtol=1e-6, atol=1e-6)
    assert torch.allclose(end, h_last, rtol=1e-6, atol=1e-6)
    # aggregates: h_end = A * h_in + H
    A = torch.empty(B, D, device=DEV)
    H = torch.empty(B, D, device=DEV)
    _lib.aggregate_fwd(x[:, hi], a[:, hi], b[:, hi], A, H)
    assert torch.allclose(A * mid + H, end, rtol=1e-5, atol=1e-6)
    assert torch.allclose(A, a[:, hi].double().prod(dim=1).float(), rtol=1e-5, atol=1e-30)
    stack_a = torch.stack([torch.ones_like(A), A])
    stack_h = torch.stack([mid, H])
    folded = _lib.carry_fold(stack_a, stack_h, 2, reverse=False)
    assert torch.allclose(folded, end, rtol=1e-5, atol=1e-6)

    # backward: the later shard hands a(t0)*dh(t0) to the earlier one
    dy = inp.dy
    ref = _oracle(inp, np.float64)
    grads = [torch.empty_like(x) for _ in range(4)]
    g_mid = torch.empty(B, D, device=DEV)
    th_lo = torch.empty(B, (half + 15) // 16, D, device=DEV)
    th_hi = torch.empty(B, (L - half + 15) // 16, D, device=DEV)
    _lib.scan_fwd(x[:, lo], a[:, lo], b[:, lo], c[:, lo], y[:, lo], tile_h=th_lo, h_last=mid)
    _lib.scan_fwd(x[:, hi], a[:, hi], b[:, hi], c[:, hi], y[:, hi], tile_h=th_hi, h_in=mid)
    out_hi = [torch.empty(B, L - half, D, device=DEV) for _ in range(4)]
    out_lo = [torch.empty(B, half, D, device=DEV) for _ in range(4)]
    _lib.scan_bwd(x[:, hi], a[:, hi], b[:, hi], c[:, hi], dy[:, hi], *out_hi, tile_h=th_hi, g_first=g_mid)
    _lib.scan_bwd(x[:, lo], a[:, lo], b[:, lo], c[:, lo], dy[:, lo], *out_lo, tile_h=th_lo, g_in=g_mid)
    torch.cuda.synchronize()
    for k, lo_t, hi_t in zip(("dx", "da", "db", "dc"), out_lo, out_hi):
        assert_close_f32(torch.cat([lo_t, hi_t], dim=1), ref[k], k)
    P = torch.empty(B, D, device=DEV)
    Q = torch.empty(B, D, device=DEV)
    _lib.aggregate_bwd(a[:, hi], c[:, hi], dy[:, hi], P, Q)
    assert torch.allclose(Q, g_mid, rtol=1e-5, atol=1e-6)


def test_kernel_level_entry_points():
    """block_scan_forward_3d -> (cumprod a, h); block_scan_backward_3d(a,b,c,x,h,dy)."""
    from quick_ssm_b200.triton_backwards import block_scan_backward_3d
    from quick_ssm_b200.triton_forwards import block_scan_forward_3d
    for shape, seed in [((2, 512, 8), 42), ((1, 4, 1), 3), ((1, 1024, 1), 4), ((2, 2048, 8), 0)]:
        torch.manual_seed(seed)
        x = torch.randn(*shape)
        a = torch.rand(*shape) * 0.1 + 0.9
        b = torch.randn(*shape) * 0.1
        c = torch.randn(*shape)
        dy = torch.randn(*shape)
        out_a, h = block_scan_forward_3d(x.to(DEV), a.to(DEV), b.to(DEV), BLOCK_L=128)
        h_ref, _, _ = so.scan_forward(x, a, b, dtype=np.float64)
        assert_close_f32(h, h_ref, "h")
        assert torch.allclose(out_a.cpu().double(), torch.cumprod(a.double(), dim=1), rtol=1e-4, atol=1e-30)
        grads = block_scan_backward_3d(a.to(DEV), b.to(DEV), c.to(DEV), x.to(DEV), h, dy.to(DEV))
        ref = so.scan_backward(x, a, b, c, dy, dtype=np.float64)
        for name, g, r in zip(("dx", "da", "db", "dc"), grads, ref):
            assert g.dtype == torch.float32
            assert_close_f32(g, r, name)
    e = torch.empty(2, 0, 4, device=DEV)
    assert block_scan_forward_3d(e, e, e)[1].shape == e.shape


def test_segment_aggregates_are_reused_by_the_scan():
    """n_seg = -k: the scan takes the per-segment aggregates an aggregate call left in the workspace."""
    inp = make_inputs(2, 3000, 70, dtype=torch.bfloat16, seed=12).to(DEV)
    x, a, b, c = inp.tensors()
    B, L, D = x.shape
    k = 6
    h0 = torch.randn(B, D, device=DEV)
    ref = torch.empty_like(x)
    _lib.scan_fwd(x, a, b, c, ref, h_in=h0, n_seg=k)
    ws = torch.empty(3 * B * k * D * 4, dtype=torch.uint8, device=DEV)
    A = torch.empty(B, D, device=DEV)
    H = torch.empty(B, D, device=DEV)
    _lib.aggregate_fwd(x, a, b, A, H, n_seg=k, ws=ws)
    got = torch.empty_like(x)
    _lib.scan_fwd(x, a, b, c, got, h_in=h0, n_seg=-k, ws=ws)
    assert torch.equal(got, ref)
    # backward twin
    th = torch.empty(B, (L + 15) // 16, D, device=DEV)
    _lib.scan_fwd(x, a, b, c, ref, tile_h=th, h_in=h0)
    g0 = torch.randn(B, D, device=DEV)
    want = [torch.empty_like(x) for _ in range(4)]
    _lib.scan_bwd(x, a, b, c, inp.dy, *want, tile_h=th, g_in=g0, n_seg=k)
    P = torch.empty(B, D, device=DEV)
    Q = torch.empty(B, D, device=DEV)
    _lib.aggregate_bwd(a, c, inp.dy, P, Q, n_seg=k, ws=ws)
    have = [torch.empty_like(x) for _ in range(4)]
    _lib.scan_bwd(x, a, b, c, inp.dy, *have, tile_h=th, g_in=g0, n_seg=-k, ws=ws)
    _lib.check_device_status(synchronize=True)
    for w, h in zip(want, have):
        assert torch.equal(w, h)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (1, 5000, 72)), (torch.bfloat16, (2, 3001, 200)),
                                         (torch.float16, (3, 700, 64))], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("chunk_rows", [64, 256])
def test_chained_single_pass_forward(tune, dtype, shape, chunk_rows):
    """The single-pass forward for few chains (chunks claimed from a ticket counter, carries found by
    looking back over chunk descriptors), forced on small shapes: forward, boundary states (through the
    backward that consumes them), seed and end state."""
    tune("CHAINED", "2")
    tune("CHUNK_ROWS", str(chunk_rows))
    inp = make_inputs(*shape, dtype=dtype, seed=23)
    ref = _oracle(inp, np.float64 if dtype == torch.float32 else np.float32)
    got = _run_scan(inp)
    _check(got, ref, dtype)
    # seeded, with the end state
    x, a, b, c = (t.to(DEV) for t in inp.tensors())
    B, L, D = x.shape
    h0 = torch.randn(B, D, device=DEV)
    y = torch.empty_like(x)
    h_last = torch.empty(B, D, device=DEV)
    _lib.scan_fwd(x, a, b, c, y, h_in=h0, h_last=h_last)
    tune("CHAINED", "0")
    y_ref = torch.empty_like(x)
    h_ref = torch.empty(B, D, device=DEV)
    _lib.scan_fwd(x, a, b, c, y_ref, h_in=h0, h_last=h_ref, n_seg=1)
    _lib.check_device_status(synchronize=True)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-3)
    assert torch.allclose(y.float(), y_ref.float(), **tol)
    assert torch.allclose(h_last, h_ref, rtol=1e-4, atol=1e-5)


def test_chained_single_pass_is_deterministic(tune):
    """Chunks run concurrently and find their carries in whatever state the predecessors are in, but the
    carry is always folded chunk by chunk in time order: results are bit-identical from run to run and
    for any number of warps working at once."""
    tune("CHAINED", "2")
    tune("CHUNK_ROWS", "64")
    inp = make_inputs(2, 20000, 128, dtype=torch.bfloat16, seed=31)
    runs = []
    for grid in ("0", "0", "37", "1000"):
        tune("CHAINED_GRID", grid)
        runs.append(_run_scan(inp))
    for other in runs[1:]:
        for k in runs[0]:
            assert torch.equal(runs[0][k], other[k]), k


@pytest.mark.parametrize("slots", [2, 4, 8])
def test_chained_look_back_survives_descriptor_slots_changing_hands(tune, slots):
    """A descriptor ring far smaller than the chunks of a chain in flight: chunks take over slots while
    readers that loaded their window earlier still look for the old owner.  The look-back must notice (a
    larger tag), start over and still deliver the same carries: results equal the oracle and are
    bit-identical to a run with a roomy ring."""
    tune("CHAINED", 2)
    tune("CHUNK_ROWS", 32)
    inp = make_inputs(1, 40000, 64, dtype=torch.float32, seed=37)   # one chain, 1250 chunks, hundreds of warps on it
    ref = _oracle(inp, np.float64)
    roomy = _run_scan(inp)
    tune("CHAINED_SLOTS", slots)
    tight = _run_scan(inp)
    _check(tight, ref, torch.float32)
    for k in roomy:
        assert torch.equal(roomy[k], tight[k]), k


@pytest.mark.parametrize("shape,dtype", [((2, 100, 72), torch.float32), ((3, 77, 200), torch.bfloat16),
                                         ((1, 50, 3), torch.float32), ((2, 300, 330), torch.float16)],
                         ids=["fp32", "bf16", "fp32_guarded_path", "fp16_wide"])
def test_no_write_outside_the_outputs(shape, dtype):
    """Outputs live inside sentinel-filled buffers; rows before and after them must stay untouched
    (partial tiles, partial strips and the guarded path all clip their stores)."""
    B, L, D = shape
    inp = make_inputs(B, L, D, dtype=dtype, seed=41).to(DEV)
    x, a, b, c = inp.tensors()
    pad = 64
    sentinel = -8192.0

    def guarded(dt):
        buf = torch.full((B * L * D + 2 * pad,), sentinel, dtype=dt, device=DEV)
        return buf, buf[pad:pad + B * L * D].view(B, L, D)

    ybuf, y = guarded(dtype)
    nt = (L + 15) // 16
    thbuf = torch.full((B * nt * D + 2 * pad,), sentinel, dtype=torch.float32, device=DEV)
    th = thbuf[pad:pad + B * nt * D].view(B, nt, D)
    gbufs, grads = zip(*(guarded(dtype) for _ in range(4)))
    for n_seg in (0, 3):
        _lib.scan_fwd(x, a, b, c, y, tile_h=th, n_seg=n_seg)
        _lib.scan_bwd(x, a, b, c, inp.dy, *grads, tile_h=th, n_seg=n_seg)
    _lib.check_device_status(synchronize=True)
    for buf in (ybuf, thbuf) + tuple(gbufs):
        assert bool((buf[:pad].float() == sentinel).all()) and bool((buf[-pad:].float() == sentinel).all())
    assert not bool((y.float() == sentinel).any())


@pytest.mark.parametrize("env", [{"QSSM_V": "1"}, {"QSSM_V": "2"}, {"QSSM_TB": "32"}, {"QSSM_V": "1", "QSSM_TB": "32"},
                                 {"QSSM_WIDE": "0"}, {"QSSM_NO_TMA": "1"}, {"QSSM_STAGES": "2"}],
                         ids=lambda e: "_".join(f"{k[5:]}{v}" for k, v in e.items()))
def test_every_kernel_variant_gives_the_same_answer(tune, env):
    """Strip width, tile height, ring depth, wide/narrow stores and the guarded path are launch-shape
    choices: forcing each of them must not change the result beyond fp32 rounding."""
    inp = make_inputs(2, 700, 330, dtype=torch.bfloat16, seed=43)
    ref = _oracle(inp, np.float32)
    base = _run_scan(inp)
    for k, v in env.items():
        tune(k[5:], v)
    for checkpoint in (True, False):
        got = _run_scan(inp, checkpoint=checkpoint)
        _check(got, ref, torch.bfloat16)
        for k in base:
            assert torch.allclose(got[k].float(), base[k].float(), rtol=2e-2, atol=1e-3), k


@pytest.mark.parametrize("shape", [(1, 9000, 2048), (4, 203, 2048), (5, 203, 2048), (3, 203, 4070), (4, 203, 4096),
                                   (12, 150, 4096)],
                         ids=["32_strips_long", "128_strips", "160_strips", "192_strips", "256_strips", "768_strips"])
@pytest.mark.parametrize("route", ["auto", "one_pass"])
def test_fp32_launch_shapes_by_strip_count_match_float64(shape, route):
    """fp32 storage picks its launch shape by the number of 64-channel strips: below one strip per SM both
    directions take the chained kernels, above it the forward runs one warp per strip (narrow or wide strips,
    16- or 32-row tiles) while the backward stays chained up to five strips per SM and then takes 32-row tiles.
    `one_pass` forces one warp per strip in both directions (n_seg = 1), which reaches the tile-height choices
    the automatic route leaves to the chained kernels.  Ragged last tile in time, ragged last strip."""
    B, L, D = shape
    inp = make_inputs(B, L, D, dtype=torch.float32, seed=59)
    ref = _oracle(inp, np.float64)
    if route == "auto":
        if torch.cuda.get_device_properties(0).multi_processor_count == 148 and B * ((D + 63) // 64) >= 148:
            assert _lib.auto_segments(B, 1 << 16, D, torch.float32) == 1
        got = _run_scan(inp)
    else:
        x, a, b, c, dy = (t.to(DEV) for t in (inp.x, inp.a, inp.b, inp.c, inp.dy))
        y = torch.empty_like(x)
        th = torch.empty((B, (L + 15) // 16, D), dtype=torch.float32, device=DEV)
        g = [torch.empty_like(x) for _ in range(4)]
        _lib.scan_fwd(x, a, b, c, y, tile_h=th, n_seg=1)
        _lib.scan_bwd(x, a, b, c, dy, *g, tile_h=th, n_seg=1)
        _lib.check_device_status(synchronize=True)
        got = dict(y=y, dx=g[0], da=g[1], db=g[2], dc=g[3])
    _check(got, ref, torch.float32)


@pytest.mark.parametrize("shape,dtype,out_dtype", [((5, 203, 4096), torch.bfloat16, None), ((6, 150, 4070), torch.float16, None),
                                                   ((5, 203, 4096), torch.bfloat16, torch.float32)],
                         ids=["bf16_320_strips", "fp16_384_strips_ragged", "bf16_320_strips_fp32_out"])
def test_half_between_two_and_three_strips_per_sm_matches_fp32_loop(shape, dtype, out_dtype):
    """16-bit storage with 2 to 2.75 strips per SM: the forward with 16-bit output runs one warp per strip on
    32-row tiles while the backward (and the forward with fp32 output) stays on the chained kernels, so one
    autograd step mixes the two routes through the same tile states."""
    inp = make_inputs(*shape, dtype=dtype, out_dtype=out_dtype, seed=61)
    ref = _oracle(inp, np.float32)
    got = _run_scan(inp, out_dtype=out_dtype)
    _check(got, ref, dtype)


@pytest.mark.parametrize("shape,dtype,out_dtype", [((8, 200, 4096), torch.bfloat16, None),
                                                   ((8, 200, 4000), torch.float16, None),
                                                   ((9, 137, 3784), torch.bfloat16, torch.float32)],
                         ids=["bf16_full_strips", "fp16_ragged_channels", "bf16_fp32_out_ragged"])
@pytest.mark.parametrize("checkpoint", [True, False], ids=["ckpt", "saved_h"])
@pytest.mark.parametrize("fwd_tile4", ["0", "1"], ids=["fwd_auto", "fwd_four_strips"])
def test_four_strip_kernels_match_the_oracle(tune, shape, dtype, out_dtype, checkpoint, fwd_tile4):
    """Shapes wide enough for the kernels that give a CTA four adjacent strips (16-bit storage, enough
    groups of four strips to fill the GPU): a partial last tile in time, a channel count that leaves the
    last group with fewer than four strips and a partial strip, fp32 y/dy, stored h and recompute.  The
    forward takes the four-strip kernel by itself only when it stores h; QSSM_FWD_TILE4=1 forces it for
    the other forwards too.  Narrow kernels on the same input must agree within rounding."""
    tune("FWD_TILE4", fwd_tile4)
    inp = make_inputs(*shape, dtype=dtype, out_dtype=out_dtype, seed=47)
    ref = _oracle(inp, np.float32)
    got = _run_scan(inp, checkpoint=checkpoint, out_dtype=out_dtype)
    _check(got, ref, dtype)
    tune("WIDE", "0")
    narrow = _run_scan(inp, checkpoint=checkpoint, out_dtype=out_dtype)
    for k in got:
        assert torch.allclose(got[k].float(), narrow[k].float(), rtol=2e-2, atol=1e-3), k


def test_expired_wait_is_reported_and_the_context_survives(tune):
    """The failure path of the bounded waits, on a healthy GPU: a test hook starts the chunk counter of
    the single-pass kernel past the first chunk of every chain, so nothing ever publishes those chunks;
    the look-back waits of the other chunks run into their (shortened) limit, the kernel records the
    status code and returns, the host raises, and the next launch works as usual."""
    tune("CHAINED", "2")
    tune("CHUNK_ROWS", "64")
    tune("WAIT_MS", "100")
    inp = make_inputs(1, 2000, 64, dtype=torch.float32, seed=51).to(DEV)
    x, a, b, c = inp.tensors()
    y = torch.empty_like(x)
    tune("TEST_SKIP_FIRST_CHUNK", "1")
    _lib.scan_fwd(x, a, b, c, y)  # launches fine; the error is found on the device
    with pytest.raises(RuntimeError, match="expired"):
        _lib.check_device_status(synchronize=True)
    tune("TEST_SKIP_FIRST_CHUNK", 0)
    _lib.scan_fwd(x, a, b, c, y)
    _lib.check_device_status(synchronize=True)
    ref = _oracle(inp, np.float64)
    assert_close_f32(y, ref["y"], "y after the failed launch")


def test_views_with_odd_offsets_and_pitches():
    """Batch, time and channel slices of larger tensors are scanned in place; a channel slice that
    starts at an odd element (base not 16-byte aligned) takes the guarded path; results equal those
    of contiguous copies."""
    big = make_inputs(3, 120, 200, dtype=torch.bfloat16, seed=61).to(DEV)
    for sl in [(slice(1, 3), slice(None), slice(None)),        # batch slice
               (slice(None), slice(7, 100), slice(None)),      # time slice (still addressed in place)
               (slice(None), slice(None), slice(1, 66)),       # odd channel offset: unaligned base
               (slice(0, 2), slice(16, 48), slice(8, 136))]:   # all three, aligned
        views = [t[sl] for t in big.tensors()]
        dy = big.dy[sl]
        outs = []
        for tensors, g in ((views, dy), ([v.contiguous() for v in views], dy.contiguous())):
            leaves = [t.detach().clone().requires_grad_() if t.is_contiguous() else t.detach().requires_grad_()
                      for t in tensors]
            y = scan(*leaves)
            y.backward(g)
            outs.append([y] + [t.grad for t in leaves])
        for u, v in zip(*outs):
            assert torch.equal(u, v)
    _lib.check_device_status(synchronize=True)


def test_two_host_threads_on_their_own_streams():
    """Two host threads, each on its own CUDA stream, run forward + backward repeatedly on different shapes at
    the same time (one few-strip shape on the chained kernels, one on the one-warp kernels): the per-thread
    tensor-map cache, the shared kernel-attribute cache and the per-call workspaces must keep them apart."""
    import threading
    cases = [make_inputs(1, 6000, 192, dtype=torch.bfloat16, seed=71, decay="near_unit"),
             make_inputs(6, 300, 2048, dtype=torch.float32, seed=73)]
    refs = [_oracle(cases[0], np.float32), _oracle(cases[1], np.float64)]
    results, errors = [None, None], []

    def work(i):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                dev = [t.to(DEV) for t in (*cases[i].tensors(), cases[i].dy)]
                for _ in range(6):
                    x, a, b, c = (t.detach().requires_grad_() for t in dev[:4])
                    y = scan(x, a, b, c)
                    y.backward(dev[4])
                    results[i] = dict(y=y.detach(), dx=x.grad, da=a.grad, db=b.grad, dc=c.grad)
                stream.synchronize()
        except Exception as e:  # surfaced in the main thread below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    _lib.check_device_status(synchronize=True)
    for i, dt in enumerate((torch.bfloat16, torch.float32)):
        if dt == torch.bfloat16:
            for k in ("y", "dx", "da", "db", "dc"):
                assert_close_half(results[i][k], refs[i][k], k, scale_atol=max(1.0, float(np.abs(refs[i][k]).max())))
        else:
            _check(results[i], refs[i], dt)
