"""Callers of the scan on the GPU: the SSM layer stack (16-bit gates, fp32 scan output) and the
sequence-sharded scan over NCCL when the box has more than one GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scan_oracle as so
from quick_ssm_b200 import SSM, _lib
from quick_ssm_b200.synth import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("compute_dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_ssm_layer_gpu_matches_torch_backend(compute_dtype):
    torch.manual_seed(0)
    layer = SSM(hidden_size=64, state_size_mult=4.0, compute_dtype=compute_dtype, device="cuda")
    x = torch.randn(2, 200, 64, device="cuda")
    outs = {}
    for backend in ("auto", "torch"):
        xi = x.clone().requires_grad_()
        layer.zero_grad()
        y = layer(xi, block_l=128, checkpoint=True, tile_b=1, tile_d=512, scan_out_dtype=torch.float32,
                  backend=backend)
        y.pow(2).mean().backward()
        outs[backend] = (y.detach(), xi.grad, layer.A_proj.weight.grad.clone())
    tol = dict(rtol=1e-3, atol=1e-4) if compute_dtype == torch.float32 else dict(rtol=3e-2, atol=3e-3)
    for got, ref, name in zip(outs["auto"], outs["torch"], ("y", "dx", "dW_A")):
        assert torch.allclose(got, ref, **tol), name
    _lib.check_device_status(synchronize=True)


def test_copy_model_trains_a_few_steps():
    """The shape of the reference's copy task (copy_train.py:20-38): embed -> SSM -> head."""
    torch.manual_seed(0)
    vocab, hidden = 62, 64
    embed = torch.nn.Embedding(vocab, hidden, device="cuda")
    ssm = SSM(hidden_size=hidden, state_size_mult=4.0, compute_dtype=torch.bfloat16, device="cuda")
    head = torch.nn.Linear(hidden, vocab, device="cuda")
    params = list(embed.parameters()) + list(ssm.parameters()) + list(head.parameters())
    opt = torch.optim.AdamW(params, lr=3e-3)
    losses = []
    for _ in range(30):
        src = torch.randint(0, vocab, (16, 8), device="cuda")
        inp = torch.cat([src, torch.cat([torch.zeros_like(src[:, :1]), src[:, :-1]], 1)], 1)
        labels = torch.cat([torch.full_like(src, -100), src], 1)
        logits = head(ssm(embed(inp), block_l=128, checkpoint=True, tile_b=1, tile_d=512,
                          scan_out_dtype=torch.float32))
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, vocab), labels.reshape(-1), ignore_index=-100)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert np.isfinite(losses).all() and losses[-1] < losses[0]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, out_dir, dtype):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from quick_ssm_b200.sharded import scan_sequence_sharded
        L = 4096
        inp = make_inputs(2, L, 96, dtype=dtype, seed=3, decay="near_unit")
        per = L // world
        sl = slice(rank * per, (rank + 1) * per)
        x, a, b, c = (t[:, sl].cuda().requires_grad_() for t in inp.tensors())
        y = scan_sequence_sharded(x, a, b, c)
        y.backward(inp.dy[:, sl].cuda())
        torch.cuda.synchronize()
        torch.save({k: v.detach().float().cpu() for k, v in
                    dict(y=y, dx=x.grad, da=a.grad, db=b.grad, dc=c.grad).items()},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
def test_sequence_sharded_scan_over_nccl(tmp_path, dtype):
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path), dtype), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    inp = make_inputs(2, 4096, 96, dtype=dtype, seed=3, decay="near_unit")
    acc = np.float64 if dtype == torch.float32 else np.float32
    f = [t.float() for t in (inp.x, inp.a, inp.b, inp.c, inp.dy)]
    _, y_ref, _ = so.scan_forward(*f[:4], dtype=acc)
    g_ref = so.scan_backward(*f, dtype=acc)
    got = {k: torch.cat([p[k] for p in parts], dim=1).numpy() for k in parts[0]}
    from tolerances import assert_close_f32, assert_close_half
    check = assert_close_f32 if dtype == torch.float32 else assert_close_half
    check(got["y"], y_ref, "y")
    for k, ref in zip(("dx", "da", "db", "dc"), g_ref):
        check(got[k], ref, k)


def test_streaming_pieces_match_the_seeded_oracle():
    """Pieces of a sequence fed one after the other with the carried state: every piece is checked
    against the CPU oracle run on that piece with the oracle's own carried state (``h_in``), and the
    concatenation against the oracle over the whole sequence.  Includes single-step pieces
    (token-by-token decoding) and an empty piece."""
    from quick_ssm_b200.streaming import ScanState, scan_chunk
    from tolerances import assert_close_f32, assert_close_half
    for dtype in (torch.float32, torch.bfloat16):
        inp = make_inputs(3, 301, 72, dtype=dtype, seed=17)
        dev = inp.to("cuda")
        acc = np.float64 if dtype == torch.float32 else np.float32
        check = assert_close_f32 if dtype == torch.float32 else assert_close_half
        f = [t.float() for t in inp.tensors()]
        _, y_whole, h_whole = so.scan_forward(*f, dtype=acc)
        state, outs, pos = None, [], 0
        ref_state = np.zeros((3, 72), dtype=acc)
        for piece in (1, 1, 30, 0, 16, 17, 200, 36):
            sl = slice(pos, pos + piece)
            y, state = scan_chunk(dev.x[:, sl], dev.a[:, sl], dev.b[:, sl], dev.c[:, sl], state)
            if piece > 0:
                _, y_ref, ref_state = so.scan_forward(*(t[:, sl] for t in f), dtype=acc, h_in=ref_state)
                check(y, y_ref, f"y of piece [{pos}, {pos + piece})")
            check(state.h, ref_state, f"state after step {pos + piece}")
            outs.append(y)
            pos += piece
        assert pos == 301
        check(torch.cat(outs, dim=1), y_whole, "concatenated pieces")
        check(state.h, h_whole, "final state")
        # h itself (no output gate), seeded with an explicit zero state
        h_all, last = scan_chunk(dev.x, dev.a, dev.b, None, ScanState.zeros(3, 72))
        check(h_all, so.scan_forward(*f[:3], dtype=acc)[0], "h")
        check(last.h, h_whole, "h_last")
    _lib.check_device_status(synchronize=True)


@pytest.mark.parametrize("param_dtype,compute_dtype", [(torch.float32, torch.bfloat16), (torch.float32, torch.float32),
                                                      (torch.float32, torch.float16)],
                         ids=["fp32_bf16", "fp32_fp32", "fp32_fp16"])
def test_fused_gate_layer_matches_the_unfused_layer(param_dtype, compute_dtype):
    """SSMFused reads the projection outputs in the scan kernels; output and every gradient must agree
    with the unfused layer that builds the gates with torch element-wise kernels."""
    from quick_ssm_b200.layers import SSMFused
    torch.manual_seed(0)
    ref = SSM(hidden_size=64, state_size_mult=4.0, dtype=param_dtype, compute_dtype=compute_dtype, device="cuda")
    fused = SSMFused(hidden_size=64, state_size_mult=4.0, dtype=param_dtype, compute_dtype=compute_dtype, device="cuda")
    fused.load_state_dict(ref.state_dict())
    x = torch.randn(3, 300, 64, device="cuda", dtype=param_dtype)
    outs = []
    for layer in (ref, fused):
        xi = x.clone().requires_grad_()
        y = layer(xi, scan_out_dtype=torch.float32)
        y.pow(2).mean().backward()
        outs.append([y.detach(), xi.grad] + [p.grad for p in layer.parameters()])
    _lib.check_device_status(synchronize=True)
    tol = dict(rtol=2e-3, atol=2e-5) if compute_dtype == torch.float32 else dict(rtol=3e-2, atol=3e-4)
    names = ["y", "dx"] + [n for n, _ in ref.named_parameters()]
    for name, u, v in zip(names, *outs):
        scale = float(u.abs().max())
        assert torch.allclose(v, u, rtol=tol["rtol"], atol=tol["atol"] + 1e-2 * tol["rtol"] * scale), name


def test_gated_scan_matches_composition_of_torch_gates():
    from quick_ssm_b200.gated import _composed, gated_scan
    torch.manual_seed(1)
    # the last two shapes have enough strips for the wide-strip forward (16-bit y) next to the narrow-strip backward
    for dtype, gate, out, shape in [(torch.float32, torch.bfloat16, torch.float32, (2, 200, 136)),
                                    (torch.bfloat16, torch.bfloat16, torch.bfloat16, (2, 200, 136)),
                                    (torch.float16, torch.float16, torch.float32, (2, 200, 136)),
                                    (torch.float32, torch.float32, torch.float32, (2, 200, 136)),
                                    (torch.bfloat16, torch.bfloat16, torch.bfloat16, (10, 70, 4096)),
                                    (torch.float16, torch.float16, torch.float16, (9, 50, 4070))]:
        pre = [torch.randn(*shape, device="cuda", dtype=dtype) for _ in range(5)]
        dy = torch.randn(*shape, device="cuda", dtype=out)
        res = []
        for fn in (_composed, None):
            leaves = [t.clone().requires_grad_() for t in pre]
            y = fn(*leaves, gate, out) if fn else gated_scan(*leaves, gate_dtype=gate, out_dtype=out)
            y.backward(dy)
            res.append([y.detach()] + [t.grad for t in leaves])
        _lib.check_device_status(synchronize=True)
        for name, u, v in zip(("y", "dpa", "dpx", "dpc1", "dpc2", "dpd"), *res):
            scale = float(u.float().abs().max())
            assert torch.allclose(v.float(), u.float(), rtol=3e-2, atol=3e-3 * max(scale, 1.0)), (dtype, name)
    # a layout the fused kernels cannot take falls back to the composed path on the GPU
    odd = [torch.randn(1, 40, 7, device="cuda") for _ in range(5)]
    assert torch.allclose(gated_scan(*odd), _composed(*odd, torch.float32, torch.float32), rtol=1e-4, atol=1e-5)


def test_gated_scan_fp32_against_float64_autograd():
    """fp32 gates (no rounding, accurate sigmoid): forward and the five gradients against float64
    autograd through the sequential loop on the CPU."""
    from quick_ssm_b200 import scan
    from quick_ssm_b200.gated import gated_scan
    from tolerances import assert_close_f32
    torch.manual_seed(3)
    pre = [torch.randn(2, 150, 72) for _ in range(5)]
    dy = torch.randn(2, 150, 72)
    ref_leaves = [t.double().requires_grad_() for t in pre]
    pa, px, pc1, pc2, pd = ref_leaves
    y_ref = scan(px, torch.sigmoid(pa), torch.sigmoid(pd), torch.nn.functional.silu(pc1) * pc2, backend="torch")
    y_ref.backward(dy.double())
    leaves = [t.cuda().requires_grad_() for t in pre]
    y = gated_scan(*leaves, gate_dtype=torch.float32, out_dtype=torch.float32)
    y.backward(dy.cuda())
    _lib.check_device_status(synchronize=True)
    assert_close_f32(y, y_ref.detach(), "y")
    for name, got, ref in zip(("dpa", "dpx", "dpc1", "dpc2", "dpd"), leaves, ref_leaves):
        assert_close_f32(got.grad, ref.grad, name)
