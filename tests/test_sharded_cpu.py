"""Sequence sharding across ranks, run as two gloo processes on CPU.  The device operations are
replaced by the CPU oracle (injected through the private ``_ops`` hook), so what is tested is
the host logic: who sends which aggregate, the rank-ordered fold, the autograd wiring."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scan_oracle as so
from quick_ssm_b200.sharded import channel_shard, scan_sequence_sharded
from quick_ssm_b200.synth import make_inputs


class OracleShardOps:
    """CPU stand-in for CudaShardOps, float32 tensors only."""

    def aggregate_fwd(self, x, a, b, A_out, H_out):
        ones = np.ones((x.shape[0], x.shape[2]), dtype=np.float64)
        _, _, H = so.scan_forward(x, a, b)
        _, _, A = so.scan_forward(torch.zeros_like(x), a, torch.zeros_like(x), h_in=ones)
        A_out.copy_(torch.from_numpy(A))
        H_out.copy_(torch.from_numpy(H))

    def aggregate_bwd(self, a, c, dy, P_out, Q_out):
        z = torch.zeros_like(a)
        Q = so.scan_backward(z, a, z, c, dy)[4]
        P_out.copy_(a.double().prod(dim=1))
        Q_out.copy_(torch.from_numpy(Q))

    def fold(self, A, H, upto, reverse):
        run = torch.zeros_like(A[0])
        ks = range(A.shape[0] - 1, upto, -1) if reverse else range(0, upto)
        for k in ks:
            run = A[k] * run + H[k]
        return run

    def forward(self, x, a, b, c, y, tile_h, h_in):
        _, yy, _ = so.scan_forward(x, a, b, c, h_in=h_in)
        y.copy_(torch.from_numpy(yy))
        if tile_h is not None:
            h, _, _ = so.scan_forward(x, a, b, h_in=h_in)
            prev = np.concatenate([h_in.numpy()[:, None].astype(np.float64), h[:, :-1]], axis=1)
            tile_h.copy_(torch.from_numpy(prev[:, ::16]))

    def backward(self, x, a, b, c, dy, tile_h, g_in, grads):
        h_in = tile_h[:, 0]
        out = so.scan_backward(x, a, b, c, dy, h_in=h_in, g_in=g_in)
        for dst, src in zip(grads, out[:4]):
            dst.copy_(torch.from_numpy(src))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = make_inputs(2, 96, 6, dtype=torch.float32, seed=3)
        per = 96 // world
        sl = slice(rank * per, (rank + 1) * per)
        x, a, b, c = (t[:, sl].clone().requires_grad_() for t in inp.tensors())
        y = scan_sequence_sharded(x, a, b, c, _ops=OracleShardOps())
        (y * inp.dy[:, sl]).sum().backward()
        torch.save(dict(y=y.detach(), dx=x.grad, da=a.grad, db=b.grad, dc=c.grad),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3, 4])
def test_sequence_shards_reproduce_the_whole_scan(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    inp = make_inputs(2, 96, 6, dtype=torch.float32, seed=3)
    _, y_ref, _ = so.scan_forward(inp.x, inp.a, inp.b, inp.c)
    g_ref = so.scan_backward(inp.x, inp.a, inp.b, inp.c, inp.dy)
    got = {k: torch.cat([p[k] for p in parts], dim=1).numpy() for k in parts[0]}
    assert np.allclose(got["y"], y_ref, rtol=1e-4, atol=1e-5)
    for k, ref in zip(("dx", "da", "db", "dc"), g_ref):
        assert np.allclose(got[k], ref, rtol=1e-4, atol=1e-5), k


def test_channel_shards_cover_all_channels():
    t = torch.arange(2 * 3 * 10).reshape(2, 3, 10)
    parts = [channel_shard(t, r, 4) for r in range(4)]
    assert torch.equal(torch.cat(parts, dim=2), t)
    assert parts[0].data_ptr() == t.data_ptr()
