"""Carry exchange through peer memory (``qssm_carry_push`` / ``qssm_carry_wait_fold``).

* the slot / epoch protocol, modelled on the CPU with randomised interleavings of the ranks' kernels;
* the two kernels on ONE GPU, with every "rank's" inbox in local memory (the pointer table holds local
  addresses), against ``qssm_carry_fold`` on the same pairs;
* the bounded wait: a flag that nothing sets expires, is reported, and the context stays usable;
* on two or more GPUs, ranks as processes with inboxes in torch's symmetric memory: the sharded scan
  with the peer exchange is bit-identical to the one with the NCCL all-gather.
"""
import os
import random
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from quick_ssm_b200 import _lib
from quick_ssm_b200.synth import make_inputs


# ---------------------------------------------------------------------------------------------
# protocol model (no GPU)
# ---------------------------------------------------------------------------------------------
class _ModelRank:
    """One rank of the model: a stream of kernels [push(e), fold(e)] for e = 1, 2, ...; a push writes
    (value, flag) into slot e & 1 of every inbox, a fold may run only when all flags of its slot show
    its epoch and then reads every entry of that slot."""

    def __init__(self, rank, world, calls):
        self.rank, self.world = rank, world
        self.queue = [(kind, e) for e in range(1, calls + 1) for kind in ("push", "fold")]
        self.inbox = {(slot, k): (0, None) for slot in (0, 1) for k in range(world)}  # (flag, payload)
        self.seen = []

    def runnable(self):
        if not self.queue:
            return False
        kind, e = self.queue[0]
        if kind == "push":
            return True
        return all(self.inbox[(e & 1, k)][0] == e for k in range(self.world))


@pytest.mark.parametrize("world,wait_all", [(2, True), (4, True), (8, True), (3, False)])
def test_slot_epoch_protocol_never_overwrites_unread_data(world, wait_all):
    """With folds that wait for EVERY rank's flag, no interleaving lets a push overwrite a pair that a
    slower rank has not folded yet.  (With folds that wait only for the ranks they depend on, the
    first rank of a forward-only loop runs ahead and does overwrite: the model shows that too.)"""
    rng = random.Random(1234 + world)
    overwritten = False
    for trial in range(200):
        calls = 6
        ranks = [_ModelRank(r, world, calls) for r in range(world)]
        unread = {}  # (dst, slot, src) -> epoch written and not yet folded by dst
        while any(r.queue for r in ranks):
            ready = []
            for r in ranks:
                if not r.queue:
                    continue
                kind, e = r.queue[0]
                if kind == "push":
                    ready.append(r)
                elif wait_all and r.runnable():
                    ready.append(r)
                elif not wait_all and all(r.inbox[(e & 1, k)][0] == e for k in range(r.rank)):
                    ready.append(r)
            if not ready and not wait_all:
                overwritten = True  # a flag was overwritten by a later call: the waiter would time out
                break
            assert ready, "deadlock in the model"
            r = rng.choice(ready)
            kind, e = r.queue.pop(0)
            if kind == "push":
                for dst in ranks:
                    key = (dst.rank, e & 1, r.rank)
                    if key in unread:
                        overwritten = True
                    unread[key] = e
                    dst.inbox[(e & 1, r.rank)] = (e, (r.rank, e))
            else:
                need = range(world) if wait_all else range(r.rank)
                for k in need:
                    flag, payload = r.inbox[(e & 1, k)]
                    if wait_all:
                        assert payload == (k, e), "a fold read a pair of another call"
                    elif payload != (k, e):
                        overwritten = True
                for k in range(world):
                    if unread.get((r.rank, e & 1, k)) == e:
                        del unread[(r.rank, e & 1, k)]
                r.seen.append(e)
        if wait_all:
            assert not overwritten
    if not wait_all:
        assert overwritten, "the weaker protocol is expected to show the hazard"


# ---------------------------------------------------------------------------------------------
# the kernels on one GPU
# ---------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("world,n_chan", [(2, 192), (4, 2048), (8, 70)])
def test_push_and_fold_on_one_device_match_carry_fold(world, n_chan):
    dev = torch.device("cuda")
    nbytes = _lib.peer_inbox_bytes(world, n_chan)
    inboxes = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [t.data_ptr() for t in inboxes]
    counters = torch.zeros(32, dtype=torch.int32, device=dev)
    torch.manual_seed(world)
    for epoch in (1, 2, 3):            # every slot is used and reused
        for reverse in (False, True):
            slot = 2 * int(reverse) + (epoch & 1)
            pairs = torch.rand(world, 2, n_chan, device=dev) * 0.3 + 0.8
            for r in range(world):     # every "rank" pushes into every inbox
                _lib.carry_push(pairs[r, 0], pairs[r, 1], ptrs, counters, r, slot, epoch)
            for r in range(world):
                got = torch.empty(n_chan, device=dev)
                _lib.carry_wait_fold(ptrs[r], n_chan, r, world, slot, epoch, reverse, got, wait_ms=500)
                want = _lib.carry_fold(pairs[:, 0], pairs[:, 1], r, reverse=reverse)
                _lib.check_device_status(synchronize=True)
                assert torch.equal(got, want), (epoch, reverse, r)


@gpu
def test_a_pair_that_never_arrives_is_reported_and_the_context_survives():
    dev = torch.device("cuda")
    world, n_chan = 2, 256
    inboxes = [torch.zeros(_lib.peer_inbox_bytes(world, n_chan), dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [t.data_ptr() for t in inboxes]
    counters = torch.zeros(32, dtype=torch.int32, device=dev)
    pair = torch.ones(2, n_chan, device=dev)
    carry = torch.full((n_chan,), -7.0, device=dev)
    _lib.carry_push(pair[0], pair[1], ptrs, counters, 1, 1, 1)        # rank 1 pushes; "rank 0" never does
    _lib.carry_wait_fold(ptrs[1], n_chan, 1, world, 1, 1, False, carry, wait_ms=100)
    with pytest.raises(RuntimeError, match="expired"):
        _lib.check_device_status(synchronize=True)
    assert bool((carry == -7.0).all()), "an expired wait must leave the output alone"
    _lib.carry_push(pair[0], pair[1], ptrs, counters, 0, 1, 1)        # now it arrives
    _lib.carry_wait_fold(ptrs[1], n_chan, 1, world, 1, 1, False, carry, wait_ms=100)
    _lib.check_device_status(synchronize=True)
    assert torch.equal(carry, torch.ones(n_chan, device=dev))         # fold of rank 0's pair (1, 1) onto 0


# ---------------------------------------------------------------------------------------------
# ranks as processes on two or more GPUs
# ---------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _peer_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from quick_ssm_b200.sharded import CudaShardOps, PeerCarryExchange, scan_sequence_sharded
        B, L, D = 2, 4096, 96
        peer_ops = CudaShardOps(peer=PeerCarryExchange(dist.group.WORLD, B * D, torch.device("cuda", rank)))
        per = L // world
        sl = slice(rank * per, (rank + 1) * per)
        same = True
        for seed in (3, 4, 5):  # three forward/backward rounds: every inbox slot is used and reused
            inp = make_inputs(B, L, D, dtype=torch.float32, seed=seed, decay="near_unit")
            res = []
            for ops in (None, peer_ops):
                x, a, b, c = (t[:, sl].cuda().requires_grad_() for t in inp.tensors())
                y = scan_sequence_sharded(x, a, b, c, _ops=ops)
                y.backward(inp.dy[:, sl].cuda())
                res.append([y.detach(), x.grad, a.grad, b.grad, c.grad])
            _lib.check_device_status(synchronize=True)
            same = same and all(torch.equal(u, v) for u, v in zip(*res))
        torch.save({"same": same}, os.path.join(out_dir, f"peer{rank}.pt"))
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_carry_exchange_equals_the_all_gather(tmp_path):
    """The carry exchange through peer memory (stores into the other ranks' inboxes, flags, bounded
    wait) gives bit-identical results to the all-gather + fold it replaces, over repeated calls."""
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert torch.load(os.path.join(tmp_path, f"peer{r}.pt"))["same"]
