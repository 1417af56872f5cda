"""Sequence-parallel scan over NCCL: each rank holds a T-slice on its own GPU; the assembled result
must match the unsharded CPU oracle.  Needs at least two GPUs (skipped otherwise)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import oracle  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, gates, rows, steps, out_dir, peer=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from scanscam_b200 import _native, sharded

        exchange = None
        if peer:  # the exchange through peer memory instead of the all-gather
            exchange = sharded.PeerCarryExchange.create(rows)
            assert exchange is not None, "peer memory exchange could not be set up on this box"
        a, b, g = make_inputs(gates, (rows, steps), seed=3)
        lo, hi = rank * steps // world, (rank + 1) * steps // world
        dist.barrier()  # the ranks start their first call together (the peers' waits are bounded at a second)
        for rep in range(3 if peer else 1):  # several calls in a row: both slot generations, slot reuse
            a_l = a[:, lo:hi].contiguous().cuda().requires_grad_(True)
            b_l = b[:, lo:hi].contiguous().cuda().requires_grad_(True)
            h_l = sharded.scan_sequence_parallel(a_l, b_l, exchange=exchange)
            h_l.backward(g[:, lo:hi].contiguous().cuda())
        torch.cuda.synchronize()
        detail = _native.ctypes.c_int(0)
        _native.check(_native.load().ssb_device_status(_native.ctypes.byref(detail)))  # no wait ran out
        torch.save({"h": h_l.detach().cpu(), "ga": a_l.grad.cpu(), "gb": b_l.grad.cpu()},
                   os.path.join(out_dir, f"r{rank}.pt"))
        if exchange is not None:
            dist.barrier()  # nobody unmaps while a peer may still be storing
            exchange.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("gates,rows,steps", [("nearunit", 64, 32768), ("sigmoid2", 33, 4096), ("resets", 16, 8200),
                                              ("nearunit", 40, 131072), ("randn", 16, 8192), ("ones", 8, 4096)])
def test_sequence_parallel_scan_on_nccl(tmp_path, gates, rows, steps):
    _run_and_check(tmp_path, gates, rows, steps, peer=False)


@pytest.mark.parametrize("gates,rows,steps", [("nearunit", 40, 131072), ("randn", 16, 8192), ("ones", 8, 4096)])
def test_sequence_parallel_scan_through_peer_memory(tmp_path, gates, rows, steps):
    """The same operator with the shard maps exchanged by peer stores and flags instead of NCCL
    (PeerCarryExchange): one process per GPU, every wait bounded, three calls in a row."""
    _run_and_check(tmp_path, gates, rows, steps, peer=True)


def _run_and_check(tmp_path, gates, rows, steps, peer):
    world = min(torch.cuda.device_count(), 8)  # every GPU of the box, up to eight
    if world < 2:
        pytest.skip("needs at least two GPUs")
    while steps % world:
        world -= 1
    mp.spawn(_worker, args=(world, _free_port(), gates, rows, steps, str(tmp_path), peer), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    h = torch.cat([p["h"] for p in parts], dim=1).numpy()
    ga = torch.cat([p["ga"] for p in parts], dim=1).numpy()
    gb = torch.cat([p["gb"] for p in parts], dim=1).numpy()
    a, b, g = (x.numpy() for x in make_inputs(gates, (rows, steps), seed=3))
    h_ref = oracle.scan_forward(a, b)
    ga_ref, gb_ref = oracle.scan_backward(a, h_ref, g)
    for got, ref in ((h, h_ref), (gb, gb_ref), (ga, ga_ref)):
        assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-4
