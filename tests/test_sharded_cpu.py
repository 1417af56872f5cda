"""Sequence-parallel host logic on CPU: gloo process groups of 2 and 3 ranks, with the local
kernels replaced by oracle-backed stand-ins (tests/_oracle_ops.py)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _oracle_ops import OracleShardOps  # noqa: E402

from scanscam_b200 import sharded  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, gates, rows, steps, out_dir, cut=sharded.DEFAULT_CUT):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, b, g = make_inputs(gates, (rows, steps), seed=3)
        lo, hi = rank * steps // world, (rank + 1) * steps // world
        a_l = a[:, lo:hi].contiguous().requires_grad_(True)
        b_l = b[:, lo:hi].contiguous().requires_grad_(True)
        h_l = sharded.scan_sequence_parallel(a_l, b_l, None, OracleShardOps, cut)
        h_l.backward(g[:, lo:hi].contiguous())
        torch.save({"h": h_l.detach(), "ga": a_l.grad, "gb": b_l.grad}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,gates,steps,cut", [(2, "sigmoid2", 96, sharded.DEFAULT_CUT), (3, "randn", 96, 0.0),
                                                   (2, "resets", 96, 0.0), (2, "ones", 96, sharded.DEFAULT_CUT),
                                                   (2, "sigmoid2", 1200, sharded.DEFAULT_CUT), (3, "randn", 300, sharded.DEFAULT_CUT)])
def test_sequence_parallel_scan_on_gloo(tmp_path, world, gates, steps, cut):
    """Gates whose products vanish inside a shard (sigmoid2 over 600 steps, randn), gates whose
    products never do (ones), exact zeros (resets); with the default cut and with cut = 0."""
    rows = 6
    mp.spawn(_worker, args=(world, _free_port(), gates, rows, steps, str(tmp_path), cut), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    h = torch.cat([p["h"] for p in parts], dim=1).numpy()
    ga = torch.cat([p["ga"] for p in parts], dim=1).numpy()
    gb = torch.cat([p["gb"] for p in parts], dim=1).numpy()
    a, b, g = (x.numpy() for x in make_inputs(gates, (rows, steps), seed=3))
    h_ref = oracle.scan_forward(a, b)
    ga_ref, gb_ref = oracle.scan_backward(a, h_ref, g)
    scale = lambda x: np.abs(x).max() + 1e-30  # noqa: E731
    assert np.abs(h - h_ref).max() / scale(h_ref) < 1e-5
    assert np.abs(gb - gb_ref).max() / scale(gb_ref) < 1e-5
    assert np.abs(ga - ga_ref).max() / scale(ga_ref) < 1e-5


def test_single_process_is_the_plain_scan():
    a, b, g = make_inputs("sigmoid0", (4, 50), seed=1)
    h, h_in = sharded.sharded_scan_forward(a, b, None, OracleShardOps)
    assert torch.equal(h_in, torch.zeros(4))
    assert np.array_equal(h.numpy(), oracle.scan_forward(a.numpy(), b.numpy()))
    ga, gb = sharded.sharded_scan_backward(a, h, g, h_in, None, OracleShardOps)
    ga_ref, gb_ref = oracle.scan_backward(a.numpy(), h.numpy(), g.numpy())
    assert np.array_equal(gb.numpy(), gb_ref) and np.array_equal(ga.numpy(), ga_ref)


@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_virtual_shards_compose_to_the_unsharded_result(n_shards):
    """The carry algebra alone, no process group: G shards on one host."""
    a, b, g = make_inputs("nearunit", (3, 64 * n_shards), seed=2)
    step = a.shape[1] // n_shards
    sl = [slice(s * step, (s + 1) * step) for s in range(n_shards)]
    fwd_maps = torch.stack([OracleShardOps.reduce_forward(a[:, s].contiguous(), b[:, s].contiguous()) for s in sl])
    bwd_maps = torch.stack([OracleShardOps.reduce_backward(a[:, s].contiguous(), g[:, s].contiguous()) for s in sl])
    h_ref = oracle.scan_forward(a.numpy(), b.numpy())
    ga_ref, gb_ref = oracle.scan_backward(a.numpy(), h_ref, g.numpy())
    for s in range(n_shards):
        h_in = OracleShardOps.carry(fwd_maps, s, False)
        h = OracleShardOps.scan_forward(a[:, sl[s]].contiguous(), b[:, sl[s]].contiguous(), h_in)
        np.testing.assert_allclose(h.numpy(), h_ref[:, sl[s]], rtol=2e-6, atol=1e-6)
        c_in = OracleShardOps.carry(bwd_maps, s, True)
        ga, gb = OracleShardOps.scan_backward(a[:, sl[s]].contiguous(), torch.from_numpy(h_ref[:, sl[s]].copy()),
                                              g[:, sl[s]].contiguous(), c_in, h_in)
        np.testing.assert_allclose(gb.numpy(), gb_ref[:, sl[s]], rtol=2e-6, atol=1e-5)
        np.testing.assert_allclose(ga.numpy(), ga_ref[:, sl[s]], rtol=2e-5, atol=1e-4)


@pytest.mark.parametrize("gates", ["sigmoid2", "nearunit", "randn", "ones", "resets"])
def test_early_terminated_maps_stay_within_the_cut(gates):
    """map_* with cut = 0 equals the full fold; with cut > 0 it stops early on vanishing products and
    differs from the full fold by at most cut x (largest state), and it reads fewer elements."""
    rows, steps = 5, 3000
    a, b, g = make_inputs(gates, (rows, steps), seed=7)
    full_f, full_b = OracleShardOps.reduce_forward(a, b).numpy(), OracleShardOps.reduce_backward(a, g).numpy()
    for cut in (0.0, 2.0 ** -40, 1e-3):
        wf, wb = np.zeros(1, np.int64), np.zeros(1, np.int64)
        mf = OracleShardOps.map_forward(a, b, cut, wf).numpy()
        mb = OracleShardOps.map_backward(a, g, cut, wb).numpy()
        h = oracle.scan_forward(a.numpy(), b.numpy())
        scale_h = np.abs(h).max()
        ga, gb = oracle.scan_backward(a.numpy(), h, g.numpy())
        scale_c = max(np.abs(gb).max(), 1.0) * max(np.abs(a.numpy()).max(), 1.0)
        finite = np.isfinite(full_f).all(axis=1) & np.isfinite(full_b).all(axis=1)  # randn gates can overflow
        tol = 2 * cut + 2e-6  # the cut's bound plus fp32 reassociation
        assert (np.abs(mf[finite, 1] - full_f[finite, 1]) <= tol * scale_h + 1e-6 * np.abs(full_f[finite, 1])).all()
        assert (np.abs(mb[finite, 1] - full_b[finite, 1]) <= tol * scale_c + 1e-6 * np.abs(full_b[finite, 1])).all()
        assert (np.abs(mf[finite, 0]) <= np.maximum(np.abs(full_f[finite, 0]) * 1.001, cut)).all()
        if gates in ("sigmoid2", "resets") and cut > 0:
            assert wf[0] < rows * steps // 4 and wb[0] < rows * steps // 4  # products vanish within a few hundred steps
        if gates == "ones":
            assert wf[0] == rows * steps and wb[0] == rows * steps  # never vanishes: the whole shard is walked
