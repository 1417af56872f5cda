"""Seeded random shapes through the default kernel choice of every public entry point, against
the CPU oracle.  The shapes are drawn around the thresholds of the dispatch policies (row
lengths 32 * 2^k and their neighbours, 4096-step chunk multiples, channel-block counts near the
streaming / chunked / look-back switch points) so that every policy branch is exercised with
ragged sizes as well as round ones."""
import os
import random
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _gpu  # noqa: E402

import oracle  # noqa: E402
import scanscam_b200  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-4


def row_shapes(rng, count):
    shapes = []
    for _ in range(count):
        kind = rng.randrange(6)
        if kind == 0:    # power-of-two rows (TMA flat sweep) and their neighbours
            T = (32 << rng.randrange(8)) + rng.choice([0, 0, 0, -1, 1, 4, -4])
            rows = rng.randrange(1, 700)
        elif kind == 1:  # multiples of 4 that are not powers of two
            T = 4 * rng.randrange(1, 2500)
            rows = rng.randrange(1, 300)
        elif kind == 2:  # odd lengths
            T = rng.randrange(1, 9000)
            rows = rng.randrange(1, 200)
        elif kind == 3:  # a few long rows of whole 4096-step chunks (two-pass chunked form)
            T = 4096 * rng.randrange(16, 40)
            rows = rng.randrange(1, 12)
        elif kind == 4:  # long rows, any length (look-back)
            T = rng.randrange(5000, 120000)
            rows = rng.randrange(1, 24)
        else:            # many short rows
            T = rng.randrange(1, 64)
            rows = rng.randrange(1000, 20000)
        shapes.append((rows, max(T, 1)))
    return shapes


def cl_shapes(rng, count):
    shapes = []
    for _ in range(count):
        kind = rng.randrange(4)
        if kind == 0:    # enough channel blocks for the streaming kernels
            N, C, T = rng.randrange(1, 9), 4 * rng.randrange(100, 400), rng.randrange(100, 700)
        elif kind == 1:  # few channel blocks, long (chunked / look-back)
            N, C, T = rng.randrange(1, 3), 4 * rng.randrange(2, 60), rng.randrange(2048, 20000)
        elif kind == 2:  # odd channel counts (plain / look-back kernels)
            N, C, T = rng.randrange(1, 5), rng.randrange(1, 300), rng.randrange(1, 3000)
        else:            # short sequences
            N, C, T = rng.randrange(1, 40), 8 * rng.randrange(1, 80), rng.randrange(1, 140)
        shapes.append((N, T, C))
    return shapes


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_rows_layout_random_shapes(seed):
    rng = random.Random(seed)
    for rows, T in row_shapes(rng, 14):
        gates = rng.choice(["sigmoid2", "sigmoid0", "resets", "nearunit"])
        a, b, g = make_inputs(gates, (rows, T), seed=seed)
        h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
        da, db = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
        h = scanscam_b200.scan(da, db)                      # through the extension: scratch provided
        h.backward(g.cuda())
        h2 = _gpu.fwd(a.cuda(), b.cuda())                   # plain C-ABI entry points: no scratch
        ga2, gb2 = _gpu.bwd(a.cuda(), torch.from_numpy(h_ref).cuda(), g.cuda())
        for x, ref, name in ((h, h_ref, "h"), (da.grad, ga_ref, "ga"), (db.grad, gb_ref, "gb"), (h2, h_ref, "h2"),
                             (ga2, ga_ref, "ga2"), (gb2, gb_ref, "gb2")):
            err = _gpu.max_norm_err(x, ref)
            assert err < TOL, ((rows, T), gates, name, err)
    _gpu.device_ok()


@pytest.mark.parametrize("seed", [4, 5])
def test_channels_last_random_shapes(seed):
    rng = random.Random(seed)
    for shape in cl_shapes(rng, 12):
        gates = rng.choice(["sigmoid2", "sigmoid0", "resets"])
        a, b, g = make_inputs(gates, shape, seed=seed)
        h_ref = oracle.scan_forward_channels_last(a.numpy(), b.numpy())
        ga_ref, gb_ref = oracle.scan_backward_channels_last(a.numpy(), h_ref, g.numpy())
        if shape[0] * shape[1] * shape[2] > 1 and (shape[1] > 1 and shape[2] > 1):
            da, db = a.cuda().mT.requires_grad_(True), b.cuda().mT.requires_grad_(True)
            h = scanscam_b200.scan(da, db)                  # operator: channels-last branch, scratch provided
            h.backward(g.cuda().mT)
            outs = [(h.mT, h_ref, "h"), (da.grad.mT, ga_ref, "ga"), (db.grad.mT, gb_ref, "gb")]
        else:
            outs = []
        h2 = _gpu.cl_fwd(a.cuda(), b.cuda())                # plain entry points: no scratch
        ga2, gb2 = _gpu.cl_bwd(a.cuda(), torch.from_numpy(h_ref).cuda(), g.cuda())
        outs += [(h2, h_ref, "h2"), (ga2, ga_ref, "ga2"), (gb2, gb_ref, "gb2")]
        for x, ref, name in outs:
            err = _gpu.max_norm_err(x.detach().contiguous(), ref)
            assert err < TOL, (shape, gates, name, err)
    _gpu.device_ok()


@pytest.mark.parametrize("seed", [6])
def test_16bit_random_shapes(seed):
    rng = random.Random(seed)
    for dtype, half_ulp in ((torch.bfloat16, 2.0 ** -8), (torch.float16, 2.0 ** -11)):
        for rows, T in row_shapes(rng, 8):
            a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", (rows, T), seed=seed))
            h_ref = oracle.scan_forward(a.float().numpy(), b.float().numpy())
            da, db = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
            h = scanscam_b200.scan(da, db)
            h.backward(g.cuda())
            ga_ref, gb_ref = oracle.scan_backward(a.float().numpy(), h.detach().float().cpu().numpy(), g.float().numpy())
            for x, ref, name in ((h, h_ref, "h"), (da.grad, ga_ref, "ga"), (db.grad, gb_ref, "gb")):
                err = _gpu.max_norm_err(x.detach().float(), ref)
                assert err < 1.01 * half_ulp, ((rows, T), dtype, name, err)
        for N, T, C in cl_shapes(rng, 8):
            C = max(8, C // 8 * 8)
            if T < 2:
                continue
            a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", (N, T, C), seed=seed))
            h_ref = oracle.scan_forward_channels_last(a.float().numpy(), b.float().numpy())
            da, db = a.cuda().mT.requires_grad_(True), b.cuda().mT.requires_grad_(True)
            h = scanscam_b200.scan(da, db)
            h.backward(g.cuda().mT)
            ga_ref, gb_ref = oracle.scan_backward_channels_last(a.float().numpy(), h.detach().mT.float().cpu().numpy(),
                                                                g.float().numpy())
            for x, ref, name in ((h.mT, h_ref, "h"), (da.grad.mT, ga_ref, "ga"), (db.grad.mT, gb_ref, "gb")):
                err = _gpu.max_norm_err(x.detach().float().contiguous(), ref)
                assert err < 1.01 * half_ulp, ((N, T, C), dtype, name, err)
    _gpu.device_ok()
