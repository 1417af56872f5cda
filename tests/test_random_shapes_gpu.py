"""Seeded random shapes through the C-ABI with the kernels the library picks by itself
(SSB_VARIANT_AUTO / SSB_CL_VARIANT_AUTO), with and without the caller's scratch and -- rows layout
-- with and without carries entering both scans, against the CPU oracle.

test_fuzz_gpu.py walks the same dispatch rules through the Python operators, which never pass
carries and always allocate scratch; here the entry points get what a C caller may give them: a
state entering the forward, a gradient and a previous h entering the backward, scratch or none.
Lengths are drawn on and just off the boundaries the rules test for (multiples of 4, 32, 512,
4096; one more, one less).  Sizes stay near 2 M elements per tensor so that the oracle takes
milliseconds per case."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _gpu  # noqa: E402
from _gpu import AUTO  # noqa: E402

import oracle  # noqa: E402
from scanscam_b200 import _native  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-4
MAX_ELEMS = 1 << 21
GATES = ("sigmoid2", "sigmoid0", "nearunit", "resets", "randn")


def _log_uniform(rng, lo, hi):
    return int(round(float(np.exp(rng.uniform(np.log(lo), np.log(hi))))))


def _near_boundary(rng, x):
    """x, or the nearest multiple of a boundary the dispatch rules test for, give or take one."""
    kind = rng.integers(0, 4)
    if kind == 0:
        return x
    step = int(rng.choice([4, 32, 512, 4096]))
    base = max(step, (x + step // 2) // step * step)
    return int(max(1, base + int(rng.integers(-1, 2)) * (kind == 3)))


def rows_cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < n:
        T = _near_boundary(rng, _log_uniform(rng, 1, 150000))
        rows = _log_uniform(rng, 1, 6000)
        rows = int(max(1, min(rows, MAX_ELEMS // T)))
        out.append((rows, T, str(rng.choice(GATES)), bool(rng.integers(0, 2)), bool(rng.integers(0, 2)), len(out)))
    return out


def cl_cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < n:
        C = int(rng.choice([1, 3, 4, 8, 12, 16, 20, 32, 48, 64, 96, 128, 200, 256, 512]))
        T = _near_boundary(rng, _log_uniform(rng, 1, 20000))
        N = int(max(1, min(_log_uniform(rng, 1, 64), MAX_ELEMS // (T * C))))
        if N * T * C > MAX_ELEMS:
            continue
        out.append((N, T, C, str(rng.choice(GATES[:4])), bool(rng.integers(0, 2)), len(out)))
    return out


@pytest.mark.parametrize("rows,T,gates,carries,scratch,case", rows_cases(120, seed=20240531))
def test_rows_layout_auto(rows, T, gates, carries, scratch, case):
    a, b, g = make_inputs(gates, (rows, T), seed=1000 + case)
    gen = torch.Generator().manual_seed(case)
    h_in = torch.randn(rows, generator=gen) if carries else None
    gb_in = torch.randn(rows, generator=gen) if carries else None
    np_or_none = lambda x: None if x is None else x.numpy()  # noqa: E731
    h_ref = oracle.scan_forward(a.numpy(), b.numpy(), np_or_none(h_in))
    ga_ref, gb_ref = oracle.scan_backward(a.numpy(), h_ref, g.numpy(), np_or_none(gb_in), np_or_none(h_in))
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    d_h_in = None if h_in is None else h_in.cuda()
    d_c_in = None if gb_in is None else gb_in.cuda()
    lib = _native.load()
    ws = (None, 0)
    if scratch:  # what a caller that can allocate would pass: the larger of the two directions' requests
        need = max(lib.ssb_scan_workspace_bytes(rows, T, lib.ssb_scan_recommend(rows, T, d, 1, 1)) for d in (0, 1))
        ws = (torch.empty(max(need, 1), dtype=torch.uint8, device="cuda"), need) if need else (None, 0)
    h = _gpu.fwd(da, db, h_in=d_h_in, variant=AUTO, workspace=ws)
    assert _gpu.max_norm_err(h, h_ref) < TOL, (rows, T, gates)
    ga, gb = _gpu.bwd(da, torch.from_numpy(h_ref).cuda(), dg, c_in=d_c_in, h_prev=d_h_in, variant=AUTO, workspace=ws)
    assert _gpu.max_norm_err(gb, gb_ref) < TOL, (rows, T, gates)
    assert _gpu.max_norm_err(ga, ga_ref) < TOL, (rows, T, gates)
    _gpu.device_ok()


@pytest.mark.parametrize("N,T,C,gates,scratch,case", cl_cases(60, seed=977))
def test_channels_last_auto(N, T, C, gates, scratch, case):
    a, b, g = make_inputs(gates, (N, T, C), seed=2000 + case)
    h_ref = oracle.scan_forward_channels_last(a.numpy(), b.numpy())
    ga_ref, gb_ref = oracle.scan_backward_channels_last(a.numpy(), h_ref, g.numpy())
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    dh = torch.from_numpy(h_ref).cuda()
    lib = _native.load()
    st = _native.stream_of(da)
    h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
    if scratch:
        need = lib.ssb_scan_cl_workspace_bytes(N, T, C)  # the bound over every family
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
        _native.check(lib.ssb_scan_cl_fwd_f32_ex(da.data_ptr(), db.data_ptr(), h.data_ptr(), N, T, C, _native.CL_AUTO,
                                                 ws.data_ptr(), need, st))
        _native.check(lib.ssb_scan_cl_bwd_f32_ex(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                 N, T, C, _native.CL_AUTO, ws.data_ptr(), need, st))
    else:
        _native.check(lib.ssb_scan_cl_fwd_f32(da.data_ptr(), db.data_ptr(), h.data_ptr(), N, T, C, st))
        _native.check(lib.ssb_scan_cl_bwd_f32(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                              N, T, C, st))
    assert _gpu.max_norm_err(h, h_ref) < TOL, (N, T, C, gates)
    assert _gpu.max_norm_err(gb, gb_ref) < TOL, (N, T, C, gates)
    assert _gpu.max_norm_err(ga, ga_ref) < TOL, (N, T, C, gates)
    _gpu.device_ok()
