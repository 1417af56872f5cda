"""Helpers for the GPU parity tests: call the C-ABI with torch device buffers, compare with the
CPU oracle."""
import os

import numpy as np
import torch

import oracle
from scanscam_b200 import _native

AUTO, WARP, TMA, FLAT = _native.VARIANT_AUTO, _native.VARIANT_WARP, _native.VARIANT_TMA, _native.VARIANT_FLAT
LOOKBACK = _native.VARIANT_LOOKBACK
FLAT_ANY = _native.VARIANT_FLAT_ANY


def lookback_variant(tuning):
    return LOOKBACK | (tuning << 8)


def workspace_for(rows, T, variant, device="cuda"):
    """(tensor or None, nbytes) of scratch the variant asks for."""
    need = _native.load().ssb_scan_workspace_bytes(rows, T, variant)
    if need == 0:
        return None, 0
    return torch.empty(need, dtype=torch.uint8, device=device), need


def tma_variant(tuning):
    return TMA | (tuning << 8)


def flat_variant(tuning):
    return FLAT | (tuning << 8)


def fwd(a, b, h_in=None, variant=AUTO, workspace=None):
    """a, b: CUDA [rows, T] contiguous float32/float64 -> h (through ssb_scan_fwd_*)."""
    lib = _native.load()
    out = torch.empty_like(a)
    rows, T = a.shape
    st = _native.stream_of(a)
    if a.dtype == torch.float32:
        ws, ws_bytes = workspace_for(rows, T, variant, a.device) if workspace is None else workspace
        rc = lib.ssb_scan_fwd_f32_ex(a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, T, _native.ptr(h_in),
                                     variant, _native.ptr(ws), ws_bytes, st)
    else:
        rc = lib.ssb_scan_fwd_f64(a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, T, _native.ptr(h_in), st)
    _native.check(rc)
    return out


def bwd(a, h, g, c_in=None, h_prev=None, variant=AUTO, workspace=None):
    lib = _native.load()
    ga, gb = torch.empty_like(a), torch.empty_like(a)
    rows, T = a.shape
    st = _native.stream_of(a)
    if a.dtype == torch.float32:
        ws, ws_bytes = workspace_for(rows, T, variant, a.device) if workspace is None else workspace
        rc = lib.ssb_scan_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T,
                                     _native.ptr(c_in), _native.ptr(h_prev), variant, _native.ptr(ws), ws_bytes, st)
    else:
        rc = lib.ssb_scan_bwd_f64(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T,
                                  _native.ptr(c_in), _native.ptr(h_prev), st)
    _native.check(rc)
    return ga, gb


def cl_variant(mode):
    """Test shorthand -> ssb_cl_variant_t value.  True: look-back, default tile.  "plain": the plain
    kernels.  Integers keep the numbering of the tuning tables: 2..31 look-back tile shapes,
    32..37 look-back on TMA-staged tiles, 64..71 streaming tile shapes, 96 the chunked form."""
    if mode is True:
        return _native.CL_LOOKBACK
    if mode == "plain":
        return _native.CL_PLAIN
    if mode == "narrow":
        return _native.CL_NARROW
    if isinstance(mode, int) and mode == 96:
        return _native.CL_CHUNKED
    if isinstance(mode, int) and mode >= 64:
        return _native.CL_STREAM | ((mode - 64) << 8)
    if isinstance(mode, int) and mode >= 32:
        return _native.CL_LOOKBACK_TMA | ((mode - 32) << 8)
    if isinstance(mode, int) and mode > 1:
        return _native.CL_LOOKBACK | (mode << 8)
    raise ValueError(mode)


def cl_workspace(a, variant=None, backward=False):
    """Scratch for a channels-last call: what the variant asks for, or the bound over all variants."""
    lib = _native.load()
    need = (lib.ssb_scan_cl_workspace_bytes(*a.shape) if variant is None
            else lib.ssb_scan_cl_variant_workspace_bytes(*a.shape, variant, int(backward)))
    return torch.empty(max(need, 1), dtype=torch.uint8, device=a.device), need


def cl_fwd(a, b, scratch=False):
    """scratch=False: the plain entry points (no scratch).  Otherwise a family pinned through the
    _ex entry point with the scratch that family asks for (float32 only); see cl_variant."""
    lib = _native.load()
    out = torch.empty_like(a)
    N, T, C = a.shape
    if scratch:
        variant = cl_variant(scratch)
        ws, need = cl_workspace(a, variant, False)
        _native.check(lib.ssb_scan_cl_fwd_f32_ex(a.data_ptr(), b.data_ptr(), out.data_ptr(), N, T, C, variant,
                                                 ws.data_ptr() if need else None, need, _native.stream_of(a)))
        return out
    fn = lib.ssb_scan_cl_fwd_f32 if a.dtype == torch.float32 else lib.ssb_scan_cl_fwd_f64
    _native.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), N, T, C, _native.stream_of(a)))
    return out


def cl_bwd(a, h, g, scratch=False):
    lib = _native.load()
    ga, gb = torch.empty_like(a), torch.empty_like(a)
    N, T, C = a.shape
    if scratch:
        variant = cl_variant(scratch)
        ws, need = cl_workspace(a, variant, True)
        _native.check(lib.ssb_scan_cl_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                 N, T, C, variant, ws.data_ptr() if need else None, need,
                                                 _native.stream_of(a)))
        return ga, gb
    fn = lib.ssb_scan_cl_bwd_f32 if a.dtype == torch.float32 else lib.ssb_scan_cl_bwd_f64
    _native.check(fn(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), N, T, C,
                     _native.stream_of(a)))
    return ga, gb


def device_ok():
    """Synchronises and asserts that no kernel reported a timed-out wait."""
    detail = _native.ctypes.c_int(0)
    _native.check(_native.load().ssb_device_status(_native.ctypes.byref(detail)))


def max_norm_err(x, ref):
    """max|x - ref| / max|ref| : the parity metric (elementwise relative error is meaningless
    near zero crossings, where the fp32 oracle itself is several percent from fp64)."""
    x = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x
    err = float(np.abs(x.astype(np.float64) - ref.astype(np.float64)).max() / (float(np.abs(ref).max()) + 1e-300))
    report = os.environ.get("SSB_PARITY_REPORT")  # opt-in: one line per comparison, for the error survey
    if report:
        with open(report, "a") as f:
            f.write(f"{os.environ.get('PYTEST_CURRENT_TEST', '?').split(' ')[0]}\t{err:.3e}\n")
    return err


def allclose_ref(x, ref, atol=1e-4, rtol=1e-5):
    """The reference tests' own criterion (scanscam/cuda_test.py:79-80: atol=1e-4, default rtol)."""
    x = x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x
    return bool(np.all(np.abs(x - ref) <= atol + rtol * np.abs(ref)))


def oracle_all(a, b, g):
    """CPU oracle on torch CPU tensors -> numpy (h, ga, gb); bwd is fed the oracle's own h."""
    an, bn, gn = a.numpy(), b.numpy(), g.numpy()
    h = oracle.scan_forward(an, bn)
    ga, gb = oracle.scan_backward(an, h, gn)
    return h, ga, gb
