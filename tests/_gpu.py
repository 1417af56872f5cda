"""Helpers for the GPU parity tests: call the C-ABI with torch device buffers, compare with the
CPU oracle."""
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


def cl_workspace(a):
    need = _native.load().ssb_scan_cl_workspace_bytes(*a.shape)
    return torch.empty(max(need, 1), dtype=torch.uint8, device=a.device), need


def cl_fwd(a, b, scratch=False):
    """scratch=True: the look-back kernels (float32 only), with a workspace as a caller would pass."""
    lib = _native.load()
    out = torch.empty_like(a)
    N, T, C = a.shape
    if scratch == "plain":  # the plain kernels, whatever the library would pick
        lib.ssb_scan_cl_set_tuning(0x200)
        rc = lib.ssb_scan_cl_fwd_f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), N, T, C, _native.stream_of(a))
        lib.ssb_scan_cl_set_tuning(0)
        _native.check(rc)
        return out
    if scratch:
        ws, need = cl_workspace(a)
        lib.ssb_scan_cl_set_tuning(scratch if isinstance(scratch, int) and scratch > 1 else 1)  # always look-back
        _native.check(lib.ssb_scan_cl_fwd_f32_ex(a.data_ptr(), b.data_ptr(), out.data_ptr(), N, T, C, ws.data_ptr(),
                                                 need, _native.stream_of(a)))
        lib.ssb_scan_cl_set_tuning(0)
        return out
    fn = lib.ssb_scan_cl_fwd_f32 if a.dtype == torch.float32 else lib.ssb_scan_cl_fwd_f64
    _native.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), N, T, C, _native.stream_of(a)))
    return out


def cl_bwd(a, h, g, scratch=False):
    lib = _native.load()
    ga, gb = torch.empty_like(a), torch.empty_like(a)
    N, T, C = a.shape
    if scratch == "plain":
        lib.ssb_scan_cl_set_tuning(0x200)
        rc = lib.ssb_scan_cl_bwd_f32(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), N, T, C,
                                     _native.stream_of(a))
        lib.ssb_scan_cl_set_tuning(0)
        _native.check(rc)
        return ga, gb
    if scratch:
        ws, need = cl_workspace(a)
        lib.ssb_scan_cl_set_tuning(scratch if isinstance(scratch, int) and scratch > 1 else 1)
        _native.check(lib.ssb_scan_cl_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                 N, T, C, ws.data_ptr(), need, _native.stream_of(a)))
        lib.ssb_scan_cl_set_tuning(0)
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
    return float(np.abs(x.astype(np.float64) - ref.astype(np.float64)).max() / (float(np.abs(ref).max()) + 1e-300))


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
