"""The entry point for callers that cannot allocate device memory (ssb_scan_fwd_f32_static).

Some users of the library have no allocator to take scratch from at call time -- a serving
process that carved up the whole GPU at start-up, or a foreign-language binding without a CUDA
memory API -- so the library carries a fixed scratch area of its own for them.  These checks
go through the C-ABI like any such caller would: raw device pointers, no workspace argument.

Collected last on purpose (file name): if it fails under `pytest -x`, every other test has
already run.  It makes no assumption about what ran before it in the process; the built-in
scratch may hold records from earlier launches, which is exactly the situation it must handle.
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _gpu  # noqa: E402

import oracle  # noqa: E402
from scanscam_b200 import _native  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-4  # max-norm relative error, the bound the parity tests use


def static_forward(a, b, h_in=None):
    lib = _native.load()
    out = torch.empty_like(a)
    rows, T = a.shape
    _native.check(lib.ssb_scan_fwd_f32_static(a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, T,
                                              _native.ptr(h_in), _native.stream_of(a)))
    return out


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    """Same kernel, scratch from the library instead of from the caller; the second call is a
    different, larger problem, so it meets the first call's leftovers in the shared scratch.
    Each result is compared with the existing entry point (caller's workspace) and, because that is
    the same kernel, also with the CPU oracle started from the same carries."""
    for seed, (rows, T), gates in ((1, (24, 40960), "nearunit"), (2, (300, 8200), "resets")):
        a, b, _ = make_inputs(gates, (rows, T), seed=seed)
        carry = torch.randn(rows, generator=torch.Generator().manual_seed(seed))
        da, db, dc = a.cuda(), b.cuda(), carry.cuda()
        expected = _gpu.fwd(da, db, h_in=dc, variant=_gpu.LOOKBACK)   # existing entry point, caller's workspace
        got = static_forward(da, db, dc)
        _gpu.device_ok()
        err = float((got - expected).abs().max() / expected.abs().max())
        assert err < TOL, (rows, T, err)
        assert torch.allclose(got, expected, atol=1e-4, rtol=1e-5)
        h_ref = oracle.scan_forward(a.numpy(), b.numpy(), h_in=carry.numpy())
        assert _gpu.max_norm_err(got, h_ref) < TOL and _gpu.allclose_ref(got, h_ref)


def test_without_a_carry_and_without_touching_the_allocator():
    """h_in = NULL is the reference's case (the scan starts from zero).  And the property the entry
    point exists for: between the moment the tensors exist and the moment the result is complete,
    the amount of free device memory does not change -- nothing was allocated, by the runtime or
    by any library (the first call on the device has already looked up the scratch address)."""
    rows, T = 40, 24576
    a, b, _ = make_inputs("sigmoid2", (rows, T), seed=3)
    da, db = a.cuda(), b.cuda()
    h_ref = oracle.scan_forward(a.numpy(), b.numpy())
    assert _gpu.max_norm_err(static_forward(da, db), h_ref) < TOL      # first call on this device, at the latest
    lib = _native.load()
    out = torch.empty_like(da)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    _native.check(lib.ssb_scan_fwd_f32_static(da.data_ptr(), db.data_ptr(), out.data_ptr(), rows, T, None,
                                              _native.stream_of(da)))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert _gpu.max_norm_err(out, h_ref) < TOL and _gpu.allclose_ref(out, h_ref)
    _gpu.device_ok()


def test_problems_beyond_the_built_in_scratch_are_refused():
    lib = _native.load()
    rows, T = 33000, 4100                       # 2 spans per row -> 66 000 spans > 65 536
    assert lib.ssb_scan_workspace_bytes(rows, T, _gpu.LOOKBACK) > 256 + 16 * 65536
    a = torch.empty(rows, T, device="cuda")     # never read: the call must refuse before launching
    out = torch.empty_like(a)
    rc = lib.ssb_scan_fwd_f32_static(a.data_ptr(), a.data_ptr(), out.data_ptr(), rows, T, None, _native.stream_of(a))
    assert rc == _native.ERR_WORKSPACE
    msg = lib.ssb_last_error().decode()
    assert "built-in scratch" in msg and "65536" in msg
    # shapes that need no scratch are pointed to the ordinary entry point
    short = torch.rand(8, 1024, device="cuda")
    rc = lib.ssb_scan_fwd_f32_static(short.data_ptr(), short.data_ptr(), out.data_ptr(), 8, 1024, None,
                                     _native.stream_of(short))
    assert rc == _native.ERR_UNSUPPORTED
    assert lib.ssb_scan_fwd_f32_static(None, None, None, 0, 8192, None, None) == _native.OK   # empty problem
    _gpu.device_ok()
