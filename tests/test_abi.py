"""The C-ABI library: loads without a GPU, exports every declared symbol, and validates
arguments before touching the device."""
import ctypes
import os
import re

import pytest

from scanscam_b200 import _native

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(REPO, "include", "scanscam_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ssb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("ssb_scan_fwd_f32", "ssb_scan_bwd_f32", "ssb_scan_cl_fwd_f32", "ssb_scan_cl_bwd_f32",
                 "ssb_shard_reduce_fwd_f32", "ssb_shard_carry_f32", "ssb_device_status"):
        assert must in names


def test_library_exports_every_declared_symbol(native):
    for name in declared_symbols():
        assert hasattr(native, name), f"{name} declared in the header but not exported"


def test_ctypes_signatures_cover_the_header(native):
    assert sorted(_native.SIGNATURES) == declared_symbols()


def test_version_and_status_strings(native):
    assert native.ssb_version() >= 100
    assert native.ssb_status_string(_native.OK) == b"ok"
    for code in range(1, 7):
        assert native.ssb_status_string(code) not in (b"ok", b"unknown status")
    assert native.ssb_status_string(99) == b"unknown status"


def test_argument_validation_happens_on_the_host(native):
    """These calls return before any CUDA call, so they are safe without a device."""
    null = None
    assert native.ssb_scan_fwd_f32(null, null, null, -1, 4, null, null) == _native.ERR_BAD_ARG
    assert b"negative" in native.ssb_last_error()
    assert native.ssb_scan_fwd_f32(null, null, null, 2**40, 2**40, null, null) == _native.ERR_BAD_ARG
    assert native.ssb_scan_fwd_f32(null, null, null, 8, 16, null, null) == _native.ERR_BAD_ARG  # NULL data
    assert native.ssb_scan_bwd_f32(null, null, null, null, null, 8, 16, null, null, null) == _native.ERR_BAD_ARG
    assert native.ssb_scan_cl_fwd_f64(null, null, null, 2, -3, 4, null) == _native.ERR_BAD_ARG
    assert native.ssb_shard_carry_f32(null, 2, 5, 0, 4, null, null) == _native.ERR_BAD_ARG
    # empty problems are a no-op, whatever the pointers
    assert native.ssb_scan_fwd_f32(null, null, null, 0, 128, null, null) == _native.OK
    assert native.ssb_scan_fwd_f64(null, null, null, 16, 0, null, null) == _native.OK
    assert native.ssb_scan_bwd_f32(null, null, null, null, null, 0, 0, null, null, null) == _native.OK
    assert native.ssb_scan_cl_bwd_f32(null, null, null, null, null, 3, 0, 5, null) == _native.OK
    # misaligned pointers are refused (fake non-NULL addresses; never dereferenced on the host)
    p = ctypes.c_void_p(0x1002)
    q = ctypes.c_void_p(0x1000)
    assert native.ssb_scan_fwd_f32(p, q, q, 4, 8, null, null) == _native.ERR_ALIGNMENT
    assert native.ssb_scan_fwd_f64(ctypes.c_void_p(0x1004), q, q, 4, 8, null, null) == _native.ERR_ALIGNMENT


def test_check_raises_with_the_library_message(native):
    rc = native.ssb_scan_fwd_f32(None, None, None, -5, 1, None, None)
    with pytest.raises(_native.NativeError) as err:
        _native.check(rc)
    assert err.value.status == _native.ERR_BAD_ARG and "negative" in str(err.value)


def test_workspace_query(native):
    assert native.ssb_scan_workspace_bytes(1024, 4096, _native.VARIANT_WARP) == 0
    assert native.ssb_scan_workspace_bytes(1024, 4096, _native.VARIANT_TMA) == 0


def test_kernel_recommendation_for_row_lengths_that_need_no_device(native):
    """The part of the default policy that does not depend on a driver being present."""
    flat = _native.VARIANT_FLAT
    assert native.ssb_scan_recommend(4096, 4092, 0, 1, 0) == flat | (6 << 8)   # fills the 4096-element span
    assert native.ssb_scan_recommend(4096, 3000, 0, 1, 0) == flat | (4 << 8)   # 27 % of it idle: the smaller span
    assert native.ssb_scan_recommend(4096, 2200, 1, 1, 0) == flat | (4 << 8)
    assert native.ssb_scan_recommend(4096, 4100, 0, 1, 0) == flat | (4 << 8)   # a full piece and a 4-element one
    assert native.ssb_scan_recommend(4096, 6000, 0, 1, 0) == flat | (6 << 8)
    assert native.ssb_scan_recommend(4096, 6000, 1, 1, 0) == flat | (9 << 8)
    assert native.ssb_scan_recommend(64, 1001, 0, 1, 0) == _native.VARIANT_WARP
    assert native.ssb_scan_recommend(64, 1000, 0, 0, 0) == _native.VARIANT_WARP  # unaligned tensors
    # small problems (a few spans per SM): short spans so that the grid gets going at once
    assert native.ssb_scan_recommend(1024, 1024, 0, 1, 0) == flat | (12 << 8)
    assert native.ssb_scan_recommend(1024, 1024, 1, 1, 0) == flat | (12 << 8)
    assert native.ssb_scan_recommend(64, 4092, 0, 1, 0) == flat | (12 << 8)


def test_channels_last_recommendation_and_scratch_sizes(native):
    """No hidden state: the choice is a function of the shape and of the scratch on offer, and the
    scratch query answers for the variant that will run (nothing for the kernels that need none)."""
    plain, chunked = _native.CL_PLAIN, _native.CL_CHUNKED
    v = native.ssb_scan_cl_recommend(3, 107, 197, 0, 1, 1)          # odd channel count, short: plain or look-back, never TMA
    assert (v & 0xff) in (plain, _native.CL_LOOKBACK)
    assert native.ssb_scan_cl_recommend(3, 107, 197, 0, 1, 0) == plain
    assert native.ssb_scan_cl_variant_workspace_bytes(8, 4096, 512, plain, 0) == 0
    assert native.ssb_scan_cl_variant_workspace_bytes(8, 4096, 512, _native.CL_STREAM, 1) == 0
    need = native.ssb_scan_cl_variant_workspace_bytes(4, 65536, 256, chunked, 0)
    assert 0 < need < 4 * 65536 * 256 * 4 // 100                     # chunk maps and carries: far below a tensor
    assert native.ssb_scan_cl_variant_workspace_bytes(4, 65536, 256, _native.CL_LOOKBACK, 0) > need
    assert native.ssb_scan_cl_workspace_bytes(4, 65536, 256) >= native.ssb_scan_cl_variant_workspace_bytes(
        4, 65536, 256, _native.CL_LOOKBACK, 1)
    assert native.ssb_scan_cl_sigmoid_workspace_bytes(0, 5, 5) == 0
