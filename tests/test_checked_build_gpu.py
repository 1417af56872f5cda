"""The checked build (-DSSB_CHECKED): the same kernels with a range test in front of every global
access they compute an address for.  It is this repository's stand-in for a memory checker: run
the parity suite's edge cases through it and expect (a) the same results and (b) a clean status
word -- an index outside its tensor would have been skipped and reported, not dereferenced.

The parity tests reach the kernels through ctypes, so pointing SCANSCAM_B200_LIB at the checked
library in a child process is enough to run them against it.  The reporting path itself is
exercised with an index VALUE that is out of range (no memory access is involved).
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent(
    """
    import sys
    sys.path.insert(0, sys.argv[1])
    import ctypes
    import pytest, torch
    from scanscam_b200 import _native
    lib = _native.load()
    assert lib.ssb_checked_build() == 1, _native.LIB_PATH
    # the reporting path: an out-of-range index value is reported once, and the context lives on
    _native.check(lib.ssb_selftest_index_check(None))
    detail = ctypes.c_int(0)
    assert lib.ssb_device_status(ctypes.byref(detail)) == _native.ERR_DEVICE_CHECK and detail.value == 99
    assert lib.ssb_device_status(ctypes.byref(detail)) == _native.OK
    x = torch.rand(8, 1000, device="cuda")
    out = torch.empty_like(x)
    _native.check(lib.ssb_scan_fwd_f32(x.data_ptr(), x.data_ptr(), out.data_ptr(), 8, 1000, None, None))
    assert lib.ssb_device_status(ctypes.byref(detail)) == _native.OK
    # the edge cases of the parity suite; every test ends with a status check of its own
    select = ("golden or reference_shape_grid or row_packing or fp64 or edge_shapes or unaligned or lookback_long_rows or "
              "shard_maps or shard_carries or channels_last_with_scratch or virtual_t_shards or random_shapes")
    rc = pytest.main(["-x", "-q", "-m", "gpu", "-k", select, sys.argv[1] + "/tests/test_parity_gpu.py",
                      sys.argv[1] + "/tests/test_fuzz_gpu.py"])
    assert lib.ssb_device_status(ctypes.byref(detail)) == _native.OK, detail.value
    print("CHECKED_BUILD_RC", int(rc))
    sys.exit(int(rc))
    """
)


def test_edge_cases_run_clean_under_the_checked_build():
    from scanscam_b200 import build

    checked = build.LIB_CHECKED
    if not os.path.exists(checked):
        checked = build.build_library(checked=True)  # nvcc only; a few minutes at most
    env = dict(os.environ, SCANSCAM_B200_LIB=checked)
    out = subprocess.run([sys.executable, "-c", CHILD, REPO], capture_output=True, text=True, env=env, timeout=3000)
    sys.stdout.write(out.stdout[-3000:])
    sys.stderr.write(out.stderr[-3000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "CHECKED_BUILD_RC 0" in out.stdout


def test_the_ordinary_build_says_what_it_is():
    from scanscam_b200 import _native

    lib = _native.load()
    if os.environ.get("SCANSCAM_B200_LIB"):
        pytest.skip("another build of the library was selected for this session")
    assert lib.ssb_checked_build() == 0
    assert lib.ssb_selftest_index_check(None) == _native.ERR_UNSUPPORTED
