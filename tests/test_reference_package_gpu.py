"""The reference's own, unmodified Python package running over this build's `scanscam_ext`.

The reference's wrappers do ``import scanscam_ext`` and call its functions with caller-allocated
outputs (scanscam/cuda.py:7-13,39); the module built here exports the same seven names with the
same argument order (src/scanscam_cuda.cu:725-737).  This test puts the directory that holds the
built ``scanscam_ext.so`` in front of ``sys.path``, imports the reference package from the
directory named by ``SCANSCAM_REFERENCE_DIR`` (a checkout of the reference, i.e. the directory
that contains ``scanscam/``) and replays the reference's CUDA test grid
(scanscam/cuda_test.py:19-163) through ``scanscam.cuda.*`` and ``scanscam.scan``, checking against
the CPU oracle with the reference tests' own criterion (atol 1e-4, default rtol).

It runs in a child process so that the import order is the one a user of the reference would
have, whatever this test session imported before.  Skipped when no checkout is given.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.environ.get("SCANSCAM_REFERENCE_DIR", "")

CHILD = textwrap.dedent(
    """
    import os, sys
    repo, ref = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref)                                   # the reference checkout: provides `scanscam`
    sys.path.insert(0, os.path.join(repo, "scanscam_b200"))   # first on the path: provides `scanscam_ext`
    sys.path.append(repo)                                     # for the oracle (test infrastructure)
    import numpy as np
    import torch
    import scanscam_ext
    assert os.path.dirname(os.path.abspath(scanscam_ext.__file__)) == os.path.join(repo, "scanscam_b200"), scanscam_ext.__file__
    import scanscam
    import scanscam.cuda as rc
    assert os.path.abspath(scanscam.__file__).startswith(os.path.abspath(ref)), scanscam.__file__
    assert rc.has_cuda_ops, "the reference package did not recognise scanscam_ext"
    import oracle

    def close(x, ref):
        return bool(np.all(np.abs(x.detach().cpu().numpy() - ref) <= 1e-4 + 1e-5 * np.abs(ref)))

    torch.manual_seed(0)
    n = 0
    # scanscam/cuda_test.py:19-80 -- forward, contiguous and permuted inputs, all three strategies' names
    fwd_shapes = [(32, 5), (16, 2, 5), (32, 64), (32, 128), (32, 256), (32, 512), (32, 513), (1, 1024), (32, 1024),
                  (32, 1025), (1, 1025), (32, 4095), (32, 4096), (32, 4097), (32, 4100), (32, 16384), (32, 16388)]
    for shape in fwd_shapes:
        for permute in (False, True):
            x, y = torch.randn(shape, device="cuda"), torch.randn(shape, device="cuda")
            if permute:
                x, y = x.mT.contiguous().mT, y.mT.contiguous().mT
            ref = oracle.scan_forward(x.contiguous().cpu().numpy(), y.contiguous().cpu().numpy())
            for fn in (rc.simple_linear_scan_forward, rc.coalesced_linear_scan_forward, rc.blocked_linear_scan_forward):
                assert close(fn(x, y), ref), (fn.__name__, shape, permute)
                n += 1
    # scanscam/cuda_test.py:83-126 -- backward (arguments are gate, output, out_grad)
    for shape in [(32, 5), (16, 2, 5), (32, 64), (1, 1024), (32, 1024), (32, 1025), (1, 1025)]:
        for permute in (False, True):
            x, y, z = (torch.randn(shape, device="cuda") for _ in range(3))
            if permute:
                x, y, z = (t.mT.contiguous().mT for t in (x, y, z))
            ga_ref, gb_ref = oracle.scan_backward(*(t.contiguous().cpu().numpy() for t in (x, y, z)))
            for fn in (rc.simple_linear_scan_backward, rc.blocked_linear_scan_backward):
                ga, gb = fn(x, y, z)
                assert close(ga, ga_ref) and close(gb, gb_ref), (fn.__name__, shape, permute)
                n += 1
    # scanscam/cuda_test.py:129-163 -- channels-last, the three channels_per_block values the tests use
    for shape in [(8, 4096, 512), (512, 4096, 8), (3, 107, 197), (3, 293, 283), (5, 6113, 107)]:
        x, y, z = (torch.randn(shape, device="cuda") for _ in range(3))
        h_ref = oracle.scan_forward_channels_last(x.cpu().numpy(), y.cpu().numpy())
        ga_ref, gb_ref = oracle.scan_backward_channels_last(x.cpu().numpy(), y.cpu().numpy(), z.cpu().numpy())
        for cpb in (1, 8, 32):
            assert close(rc.transposed_linear_scan_forward(x, y, cpb), h_ref), (shape, cpb)
            ga, gb = rc.transposed_linear_scan_backward(x, y, z, cpb)
            assert close(ga, ga_ref) and close(gb, gb_ref), (shape, cpb)
            n += 2
    # the operator itself (scanscam/op.py:13-55): autograd through the rows layout, forward on a
    # channels-last input (the reference's own backward for that layout raises, op.py:46-48)
    a = torch.sigmoid(torch.randn(4, 64, 1024, device="cuda") + 2).requires_grad_(True)
    b = torch.randn(4, 64, 1024, device="cuda", requires_grad=True)
    g = torch.randn(4, 64, 1024, device="cuda")
    h = scanscam.scan(a, b)
    h.backward(g)
    h_ref = oracle.scan_forward(a.detach().cpu().numpy(), b.detach().cpu().numpy())
    ga_ref, gb_ref = oracle.scan_backward(a.detach().cpu().numpy(), h_ref, g.cpu().numpy())
    assert close(h, h_ref) and close(a.grad, ga_ref) and close(b.grad, gb_ref)
    xt, yt = torch.randn(3, 300, 64, device="cuda").mT, torch.randn(3, 300, 64, device="cuda").mT
    ht = scanscam.scan(xt, yt)
    assert close(ht.contiguous(), oracle.scan_forward(xt.contiguous().cpu().numpy(), yt.contiguous().cpu().numpy()))
    n += 2
    torch.cuda.synchronize()
    print(f"REFERENCE_PACKAGE_OK {n} comparisons; scanscam from {scanscam.__file__}; scanscam_ext from {scanscam_ext.__file__}")
    """
)


@pytest.mark.skipif(not REF_DIR or not os.path.isdir(os.path.join(REF_DIR, "scanscam")),
                    reason="set SCANSCAM_REFERENCE_DIR to a checkout of the reference (the directory holding scanscam/)")
def test_unmodified_reference_package_over_this_extension():
    out = subprocess.run([sys.executable, "-c", CHILD, REPO, os.path.abspath(REF_DIR)], capture_output=True, text=True,
                         timeout=1200)
    sys.stdout.write(out.stdout)
    sys.stderr.write(out.stderr[-4000:])
    assert out.returncode == 0, out.stderr[-4000:]
    assert "REFERENCE_PACKAGE_OK" in out.stdout
