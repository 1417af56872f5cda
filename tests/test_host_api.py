"""Host-side mirror of the reference's Python interface (no GPU needed)."""
import pytest
import torch

import scanscam_b200
from scanscam_b200 import cuda, decorator, op


def test_public_names_match_the_reference():
    assert scanscam_b200.scan is op.scan
    assert issubclass(op.Scan, torch.autograd.Function)
    for name in ("simple_linear_scan_forward", "coalesced_linear_scan_forward", "blocked_linear_scan_forward",
                 "simple_linear_scan_backward", "blocked_linear_scan_backward",
                 "transposed_linear_scan_forward", "transposed_linear_scan_backward"):
        assert callable(getattr(cuda, name)), name
    assert cuda.has_cuda_ops is True  # the extension is built in-tree and importable without a GPU


def test_extension_module_exports_the_reference_functions():
    import scanscam_ext  # registered by scanscam_b200.cuda

    for name in ("simple_linear_scan", "coalesced_linear_scan", "blocked_linear_scan",
                 "simple_linear_scan_backward", "blocked_linear_scan_backward",
                 "transposed_linear_scan", "transposed_linear_scan_backward"):
        assert hasattr(scanscam_ext, name), name
    # no CPU entry points: this build has no CPU path
    assert not hasattr(scanscam_ext, "simple_linear_scan_cpu")


def test_is_transpose_contig():
    x = torch.zeros(2, 5, 7)
    assert not op.is_transpose_contig(x)
    assert op.is_transpose_contig(x.mT)
    assert not op.is_transpose_contig(torch.zeros(5, 7).mT)      # 2-D never qualifies
    assert not op.is_transpose_contig(x.mT.contiguous())


def test_flattening_decorator_semantics():
    seen = {}

    @decorator.preprocess_scan_args
    def fwd(x, y):
        seen["shape"] = (tuple(x.shape), tuple(y.shape))
        return x + y

    out = fwd(torch.ones(3, 4, 5), torch.ones(3, 4, 5))
    assert seen["shape"] == ((12, 5), (12, 5)) and out.shape == (3, 4, 5)
    with pytest.raises(AssertionError):
        fwd(torch.ones(3, 4), torch.ones(3, 5))
    with pytest.raises(AssertionError):
        fwd(torch.ones(5), torch.ones(5))  # fewer than two axes

    @decorator.preprocess_backward_scan_args
    def bwd(x, y, z):
        assert x.dim() == y.dim() == z.dim() == 2
        return x * 2, z * 3

    ga, gb = bwd(torch.ones(2, 3, 4), torch.ones(2, 3, 4), torch.ones(2, 3, 4))
    assert ga.shape == gb.shape == (2, 3, 4) and float(gb[0, 0, 0]) == 3.0
    with pytest.raises(AssertionError):
        bwd(torch.ones(2, 3), torch.ones(2, 3), torch.ones(3, 2))


def test_cpu_tensors_are_refused_not_silently_served():
    a, b = torch.rand(4, 8), torch.rand(4, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        scanscam_b200.scan(a, b)
    with pytest.raises(RuntimeError, match="no CPU path"):
        scanscam_b200.scan_sigmoid_gate(a, b)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        cuda.blocked_linear_scan_forward(a, b)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        cuda.transposed_linear_scan_forward(torch.rand(2, 3, 4), torch.rand(2, 3, 4), 32)


def test_transposed_wrappers_assert_like_the_reference():
    x = torch.rand(2, 3, 4)
    with pytest.raises(AssertionError):
        cuda.transposed_linear_scan_forward(x, torch.rand(2, 3, 5), 32)
    with pytest.raises(AssertionError):
        cuda.transposed_linear_scan_forward(x.mT, x.mT, 32)  # not contiguous
    with pytest.raises(AssertionError):
        cuda.transposed_linear_scan_backward(x[0], x[0], x[0], 32)  # not 3-D


def test_workload_table():
    from scanscam_b200 import workloads

    w = workloads.WORKLOADS["cfg2"]
    assert w.shape == (8, 2048, 4096) and w.rows == 16384 and w.elements == 67108864
    a, b, g = workloads.make_inputs("resets", (4, 256), seed=0)
    assert (a == 0).float().mean() > 0.03 and a.min() >= 0 and a.max() < 1
    a2, _, _ = workloads.make_inputs("resets", (4, 256), seed=0)
    assert torch.equal(a, a2)
    a, b, _ = workloads.make_inputs("nearunit", (2, 1000))
    assert a.min() >= 0.99 and a.max() <= 1.0 and abs(float(b.std()) - 0.1) < 0.02
    a, _, _ = workloads.make_inputs("sigmoid2", (8, 4096))
    assert 0.86 < float(a.median()) < 0.90
