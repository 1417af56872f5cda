"""The Python operator layer on a GPU: scan()/Scan through autograd on both layouts, the
wrapper names of the reference's cuda module, and the reference's error behaviour."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _gpu  # noqa: E402

import oracle  # noqa: E402
import scanscam_b200  # noqa: E402
from scanscam_b200 import cuda, op, sharded  # noqa: E402
from scanscam_b200.workloads import make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu

GRID = [(32, 5), (16, 2, 5), (32, 64), (1, 1024), (32, 1024), (32, 1025), (1, 1025)]


@pytest.mark.parametrize("shape", GRID + [(4, 8, 4096)])
@pytest.mark.parametrize("permute", [False, True])
def test_scan_autograd_matches_oracle(shape, permute):
    """permute=True feeds the layouts of scanscam/cuda_test.py:28-29: x.mT.contiguous().mT."""
    a, b, g = make_inputs("randn", shape, seed=21)
    T = shape[-1]
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, T) for x in (a, b, g)))
    da, db = a.cuda(), b.cuda()
    if permute:
        da, db = da.mT.contiguous().mT, db.mT.contiguous().mT
    da.requires_grad_(True)
    db.requires_grad_(True)
    h = scanscam_b200.scan(da, db)
    assert h.shape == da.shape
    h.backward(g.cuda())
    assert _gpu.allclose_ref(h.reshape(-1, T), h_ref)
    assert _gpu.allclose_ref(db.grad.reshape(-1, T), gb_ref)
    assert _gpu.allclose_ref(da.grad.reshape(-1, T), ga_ref)


def test_channels_last_path_is_taken_and_correct():
    a, b, g = make_inputs("sigmoid2", (3, 50, 200), seed=5)      # [N, C, T] logical
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, 200) for x in (a, b, g)))
    da = a.cuda().mT.contiguous().mT.requires_grad_(True)          # dense as [N, T, C]
    db = b.cuda().mT.contiguous().mT.requires_grad_(True)
    assert op.is_transpose_contig(da)
    h = scanscam_b200.scan(da, db)
    assert op.is_transpose_contig(h)                                # stays channels-last
    h.backward(g.cuda().mT.contiguous().mT)                         # the branch the reference gets wrong
    assert _gpu.allclose_ref(h.reshape(-1, 200), h_ref)
    assert _gpu.allclose_ref(db.grad.reshape(-1, 200), gb_ref)
    assert _gpu.allclose_ref(da.grad.reshape(-1, 200), ga_ref)


# the reference's channels-last grid, scanscam/cuda_test.py:129-163 (largest case trimmed in N)
@pytest.mark.parametrize("shape", [(8, 4096, 512), (64, 4096, 8), (3, 107, 197), (3, 293, 283), (5, 6113, 107)])
@pytest.mark.parametrize("cpb", [1, 32])
def test_transposed_wrappers(shape, cpb):
    a, b, g = make_inputs("randn", shape, seed=31)
    an, bn, gn = a.numpy(), b.numpy(), g.numpy()
    h_ref = oracle.scan_forward_channels_last(an, bn)
    ga_ref, gb_ref = oracle.scan_backward_channels_last(an, h_ref, gn)
    h = cuda.transposed_linear_scan_forward(a.cuda(), b.cuda(), cpb)
    ga, gb = cuda.transposed_linear_scan_backward(a.cuda(), torch.from_numpy(h_ref).cuda(), g.cuda(), cpb)
    for got, ref in ((h, h_ref), (gb, gb_ref), (ga, ga_ref)):
        assert _gpu.max_norm_err(got, ref) < 1e-4
        # The reference's criterion (scanscam/cuda_test.py:140) holds element by element except where
        # a value of order 1 is the difference of terms of order 1e4 (randn gates over 4096 steps):
        # allow a few such elements per million.
        bad = np.abs(got.cpu().numpy() - ref) > 1e-4 + 1e-5 * np.abs(ref)
        assert bad.mean() < 5e-6, bad.sum()


@pytest.mark.parametrize("fn_name", ["simple_linear_scan_forward", "coalesced_linear_scan_forward",
                                     "blocked_linear_scan_forward"])
def test_forward_wrapper_names(fn_name):
    a, b, _ = make_inputs("randn", (16, 2, 1025), seed=2)
    h_ref = oracle.scan_forward(a.numpy(), b.numpy())
    h = getattr(cuda, fn_name)(a.cuda(), b.cuda())
    assert h.shape == (16, 2, 1025) and _gpu.allclose_ref(h, h_ref)


@pytest.mark.parametrize("fn_name", ["simple_linear_scan_backward", "blocked_linear_scan_backward"])
def test_backward_wrapper_names(fn_name):
    a, b, g = make_inputs("randn", (16, 2, 1025), seed=3)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, 1025) for x in (a, b, g)))
    ga, gb = getattr(cuda, fn_name)(a.cuda(), torch.from_numpy(h_ref).cuda().reshape(a.shape), g.cuda())
    assert ga.shape == a.shape
    assert _gpu.allclose_ref(ga.reshape(-1, 1025), ga_ref) and _gpu.allclose_ref(gb.reshape(-1, 1025), gb_ref)


def test_gradcheck_fp64():
    a = torch.rand(3, 37, dtype=torch.float64, device="cuda", requires_grad=True)
    b = torch.randn(3, 37, dtype=torch.float64, device="cuda", requires_grad=True)
    assert torch.autograd.gradcheck(scanscam_b200.scan, (a, b), eps=1e-6, atol=1e-6)


def test_error_behaviour_matches_the_reference():
    x = torch.rand(4, 8, device="cuda")
    with pytest.raises(AssertionError):
        scanscam_b200.scan(x, torch.rand(4, 9, device="cuda"))
    with pytest.raises(AssertionError):
        scanscam_b200.scan(torch.rand(8, device="cuda"), torch.rand(8, device="cuda"))
    with pytest.raises(NotImplementedError, match="not implemented for 'Int'"):
        scanscam_b200.scan(x.int(), x.int())
    # 16-bit floating types are an addition (rows layout: any shape; channels-last: C % 8 == 0);
    # other channel counts raise as the reference does for every half-precision input
    xt = torch.rand(2, 8, 4, device="cuda").half().mT
    with pytest.raises(NotImplementedError, match="not implemented for 'Half'"):
        scanscam_b200.scan(xt, xt)
    import scanscam_ext

    with pytest.raises(RuntimeError, match="contiguous"):
        scanscam_ext.blocked_linear_scan(x.t(), x.t(), torch.empty(8, 4, device="cuda"))
    with pytest.raises(RuntimeError, match="same dtype"):
        scanscam_ext.blocked_linear_scan(x, x.double(), torch.empty_like(x))


def test_runs_on_the_current_stream():
    a, b, _ = make_inputs("sigmoid2", (64, 4096), seed=8)
    h_ref = oracle.scan_forward(a.numpy(), b.numpy())
    side = torch.cuda.Stream()
    da, db = a.cuda(), b.cuda()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        h = scanscam_b200.scan(da, db)
    side.synchronize()
    assert _gpu.allclose_ref(h, h_ref)


def test_sequence_parallel_module_single_rank():
    """Without a process group the sequence-parallel entry point is the plain scan."""
    a, b, g = make_inputs("nearunit", (8, 8192), seed=13)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    h = sharded.scan_sequence_parallel(da, db)
    h.backward(g.cuda())
    assert _gpu.max_norm_err(h, h_ref) < 1e-4
    assert _gpu.max_norm_err(db.grad, gb_ref) < 1e-4 and _gpu.max_norm_err(da.grad, ga_ref) < 1e-4


@pytest.mark.parametrize("shape,chunks", [((37, 1024), 4), ((5, 3, 260), 3), ((8, 4096), 16)])
def test_host_pipeline_matches_oracle(shape, chunks):
    """Host-buffer entry point: pinned tensors in, results back on the host, chunks pipelined."""
    from scanscam_b200 import host

    a, b, g = make_inputs("sigmoid2", shape, seed=41)
    T = shape[-1]
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, T) for x in (a, b, g)))
    h, ga, gb = host.scan_forward_backward_host(a.pin_memory(), b.pin_memory(), g.pin_memory(), chunks=chunks)
    assert h.device.type == "cpu" and h.shape == a.shape
    assert _gpu.allclose_ref(h.reshape(-1, T), h_ref)
    assert _gpu.allclose_ref(ga.reshape(-1, T), ga_ref) and _gpu.allclose_ref(gb.reshape(-1, T), gb_ref)
    # a reused pipeline gives the same answer on a second call (staging slots are recycled correctly)
    pipe = host.HostScanPipeline(h_ref.shape[0], T, chunks=chunks)
    flat = [x.reshape(-1, T).contiguous().pin_memory() for x in (a, b, g)]
    out1 = pipe.run(*flat)
    torch.cuda.synchronize()
    first = [o.clone() for o in out1]
    out2 = pipe.run(*flat, out=out1)
    torch.cuda.synchronize()
    assert all(torch.equal(x, y) for x, y in zip(first, out2))


def test_scan_can_be_captured_in_a_cuda_graph():
    """Forward + backward kernels recorded once and replayed on new data (rows that fit a span:
    no scratch is involved, so nothing is allocated by the library during capture)."""
    a, b, g = make_inputs("sigmoid2", (64, 2048), seed=51)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
    _gpu.fwd(da, db)  # warm-up outside capture (occupancy queries are cached on first use)
    _gpu.bwd(da, da, dg)
    torch.cuda.synchronize()
    from scanscam_b200 import _native

    lib = _native.load()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        st = torch.cuda.current_stream().cuda_stream
        _native.check(lib.ssb_scan_fwd_f32(da.data_ptr(), db.data_ptr(), h.data_ptr(), 64, 2048, None, st))
        _native.check(lib.ssb_scan_bwd_f32(da.data_ptr(), h.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                           64, 2048, None, None, st))
    for seed in (52, 53):
        a2, b2, g2 = make_inputs("sigmoid2", (64, 2048), seed=seed)
        da.copy_(a2); db.copy_(b2); dg.copy_(g2)
        graph.replay()
        torch.cuda.synchronize()
        h_ref, ga_ref, gb_ref = _gpu.oracle_all(a2, b2, g2)
        assert _gpu.allclose_ref(h, h_ref) and _gpu.allclose_ref(ga, ga_ref) and _gpu.allclose_ref(gb, gb_ref)


def test_chunked_channels_last_can_be_captured_in_a_cuda_graph():
    """The two-pass channels-last form -- map kernel, then the scan kernel as its programmatic
    dependent -- recorded once with the caller's scratch and replayed on new data."""
    from scanscam_b200 import _native

    lib = _native.load()
    N, T, C = 2, 6144, 64
    a, b, g = make_inputs("sigmoid2", (N, T, C), seed=61)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
    v = _native.CL_CHUNKED
    need = max(lib.ssb_scan_cl_variant_workspace_bytes(N, T, C, v, d) for d in (0, 1))
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")

    def both(st):
        _native.check(lib.ssb_scan_cl_fwd_f32_ex(da.data_ptr(), db.data_ptr(), h.data_ptr(), N, T, C, v, ws.data_ptr(), need, st))
        _native.check(lib.ssb_scan_cl_bwd_f32_ex(da.data_ptr(), h.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                 N, T, C, v, ws.data_ptr(), need, st))

    both(torch.cuda.current_stream().cuda_stream)  # warm-up outside capture (occupancy queries are cached on first use)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        both(torch.cuda.current_stream().cuda_stream)
    for seed in (62, 63):
        a2, b2, g2 = make_inputs("sigmoid2", (N, T, C), seed=seed)
        da.copy_(a2); db.copy_(b2); dg.copy_(g2)
        graph.replay()
        torch.cuda.synchronize()
        h_ref = oracle.scan_forward_channels_last(a2.numpy(), b2.numpy())
        ga_ref, gb_ref = oracle.scan_backward_channels_last(a2.numpy(), h_ref, g2.numpy())
        assert _gpu.allclose_ref(h, h_ref) and _gpu.allclose_ref(ga, ga_ref) and _gpu.allclose_ref(gb, gb_ref)
    _gpu.device_ok()


@pytest.mark.parametrize("shape", [(64, 4096), (3, 5, 1024), (2, 20000), (1000, 8), (7, 1001)])
def test_fused_sigmoid_gate_matches_unfused_oracle(shape):
    """scan_sigmoid_gate(z, b) against the CPU oracle fed sigmoid(z) computed in fp32 on the host;
    the last shape (T % 4 != 0) goes through the unfused composition."""
    z, b, g = make_inputs("randn", shape, seed=61)
    z = z * 2 + 1.5
    T = shape[-1]
    a = torch.sigmoid(z)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, T) for x in (a, b, g)))
    gz_ref = ga_ref * (a * (1 - a)).reshape(-1, T).numpy()
    dz, db = z.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    h = scanscam_b200.scan_sigmoid_gate(dz, db)
    h.backward(g.cuda())
    assert _gpu.max_norm_err(h.reshape(-1, T), h_ref) < 1e-4
    assert _gpu.max_norm_err(db.grad.reshape(-1, T), gb_ref) < 1e-4
    assert _gpu.max_norm_err(dz.grad.reshape(-1, T), gz_ref) < 1e-4
    assert _gpu.allclose_ref(h.reshape(-1, T), h_ref, atol=1e-4, rtol=1e-4)
    # and against the library's own unfused path
    dz2, db2 = z.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    h2 = scanscam_b200.scan(torch.sigmoid(dz2), db2)
    h2.backward(g.cuda())
    assert float((h - h2).detach().abs().max() / h2.detach().abs().max()) < 1e-5
    assert float((dz.grad - dz2.grad).abs().max() / dz2.grad.abs().max()) < 1e-5


@pytest.mark.parametrize("shape,dtype,permute", [((8, 16, 4096), torch.float32, False), ((3, 5, 1000), torch.float32, False),
                                                  ((2, 3, 7, 64), torch.float32, False), ((4, 33), torch.float64, False),
                                                  ((2, 50, 96), torch.float32, True)])
def test_scan_recompute_matches_scan(shape, dtype, permute):
    """scan_recompute keeps (gate, value) for the backward, not the output, and returns the same
    values and gradients as scan."""
    a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", shape, seed=95))

    def leaf(x):
        x = x.cuda()
        if permute:  # dense in [N, T, C] order, viewed as [N, C, T]
            x = x.mT.contiguous().mT
        return x.requires_grad_(True)

    a1, b1, a2, b2 = leaf(a), leaf(b), leaf(a), leaf(b)
    h1 = scanscam_b200.scan(a1, b1)
    h2 = scanscam_b200.scan_recompute(a2, b2)
    saved = h2.grad_fn.saved_tensors
    assert len(saved) == 2 and saved[0].data_ptr() == a2.data_ptr() and saved[1].data_ptr() == b2.data_ptr()
    dg = g.cuda()
    h1.backward(dg)
    h2.backward(dg)
    assert torch.equal(h1, h2)
    tol = 1e-5 if dtype == torch.float32 else 1e-12
    for x, y in ((a1.grad, a2.grad), (b1.grad, b2.grad)):
        assert float((x - y).abs().max() / y.abs().max()) < tol
    T = shape[-1]
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(*(x.reshape(-1, T) for x in (a, b, g)))
    assert _gpu.max_norm_err(a2.grad.contiguous().reshape(-1, T), ga_ref) < 1e-4
    assert _gpu.max_norm_err(b2.grad.contiguous().reshape(-1, T), gb_ref) < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 16, 4096), (3, 5, 1000), (6, 33)])
def test_scan_with_16bit_tensors(dtype, shape):
    """scan() on bf16 / fp16 tensors: fp32 arithmetic inside, outputs and gradients rounded once.
    Checked against the oracle run in fp32 on the same (already rounded) inputs."""
    a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", shape, seed=97))
    T = shape[-1]
    h_ref = oracle.scan_forward(a.float().reshape(-1, T).numpy(), b.float().reshape(-1, T).numpy())
    da, db = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    h = scanscam_b200.scan(da, db)
    assert h.dtype == dtype
    h.backward(g.cuda())
    # the backward reads the h the forward stored, i.e. the rounded one
    ga_ref, gb_ref = oracle.scan_backward(a.float().reshape(-1, T).numpy(), h.detach().float().cpu().reshape(-1, T).numpy(),
                                          g.float().reshape(-1, T).numpy())
    half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    for x, ref in ((h, h_ref), (da.grad, ga_ref), (db.grad, gb_ref)):
        assert x.dtype == dtype
        assert _gpu.max_norm_err(x.detach().float().reshape(-1, T), ref) < 1.01 * half_ulp


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 16, 4096), (3, 5, 1000)])
def test_fused_operators_with_16bit_tensors(dtype, shape):
    """scan_sigmoid_gate and scan_recompute on bf16 / fp16 tensors against the plain operator run in
    fp32 on the same inputs (the second shape takes the unfused / forward-again fallbacks)."""
    z, b, g = make_inputs("randn", shape, seed=113)
    z, b, g = (z + 1).to(dtype).cuda(), b.to(dtype).cuda(), g.to(dtype).cuda()
    half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11

    def close(x, ref, slack=3.0):
        assert x.dtype == dtype
        return float((x.detach().float() - ref).abs().max() / ref.abs().max()) < slack * half_ulp

    zf, bf = z.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = scanscam_b200.scan(torch.sigmoid(zf), bf)
    ref.backward(g.float())
    z1, b1 = z.clone().requires_grad_(True), b.clone().requires_grad_(True)
    h = scanscam_b200.scan_sigmoid_gate(z1, b1)
    h.backward(g)
    assert close(h, ref.detach()) and close(z1.grad, zf.grad) and close(b1.grad, bf.grad)

    a = torch.sigmoid(z.float()).to(dtype)
    af, bf2 = a.float().requires_grad_(True), b.float().requires_grad_(True)
    ref2 = scanscam_b200.scan(af, bf2)
    ref2.backward(g.float())
    a2, b2 = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    h2 = scanscam_b200.scan_recompute(a2, b2)
    h2.backward(g)
    assert close(h2, ref2.detach()) and close(a2.grad, af.grad) and close(b2.grad, bf2.grad)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 256, 600), (1, 64, 5000), (2, 24, 100), (24, 512, 300), (20, 520, 260)])
def test_scan_channels_last_with_16bit_tensors(dtype, shape):
    """scan() on channels-last bf16 / fp16 inputs ([N, C, T] views of dense [N, T, C]) against the
    fp32 oracle on the rounded inputs."""
    N, C, T = shape
    a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", (N, T, C), seed=121))
    h_ref = oracle.scan_forward_channels_last(a.float().numpy(), b.float().numpy())
    da, db = a.cuda().mT.requires_grad_(True), b.cuda().mT.requires_grad_(True)
    assert op.is_transpose_contig(da)
    h = scanscam_b200.scan(da, db)
    assert h.dtype == dtype and op.is_transpose_contig(h)
    h.backward(g.cuda().mT)
    ga_ref, gb_ref = oracle.scan_backward_channels_last(a.float().numpy(), h.detach().mT.float().cpu().numpy(), g.float().numpy())
    half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    for x, ref in ((h.mT, h_ref), (da.grad.mT, ga_ref), (db.grad.mT, gb_ref)):
        assert _gpu.max_norm_err(x.detach().float().contiguous(), ref) < 1.01 * half_ulp


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 256, 600), (1, 64, 5000), (2, 24, 100), (3, 12, 50), (24, 512, 300), (20, 520, 260)])
def test_fused_sigmoid_gate_channels_last(dtype, shape):
    """scan_sigmoid_gate on channels-last inputs ([N, C, T] views of dense [N, T, C]): the fused
    streaming kernels (the last shape's 12 channels fall back to the unfused composition for the
    16-bit types) against the plain operator run in fp32 on the same inputs."""
    N, C, T = shape
    z, b, g = make_inputs("randn", (N, T, C), seed=151)
    z, b, g = (z + 1).to(dtype).cuda(), b.to(dtype).cuda(), g.to(dtype).cuda()
    if dtype != torch.float32 and C % 8:
        with pytest.raises(NotImplementedError):  # neither fused nor unfused: 16-bit channels-last needs C % 8 == 0
            scanscam_b200.scan_sigmoid_gate(z.mT, b.mT)
        return
    tol = {torch.float32: 2e-6, torch.bfloat16: 3 * 2.0 ** -8, torch.float16: 3 * 2.0 ** -11}[dtype]
    zf, bf = z.float().mT.requires_grad_(True), b.float().mT.requires_grad_(True)
    ref = scanscam_b200.scan(torch.sigmoid(zf), bf)
    ref.backward(g.float().mT)
    z1, b1 = z.mT.requires_grad_(True), b.mT.requires_grad_(True)
    h = scanscam_b200.scan_sigmoid_gate(z1, b1)
    assert h.dtype == dtype and op.is_transpose_contig(h)
    h.backward(g.mT)
    for x, r in ((h, ref), (z1.grad, zf.grad), (b1.grad, bf.grad)):
        assert float((x.detach().float() - r.detach()).abs().max() / r.detach().abs().max()) < tol


@pytest.mark.parametrize("shape", [(8, 4096, 512), (16, 1024, 256)])
def test_channels_last_wrappers_hold_no_scratch_when_the_kernel_needs_none(shape):
    """Shapes whose channels-last kernels stream a whole sequence per CTA use no workspace: a call
    through the reference's wrapper names must not hold more device memory than its inputs and its
    outputs (the reference allocates nothing beyond them either, scanscam/cuda.py:76-77,90-93)."""
    from scanscam_b200 import _native

    lib = _native.load()
    assert lib.ssb_scan_cl_variant_workspace_bytes(*shape, lib.ssb_scan_cl_recommend(*shape, 0, 1, 1), 0) == 0
    assert lib.ssb_scan_cl_variant_workspace_bytes(*shape, lib.ssb_scan_cl_recommend(*shape, 1, 1, 1), 1) == 0
    x, y, z = (torch.randn(shape, device="cuda") for _ in range(3))
    cuda.transposed_linear_scan_forward(x, y, 32)  # warm-up: one-time allocations of the runtime
    torch.cuda.synchronize()
    one = x.numel() * 4
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    h = cuda.transposed_linear_scan_forward(x, y, 32)
    torch.cuda.synchronize()
    assert torch.cuda.max_memory_allocated() - base <= one + (1 << 20), (torch.cuda.max_memory_allocated() - base, one)
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    ga, gb = cuda.transposed_linear_scan_backward(x, h, z, 32)
    torch.cuda.synchronize()
    assert torch.cuda.max_memory_allocated() - base <= 2 * one + (1 << 20)
    _gpu.device_ok()
