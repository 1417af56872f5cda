"""Parity of the CUDA kernels with the CPU oracle, through the C-ABI (ctypes + raw device
pointers).  Tolerances: the reference tests' allclose(atol=1e-4, rtol=1e-5) on the reference's
shape grid, and max-norm relative error <= 1e-4 on the benchmark configurations (observed
errors are ~1e-6; anything near 1e-5 would already mean a bug, not reassociation)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _gpu  # noqa: E402
from _gpu import AUTO, FLAT, FLAT_ANY, LOOKBACK, TMA, WARP  # noqa: E402

import oracle  # noqa: E402
from scanscam_b200 import _native  # noqa: E402
from scanscam_b200.workloads import WORKLOADS, make_inputs, workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-4

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "scan_golden.npz"))
GOLDEN_ROWS = sorted({k.split("/")[0] for k in GOLDEN.files if not k.startswith("cl_")})
GOLDEN_CL = sorted({k.split("/")[0] for k in GOLDEN.files if k.startswith("cl_")})

# the reference's own shape grids (scanscam/cuda_test.py:19-126)
REF_SHAPES = [(32, 5), (16, 2, 5), (32, 64), (32, 128), (32, 256), (32, 512), (32, 513), (1, 1024), (32, 1024),
              (32, 1025), (1, 1025), (32, 4095), (32, 4096), (32, 4097), (32, 4100), (32, 16384), (32, 16388)]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda() if isinstance(x, np.ndarray) else x.cuda()


def variants_for(T, dtype=torch.float32):
    v = [AUTO, WARP]
    if dtype == torch.float32 and T % 32 == 0:
        v += [TMA, _gpu.tma_variant(1), _gpu.tma_variant(6)]
    if dtype == torch.float32 and T % 4 == 0:
        v += [_gpu.flat_variant(t) for t in range(7)]
    if dtype == torch.float32:
        v += [FLAT_ANY, FLAT_ANY | (1 << 8)]  # any T, two span shapes
    if dtype == torch.float32 and T % 32 == 0 and (T // 32) & (T // 32 - 1) == 0:
        # TMA-staged flat sweep: tuning ids 32+k, usable while a row fits the id's span (lines of 32)
        min_lines = [128, 128, 64, 64, 64, 128, 32]
        v += [_gpu.tma_variant(32 + k) for k, lines in enumerate(min_lines) if T // 32 <= lines]
    if dtype == torch.float32 and T % 4096 == 0 and T >= 8192:
        v.append(_gpu.tma_variant(48))  # the same sweep over rows of several spans, state chained from span to span
    return v


@pytest.mark.parametrize("name", GOLDEN_ROWS)
def test_golden_vectors(name):
    c = {k: GOLDEN[f"{name}/{k}"] for k in ("a", "b", "g", "h", "ga", "gb")}
    shape = c["a"].shape
    T = shape[-1]
    a, b, g, h_ref = (dev(c[k].reshape(-1, T)) for k in ("a", "b", "g", "h"))
    for variant in variants_for(T, a.dtype):
        h = _gpu.fwd(a, b, variant=variant)
        ga, gb = _gpu.bwd(a, h_ref, g, variant=variant)
        for got, key in ((h, "h"), (ga, "ga"), (gb, "gb")):
            ref = c[key].reshape(-1, T)
            assert _gpu.allclose_ref(got, ref), (name, variant, key, _gpu.max_norm_err(got, ref))
            assert _gpu.max_norm_err(got, ref) < TOL
    _gpu.device_ok()


@pytest.mark.parametrize("name", GOLDEN_CL)
def test_golden_vectors_channels_last(name):
    c = {k: GOLDEN[f"{name}/{k}"] for k in ("a", "b", "g", "h", "ga", "gb")}
    a, b, g, h_ref = (dev(c[k]) for k in ("a", "b", "g", "h"))
    for scratch in ([False, True, "plain", 64, 65] if a.dtype == torch.float32 else [False]):
        if isinstance(scratch, int) and scratch >= 64 and a.shape[2] % 4:
            continue
        h = _gpu.cl_fwd(a, b, scratch=scratch)
        ga, gb = _gpu.cl_bwd(a, h_ref, g, scratch=scratch)
        for got, key in ((h, "h"), (ga, "ga"), (gb, "gb")):
            assert _gpu.allclose_ref(got, c[key]), (name, scratch, key, _gpu.max_norm_err(got, c[key]))
    _gpu.device_ok()


# [N, T, C]: wide, narrow, odd C (scalar path), C % 4 == 0 but not a multiple of 128, one long
# sequence with few channels (many tiles chained by look-back), T below one tile, unaligned base
@pytest.mark.parametrize("shape", [(2, 300, 512), (3, 107, 197), (5, 613, 107), (2, 1000, 36), (1, 20000, 8),
                                   (1, 70000, 128), (4, 5, 64), (2, 64, 4), (16, 257, 256), (32, 300, 256), (3, 700, 1100),
                                   (300, 961, 8), (70, 2000, 16), (5, 1, 8), (200, 1920, 4)])
@pytest.mark.parametrize("gates", ["randn", "nearunit"])
def test_channels_last_with_scratch(shape, gates):
    a, b, g = make_inputs(gates, shape, seed=29)
    an, bn, gn = a.numpy(), b.numpy(), g.numpy()
    h_ref = oracle.scan_forward_channels_last(an, bn)
    ga_ref, gb_ref = oracle.scan_backward_channels_last(an, h_ref, gn)
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    modes = [True, 12, 7, False]  # look-back: default tile and two other tile shapes; the library's own choice
    if a.dtype == torch.float32:
        modes.append("plain")
    if shape[2] in (4, 8, 16):
        modes.append("narrow")  # whole batch elements per CTA, untiled bulk copies
    if shape[2] % 4 == 0:
        modes += [32, 33, 34, 35, 36, 37]  # TMA-staged tiles, every tile shape of the table
        modes += [96]  # streaming kernels over chunks of T: chunk maps, carries, scan
        modes += list(range(64, 72))  # streaming kernels (a CTA walks all of T), every tile shape
    for scratch in modes:
        h = _gpu.cl_fwd(da, db, scratch=scratch)
        ga, gb = _gpu.cl_bwd(da, dh, dg, scratch=scratch)
        for got, ref, name in ((h, h_ref, "h"), (gb, gb_ref, "gb"), (ga, ga_ref, "ga")):
            assert _gpu.max_norm_err(got, ref) < TOL, (shape, gates, scratch, name, _gpu.max_norm_err(got, ref))
            if gates == "nearunit" or shape[1] <= 1000:
                assert _gpu.allclose_ref(got, ref), (shape, gates, scratch, name)
    _gpu.device_ok()


def test_channels_last_unaligned_view_with_scratch():
    a, b, g = make_inputs("sigmoid2", (2, 200, 64), seed=4)
    h_ref = oracle.scan_forward_channels_last(a.numpy(), b.numpy())

    def shifted(x):
        buf = torch.empty(x.numel() + 1, device="cuda")
        view = buf[1:].view(x.shape)
        view.copy_(x)
        return view

    h = _gpu.cl_fwd(shifted(a), shifted(b), scratch=True)
    assert _gpu.allclose_ref(h, h_ref)


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("gates", ["randn", "sigmoid2"])
def test_reference_shape_grid(shape, gates):
    a, b, g = make_inputs(gates, shape, seed=hash(shape) % 1000)
    T = shape[-1]
    a2, b2, g2 = (x.reshape(-1, T) for x in (a, b, g))
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a2, b2, g2)
    da, db, dg, dh = a2.cuda(), b2.cuda(), g2.cuda(), dev(h_ref)
    for variant in variants_for(T):
        h = _gpu.fwd(da, db, variant=variant)
        ga, gb = _gpu.bwd(da, dh, dg, variant=variant)
        assert _gpu.allclose_ref(h, h_ref), (variant, _gpu.max_norm_err(h, h_ref))
        assert _gpu.allclose_ref(gb, gb_ref), (variant, _gpu.max_norm_err(gb, gb_ref))
        assert _gpu.allclose_ref(ga, ga_ref), (variant, _gpu.max_norm_err(ga, ga_ref))
    _gpu.device_ok()


@pytest.mark.parametrize("shape", [(1000, 4), (77, 100), (13, 1028), (5, 5000), (3, 4092), (2, 8196), (300, 36),
                                   (7, 3), (1000, 1), (5, 2), (33, 4097), (3, 12289), (2, 100003), (9, 4091), (700, 37)])
def test_row_packing_shapes(shape):
    """T % 4 == 0 but not a divisor of the 4096-element span: whole rows are packed per span,
    long rows are walked in pieces with a ragged last piece."""
    a, b, g = make_inputs("randn", shape, seed=17)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    h_in = torch.randn(shape[0], device="cuda")
    c_in = torch.randn(shape[0], device="cuda")
    h_ref2 = oracle.scan_forward(a.numpy(), b.numpy(), h_in=h_in.cpu().numpy())
    ga_ref2, gb_ref2 = oracle.scan_backward(a.numpy(), h_ref, g.numpy(), gb_in=c_in.cpu().numpy(),
                                            h_prev=h_in.cpu().numpy())
    for variant in variants_for(shape[1]):
        h = _gpu.fwd(da, db, variant=variant)
        ga, gb = _gpu.bwd(da, dh, dg, variant=variant)
        assert _gpu.allclose_ref(h, h_ref), (variant, _gpu.max_norm_err(h, h_ref))
        assert _gpu.allclose_ref(gb, gb_ref) and _gpu.allclose_ref(ga, ga_ref), variant
        h2 = _gpu.fwd(da, db, h_in=h_in, variant=variant)
        assert _gpu.allclose_ref(h2, h_ref2), (variant, "carry-in")
        ga2, gb2 = _gpu.bwd(da, dh, dg, c_in=c_in, h_prev=h_in, variant=variant)
        assert _gpu.allclose_ref(gb2, gb_ref2) and _gpu.allclose_ref(ga2, ga_ref2), (variant, "bwd carries")
    _gpu.device_ok()


@pytest.mark.parametrize("shape", [(3, 7), (5, 64), (2, 1000), (9, 2049), (2, 4098)])
def test_fp64(shape):
    a, b, g = make_inputs("randn", shape, seed=7, dtype=torch.float64)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    h = _gpu.fwd(a.cuda(), b.cuda())
    ga, gb = _gpu.bwd(a.cuda(), dev(h_ref), g.cuda())
    for got, ref in ((h, h_ref), (ga, ga_ref), (gb, gb_ref)):
        assert _gpu.max_norm_err(got, ref) < 1e-12


def test_unaligned_base_pointers():
    """Views that start 4 bytes into an allocation: the 16-byte fast paths must not be taken."""
    a, b, g = make_inputs("sigmoid2", (8, 1028), seed=4)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)

    def shifted(x):
        buf = torch.empty(x.numel() + 1, device="cuda")
        view = buf[1:].view(x.shape)
        view.copy_(x)
        assert view.data_ptr() % 16 == 4
        return view

    da, db, dg, dh = shifted(a), shifted(b), shifted(g), shifted(torch.from_numpy(h_ref))
    h = _gpu.fwd(da, db)
    ga, gb = _gpu.bwd(da, dh, dg)
    assert _gpu.allclose_ref(h, h_ref) and _gpu.allclose_ref(ga, ga_ref) and _gpu.allclose_ref(gb, gb_ref)
    with pytest.raises(_native.NativeError) as err:
        _gpu.fwd(da, db, variant=TMA)
    assert err.value.status == _native.ERR_UNSUPPORTED


def test_edge_shapes_and_errors():
    one = torch.full((3, 1), 2.0, device="cuda")
    assert torch.equal(_gpu.fwd(one, one), one)
    ga, gb = _gpu.bwd(one, one, one)
    assert torch.equal(gb, one) and torch.equal(ga, torch.zeros_like(one))
    empty = torch.empty((4, 0), device="cuda")
    assert _gpu.fwd(empty, empty).shape == (4, 0)
    a = torch.rand(4, 100, device="cuda")
    with pytest.raises(_native.NativeError) as err:
        _gpu.fwd(a, a, variant=TMA)  # T % 32 != 0
    assert err.value.status == _native.ERR_UNSUPPORTED
    with pytest.raises(_native.NativeError):
        _gpu.fwd(a, a, variant=99)
    _gpu.device_ok()


@pytest.mark.parametrize("gates,shape", [("sigmoid2", (64, 4096)), ("resets", (40, 2048)), ("nearunit", (4, 65536))])
@pytest.mark.parametrize("variant", [WARP, TMA, FLAT, _gpu.flat_variant(2), _gpu.flat_variant(3), _gpu.tma_variant(32),
                                     _gpu.tma_variant(34), _gpu.tma_variant(10), _gpu.tma_variant(1)])
def test_shard_carries(gates, shape, variant):
    """A call with carry-in must continue a scan exactly where another call stopped."""
    a, b, g = make_inputs(gates, shape, seed=9)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    T = shape[1]
    cut = T // 2
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    left = [x[:, :cut].contiguous() for x in (da, db, dg, dh)]
    right = [x[:, cut:].contiguous() for x in (da, db, dg, dh)]
    try:
        h_l = _gpu.fwd(left[0], left[1], variant=variant)
    except _native.NativeError as e:  # the TMA flat sweep only takes rows that fit one span
        assert e.status == _native.ERR_UNSUPPORTED and (variant >> 8) >= 32
        pytest.skip("shape outside this variant's range")
    h_r = _gpu.fwd(right[0], right[1], h_in=h_l[:, -1].contiguous(), variant=variant)
    assert _gpu.max_norm_err(torch.cat([h_l, h_r], 1), h_ref) < TOL
    ga_r, gb_r = _gpu.bwd(right[0], right[3], right[2], h_prev=left[3][:, -1].contiguous(), variant=variant)
    c_in = (right[0][:, 0] * gb_r[:, 0]).contiguous()
    ga_l, gb_l = _gpu.bwd(left[0], left[3], left[2], c_in=c_in, variant=variant)
    assert _gpu.max_norm_err(torch.cat([gb_l, gb_r], 1), gb_ref) < TOL
    assert _gpu.max_norm_err(torch.cat([ga_l, ga_r], 1), ga_ref) < TOL
    _gpu.device_ok()


@pytest.mark.parametrize("n_shards", [2, 8])
def test_virtual_t_shards_on_one_gpu(n_shards):
    """reduce -> (gather) -> carry -> scan-with-carry, all shards on one device, vs. unsharded."""
    lib = _native.load()
    rows, T = 48, 4096 * n_shards
    a, b, g = make_inputs("nearunit", (rows, T), seed=12)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    step = T // n_shards
    parts = [[x[:, s * step:(s + 1) * step].contiguous() for x in (da, db, dg, dh)] for s in range(n_shards)]
    st = _native.stream_of(da)
    fmaps = torch.empty(n_shards, rows, 2, device="cuda")
    bmaps = torch.empty(n_shards, rows, 2, device="cuda")
    for s, (pa, pb, pg, _) in enumerate(parts):
        ws_bytes = lib.ssb_shard_reduce_workspace_bytes(rows, step) if s % 2 == 0 else 0  # both code paths
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
        _native.check(lib.ssb_shard_reduce_fwd_f32(pa.data_ptr(), pb.data_ptr(), fmaps[s].data_ptr(), rows, step,
                                                   ws.data_ptr() if ws_bytes else None, ws_bytes, st))
        _native.check(lib.ssb_shard_reduce_bwd_f32(pa.data_ptr(), pg.data_ptr(), bmaps[s].data_ptr(), rows, step,
                                                   ws.data_ptr() if ws_bytes else None, ws_bytes, st))
    hs, gas, gbs = [], [], []
    for s, (pa, pb, pg, ph) in enumerate(parts):
        h_in = torch.empty(rows, device="cuda")
        c_in = torch.empty(rows, device="cuda")
        _native.check(lib.ssb_shard_carry_f32(fmaps.data_ptr(), n_shards, s, 0, rows, h_in.data_ptr(), st))
        _native.check(lib.ssb_shard_carry_f32(bmaps.data_ptr(), n_shards, s, 1, rows, c_in.data_ptr(), st))
        hs.append(_gpu.fwd(pa, pb, h_in=h_in))
        ga, gb = _gpu.bwd(pa, ph, pg, c_in=c_in, h_prev=h_in)
        gas.append(ga)
        gbs.append(gb)
    assert _gpu.max_norm_err(torch.cat(hs, 1), h_ref) < TOL
    assert _gpu.max_norm_err(torch.cat(gbs, 1), gb_ref) < TOL
    assert _gpu.max_norm_err(torch.cat(gas, 1), ga_ref) < TOL
    # the maps themselves: A is the product of the shard's gates, B its zero-started end value
    A_ref = a[:, :step].double().prod(dim=1)
    np.testing.assert_allclose(fmaps[0, :, 0].cpu().double().numpy(), A_ref.numpy(), rtol=1e-4)
    np.testing.assert_allclose(fmaps[0, :, 1].cpu().numpy(), h_ref[:, step - 1], rtol=1e-5, atol=1e-6)
    _gpu.device_ok()


@pytest.mark.parametrize("gates", ["nearunit", "sigmoid2", "randn", "ones", "resets"])
@pytest.mark.parametrize("shape", [(48, 40960), (3, 2048), (200, 6148), (5, 4098)])
def test_shard_maps_with_early_termination(gates, shape):
    """ssb_shard_map_*: cut = 0 (and cut < 0) equals the full reduction; cut = 2^-40 stays within
    the cut's bound, walks only as far as the gate product needs, and walks everything when the
    product never vanishes.  (5, 4098): T % 4 != 0, the fallback that always reads the whole shard."""
    lib = _native.load()
    rows, T = shape
    a, b, g = make_inputs(gates, shape, seed=31)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    st = _native.stream_of(da)
    full = torch.empty(2, rows, 2, device="cuda")
    _native.check(lib.ssb_shard_reduce_fwd_f32(da.data_ptr(), db.data_ptr(), full[0].data_ptr(), rows, T, None, 0, st))
    _native.check(lib.ssb_shard_reduce_bwd_f32(da.data_ptr(), dg.data_ptr(), full[1].data_ptr(), rows, T, None, 0, st))
    full = full.cpu().double().numpy()
    an = a.double().numpy()
    h_ref = oracle.scan_forward(a.numpy(), b.numpy())
    _, gb_ref = oracle.scan_backward(a.numpy(), h_ref, g.numpy())
    finite = np.isfinite(full).all(axis=(0, 2)) & np.isfinite(h_ref).all(axis=1) & np.isfinite(gb_ref).all(axis=1)
    scale = [max(float(np.abs(h_ref[finite]).max()), 1e-30),
             max(float(np.abs(gb_ref[finite]).max() * max(np.abs(an).max(), 1.0)), 1e-30)]
    for cut in (-1.0, 0.0, 2.0 ** -40):
        got = torch.empty(2, rows, 2, device="cuda")
        walked = torch.zeros(2, dtype=torch.int64, device="cuda")
        _native.check(lib.ssb_shard_map_fwd_f32(da.data_ptr(), db.data_ptr(), got[0].data_ptr(), rows, T, cut,
                                                walked[0:].data_ptr(), st))
        _native.check(lib.ssb_shard_map_bwd_f32(da.data_ptr(), dg.data_ptr(), got[1].data_ptr(), rows, T, cut,
                                                walked[1:].data_ptr(), st))
        got, walked = got.cpu().double().numpy(), walked.cpu().numpy()
        for d in range(2):
            err = np.abs(got[d, finite, 1] - full[d, finite, 1]).max(initial=0.0) / scale[d]
            assert err <= 2 * max(cut, 0.0) + 1e-5, (d, cut, err)
            assert (np.abs(got[d, finite, 0]) <= np.maximum(np.abs(full[d, finite, 0]) * 1.01 + 1e-37, max(cut, 0.0))).all()
        assert (walked <= rows * T).all() and (walked > 0).all()
        if cut < 0 or gates == "ones" or T % 4 != 0:
            assert (walked == rows * T).all()  # no early stop: the whole shard is read
        elif gates == "nearunit" and T >= 40960:
            # 0.995^t reaches 2^-40 after ~5.5 K steps and zero after ~20.6 K (2048-element chunks)
            limit = 8192 if cut > 0 else 24576
            assert (walked <= rows * limit).all(), (cut, walked)
        elif gates in ("sigmoid2", "resets") and T >= 6148:
            assert (walked <= rows * 4096).all(), (cut, walked)
    _gpu.device_ok()


@pytest.mark.parametrize("gates,n_shards,cut", [("nearunit", 4, 2.0 ** -40), ("nearunit", 2, 0.0), ("randn", 4, 2.0 ** -40),
                                                ("ones", 2, 2.0 ** -40), ("sigmoid2", 8, 2.0 ** -40)])
def test_virtual_t_shards_through_the_sharded_module(gates, n_shards, cut):
    """scanscam_b200.sharded's own steps (map -> gather -> carry -> scan) with the CUDA ops, the
    gather replaced by stacking the shards' maps on one device; result vs. the unsharded oracle."""
    from scanscam_b200 import sharded

    ops = sharded.CudaShardOps
    rows, step = 40, 24576 if gates == "nearunit" else 4096
    T = step * n_shards
    a, b, g = make_inputs(gates, (rows, T), seed=5)
    if gates == "ones":
        b, g = b * 0.01, g * 0.01  # keep the running sums small against fp32 cancellation
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    parts = [[x[:, s * step:(s + 1) * step].contiguous() for x in (da, db, dg)] for s in range(n_shards)]
    fmaps = torch.stack([ops.map_forward(pa, pb, cut) for pa, pb, _ in parts])
    bmaps = torch.stack([ops.map_backward(pa, pg, cut) for pa, _, pg in parts])
    hs, gas, gbs = [], [], []
    for s, (pa, pb, pg) in enumerate(parts):
        h_in, c_in = ops.carry(fmaps, s, False), ops.carry(bmaps, s, True)
        h = ops.scan_forward(pa, pb, h_in)
        ga, gb = ops.scan_backward(pa, h, pg, c_in, h_in)
        hs.append(h), gas.append(ga), gbs.append(gb)
    assert _gpu.max_norm_err(torch.cat(hs, 1), h_ref) < TOL
    assert _gpu.max_norm_err(torch.cat(gbs, 1), gb_ref) < TOL
    assert _gpu.max_norm_err(torch.cat(gas, 1), ga_ref) < TOL
    _gpu.device_ok()


@pytest.mark.parametrize("world,rows,step", [(4, 40, 8192), (8, 700, 2048), (2, 257, 4096)])
def test_peer_exchange_emulated_on_one_gpu(world, rows, step):
    """ssb_shard_map_publish_f32 / ssb_shard_carry_peer_f32 with `world` "ranks" that are buffers on
    ONE device: every rank's publish is launched before any rank's carry, so no kernel ever waits for
    a later launch (the flags it polls are already up).  Three epochs in a row exercise both slot
    generations and the reuse of a slot; carries are compared with ssb_shard_carry_f32 on the maps
    of the collective path.  The largest supported world (8) and row counts that need several CTAs
    of the carry kernel are among the cases."""
    lib = _native.load()
    a, b, g = make_inputs("nearunit", (rows, step * world), seed=17)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    nbytes = lib.ssb_peer_exchange_bytes(world, rows)
    assert nbytes > 0 and lib.ssb_peer_exchange_bytes(9, rows) == 0
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    structs = []
    for r in range(world):
        ex = _native.PeerExchangeStruct()
        ex.world, ex.rank, ex.rows = world, r, rows
        for q in range(world):
            ex.buffers[q] = bufs[q].data_ptr()
        structs.append(ex)
    st = _native.stream_of(da)
    cut = 2.0 ** -40
    for epoch in (1, 2, 3):
        scale = float(epoch)  # different data every epoch: a stale slot would show
        parts = [[(x[:, r * step:(r + 1) * step] * (scale if i else 1.0)).contiguous() for i, x in enumerate((da, db, dg))]
                 for r in range(world)]
        for backward in (0, 1):
            ref_maps = torch.empty(world, rows, 2, device="cuda")
            for r, (pa, pb, pg) in enumerate(parts):
                other = pg if backward else pb
                fn = lib.ssb_shard_map_bwd_f32 if backward else lib.ssb_shard_map_fwd_f32
                _native.check(fn(pa.data_ptr(), other.data_ptr(), ref_maps[r].data_ptr(), rows, step, cut, None, st))
                _native.check(lib.ssb_shard_map_publish_f32(pa.data_ptr(), other.data_ptr(), rows, step, cut, backward,
                                                            _native.ctypes.byref(structs[r]), epoch, None, st))
            for r in range(world):
                got, want = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
                _native.check(lib.ssb_shard_carry_peer_f32(_native.ctypes.byref(structs[r]), epoch, backward, got.data_ptr(), st))
                _native.check(lib.ssb_shard_carry_f32(ref_maps.data_ptr(), world, r, backward, rows, want.data_ptr(), st))
                assert torch.equal(got, want), (epoch, backward, r, float((got - want).abs().max()))
    # refusals: a shape the publishing kernel does not take, a descriptor that makes no sense
    odd = torch.rand(rows, 1001, device="cuda")
    assert lib.ssb_shard_map_publish_f32(odd.data_ptr(), odd.data_ptr(), rows, 1001, cut, 0, _native.ctypes.byref(structs[0]), 4,
                                         None, st) == _native.ERR_UNSUPPORTED
    bad = _native.PeerExchangeStruct()
    bad.world, bad.rank, bad.rows = world, world + 3, rows
    assert lib.ssb_shard_carry_peer_f32(_native.ctypes.byref(bad), 1, 0, odd.data_ptr(), st) == _native.ERR_BAD_ARG
    _gpu.device_ok()


def test_channels_last_stream_tile_choice():
    """ssb_scan_cl_recommend on a 148-SM part: the streaming tile shape follows the rounds estimate, per
    direction (units of 32 channels just above a multiple of the SM count keep 32-channel blocks; where
    halving the units halves the rounds, 64-channel blocks; the backward's 256-step tiles from 149
    units up)."""
    lib = _native.load()
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the expected choices are those of a 148-SM GPU")
    S = _native.CL_STREAM
    expect = {(8, 4096, 512): (0, 0), (12, 4096, 512): (2, 1), (16, 4096, 512): (1, 1), (20, 4096, 512): (0, 2),
              (24, 4096, 512): (0, 2), (32, 4096, 512): (1, 1), (64, 4096, 512): (1, 2)}
    for shape, (fwd_id, bwd_id) in expect.items():
        assert lib.ssb_scan_cl_recommend(*shape, 0, 1, 1) == S | (fwd_id << 8), shape
        assert lib.ssb_scan_cl_recommend(*shape, 1, 1, 1) == S | (bwd_id << 8), shape
        assert lib.ssb_scan_cl_variant_workspace_bytes(*shape, S | (fwd_id << 8), 0) == 0


def test_cfg3_full_size_under_auto_sampled():
    """cfg3 as configured -- [1024, 2^20], near-unit gates, the kernels AUTO picks at that size --
    at full size on the GPU; a strided sample of 16 rows against the oracle, the backward fed with
    the oracle's h (isolates it) and with the kernel's own h (end to end)."""
    w = WORKLOADS["cfg3"]
    rows, T = w.rows, w.steps
    gen = torch.Generator(device="cuda").manual_seed(0)
    da = torch.rand(rows, T, generator=gen, device="cuda").mul_(0.01).add_(0.99)
    db = torch.randn(rows, T, generator=gen, device="cuda").mul_(0.1)
    dg = torch.randn(rows, T, generator=gen, device="cuda")
    lib = _native.load()
    v_f, v_b = lib.ssb_scan_recommend(rows, T, 0, 1, 1), lib.ssb_scan_recommend(rows, T, 1, 1, 1)
    h = _gpu.fwd(da, db, variant=v_f)
    ga, gb = _gpu.bwd(da, h, dg, variant=v_b)
    idx = torch.arange(5, rows, 64, device="cuda")  # 16 rows
    assert idx.numel() == 16
    sa, sb, sg = (x[idx].contiguous() for x in (da, db, dg))
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(sa.cpu(), sb.cpu(), sg.cpu())
    assert _gpu.max_norm_err(h[idx], h_ref) < TOL
    assert _gpu.max_norm_err(gb[idx], gb_ref) < TOL and _gpu.max_norm_err(ga[idx], ga_ref) < TOL
    del ga, gb
    dh = torch.empty_like(h)
    dh.copy_(h)
    dh[idx] = dev(h_ref)  # the sampled rows get the oracle's h
    del h
    ga2, gb2 = _gpu.bwd(da, dh, dg, variant=v_b)
    assert _gpu.max_norm_err(gb2[idx], gb_ref) < TOL and _gpu.max_norm_err(ga2[idx], ga_ref) < TOL
    _gpu.device_ok()


def test_auto_uses_the_callers_workspace_when_it_is_large_enough():
    """SSB_VARIANT_AUTO through the _ex entry points: with a workspace of the size
    ssb_scan_workspace_bytes reports for the recommended variant, a few very long rows run the
    kernels that split a row across CTAs (they write their records / chunk maps to the workspace);
    with a workspace that is too small the call falls back to the no-scratch choice and leaves it
    untouched.  Results are the oracle's either way."""
    lib = _native.load()
    rows, T = 16, 1 << 20
    a, b, g = make_inputs("nearunit", (rows, T), seed=41)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    for backward in (0, 1):
        variant = lib.ssb_scan_recommend(rows, T, backward, 1, 1)
        assert (variant & 0xff) == LOOKBACK
        need = lib.ssb_scan_workspace_bytes(rows, T, variant)
        assert need > 0
        for nbytes in (need, 4096):
            ws = torch.full((nbytes,), 0xAB, dtype=torch.uint8, device="cuda")
            if backward:
                ga, gb = _gpu.bwd(da, dh, dg, variant=AUTO, workspace=(ws, nbytes))
                assert _gpu.max_norm_err(gb, gb_ref) < TOL and _gpu.max_norm_err(ga, ga_ref) < TOL
            else:
                assert _gpu.max_norm_err(_gpu.fwd(da, db, variant=AUTO, workspace=(ws, nbytes)), h_ref) < TOL
            touched = bool((ws != 0xAB).any().item())
            assert touched == (nbytes == need), (backward, nbytes, touched)
    _gpu.device_ok()


# ---- long rows: spans of one row on different CTAs, carries by decoupled look-back ----------
LONG_SHAPES = [(3, 8192), (1, 1048576), (5, 40000), (64, 16384), (700, 8196), (2, 4100), (17, 262144), (6, 1048576)]


@pytest.mark.parametrize("shape", LONG_SHAPES)
@pytest.mark.parametrize("gates", ["nearunit", "randn", "resets"])
def test_lookback_long_rows(shape, gates):
    rows, T = shape
    a, b, g = make_inputs(gates, shape, seed=23)
    carry = torch.randn(rows) * 0.5
    an, bn, gn, cn = a.numpy(), b.numpy(), g.numpy(), carry.numpy()
    h_ref = oracle.scan_forward(an, bn, h_in=cn)
    ga_ref, gb_ref = oracle.scan_backward(an, h_ref, gn, gb_in=cn, h_prev=cn)
    da, db, dg, dh, dc = a.cuda(), b.cuda(), g.cuda(), dev(h_ref), carry.cuda()
    lib = _native.load()
    ran = 0
    for tuning in list(range(7)) + [16, 17]:  # 16, 17: the chunked forms (no look-back): 4096-step chunks; long chunks with early-terminated maps
        variant = _gpu.lookback_variant(tuning)
        if lib.ssb_scan_workspace_bytes(rows, T, variant) == 0:
            continue
        ws = _gpu.workspace_for(rows, T, variant)
        if ws[0] is not None:
            ws[0].fill_(0xAB)  # stale contents must not matter
        try:
            h = _gpu.fwd(da, db, h_in=dc, variant=variant, workspace=ws)
        except _native.NativeError as e:  # row not longer than this tuning's span
            assert e.status == _native.ERR_UNSUPPORTED
            continue
        ga, gb = _gpu.bwd(da, dh, dg, c_in=dc, h_prev=dc, variant=variant, workspace=ws)
        ran += 1
        for got, ref, name in ((h, h_ref, "h"), (gb, gb_ref, "gb"), (ga, ga_ref, "ga")):
            err = _gpu.max_norm_err(got, ref)
            assert err < TOL, (shape, gates, tuning, name, err)
        if gates != "randn":  # randn gates swing over many orders of magnitude; max-norm is the fair metric there
            assert _gpu.allclose_ref(h, h_ref) and _gpu.allclose_ref(gb, gb_ref)
    assert ran >= 3
    if T % 4096 == 0 and T >= 8192:  # the flat sweep that walks a row span by span, same carries
        variant = _gpu.tma_variant(48)
        h = _gpu.fwd(da, db, h_in=dc, variant=variant)
        ga, gb = _gpu.bwd(da, dh, dg, c_in=dc, h_prev=dc, variant=variant)
        for got, ref, name in ((h, h_ref, "h"), (gb, gb_ref, "gb"), (ga, ga_ref, "ga")):
            assert _gpu.max_norm_err(got, ref) < TOL, (shape, gates, "tma48", name)
    _gpu.device_ok()


def test_lookback_workspace_contract():
    lib = _native.load()
    a = torch.rand(4, 16384, device="cuda")
    v = _gpu.lookback_variant(0)
    need = lib.ssb_scan_workspace_bytes(4, 16384, v)
    assert need == 256 + 4 * 4 * 16          # header + rows * pieces(4096-element spans) * 16-byte records
    assert lib.ssb_scan_workspace_bytes(4, 16384, WARP) == 0
    with pytest.raises(_native.NativeError) as err:
        _gpu.fwd(a, a, variant=v, workspace=(None, 0))
    assert err.value.status == _native.ERR_WORKSPACE
    small = torch.empty(need - 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(_native.NativeError) as err:
        _gpu.fwd(a, a, variant=v, workspace=(small, need - 16))
    assert err.value.status == _native.ERR_WORKSPACE
    short = torch.rand(4, 1024, device="cuda")
    with pytest.raises(_native.NativeError) as err:
        _gpu.fwd(short, short, variant=v, workspace=(torch.empty(4096, dtype=torch.uint8, device="cuda"), 4096))
    assert err.value.status == _native.ERR_UNSUPPORTED
    # the recommendation: look-back only for long rows and only when the caller can supply scratch
    assert lib.ssb_scan_recommend(64, 65536, 0, 1, 1) == LOOKBACK | (17 << 8)   # few long rows: long chunks, early-terminated maps
    assert lib.ssb_scan_recommend(256, 65536, 1, 1, 1) == LOOKBACK | (17 << 8)
    assert lib.ssb_scan_recommend(300, 65536, 0, 1, 1) == LOOKBACK              # from there on look-back keeps up
    assert lib.ssb_scan_recommend(2048, 65536, 0, 1, 1) == TMA | (48 << 8)        # many long rows of whole spans
    assert lib.ssb_scan_recommend(1024, 65536, 1, 1, 0) == TMA | (48 << 8)
    assert lib.ssb_scan_recommend(1024, 65536, 0, 1, 1) == TMA | (10 << 8)        # the forward only from 2048 rows: per-warp ring below
    assert lib.ssb_scan_recommend(1024, 32768, 0, 1, 1) == LOOKBACK
    assert lib.ssb_scan_recommend(64, 65540, 0, 1, 1) == LOOKBACK               # T not a multiple of 4096
    assert lib.ssb_scan_recommend(64, 65536, 0, 1, 0) & 0xff == FLAT
    assert lib.ssb_scan_recommend(4096, 4096, 0, 1, 1) & 0xff == TMA      # power-of-two rows that fit a span
    assert lib.ssb_scan_recommend(64, 4096, 0, 1, 1) == TMA | (32 << 8)   # ... also when the whole problem is a few spans per SM
    assert lib.ssb_scan_recommend(1024, 1024, 0, 1, 1) == TMA | (34 << 8)  # small problems, power-of-two rows up to 2048 steps: 64-line spans
    assert lib.ssb_scan_recommend(1024, 1024, 1, 1, 0) == TMA | (34 << 8)
    assert lib.ssb_scan_recommend(64, 4092, 0, 1, 1) == FLAT | (12 << 8)   # small problems, other row lengths: 512-element spans
    assert lib.ssb_scan_recommend(64, 4092, 0, 1, 1) & 0xff == FLAT
    assert lib.ssb_scan_recommend(64, 4097, 1, 1, 1) & 0xff in (WARP, FLAT_ANY)
    assert lib.ssb_scan_recommend(64, 65536, 1, 0, 1) & 0xff == WARP
    _gpu.device_ok()


def test_shard_reduce_with_and_without_workspace():
    lib = _native.load()
    rows, T = 9, 70000
    _, b, g = make_inputs("nearunit", (rows, T), seed=3)
    a = 1.0 - 1e-5 * torch.rand(rows, T, generator=torch.Generator().manual_seed(3))  # product stays ~0.7
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    st = _native.stream_of(da)
    need = lib.ssb_shard_reduce_workspace_bytes(rows, T)
    assert need > 0 and lib.ssb_shard_reduce_workspace_bytes(rows, 1024) == 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = torch.empty(4, rows, 2, device="cuda")
    _native.check(lib.ssb_shard_reduce_fwd_f32(da.data_ptr(), db.data_ptr(), out[0].data_ptr(), rows, T, None, 0, st))
    _native.check(lib.ssb_shard_reduce_fwd_f32(da.data_ptr(), db.data_ptr(), out[1].data_ptr(), rows, T, ws.data_ptr(), need, st))
    _native.check(lib.ssb_shard_reduce_bwd_f32(da.data_ptr(), dg.data_ptr(), out[2].data_ptr(), rows, T, None, 0, st))
    _native.check(lib.ssb_shard_reduce_bwd_f32(da.data_ptr(), dg.data_ptr(), out[3].data_ptr(), rows, T, ws.data_ptr(), need, st))
    o = out.cpu().double().numpy()
    h_ref = oracle.scan_forward(a.double().numpy(), b.double().numpy())
    A_ref = a.double().prod(dim=1).numpy()
    for k in (0, 1):
        np.testing.assert_allclose(o[k][:, 0], A_ref, rtol=1e-3)
        np.testing.assert_allclose(o[k][:, 1], h_ref[:, -1], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(o[2], o[3], rtol=1e-4, atol=1e-5)
    _gpu.device_ok()


# ---- benchmark configurations ------------------------------------------------------------
@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg5"])
def test_benchmark_configs_against_oracle(name):
    """Full-size parity: cfg1 (the CPU-runnable case), cfg2 (headline), cfg5 (exact-zero gates)."""
    w = WORKLOADS[name]
    a, b, g = (x.reshape(w.rows, w.steps) for x in workload_inputs(name))
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    for variant in (AUTO, WARP, TMA, FLAT):
        h = _gpu.fwd(da, db, variant=variant)
        assert _gpu.max_norm_err(h, h_ref) < TOL
        ga, gb = _gpu.bwd(da, dev(h_ref), dg, variant=variant)       # isolates the backward
        assert _gpu.max_norm_err(gb, gb_ref) < TOL and _gpu.max_norm_err(ga, ga_ref) < TOL
        ga2, gb2 = _gpu.bwd(da, h, dg, variant=variant)              # end to end, kernel's own h
        assert _gpu.max_norm_err(ga2, ga_ref) < TOL
        del h, ga, gb, ga2, gb2
    _gpu.device_ok()


def test_cfg4_wide_short_rows_sampled():
    """cfg4 at full size on the GPU; the oracle checks a strided sample of rows."""
    w = WORKLOADS["cfg4"]
    a, b, g = (x.reshape(w.rows, w.steps) for x in workload_inputs("cfg4"))
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    h = _gpu.fwd(da, db)
    ga, gb = _gpu.bwd(da, h, dg)
    idx = torch.arange(0, w.rows, 37)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a[idx].contiguous(), b[idx].contiguous(), g[idx].contiguous())
    assert _gpu.max_norm_err(h[idx.cuda()], h_ref) < TOL
    assert _gpu.max_norm_err(gb[idx.cuda()], gb_ref) < TOL and _gpu.max_norm_err(ga[idx.cuda()], ga_ref) < TOL
    _gpu.device_ok()


def test_cfg3_long_context_properties():
    """cfg3's sequence length (2**20) and gate distribution on a slice of its rows: oracle parity
    on those rows, plus two size-independent properties -- linearity in the value input and
    agreement between the T-sharded composition and the single call."""
    T = WORKLOADS["cfg3"].steps
    rows = 16
    a, b, g = make_inputs("nearunit", (rows, T), seed=0)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    for variant in (TMA, WARP, FLAT, _gpu.flat_variant(3)):
        h = _gpu.fwd(da, db, variant=variant)
        ga, gb = _gpu.bwd(da, dev(h_ref), dg, variant=variant)
        assert _gpu.max_norm_err(h, h_ref) < TOL
        assert _gpu.max_norm_err(gb, gb_ref) < TOL and _gpu.max_norm_err(ga, ga_ref) < TOL
    # linearity: scan(a, b + 2*g) == scan(a, b) + 2*scan(a, g)
    lhs = _gpu.fwd(da, (db + 2 * dg).contiguous())
    rhs = _gpu.fwd(da, db) + 2 * _gpu.fwd(da, dg)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) < 1e-5
    _gpu.device_ok()


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Failure detection without a fault: a look-back poll on a record nobody publishes gives up
    after its limit (~1 s), the kernel returns, the host reads the status, later launches work."""
    import ctypes
    import time

    lib = _native.load()
    _gpu.device_ok()
    scratch = torch.empty(64, dtype=torch.uint8, device="cuda")
    t0 = time.perf_counter()
    _native.check(lib.ssb_selftest_wait_timeout(scratch.data_ptr(), 64, _native.stream_of(scratch)))
    detail = ctypes.c_int(0)
    rc = lib.ssb_device_status(ctypes.byref(detail))
    waited = time.perf_counter() - t0
    assert rc == _native.ERR_DEVICE_WAIT and detail.value == 3
    assert 0.5 < waited < 10.0
    assert lib.ssb_device_status(ctypes.byref(detail)) == _native.OK   # reported once, then cleared
    a, b, _ = make_inputs("sigmoid2", (8, 8192), seed=1)
    h = _gpu.fwd(a.cuda(), b.cuda(), variant=LOOKBACK)
    assert _gpu.allclose_ref(h, oracle.scan_forward(a.numpy(), b.numpy()))
    _gpu.device_ok()


@pytest.mark.parametrize("shape", [(40, 4096), (130, 2048), (77, 256), (300, 32), (9, 8192), (50, 24)])
def test_fused_sigmoid_entry_points_with_carries(shape):
    """ssb_scan_sigmoid_{fwd,bwd}_f32 (logits in, gradient w.r.t. logits out) with a carry entering
    every row from both sides, against the oracle fed sigmoid(z) computed on the host.  The shapes
    cover both kernel families behind the entry points."""
    rows, T = shape
    z, b, g = make_inputs("randn", shape, seed=71)
    z = z * 2 + 1.0
    a = torch.sigmoid(z)
    carry = torch.randn(rows)
    h_ref = oracle.scan_forward(a.numpy(), b.numpy(), h_in=carry.numpy())
    ga_ref, gb_ref = oracle.scan_backward(a.numpy(), h_ref, g.numpy(), gb_in=carry.numpy(), h_prev=carry.numpy())
    gz_ref = ga_ref * (a * (1 - a)).numpy()
    lib = _native.load()
    dz, db, dg, dc = z.cuda(), b.cuda(), g.cuda(), carry.cuda()
    h, gz, gb = torch.empty_like(dz), torch.empty_like(dz), torch.empty_like(dz)
    st = _native.stream_of(dz)
    _native.check(lib.ssb_scan_sigmoid_fwd_f32(dz.data_ptr(), db.data_ptr(), h.data_ptr(), rows, T, dc.data_ptr(), st))
    _native.check(lib.ssb_scan_sigmoid_bwd_f32(dz.data_ptr(), h.data_ptr(), dg.data_ptr(), gz.data_ptr(), gb.data_ptr(),
                                               rows, T, dc.data_ptr(), dc.data_ptr(), st))
    _gpu.device_ok()
    assert _gpu.max_norm_err(h, h_ref) < 1e-4
    assert _gpu.max_norm_err(gb, gb_ref) < 1e-4
    assert _gpu.max_norm_err(gz, gz_ref) < 1e-4


def test_tensor_map_paths_work_from_a_fresh_thread():
    """A thread that has made no CUDA runtime call of its own (an autograd worker, say) reaches the
    bulk-tensor kernels with every host-side lookup already cached; the tensor maps must still
    encode there."""
    import threading
    a, b, g = make_inputs("sigmoid2", (48, 4096), seed=81)
    h_ref, ga_ref, gb_ref = _gpu.oracle_all(a, b, g)
    da, db, dg = a.cuda(), b.cuda(), g.cuda()
    for variant in (AUTO, _gpu.tma_variant(0)):
        _gpu.fwd(da, db, variant=variant)  # warm every cache on this thread
        _gpu.bwd(da, _gpu.fwd(da, db), dg, variant=variant)
    torch.cuda.synchronize()
    results, errors = {}, []

    def work():
        try:
            for variant in (AUTO, _gpu.tma_variant(0)):
                h = _gpu.fwd(da, db, variant=variant)
                results[variant] = (h,) + _gpu.bwd(da, h, dg, variant=variant)
        except Exception as exc:  # noqa: BLE001 - reported by the assertion below
            errors.append(exc)

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    for h, ga, gb in results.values():
        assert _gpu.allclose_ref(h, h_ref) and _gpu.allclose_ref(ga, ga_ref) and _gpu.allclose_ref(gb, gb_ref)


@pytest.mark.parametrize("gates,shape", [("sigmoid2", (40, 4096)), ("resets", (130, 2048)), ("randn", (77, 256)),
                                         ("sigmoid2", (300, 32)), ("sigmoid0", (1000, 512)), ("nearunit", (3, 70000)),
                                         ("sigmoid2", (9, 8192)), ("resets", (50, 24)), ("sigmoid2", (7, 1001))])
def test_recompute_backward_matches_oracle(gates, shape):
    """ssb_scan_bwd_recompute_f32 takes (a, b, g) and rebuilds h itself: in one kernel for rows of
    32 * 2^k <= 4096 steps, through the forward kernel and a workspace otherwise.  Carries enter
    every row from both sides."""
    rows, T = shape
    a, b, g = make_inputs(gates, shape, seed=91)
    carry = torch.randn(rows)
    h_ref = oracle.scan_forward(a.numpy(), b.numpy(), h_in=carry.numpy())
    ga_ref, gb_ref = oracle.scan_backward(a.numpy(), h_ref, g.numpy(), gb_in=carry.numpy(), h_prev=carry.numpy())
    lib = _native.load()
    da, db, dg, dc = a.cuda(), b.cuda(), g.cuda(), carry.cuda()
    ga, gb = torch.empty_like(da), torch.empty_like(da)
    need = lib.ssb_scan_bwd_recompute_workspace_bytes(rows, T)
    in_kernel = T % 32 == 0 and T <= 4096 and (T // 32) & (T // 32 - 1) == 0
    assert (need == 0) == in_kernel
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    st = _native.stream_of(da)
    if need:
        rc = lib.ssb_scan_bwd_recompute_f32(da.data_ptr(), db.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                            rows, T, dc.data_ptr(), dc.data_ptr(), None, 0, st)
        assert rc == _native.ERR_WORKSPACE
    _native.check(lib.ssb_scan_bwd_recompute_f32(da.data_ptr(), db.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                 rows, T, dc.data_ptr(), dc.data_ptr(), ws.data_ptr(), need, st))
    _gpu.device_ok()
    assert _gpu.max_norm_err(ga, ga_ref) < TOL and _gpu.max_norm_err(gb, gb_ref) < TOL
    if gates != "randn":  # gates above 1 in magnitude grow the values beyond an absolute tolerance
        assert _gpu.allclose_ref(ga, ga_ref) and _gpu.allclose_ref(gb, gb_ref)


H16 = {"bf16": (torch.bfloat16, 2.0 ** -8), "f16": (torch.float16, 2.0 ** -11)}


@pytest.mark.parametrize("name", ["bf16", "f16"])
@pytest.mark.parametrize("gates,shape", [("sigmoid2", (40, 4096)), ("resets", (130, 2048)), ("sigmoid0", (77, 256)),
                                         ("sigmoid2", (300, 64)), ("sigmoid2", (5, 8192)), ("nearunit", (3, 70000)),
                                         ("sigmoid2", (9, 8000)), ("resets", (50, 24)), ("sigmoid2", (7, 1001)),
                                         ("sigmoid0", (33, 30)), ("sigmoid2", (37, 16384)), ("nearunit", (3, 65536)),
                                         ("resets", (200, 12288))])
def test_16bit_storage_matches_oracle(name, gates, shape):
    """ssb_scan_{fwd,bwd}_{bf16,f16}: 16-bit tensors, fp32 arithmetic and fp32 carries.  The oracle
    runs in fp32 on the same rounded inputs; every kernel output must be that result rounded once:
    within half a unit in the last place of the storage type (plus the fp32 reassociation noise,
    which can flip a rounding on a few elements, so one full unit is allowed on those)."""
    dtype, half_ulp = H16[name]
    rows, T = shape
    a, b, g = (x.to(dtype) for x in make_inputs(gates, shape, seed=101))
    carry = torch.randn(rows)
    an, bn, gn, cn = a.float().numpy(), b.float().numpy(), g.float().numpy(), carry.numpy()
    h_ref = oracle.scan_forward(an, bn, h_in=cn)
    h16 = torch.from_numpy(h_ref).to(dtype)  # what a forward in this storage type hands to the backward
    ga_ref, gb_ref = oracle.scan_backward(an, h16.float().numpy(), gn, gb_in=cn, h_prev=cn)
    lib = _native.load()
    fwd_fn, bwd_fn = getattr(lib, f"ssb_scan_fwd_{name}"), getattr(lib, f"ssb_scan_bwd_{name}")
    da, db, dg, dh, dc = a.cuda(), b.cuda(), g.cuda(), h16.cuda(), carry.cuda()
    h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
    st = _native.stream_of(da)
    _native.check(fwd_fn(da.data_ptr(), db.data_ptr(), h.data_ptr(), rows, T, dc.data_ptr(), st))
    _native.check(bwd_fn(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T,
                         dc.data_ptr(), dc.data_ptr(), st))
    _gpu.device_ok()
    for x, ref in ((h, h_ref), (ga, ga_ref), (gb, gb_ref)):
        got = x.float().cpu().numpy().astype(np.float64)
        err = np.abs(got - ref)
        unit = 2.0 * half_ulp * np.maximum(np.abs(ref), 1e-30)  # >= one unit in the last place of the result
        assert _gpu.max_norm_err(x.float(), ref) < 1.01 * half_ulp
        assert (err <= 1.001 * unit + 1e-6 * np.abs(ref).max()).all()
        exact = torch.from_numpy(ref).to(dtype).float().numpy()
        assert (got != exact).mean() < 1e-2  # all but a few rounding flips are the oracle's value rounded once


@pytest.mark.parametrize("name", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(40, 4096), (130, 2048), (300, 64), (5, 8192), (21, 12288)])
def test_16bit_fused_entry_points(name, shape):
    """Gate logits in and the h-recomputing backward on 16-bit tensors, with carries, against the
    fp32 oracle on the rounded inputs; shapes outside the bulk-tensor sweep are refused."""
    dtype, half_ulp = H16[name]
    rows, T = shape
    z, b, g = make_inputs("randn", shape, seed=111)
    z, b, g = (z * 2 + 1).to(dtype), b.to(dtype), g.to(dtype)
    a = torch.sigmoid(z.float())
    carry = torch.randn(rows)
    an, bn, gn, cn = a.numpy(), b.float().numpy(), g.float().numpy(), carry.numpy()
    h_ref = oracle.scan_forward(an, bn, h_in=cn)
    h16 = torch.from_numpy(h_ref).to(dtype)
    ga_ref, gb_ref = oracle.scan_backward(an, h16.float().numpy(), gn, gb_in=cn, h_prev=cn)
    gz_ref = ga_ref * (a * (1 - a)).numpy()
    ga_exact, gb_exact = oracle.scan_backward(an, h_ref, gn, gb_in=cn, h_prev=cn)  # what a recomputed fp32 h gives
    lib = _native.load()
    dz, db, dg, dh, dc = z.cuda(), b.cuda(), g.cuda(), h16.cuda(), carry.cuda()
    da = a.to(dtype).cuda()
    h, gz, gb = torch.empty_like(dz), torch.empty_like(dz), torch.empty_like(dz)
    st = _native.stream_of(dz)
    _native.check(getattr(lib, f"ssb_scan_sigmoid_fwd_{name}")(dz.data_ptr(), db.data_ptr(), h.data_ptr(), rows, T,
                                                                dc.data_ptr(), st))
    _native.check(getattr(lib, f"ssb_scan_sigmoid_bwd_{name}")(dz.data_ptr(), dh.data_ptr(), dg.data_ptr(), gz.data_ptr(),
                                                                gb.data_ptr(), rows, T, dc.data_ptr(), dc.data_ptr(), st))
    for x, ref in ((h, h_ref), (gz, gz_ref), (gb, gb_ref)):
        assert _gpu.max_norm_err(x.float(), ref) < 1.05 * half_ulp
    # recompute: gates given (already rounded to the storage type), h rebuilt in fp32
    a16 = da.float().cpu().numpy()
    h_ref2 = oracle.scan_forward(a16, bn, h_in=cn)
    ga_ref2, gb_ref2 = oracle.scan_backward(a16, h_ref2, gn, gb_in=cn, h_prev=cn)
    ga2, gb2 = torch.empty_like(dz), torch.empty_like(dz)
    rc = getattr(lib, f"ssb_scan_bwd_recompute_{name}")(da.data_ptr(), db.data_ptr(), dg.data_ptr(), ga2.data_ptr(),
                                                         gb2.data_ptr(), rows, T, dc.data_ptr(), dc.data_ptr(), st)
    _gpu.device_ok()
    if T > 8192:  # the recomputing kernel needs the row inside one span
        assert rc == _native.ERR_UNSUPPORTED
    else:
        _native.check(rc)
        assert _gpu.max_norm_err(ga2.float(), ga_ref2) < 1.05 * half_ulp
        assert _gpu.max_norm_err(gb2.float(), gb_ref2) < 1.05 * half_ulp
    # a row length the sweep does not take
    rc = getattr(lib, f"ssb_scan_sigmoid_fwd_{name}")(dz.data_ptr(), db.data_ptr(), h.data_ptr(), rows * T // 96, 96, None, st)
    assert rc == _native.ERR_UNSUPPORTED


@pytest.mark.parametrize("name", ["bf16", "f16"])
@pytest.mark.parametrize("shape,scratch", [((8, 700, 512), False), ((2, 300, 64), False), ((1, 9000, 64), True),
                                           ((2, 5000, 200), True), ((3, 100, 8), False), ((1, 4096, 1032), True),
                                           ((24, 300, 512), False), ((20, 260, 520), False)])  # 192 / 180 blocks: two CTAs per SM
def test_channels_last_16bit_storage(name, shape, scratch):
    """ssb_scan_cl_{fwd,bwd}_{bf16,f16}: [N,T,C] tensors in 16-bit storage; direct streaming and,
    with scratch on few-block shapes, the two-pass chunked form.  Every output within half a unit
    in the last place of the fp32 oracle's result on the same rounded inputs."""
    dtype, half_ulp = H16[name]
    N, T, C = shape
    a, b, g = (x.to(dtype) for x in make_inputs("sigmoid2", shape, seed=131))
    an, bn, gn = a.float().numpy(), b.float().numpy(), g.float().numpy()
    h_ref = oracle.scan_forward_channels_last(an, bn)
    h16 = torch.from_numpy(h_ref).to(dtype)
    ga_ref, gb_ref = oracle.scan_backward_channels_last(an, h16.float().numpy(), gn)
    lib = _native.load()
    da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), h16.cuda()
    h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
    need = lib.ssb_scan_cl_h16_workspace_bytes(N, T, C) if scratch else 0
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    wp = ws.data_ptr() if scratch else None
    st = _native.stream_of(da)
    _native.check(getattr(lib, f"ssb_scan_cl_fwd_{name}")(da.data_ptr(), db.data_ptr(), h.data_ptr(), N, T, C, wp, need, st))
    _native.check(getattr(lib, f"ssb_scan_cl_bwd_{name}")(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(),
                                                           gb.data_ptr(), N, T, C, wp, need, st))
    _gpu.device_ok()
    for x, ref in ((h, h_ref), (ga, ga_ref), (gb, gb_ref)):
        assert _gpu.max_norm_err(x.float(), ref) < 1.01 * half_ulp
        exact = torch.from_numpy(ref).to(dtype).float().numpy()
        assert (x.float().cpu().numpy() != exact).mean() < 1e-2
    rc = getattr(lib, f"ssb_scan_cl_fwd_{name}")(da.data_ptr(), db.data_ptr(), h.data_ptr(), 1, N * T * C // 4, 4, None, 0, st)
    assert rc == _native.ERR_UNSUPPORTED  # C % 8 != 0


@pytest.mark.parametrize("shape", [(3, 16384), (17, 65536), (1, 262144), (40, 16388)])
def test_fp64_few_long_rows_with_scratch(shape):
    """ssb_scan_{fwd,bwd}_f64_ex: with scratch, a few rows of whole 4096-step chunks run in two
    passes; the last shape (T % 4096 != 0) needs no scratch and takes the plain kernels."""
    rows, T = shape
    a, b, g = make_inputs("sigmoid2", shape, seed=141, dtype=torch.float64)
    carry = torch.randn(rows, dtype=torch.float64)
    an, bn, gn, cn = a.numpy(), b.numpy(), g.numpy(), carry.numpy()
    h_ref = oracle.scan_forward(an, bn, h_in=cn)
    ga_ref, gb_ref = oracle.scan_backward(an, h_ref, gn, gb_in=cn, h_prev=cn)
    lib = _native.load()
    need = lib.ssb_scan_f64_workspace_bytes(rows, T)
    assert (need > 0) == (T % 4096 == 0)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    da, db, dg, dh, dc = a.cuda(), b.cuda(), g.cuda(), dev(h_ref), carry.cuda()
    st = _native.stream_of(da)
    for wp, nb in ((ws.data_ptr(), need), (None, 0)):
        h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
        _native.check(lib.ssb_scan_fwd_f64_ex(da.data_ptr(), db.data_ptr(), h.data_ptr(), rows, T, dc.data_ptr(), wp, nb, st))
        _native.check(lib.ssb_scan_bwd_f64_ex(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T,
                                              dc.data_ptr(), dc.data_ptr(), wp, nb, st))
        for got, ref in ((h, h_ref), (ga, ga_ref), (gb, gb_ref)):
            assert _gpu.max_norm_err(got, ref) < 1e-12
    _gpu.device_ok()


@pytest.mark.parametrize("shape,scratch", [((8, 700, 512), False), ((2, 300, 64), True), ((1, 9000, 64), True),
                                           ((2, 5000, 200), True), ((3, 100, 8), False), ((1, 4096, 1028), True)])
def test_channels_last_fused_sigmoid_matches_oracle(shape, scratch):
    """ssb_scan_cl_sigmoid_{fwd,bwd}_f32 against the oracle fed sigmoid(z) computed on the host;
    direct streaming and, with scratch on few-block shapes, the two-pass chunked form."""
    N, T, C = shape
    z, b, g = make_inputs("randn", shape, seed=161)
    z = z * 2 + 1
    a = torch.sigmoid(z)
    h_ref = oracle.scan_forward_channels_last(a.numpy(), b.numpy())
    ga_ref, gb_ref = oracle.scan_backward_channels_last(a.numpy(), h_ref, g.numpy())
    gz_ref = ga_ref * (a * (1 - a)).numpy()
    lib = _native.load()
    dz, db, dg, dh = z.cuda(), b.cuda(), g.cuda(), dev(h_ref)
    h, gz, gb = torch.empty_like(dz), torch.empty_like(dz), torch.empty_like(dz)
    need = lib.ssb_scan_cl_workspace_bytes(N, T, C) if scratch else 0
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    wp = ws.data_ptr() if scratch else None
    st = _native.stream_of(dz)
    _native.check(lib.ssb_scan_cl_sigmoid_fwd_f32(dz.data_ptr(), db.data_ptr(), h.data_ptr(), N, T, C, wp, need, st))
    _native.check(lib.ssb_scan_cl_sigmoid_bwd_f32(dz.data_ptr(), dh.data_ptr(), dg.data_ptr(), gz.data_ptr(), gb.data_ptr(),
                                                  N, T, C, wp, need, st))
    _gpu.device_ok()
    for x, ref in ((h, h_ref), (gz, gz_ref), (gb, gb_ref)):
        assert _gpu.max_norm_err(x, ref) < TOL
    rc = lib.ssb_scan_cl_sigmoid_fwd_f32(dz.data_ptr(), db.data_ptr(), h.data_ptr(), 1, N * T * C // 6, 6, None, 0, st)
    assert rc == _native.ERR_UNSUPPORTED  # C % 4 != 0


@pytest.mark.skipif(os.environ.get("SCANSCAM_BIG_TESTS") != "1",
                    reason="holds ~60 GB on the device; set SCANSCAM_BIG_TESTS=1 to run")
def test_tensors_beyond_2_31_elements():
    """Index arithmetic past 2^31 elements: the channels-last streaming kernels against the plain
    kernels and a float64 loop on the tensor's tail, and the 16-bit sweep against the fp32 kernels
    on its last rows."""
    def rel(x, y):
        return float((x - y).abs().max() / y.abs().max())

    N, T, C = 4, 4096, 160000
    a = torch.rand(N, T, C, device="cuda") * 0.3 + 0.65
    b, g = torch.randn(N, T, C, device="cuda"), torch.randn(N, T, C, device="cuda")
    assert a.numel() > 2 ** 31
    h1, h2 = _gpu.cl_fwd(a, b), _gpu.cl_fwd(a, b, scratch="plain")
    assert rel(h1, h2) < 1e-5
    ga1, gb1 = _gpu.cl_bwd(a, h2, g)
    ga2, gb2 = _gpu.cl_bwd(a, h2, g, scratch="plain")
    assert rel(ga1, ga2) < 1e-5 and rel(gb1, gb2) < 1e-5
    sl = (slice(N - 1, N), slice(None), slice(C - 8, C))
    aa, bb = a[sl].double(), b[sl].double()
    hh, acc = torch.zeros_like(aa), torch.zeros(1, 8, dtype=torch.float64, device="cuda")
    for t in range(T):
        acc = aa[:, t] * acc + bb[:, t]
        hh[:, t] = acc
    assert rel(h1[sl].double(), hh) < 1e-5
    del a, b, g, h1, h2, ga1, gb1, ga2, gb2
    torch.cuda.empty_cache()
    rows, T = 700000, 4096
    a = (torch.rand(rows, T, device="cuda") * 0.3 + 0.65).bfloat16()
    b, g = torch.randn(rows, T, device="cuda").bfloat16(), torch.randn(rows, T, device="cuda").bfloat16()
    assert a.numel() > 2 ** 31
    lib = _native.load()
    h, ga, gb = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
    st = _native.stream_of(a)
    _native.check(lib.ssb_scan_fwd_bf16(a.data_ptr(), b.data_ptr(), h.data_ptr(), rows, T, None, st))
    _native.check(lib.ssb_scan_bwd_bf16(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T, None, None, st))
    af, bf = a[-4096:].float(), b[-4096:].float()
    assert rel(h[-4096:].float(), _gpu.fwd(af, bf)) < 2.0 ** -8
    gaf, gbf = _gpu.bwd(af, h[-4096:].float(), g[-4096:].float())
    assert rel(ga[-4096:].float(), gaf) < 2.0 ** -8 and rel(gb[-4096:].float(), gbf) < 2.0 ** -8
    _gpu.device_ok()
