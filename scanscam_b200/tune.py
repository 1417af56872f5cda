"""Kernel-variant sweep: times every kernel family / tuning id on given shapes.

    python -m scanscam_b200.tune cfg2,cfg5,1024x262144 [--iters 30] [--families warp,flat,tma]
    python -m scanscam_b200.tune cl:8x4096x512,cl:4x65536x256         (channels-last [N,T,C])
    python -m scanscam_b200.tune fused:16384x4096                     (gate logits in; recompute backward)
    python -m scanscam_b200.tune h16:16384x4096                       (bf16 / fp16 storage beside fp32)
    python -m scanscam_b200.tune clh16:64x4096x512                    (the same for channels-last)
    python -m scanscam_b200.tune shard:1024x131072                    (shard maps of a T-sharded sequence)
    python -m scanscam_b200.tune f64:16384x4096,clf64:64x4096x512     (the fp64 entry points)

For each shape (a named workload or ROWSxT) and variant it reports the best of three groups of
``iters`` back-to-back launches, forward and backward separately, timed with CUDA events, as
milliseconds and as algorithmic GB/s (12 B/element forward, 20 B/element backward).  This is
how the default choices in ``pick_variant`` (csrc/scanscam_b200.cu) were made.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _native
from .workloads import WORKLOADS

FLAT_IDS = range(14)                 # SSB_FLAT_CONFIGS in csrc/scanscam_b200.cu
TMA_IDS = (0, 1, 5, 6, 8, 10, 32, 33, 34, 35, 36, 37, 38, 48)  # per-warp ring ids; 32..38 flat sweep; 48 flat sweep over long rows
LOOKBACK_IDS = range(7)              # SSB_LOOKBACK_CONFIGS


def variants(families):
    out = [("auto", None)]  # the library's own choice, per direction
    if "any" in families:
        out += [("any0", _native.VARIANT_FLAT_ANY), ("any1", _native.VARIANT_FLAT_ANY | (1 << 8))]
    if "warp" in families:
        out.append(("warp", _native.VARIANT_WARP))
    if "flat" in families:
        out += [(f"flat{t}", _native.VARIANT_FLAT | (t << 8)) for t in FLAT_IDS]
    if "tma" in families:
        out += [(f"tma{t}", _native.VARIANT_TMA | (t << 8)) for t in TMA_IDS]
    if "lookback" in families:
        out += [(f"lookback{t}", _native.VARIANT_LOOKBACK | (t << 8)) for t in LOOKBACK_IDS]
        out.append(("chunked", _native.VARIANT_LOOKBACK | (16 << 8)))  # two passes over chunks of T
        out.append(("chunked17", _native.VARIANT_LOOKBACK | (17 << 8)))  # long chunks, early-terminated maps, one sweep
    return out


def time_variant(lib, rows, T, variant, tensors, iters):
    """``variant`` None: what the library recommends per direction when the caller can supply scratch."""
    a, b, g, h, ga, gb = tensors
    st = torch.cuda.current_stream().cuda_stream
    v_f = lib.ssb_scan_recommend(rows, T, 0, 1, 1) if variant is None else variant
    v_b = lib.ssb_scan_recommend(rows, T, 1, 1, 1) if variant is None else variant
    ws_bytes = max(lib.ssb_scan_workspace_bytes(rows, T, v_f), lib.ssb_scan_workspace_bytes(rows, T, v_b))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=a.device)
    ws_ptr = ws.data_ptr() if ws_bytes else None

    def fwd():
        return lib.ssb_scan_fwd_f32_ex(a.data_ptr(), b.data_ptr(), h.data_ptr(), rows, T, None, v_f, ws_ptr,
                                       ws_bytes, st)

    def bwd():
        return lib.ssb_scan_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T,
                                       None, None, v_b, ws_ptr, ws_bytes, st)

    res = {}
    for kind, fn, nbytes in (("fwd", fwd, 12), ("bwd", bwd, 20)):
        rc = fn()
        if rc != _native.OK:
            res[kind] = None  # variant does not support this shape
            continue
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / iters)
        res[kind] = {"ms": best, "GBps": nbytes * rows * T / best / 1e6}
    return res


def time_channels_last(lib, N, T, C, iters):
    """Plain kernels, look-back kernels (forced, default tile) and the library's own choice."""
    a = torch.rand(N, T, C, device="cuda") * 0.2 + 0.8
    b, g = torch.randn_like(a), torch.randn_like(a)
    h, ga, gb = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
    st = torch.cuda.current_stream().cuda_stream
    need = lib.ssb_scan_cl_workspace_bytes(N, T, C)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    n = N * T * C

    def run(fn):
        assert fn() == _native.OK
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / iters)
        return best

    rows = []
    modes = [("plain", _native.CL_PLAIN), ("lookback", _native.CL_LOOKBACK), ("auto", _native.CL_AUTO)]
    if C in (4, 8, 16):
        modes += [("narrow", _native.CL_NARROW)]  # whole batch elements per CTA, untiled bulk copies
    if C % 4 == 0:  # streaming kernels (a CTA walks all of T through a TMA ring), every tile shape
        modes += [("chunked", _native.CL_CHUNKED)]  # the same kernels over chunks of T, two passes
        modes += [(f"stream{k}", _native.CL_STREAM | (k << 8)) for k in range(8)]
    for label, variant in modes:
        p, nb = ws.data_ptr(), need
        tf = run(lambda: lib.ssb_scan_cl_fwd_f32_ex(a.data_ptr(), b.data_ptr(), h.data_ptr(), N, T, C, variant, p, nb, st))
        tb = run(lambda: lib.ssb_scan_cl_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(),
                                                    gb.data_ptr(), N, T, C, variant, p, nb, st))
        rows.append((label, 12 * n / tf / 1e6, tf, 20 * n / tb / 1e6, tb))
    return rows


def time_channels_last_16bit(lib, N, T, C, iters):
    """Channels-last entry points on fp32, bf16 and fp16 tensors of one shape (library's own choice)."""
    out = []
    st = torch.cuda.current_stream().cuda_stream
    n = N * T * C
    for name, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
        a = (torch.rand(N, T, C, device="cuda") * 0.2 + 0.8).to(dtype)
        b, g = torch.randn_like(a), torch.randn_like(a)
        h, ga, gb = (torch.empty_like(a) for _ in range(3))
        need = (lib.ssb_scan_cl_workspace_bytes if name == "f32" else lib.ssb_scan_cl_h16_workspace_bytes)(N, T, C)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
        if name == "f32":  # the library's own choice, with the scratch at hand
            def fwd(*args):
                return lib.ssb_scan_cl_fwd_f32_ex(*args[:6], _native.CL_AUTO, *args[6:])

            def bwd(*args):
                return lib.ssb_scan_cl_bwd_f32_ex(*args[:8], _native.CL_AUTO, *args[8:])
        else:
            fwd, bwd = getattr(lib, f"ssb_scan_cl_fwd_{name}"), getattr(lib, f"ssb_scan_cl_bwd_{name}")
        size = a.element_size()

        def run(fn):
            for _ in range(3):
                _native.check(fn())
            torch.cuda.synchronize()
            best = float("inf")
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1) / iters)
            return best

        tf = run(lambda: fwd(a.data_ptr(), b.data_ptr(), h.data_ptr(), N, T, C, ws.data_ptr(), need, st))
        tb = run(lambda: bwd(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), N, T, C, ws.data_ptr(), need, st))
        out.append((name, 3 * size * n / tf / 1e6, tf, 5 * size * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
        sf, sb = getattr(lib, f"ssb_scan_cl_sigmoid_fwd_{name}"), getattr(lib, f"ssb_scan_cl_sigmoid_bwd_{name}")
        if sf(a.data_ptr(), b.data_ptr(), h.data_ptr(), N, T, C, ws.data_ptr(), need, st) == _native.OK:
            tf = run(lambda: sf(a.data_ptr(), b.data_ptr(), h.data_ptr(), N, T, C, ws.data_ptr(), need, st))
            tb = run(lambda: sb(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), N, T, C, ws.data_ptr(), need, st))
            out.append((name + " fused sigmoid", 3 * size * n / tf / 1e6, tf, 5 * size * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
        del a, b, g, h, ga, gb
    return out


def time_fused_sigmoid(lib, rows, T, iters):
    """Kernel times of the plain scan, the fused-sigmoid scan and the elementwise passes it replaces."""
    z = torch.randn(rows, T, device="cuda")
    b, g = torch.randn_like(z), torch.randn_like(z)
    h, ga, gb, a = (torch.empty_like(z) for _ in range(4))
    st = torch.cuda.current_stream().cuda_stream

    def run(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    p = [t.data_ptr() for t in (z, b, g, h, ga, gb)]
    need = lib.ssb_scan_bwd_recompute_workspace_bytes(rows, T)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    return [
        ("scan forward (gates given)", run(lambda: lib.ssb_scan_fwd_f32(p[0], p[1], p[3], rows, T, None, st))),
        ("scan backward (gates given)", run(lambda: lib.ssb_scan_bwd_f32(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, st))),
        ("fused forward (logits given)", run(lambda: lib.ssb_scan_sigmoid_fwd_f32(p[0], p[1], p[3], rows, T, None, st))),
        ("fused backward (logits given)", run(lambda: lib.ssb_scan_sigmoid_bwd_f32(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, st))),
        ("recompute backward (a, b, g given)", run(lambda: lib.ssb_scan_bwd_recompute_f32(
            p[0], p[1], p[2], p[4], p[5], rows, T, None, None, ws.data_ptr(), need, st))),
        ("torch.sigmoid pass", run(lambda: torch.sigmoid(z, out=a))),
        ("torch sigmoid-backward pass", run(lambda: torch.ops.aten.sigmoid_backward(ga, a))),
    ]


def time_16bit(lib, rows, T, iters):
    """Kernel times of the bf16 / fp16 storage entry points beside fp32 on the same shape."""
    out = []
    st = torch.cuda.current_stream().cuda_stream
    for name, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
        a = (torch.rand(rows, T, device="cuda") * 0.2 + 0.8).to(dtype)
        b, g = torch.randn_like(a), torch.randn_like(a)
        h, ga, gb = (torch.empty_like(a) for _ in range(3))
        fwd, bwd = getattr(lib, f"ssb_scan_fwd_{name}"), getattr(lib, f"ssb_scan_bwd_{name}")
        p = [t.data_ptr() for t in (a, b, g, h, ga, gb)]
        size = a.element_size()

        def run(fn):
            for _ in range(3):
                _native.check(fn())
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters

        tf = run(lambda: fwd(p[0], p[1], p[3], rows, T, None, st))
        tb = run(lambda: bwd(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, st))
        n = rows * T
        out.append((name, 3 * size * n / tf / 1e6, tf, 5 * size * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
        if name != "f32" and lib.ssb_scan_sigmoid_fwd_bf16(p[0], p[1], p[3], rows, T, None, st) == _native.OK:
            sf, sb = getattr(lib, f"ssb_scan_sigmoid_fwd_{name}"), getattr(lib, f"ssb_scan_sigmoid_bwd_{name}")
            tf = run(lambda: sf(p[0], p[1], p[3], rows, T, None, st))
            tb = run(lambda: sb(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, st))
            out.append((name + " fused sigmoid", 3 * size * n / tf / 1e6, tf, 5 * size * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
        del a, b, g, h, ga, gb
    return out


def time_fp64(lib, extents, iters):
    """Kernel times of the fp64 entry points: rows layout (ROWSxT; without and with scratch) or
    channels-last (NxTxC)."""
    st = torch.cuda.current_stream().cuda_stream
    shape = tuple(extents)
    a = torch.rand(*shape, device="cuda", dtype=torch.float64) * 0.2 + 0.8
    b, g = torch.randn_like(a), torch.randn_like(a)
    h, ga, gb = (torch.empty_like(a) for _ in range(3))
    p = [t.data_ptr() for t in (a, b, g, h, ga, gb)]
    n = a.numel()

    def run(fn):
        for _ in range(3):
            _native.check(fn())
        best = float("inf")
        for _ in range(3):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / iters)
        return best

    out = []
    if len(shape) == 3:
        N, T, C = shape
        tf = run(lambda: lib.ssb_scan_cl_fwd_f64(p[0], p[1], p[3], N, T, C, st))
        tb = run(lambda: lib.ssb_scan_cl_bwd_f64(p[0], p[3], p[2], p[4], p[5], N, T, C, st))
        out.append(("f64 channels-last", 24 * n / tf / 1e6, tf, 40 * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
        return out
    rows, T = shape
    tf = run(lambda: lib.ssb_scan_fwd_f64(p[0], p[1], p[3], rows, T, None, st))
    tb = run(lambda: lib.ssb_scan_bwd_f64(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, st))
    out.append(("f64", 24 * n / tf / 1e6, tf, 40 * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
    need = lib.ssb_scan_f64_workspace_bytes(rows, T)
    if need:
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        tf = run(lambda: lib.ssb_scan_fwd_f64_ex(p[0], p[1], p[3], rows, T, None, ws.data_ptr(), need, st))
        tb = run(lambda: lib.ssb_scan_bwd_f64_ex(p[0], p[3], p[2], p[4], p[5], rows, T, None, None, ws.data_ptr(), need, st))
        out.append(("f64 with scratch", 24 * n / tf / 1e6, tf, 40 * n / tb / 1e6, tb, n / (tf + tb) / 1e6))
    return out


MODES = {"fused": 2, "h16": 2, "clh16": 3, "cl": 3, "shard": 2, "f64": 2, "clf64": 3}  # prefix -> number of extents


def parse_shape(name: str):
    """``cfg2`` | ``ROWSxT`` | ``MODE:AxB[xC]`` -> (mode or "rows", extents).  Raises ValueError."""
    if name in WORKLOADS:
        return "rows", (WORKLOADS[name].rows, WORKLOADS[name].steps)
    mode, _, dims = name.rpartition(":")
    mode = mode or "rows"
    if mode != "rows" and mode not in MODES:
        raise ValueError(f"unknown sweep mode {mode!r} in {name!r}")
    try:
        extents = tuple(int(v) for v in dims.lower().split("x"))
    except ValueError:
        raise ValueError(f"cannot read the extents of {name!r}") from None
    if len(extents) != (2 if mode == "rows" else MODES[mode]) or min(extents) <= 0:
        raise ValueError(f"{name!r}: expected {2 if mode == 'rows' else MODES[mode]} positive extents")
    return mode, extents


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("shapes", help="comma-separated: a workload name, ROWSxT, cl:NxTxC, fused:ROWSxT, h16:ROWSxT, "
                                   "clh16:NxTxC, shard:ROWSxT, f64:ROWSxT, clf64:NxTxC")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--families", default="warp,flat,tma,lookback")
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)
    args.parsed = [(name, *parse_shape(name)) for name in args.shapes.split(",")]
    known = {"warp", "flat", "tma", "lookback", "any"}
    bad = set(args.families.split(",")) - known
    if bad:
        ap.error(f"unknown kernel families {sorted(bad)}; choose from {sorted(known)}")
    return args


def time_shard_maps(lib, rows, T, iters):
    """The shard maps of a T-sharded sequence (near-unit gates): full reduction, early-terminated walks."""
    a = torch.rand(rows, T, device="cuda") * 0.01 + 0.99
    b, g = torch.randn_like(a) * 0.1, torch.randn_like(a)
    agg = torch.empty(rows, 2, device="cuda")
    walked = torch.zeros(1, dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    out = []
    for label, cut in (("full walk (cut < 0)", -1.0), ("exact zero (cut = 0)", 0.0), ("cut = 2^-40", 2.0 ** -40)):
        for kind, fn, other in (("fwd", lib.ssb_shard_map_fwd_f32, b), ("bwd", lib.ssb_shard_map_bwd_f32, g)):
            for _ in range(3):
                _native.check(fn(a.data_ptr(), other.data_ptr(), agg.data_ptr(), rows, T, cut, None, st))
            walked.zero_()
            _native.check(fn(a.data_ptr(), other.data_ptr(), agg.data_ptr(), rows, T, cut, walked.data_ptr(), st))
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn(a.data_ptr(), other.data_ptr(), agg.data_ptr(), rows, T, cut, None, st)
            e1.record()
            torch.cuda.synchronize()
            out.append((f"{label} {kind}", e0.elapsed_time(e1) / iters, walked.item() / rows))
    return out


def main(argv=None):
    args = parse_args(argv)
    lib = _native.load()
    results = {}
    for name, mode, extents in args.parsed:
        if mode == "shard":  # shard maps of a T-sharded sequence: shard:ROWSxT
            rows, T = extents
            print(f"# shard maps, rows={rows} T={T} (near-unit gates)")
            for label, ms, steps in time_shard_maps(lib, rows, T, args.iters):
                results[f"{name}/{label}"] = {"ms": ms, "steps_walked_per_row": steps}
                print(f"{label:28s} {ms:8.4f} ms  {steps:10.0f} steps walked per row", flush=True)
            continue
        if mode in ("f64", "clf64"):  # fp64 entry points: f64:ROWSxT, clf64:NxTxC
            print(f"# fp64, {'[N,T,C]' if mode == 'clf64' else 'rows x T'} = {'x'.join(map(str, extents))}")
            print(f"{'entry points':18s} {'fwd GB/s':>9s} {'fwd ms':>8s} {'bwd GB/s':>9s} {'bwd ms':>8s} {'Gelem/s':>8s}")
            for label, fg, tf, bg, tb, ge in time_fp64(lib, extents, args.iters):
                results[f"{name}/{label}"] = {"fwd": {"ms": tf, "GBps": fg}, "bwd": {"ms": tb, "GBps": bg}, "gelem_s": ge}
                print(f"{label:18s} {fg:9.0f} {tf:8.4f} {bg:9.0f} {tb:8.4f} {ge:8.1f}", flush=True)
            continue
        if name.startswith("fused:"):  # gate logits in: fused:ROWSxT
            rows, T = (int(v) for v in name[6:].lower().split("x"))
            print(f"# fused sigmoid gate, rows={rows} T={T} ({rows * T * 4 / 1e6:.0f} MB per tensor)")
            for label, ms in time_fused_sigmoid(lib, rows, T, args.iters):
                results[f"{name}/{label}"] = {"ms": ms}
                print(f"{label:36s} {ms:8.4f} ms", flush=True)
            continue
        if name.startswith("h16:"):  # 16-bit storage beside fp32: h16:ROWSxT
            rows, T = (int(v) for v in name[4:].lower().split("x"))
            print(f"# storage types, rows={rows} T={T} ({rows * T / 1e6:.0f} M elements per tensor)")
            print(f"{'storage':18s} {'fwd GB/s':>9s} {'fwd ms':>8s} {'bwd GB/s':>9s} {'bwd ms':>8s} {'Gelem/s':>8s}")
            for label, fg, tf, bg, tb, ge in time_16bit(lib, rows, T, args.iters):
                results[f"{name}/{label}"] = {"fwd": {"ms": tf, "GBps": fg}, "bwd": {"ms": tb, "GBps": bg}, "gelem_s": ge}
                print(f"{label:18s} {fg:9.0f} {tf:8.4f} {bg:9.0f} {tb:8.4f} {ge:8.1f}", flush=True)
            continue
        if name.startswith("clh16:"):  # channels-last, storage types: clh16:NxTxC
            N, T, C = (int(v) for v in name[6:].lower().split("x"))
            print(f"# channels-last storage types, [N,T,C] = {N}x{T}x{C} ({N * T * C / 1e6:.0f} M elements per tensor)")
            print(f"{'storage':18s} {'fwd GB/s':>9s} {'fwd ms':>8s} {'bwd GB/s':>9s} {'bwd ms':>8s} {'Gelem/s':>8s}")
            for label, fg, tf, bg, tb, ge in time_channels_last_16bit(lib, N, T, C, args.iters):
                results[f"{name}/{label}"] = {"fwd": {"ms": tf, "GBps": fg}, "bwd": {"ms": tb, "GBps": bg}, "gelem_s": ge}
                print(f"{label:18s} {fg:9.0f} {tf:8.4f} {bg:9.0f} {tb:8.4f} {ge:8.1f}", flush=True)
            continue
        if name.startswith("cl:"):  # channels-last: cl:NxTxC
            N, T, C = (int(v) for v in name[3:].lower().split("x"))
            print(f"# channels-last [N,T,C] = {N}x{T}x{C} ({N * T * C * 4 / 1e6:.0f} MB per tensor)")
            print(f"{'kernels':10s} {'fwd GB/s':>9s} {'fwd ms':>8s} {'bwd GB/s':>9s} {'bwd ms':>8s}")
            for label, fg, tf, bg, tb in time_channels_last(lib, N, T, C, args.iters):
                results[f"{name}/{label}"] = {"fwd": {"ms": tf, "GBps": fg}, "bwd": {"ms": tb, "GBps": bg}}
                print(f"{label:10s} {fg:9.0f} {tf:8.4f} {bg:9.0f} {tb:8.4f}", flush=True)
            continue
        if name in WORKLOADS:
            rows, T = WORKLOADS[name].rows, WORKLOADS[name].steps
        else:
            rows, T = (int(v) for v in name.lower().split("x"))
        a = torch.rand(rows, T, device="cuda") * 0.2 + 0.8
        tensors = [a, torch.randn_like(a), torch.randn_like(a)] + [torch.empty_like(a) for _ in range(3)]
        print(f"# {name}: rows={rows} T={T} ({rows * T * 4 / 1e6:.0f} MB per tensor)")
        print(f"{'variant':10s} {'fwd GB/s':>9s} {'fwd ms':>8s} {'bwd GB/s':>9s} {'bwd ms':>8s}")
        for label, v in variants(args.families.split(",")):
            r = time_variant(lib, rows, T, v, tensors, args.iters)
            results[f"{name}/{label}"] = r

            def cell(x):
                return f"{x['GBps']:9.0f} {x['ms']:8.4f}" if x else f"{'-':>9s} {'-':>8s}"

            print(f"{label:10s} {cell(r['fwd'])} {cell(r['bwd'])}", flush=True)
        del tensors, a
    detail = _native.ctypes.c_int(0)
    _native.check(lib.ssb_device_status(_native.ctypes.byref(detail)))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
