"""Prints the parity figures of the benchmark configurations: max-norm relative error of every
kernel family against the CPU oracle (fp32, and against an fp64 run of the same oracle).

    python tests/parity_report.py [cfg1,cfg2,cfg5,cfg4s,cfg3s,h16,cl]

cfg4s / cfg3s are row samples of cfg4 / cfg3 (every 64th row of cfg4; 8 rows of cfg3 at its full
sequence length 2**20): the oracle is single-threaded.  h16 = the tolerance study of bf16 / fp16
storage, cl = the channels-last kernel sets.  Test infrastructure, like the rest of
this directory; run on a GPU.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
import _gpu  # noqa: E402

import oracle  # noqa: E402
from scanscam_b200 import _native  # noqa: E402
from scanscam_b200.workloads import WORKLOADS, make_inputs  # noqa: E402


def inputs(name):
    if name == "cfg4s":
        w = WORKLOADS["cfg4"]
        return make_inputs(w.gates, (w.rows // 64, w.steps), seed=0)
    if name == "cfg3s":
        w = WORKLOADS["cfg3"]
        return make_inputs(w.gates, (8, w.steps), seed=0)
    w = WORKLOADS[name]
    return make_inputs(w.gates, (w.rows, w.steps), seed=0)


def err(x, ref):
    return float(np.abs(x.cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max())


def rms_err(x, ref):
    d = x.cpu().numpy().astype(np.float64) - ref
    return float(np.sqrt((d * d).mean()) / np.sqrt((ref.astype(np.float64) ** 2).mean()))


def report_16bit(lib):
    """Tolerance study for 16-bit storage: (1) against the fp32 oracle on the same rounded inputs
    (what the kernels add: one rounding per output), (2) against the fp64 oracle on the original
    fp32 inputs (what a caller loses by storing its tensors in 16 bits at all)."""
    for wl, shape in (("cfg2", (1024, 4096)), ("cfg5", (4096, 2048)), ("cfg3", (8, 1 << 20))):
        a, b, g = make_inputs(WORKLOADS[wl].gates, shape, seed=0)
        rows, T = shape
        h64 = oracle.scan_forward(a.double().numpy(), b.double().numpy())
        ga64, gb64 = oracle.scan_backward(a.double().numpy(), h64, g.double().numpy())
        print(f"# 16-bit storage, {wl} gates, rows={rows} T={T}")
        for name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16)):
            a16, b16, g16 = a.to(dtype), b.to(dtype), g.to(dtype)
            h32 = oracle.scan_forward(a16.float().numpy(), b16.float().numpy())
            da, db, dg = a16.cuda(), b16.cuda(), g16.cuda()
            h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
            st = _native.stream_of(da)
            _native.check(getattr(lib, f"ssb_scan_fwd_{name}")(da.data_ptr(), db.data_ptr(), h.data_ptr(), rows, T, None, st))
            _native.check(getattr(lib, f"ssb_scan_bwd_{name}")(da.data_ptr(), h.data_ptr(), dg.data_ptr(), ga.data_ptr(),
                                                                gb.data_ptr(), rows, T, None, None, st))
            ga32, gb32 = oracle.scan_backward(a16.float().numpy(), h.float().cpu().numpy(), g16.float().numpy())
            print(f"  {name:5s} vs fp32 oracle on the rounded inputs (max-norm): h {err(h.float(), h32):.2e} ga {err(ga.float(), ga32):.2e} "
                  f"gb {err(gb.float(), gb32):.2e}   half a unit in the last place = {2.0 ** (-8 if name == 'bf16' else -11):.2e}")
            print(f"        vs fp64 oracle on the original inputs: max-norm h {err(h.float(), h64):.2e} ga {err(ga.float(), ga64):.2e} "
                  f"gb {err(gb.float(), gb64):.2e}   rms h {rms_err(h.float(), h64):.2e} ga {rms_err(ga.float(), ga64):.2e} "
                  f"gb {rms_err(gb.float(), gb64):.2e}", flush=True)
        _gpu.device_ok()


def report_channels_last(lib):
    for shape in ((8, 4096, 512), (4, 65536, 256), (2, 5000, 108)):
        a, b, g = make_inputs("sigmoid2", shape, seed=0)
        h32 = oracle.scan_forward_channels_last(a.numpy(), b.numpy())
        ga32, gb32 = oracle.scan_backward_channels_last(a.numpy(), h32, g.numpy())
        da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), torch.from_numpy(h32).cuda()
        print(f"# channels-last [N,T,C] = {list(shape)}")
        for label, mode in (("auto", True), ("plain", "plain"), ("lookback", 12), ("stream0", 64), ("chunked", 96)):
            if isinstance(mode, int) and mode >= 64 and shape[2] % 4:
                continue
            if mode is True:
                lib.ssb_scan_cl_set_tuning(0)
                ws, need = _gpu.cl_workspace(da)
                h, ga, gb = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
                st = _native.stream_of(da)
                _native.check(lib.ssb_scan_cl_fwd_f32_ex(da.data_ptr(), db.data_ptr(), h.data_ptr(), *shape, ws.data_ptr(), need, st))
                _native.check(lib.ssb_scan_cl_bwd_f32_ex(da.data_ptr(), dh.data_ptr(), dg.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                                                         *shape, ws.data_ptr(), need, st))
            else:
                h = _gpu.cl_fwd(da, db, scratch=mode)
                ga, gb = _gpu.cl_bwd(da, dh, dg, scratch=mode)
            print(f"  {label:9s} vs fp32 oracle: h {err(h, h32):.2e} ga {err(ga, ga32):.2e} gb {err(gb, gb32):.2e}", flush=True)
        _gpu.device_ok()


def main():
    names = sys.argv[1].split(",") if len(sys.argv) > 1 else ["cfg1", "cfg2", "cfg5", "cfg4s", "cfg3s", "h16", "cl"]
    lib = _native.load()
    for name in names:
        if name == "h16":
            report_16bit(lib)
            continue
        if name == "cl":
            report_channels_last(lib)
            continue
        a, b, g = inputs(name)
        rows, T = a.shape
        h32 = oracle.scan_forward(a.numpy(), b.numpy())
        ga32, gb32 = oracle.scan_backward(a.numpy(), h32, g.numpy())
        h64 = oracle.scan_forward(a.double().numpy(), b.double().numpy())
        ga64, gb64 = oracle.scan_backward(a.double().numpy(), h64, g.double().numpy())
        print(f"# {name}: rows={rows} T={T}; fp32 oracle vs fp64 oracle: h {err(torch.from_numpy(h32), h64):.2e} "
              f"ga {err(torch.from_numpy(ga32), ga64):.2e} gb {err(torch.from_numpy(gb32), gb64):.2e}")
        da, db, dg, dh = a.cuda(), b.cuda(), g.cuda(), torch.from_numpy(h32).cuda()
        families = [("auto", lib.ssb_scan_recommend(rows, T, 0, 1, 1), lib.ssb_scan_recommend(rows, T, 1, 1, 1)),
                    ("warp", _gpu.WARP, _gpu.WARP), ("flat", _gpu.FLAT | (6 << 8), _gpu.FLAT | (6 << 8)),
                    ("flat_any", _gpu.FLAT_ANY | (1 << 8), _gpu.FLAT_ANY | (1 << 8)),
                    ("tma", _gpu.TMA | (1 << 8), _gpu.TMA | (1 << 8)), ("tma_flat", _gpu.TMA | (32 << 8), _gpu.TMA | (37 << 8)),
                    ("lookback", _gpu.LOOKBACK, _gpu.LOOKBACK)]
        for label, vf, vb in families:
            try:
                h = _gpu.fwd(da, db, variant=vf)
                ga, gb = _gpu.bwd(da, dh, dg, variant=vb)
            except _native.NativeError:
                continue
            print(f"  {label:9s} vs fp32 oracle: h {err(h, h32):.2e} ga {err(ga, ga32):.2e} gb {err(gb, gb32):.2e}   "
                  f"vs fp64: h {err(h, h64):.2e} ga {err(ga, ga64):.2e} gb {err(gb, gb64):.2e}", flush=True)
        _gpu.device_ok()


if __name__ == "__main__":
    main()
