"""Prints the parity figures of the benchmark configurations: max-norm relative error of every
kernel family against the CPU oracle (fp32, and against an fp64 run of the same oracle).

    python tests/parity_report.py [cfg1,cfg2,cfg5,cfg4s,cfg3s]

cfg4s / cfg3s are row samples of cfg4 / cfg3 (every 64th row of cfg4; 8 rows of cfg3 at its full
sequence length 2**20): the oracle is single-threaded.  Test infrastructure, like the rest of
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


def main():
    names = sys.argv[1].split(",") if len(sys.argv) > 1 else ["cfg1", "cfg2", "cfg5", "cfg4s", "cfg3s"]
    lib = _native.load()
    for name in names:
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
                    ("tma", _gpu.TMA | (1 << 8), _gpu.TMA | (1 << 8)), ("lookback", _gpu.LOOKBACK, _gpu.LOOKBACK)]
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
