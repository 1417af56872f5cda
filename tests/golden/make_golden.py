"""Generate the golden vectors in this directory by running the reference itself.

Run where a checkout of unixpickle/scanscam is available (path as first argument, or the
environment variable SCANSCAM_REFERENCE_DIR) and
after ``python oracle/build_ref.py`` has compiled its CPU extension:

    python tests/golden/make_golden.py [path-to-reference]

For every case the script draws seeded inputs with numpy (PCG64, stable across numpy
versions), calls the reference's public CPU wrappers
``scanscam.cpu.simple_linear_scan_forward/backward`` (scanscam/cpu.py:16-35) and the
pure-PyTorch loops ``scanscam.baseline.naive_linear_scan_forward/backward``
(scanscam/baseline.py:8-40), checks that the two agree bit for bit, and stores inputs
and outputs in ``scan_golden.npz``.  Channels-last cases are obtained the way the
reference's tests obtain them: the same functions on ``.mT`` views
(scanscam/cuda_test.py:138-141,153-158).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))

# (name, shape, gate distribution, dtype)
CASES = [
    ("randn_32x5", (32, 5), "randn", "float32"),
    ("randn_16x2x5", (16, 2, 5), "randn", "float32"),
    ("randn_32x64", (32, 64), "randn", "float32"),
    ("randn_1x1024", (1, 1024), "randn", "float32"),
    ("randn_1x1025", (1, 1025), "randn", "float32"),
    ("randn_4x1025", (4, 1025), "randn", "float32"),
    ("randn_2x4100", (2, 4100), "randn", "float32"),
    ("sigmoid2_2x4x256", (2, 4, 256), "sigmoid2", "float32"),     # gates ~0.88
    ("nearunit_1x8192", (1, 8192), "nearunit", "float32"),        # U(0.99, 1), b ~ 0.1*N(0,1)
    ("sigmoid0_8x512", (8, 512), "sigmoid0", "float32"),
    ("resets_2x2048", (2, 2048), "resets", "float32"),            # exact zeros w.p. 0.1
    ("randn_f64_4x33", (4, 33), "randn", "float64"),
    ("sigmoid2_f64_2x1030", (2, 1030), "sigmoid2", "float64"),
]
CL_CASES = [
    ("cl_randn_3x107x19", (3, 107, 19), "randn", "float32"),
    ("cl_sigmoid2_2x300x24", (2, 300, 24), "sigmoid2", "float32"),
    ("cl_randn_f64_2x17x5", (2, 17, 5), "randn", "float64"),
]


def draw(rng: np.random.Generator, shape, dist: str, dtype: str):
    """Seeded inputs: gate a, value b, upstream gradient g."""
    n = rng.standard_normal(shape)
    if dist == "randn":
        a = n
        b = rng.standard_normal(shape)
    elif dist == "sigmoid2":
        a = 1.0 / (1.0 + np.exp(-(n + 2.0)))
        b = rng.standard_normal(shape)
    elif dist == "sigmoid0":
        a = 1.0 / (1.0 + np.exp(-n))
        b = rng.standard_normal(shape)
    elif dist == "nearunit":
        a = 0.99 + 0.01 * rng.random(shape)
        b = 0.1 * rng.standard_normal(shape)
    elif dist == "resets":
        a = rng.random(shape) * (rng.random(shape) >= 0.1)
        b = rng.standard_normal(shape)
    else:
        raise ValueError(dist)
    g = rng.standard_normal(shape)
    return tuple(np.ascontiguousarray(x, dtype=dtype) for x in (a, b, g))


def main(ref_root: str) -> None:
    sys.path.insert(0, REPO)
    import oracle

    # The reference's wrappers import an extension called ``scanscam_ext``; hand them
    # the module built from the reference's own sources.
    sys.modules["scanscam_ext"] = oracle.load_reference()
    sys.path.insert(0, ref_root)
    import scanscam.baseline as ref_naive
    import scanscam.cpu as ref_cpu

    assert ref_cpu.has_cpu_ops and ref_cpu.__file__.startswith(ref_root)
    store = {}
    for idx, (name, shape, dist, dtype) in enumerate(CASES):
        a, b, g = draw(np.random.default_rng(1000 + idx), shape, dist, dtype)
        ta, tb, tg = (torch.from_numpy(x) for x in (a, b, g))
        h = ref_cpu.simple_linear_scan_forward(ta, tb)
        ga, gb = ref_cpu.simple_linear_scan_backward(ta, h, tg)
        h2 = ref_naive.naive_linear_scan_forward(ta, tb)
        ga2, gb2 = ref_naive.naive_linear_scan_backward(ta, h, tg)
        same = all(torch.equal(x, y) for x, y in ((h, h2), (ga, ga2), (gb, gb2)))
        print(f"{name:24s} cpu-ext == naive loops bit for bit: {same}")
        assert torch.allclose(h, h2, atol=1e-4) and torch.allclose(gb, gb2, atol=1e-4)
        for k, v in (("a", a), ("b", b), ("g", g), ("h", h.numpy()), ("ga", ga.numpy()),
                     ("gb", gb.numpy())):
            store[f"{name}/{k}"] = v
    for idx, (name, shape, dist, dtype) in enumerate(CL_CASES):
        a, b, g = draw(np.random.default_rng(2000 + idx), shape, dist, dtype)
        ta, tb, tg = (torch.from_numpy(x) for x in (a, b, g))
        h = ref_cpu.simple_linear_scan_forward(ta.mT, tb.mT).mT.contiguous()
        ga, gb = (x.mT.contiguous() for x in ref_cpu.simple_linear_scan_backward(ta.mT, h.mT, tg.mT))
        print(f"{name:24s} done")
        for k, v in (("a", a), ("b", b), ("g", g), ("h", h.numpy()), ("ga", ga.numpy()),
                     ("gb", gb.numpy())):
            store[f"{name}/{k}"] = v
    out = os.path.join(HERE, "scan_golden.npz")
    np.savez_compressed(out, **store)
    print(f"wrote {out}: {os.path.getsize(out) / 1024:.0f} KiB, {len(store)} arrays")


if __name__ == "__main__":
    sys.path.insert(0, REPO)
    from oracle.build_ref import DEFAULT_REFERENCE

    main(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE)
