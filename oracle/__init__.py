"""CPU oracle for the gated linear scan -- TEST INFRASTRUCTURE, never a product path.

Only the test-suite, the repository's smoke check and the benchmark's CPU-baseline
leg may import this package.  It wraps ``oracle/scan_oracle.c`` (a plain-C
restatement of the reference's ``src/scanscam_cpu.hpp:9-28`` and ``:54-78``) with
numpy, and can also load the reference's own CPU extension when
``oracle/build_ref.py`` has compiled it into ``oracle/_ref/``.

All functions take and return numpy arrays (float32 or float64), C-contiguous.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libscan_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``scan_oracle.c`` with the Makefile beside it; returns the library path."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "scan_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        p, i64 = ctypes.c_void_p, ctypes.c_int64
        for sfx in ("f32", "f64"):
            getattr(lib, f"oracle_scan_fwd_{sfx}").argtypes = [p, p, p, i64, i64, p]
            getattr(lib, f"oracle_scan_bwd_{sfx}").argtypes = [p, p, p, p, p, i64, i64, p, p]
            getattr(lib, f"oracle_scan_cl_fwd_{sfx}").argtypes = [p, p, p, i64, i64, i64]
            getattr(lib, f"oracle_scan_cl_bwd_{sfx}").argtypes = [p, p, p, p, p, i64, i64, i64]
            for name in ("fwd", "bwd", "cl_fwd", "cl_bwd"):
                getattr(lib, f"oracle_scan_{name}_{sfx}").restype = None
        _lib = lib
    return _lib


def _sfx(x: np.ndarray) -> str:
    if x.dtype == np.float32:
        return "f32"
    if x.dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle supports float32/float64, got {x.dtype}")


def _c(x, dtype=None) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=dtype)


def _ptr(x: Optional[np.ndarray]):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def scan_forward(gate, value, h_in=None) -> np.ndarray:
    """h_t = a_t*h_{t-1} + b_t over the last axis of ``[..., T]`` arrays.

    Mirrors ``scanscam.cpu.simple_linear_scan_forward`` (scanscam/cpu.py:16-22),
    including the flattening of leading axes (scanscam/decorator.py:18-23).
    ``h_in`` (one value per row) is the carry entering the first step; the
    reference always starts from zero.
    """
    gate, value = _c(gate), _c(value, gate.dtype if hasattr(gate, "dtype") else None)
    assert gate.shape == value.shape and gate.ndim >= 2
    T = gate.shape[-1]
    rows = gate.size // T if T else 0
    out = np.empty_like(gate)
    if h_in is not None:
        h_in = _c(h_in, gate.dtype).reshape(rows)
    getattr(_load(), f"oracle_scan_fwd_{_sfx(gate)}")(
        _ptr(gate), _ptr(value), _ptr(out), rows, T, _ptr(h_in))
    return out


def scan_backward(gate, output, out_grad, gb_in=None, h_prev=None) -> Tuple[np.ndarray, np.ndarray]:
    """Returns ``(grad_gate, grad_value)``; mirrors ``scanscam.cpu.simple_linear_scan_backward``
    (scanscam/cpu.py:25-35 -> src/scanscam_cpu.hpp:54-78).

    ``gb_in`` is the already-gated gradient flowing in from the step after the last one
    (a_{T}*gb_{T} of a longer sequence); ``h_prev`` is h just before the first step.
    """
    gate = _c(gate)
    output, out_grad = _c(output, gate.dtype), _c(out_grad, gate.dtype)
    assert gate.shape == output.shape == out_grad.shape and gate.ndim >= 2
    T = gate.shape[-1]
    rows = gate.size // T if T else 0
    ga, gb = np.empty_like(gate), np.empty_like(gate)
    if gb_in is not None:
        gb_in = _c(gb_in, gate.dtype).reshape(rows)
    if h_prev is not None:
        h_prev = _c(h_prev, gate.dtype).reshape(rows)
    getattr(_load(), f"oracle_scan_bwd_{_sfx(gate)}")(
        _ptr(gate), _ptr(output), _ptr(out_grad), _ptr(ga), _ptr(gb), rows, T,
        _ptr(gb_in), _ptr(h_prev))
    return ga, gb


def scan_forward_channels_last(gate, value) -> np.ndarray:
    """Scan over axis 1 of dense ``[N, T, C]`` arrays (the layout of the reference's
    ``transposed_linear_scan``, src/scanscam_cuda.cu:471-582)."""
    gate = _c(gate)
    value = _c(value, gate.dtype)
    assert gate.shape == value.shape and gate.ndim == 3
    N, T, C = gate.shape
    out = np.empty_like(gate)
    getattr(_load(), f"oracle_scan_cl_fwd_{_sfx(gate)}")(
        _ptr(gate), _ptr(value), _ptr(out), N, T, C)
    return out


def scan_backward_channels_last(gate, output, out_grad) -> Tuple[np.ndarray, np.ndarray]:
    """Backward of :func:`scan_forward_channels_last` (src/scanscam_cuda.cu:584-723)."""
    gate = _c(gate)
    output, out_grad = _c(output, gate.dtype), _c(out_grad, gate.dtype)
    assert gate.shape == output.shape == out_grad.shape and gate.ndim == 3
    N, T, C = gate.shape
    ga, gb = np.empty_like(gate), np.empty_like(gate)
    getattr(_load(), f"oracle_scan_cl_bwd_{_sfx(gate)}")(
        _ptr(gate), _ptr(output), _ptr(out_grad), _ptr(ga), _ptr(gb), N, T, C)
    return ga, gb


# --------------------------------------------------------------------------------------
# The reference's own CPU extension, compiled from its sources by oracle/build_ref.py.
# --------------------------------------------------------------------------------------
_REF_DIR = os.path.join(_HERE, "_ref")
_ref_mod = None


def reference_available() -> bool:
    return any(f.startswith("scanscam_ref_ext") and f.endswith(".so")
               for f in (os.listdir(_REF_DIR) if os.path.isdir(_REF_DIR) else []))


def load_reference():
    """Import the reference CPU extension built into ``oracle/_ref/`` (torch tensors in,
    results written into caller-allocated tensors, as src/scanscam_cpu.hpp:30-52,80-113)."""
    global _ref_mod
    if _ref_mod is None:
        import importlib.util

        import torch  # noqa: F401  (the extension links against libtorch)

        so = [f for f in os.listdir(_REF_DIR)
              if f.startswith("scanscam_ref_ext") and f.endswith(".so")]
        if not so:
            raise ImportError("reference CPU extension not built; run oracle/build_ref.py")
        spec = importlib.util.spec_from_file_location(
            "scanscam_ref_ext", os.path.join(_REF_DIR, so[0]))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ref_mod = mod
    return _ref_mod


def reference_forward(gate, value):
    """The reference's ``simple_linear_scan_cpu`` on torch CPU tensors ``[rows, T]``."""
    import torch

    out = torch.empty_like(gate)
    load_reference().simple_linear_scan_cpu(gate.contiguous(), value.contiguous(), out)
    return out


def reference_backward(gate, output, out_grad):
    """The reference's ``simple_linear_scan_backward_cpu``; returns ``(grad_gate, grad_value)``."""
    import torch

    ga, gb = torch.empty_like(gate), torch.empty_like(gate)
    load_reference().simple_linear_scan_backward_cpu(
        gate.contiguous(), output.contiguous(), out_grad.contiguous(), ga, gb)
    return ga, gb
