"""scanscam_b200 -- B200 (sm_100a) implementation of scanscam's first-order gated linear scan.

Drop-in for the CUDA path of unixpickle/scanscam: ``scan(gate, value)`` and the autograd
Function ``op.Scan`` keep the reference's signatures (scanscam/__init__.py:1-3,
scanscam/op.py:13-55), ``cuda`` mirrors the reference's wrapper module (scanscam/cuda.py), and
the extension module is importable as ``scanscam_ext``.  There is no CPU path: tensors must
live on a CUDA device and the native libraries must be built (``python -m scanscam_b200.build``).
"""
import importlib

__all__ = ["scan", "Scan", "is_transpose_contig", "scan_sigmoid_gate", "scan_recompute", "ScanRecompute"]
__version__ = "0.2.0"

# The operator modules load the native extension when they are imported.  They are resolved on
# first use, so that the helper modules that need no device (``workloads``, ``build``, ``_native``)
# can be imported without pulling the CUDA libraries into the process.
_LAZY = {"scan": "op", "Scan": "op", "is_transpose_contig": "op", "scan_sigmoid_gate": "fused",
         "scan_recompute": "recompute", "ScanRecompute": "recompute"}


def __getattr__(name):
    if name in _LAZY:
        value = getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
