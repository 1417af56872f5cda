"""scanscam_b200 -- B200 (sm_100a) implementation of scanscam's first-order gated linear scan.

Drop-in for the CUDA path of unixpickle/scanscam: ``scan(gate, value)`` and the autograd
Function ``op.Scan`` keep the reference's signatures (scanscam/__init__.py:1-3,
scanscam/op.py:13-55), ``cuda`` mirrors the reference's wrapper module (scanscam/cuda.py), and
the extension module is importable as ``scanscam_ext``.  There is no CPU path: tensors must
live on a CUDA device and the native libraries must be built (``python -m scanscam_b200.build``).
"""
from .fused import scan_sigmoid_gate
from .op import Scan, is_transpose_contig, scan
from .recompute import ScanRecompute, scan_recompute

__all__ = ["scan", "Scan", "is_transpose_contig", "scan_sigmoid_gate", "scan_recompute", "ScanRecompute"]
__version__ = "0.1.0"
