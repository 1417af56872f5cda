"""CUDA wrappers with the names and calling conventions of the reference's ``scanscam/cuda.py``.

Every wrapper makes its inputs contiguous, allocates the outputs and calls the extension module
``scanscam_ext`` (built from ``csrc/torch_ext.cpp`` over the C-ABI library).  The reference's
three forward names (scanscam/cuda.py:16-40) and two backward names (:43-66) differ only in
kernel strategy there; here they share one kernel family, chosen from the shape.
``has_cuda_ops`` has the reference's meaning (scanscam/cuda.py:7-13).  When the extension is
missing the wrappers raise; nothing falls back to another implementation.
"""
from __future__ import annotations

import sys
from typing import Optional, Tuple

import torch

from .decorator import preprocess_backward_scan_args, preprocess_scan_args

_import_error: Optional[BaseException] = None
scanscam_ext = None
has_cuda_ops = False


def _load_extension() -> None:
    """(Re)tries to import the extension module; sets ``scanscam_ext`` and ``has_cuda_ops``."""
    global scanscam_ext, has_cuda_ops, _import_error
    try:
        import importlib

        module = importlib.import_module(__package__ + ".scanscam_ext")
    except ImportError as exc:
        scanscam_ext, has_cuda_ops, _import_error = None, False, exc
        return
    # Let ``import scanscam_ext`` find the same module, as code written for the reference expects.
    sys.modules.setdefault("scanscam_ext", module)
    scanscam_ext, _import_error = module, None
    has_cuda_ops = hasattr(module, "simple_linear_scan")


_load_extension()


def _ext():
    if scanscam_ext is None:
        _load_extension()  # it may have been built since this module was imported
    if scanscam_ext is None:
        raise RuntimeError(
            "scanscam_b200: the native extension is not built or failed to load "
            f"({_import_error}); run `python -m scanscam_b200.build`. There is no fallback path."
        )
    return scanscam_ext


def _make_forward(ext_fn: str, doc: str):
    @preprocess_scan_args
    def forward(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        gate, value = x.contiguous(), y.contiguous()
        result = torch.empty_like(gate)
        getattr(_ext(), ext_fn)(gate, value, result)
        return result

    forward.__name__ = forward.__qualname__ = f"{ext_fn}_forward"
    forward.__doc__ = doc
    return forward


def _make_backward(ext_fn: str, doc: str):
    @preprocess_backward_scan_args
    def backward(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        gate, output, out_grad = x.contiguous(), y.contiguous(), z.contiguous()
        grad_gate, grad_value = torch.empty_like(gate), torch.empty_like(gate)
        getattr(_ext(), ext_fn)(gate, output, out_grad, grad_gate, grad_value)
        return grad_gate, grad_value

    backward.__name__ = backward.__qualname__ = ext_fn
    backward.__doc__ = doc
    return backward


_FWD_DOC = "h_t = x_t*h_{t-1} + y_t over the last axis of ``[N, ..., T]`` tensors (x = gate, y = value)."
_BWD_DOC = ("Gradients of the scan: x = gate, y = forward output, z = upstream gradient; "
            "returns ``(grad_gate, grad_value)``.")

simple_linear_scan_forward = _make_forward("simple_linear_scan", _FWD_DOC)
coalesced_linear_scan_forward = _make_forward("coalesced_linear_scan", _FWD_DOC)
blocked_linear_scan_forward = _make_forward("blocked_linear_scan", _FWD_DOC)
simple_linear_scan_backward = _make_backward("simple_linear_scan_backward", _BWD_DOC)
blocked_linear_scan_backward = _make_backward("blocked_linear_scan_backward", _BWD_DOC)


def _check_channels_last(*tensors: torch.Tensor) -> None:
    first = tensors[0]
    for t in tensors:
        assert t.shape == first.shape
    assert first.dim() == 3
    for t in tensors:
        assert t.is_contiguous()


def transposed_linear_scan_forward(x: torch.Tensor, y: torch.Tensor, channels_per_block: int) -> torch.Tensor:
    """Scan over axis 1 of contiguous ``[N, T, C]`` tensors (scanscam/cuda.py:69-78).

    ``channels_per_block`` is accepted for compatibility; it was a tuning knob of the
    reference's kernel and does not affect results.
    """
    _check_channels_last(x, y)
    result = torch.empty_like(x)
    _ext().transposed_linear_scan(x, y, result, channels_per_block)
    return result


def transposed_linear_scan_backward(
    x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, channels_per_block: int
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Backward of :func:`transposed_linear_scan_forward` on ``[N, T, C]`` (scanscam/cuda.py:81-95)."""
    _check_channels_last(x, y, z)
    grad_gate, grad_value = torch.empty_like(x), torch.empty_like(x)
    _ext().transposed_linear_scan_backward(x, y, z, grad_gate, grad_value, channels_per_block)
    return grad_gate, grad_value
