"""Argument flattening for scan implementations that work on ``[rows, T]`` matrices.

Same behaviour as the reference's decorators (scanscam/decorator.py:12-46): all arguments must
have equal shapes (``AssertionError`` otherwise) and at least two axes; leading axes are folded
into one with ``reshape`` and the results are unfolded again.
"""
from __future__ import annotations

import functools
from typing import Callable, Tuple

import torch

ScanFn = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]
ReverseScanFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]


def _as_rows(first: torch.Tensor, *rest: torch.Tensor):
    for other in rest:
        assert other.shape == first.shape
    assert first.dim() >= 2
    steps = first.shape[-1]
    return tuple(t.reshape(-1, steps) for t in (first, *rest))


def preprocess_scan_args(fn: ScanFn) -> ScanFn:
    """Lets a ``[rows, T]`` forward implementation accept ``[N, ..., T]`` tensors."""

    @functools.wraps(fn)
    def flattened(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        rx, ry = _as_rows(x, y)
        return fn(rx, ry).reshape(x.shape)

    return flattened


def preprocess_backward_scan_args(fn: ReverseScanFn) -> ReverseScanFn:
    """Lets a ``[rows, T]`` backward implementation accept ``[N, ..., T]`` tensors."""

    @functools.wraps(fn)
    def flattened(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        rx, ry, rz = _as_rows(x, y, z)
        grad_gate, grad_value = fn(rx, ry, rz)
        return grad_gate.reshape(x.shape), grad_value.reshape(x.shape)

    return flattened
