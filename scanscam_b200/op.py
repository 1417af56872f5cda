"""The public operator: ``scan(gate, value)`` and its autograd Function.

Mirrors scanscam/op.py:9-55 of the reference with three deliberate differences:

* CUDA only.  A non-CUDA tensor, or a missing native extension, raises; the reference would
  fall back to CPU kernels or to a per-timestep PyTorch loop (scanscam/op.py:32-35,52-55).
* The backward of channels-last inputs calls the channels-last backward kernel.  The reference
  passes four arguments to a three-argument wrapper there and raises ``TypeError``
  (scanscam/op.py:45-49); the evident intent is implemented instead.
* Every branch of ``backward`` returns both gradients (the reference's CPU branch drops them,
  scanscam/op.py:52-53; that branch does not exist here).
"""
from __future__ import annotations

from typing import Any, Tuple

import torch

from . import cuda

_CHANNELS_PER_BLOCK = 32  # forwarded for API compatibility; no effect on these kernels


def is_transpose_contig(x: torch.Tensor) -> bool:
    """True for a 3-D tensor that is dense in ``[N, T, C]`` order but viewed as ``[N, C, T]``."""
    return x.dim() == 3 and not x.is_contiguous() and x.mT.is_contiguous()


def scan(gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """First-order gated linear scan ``h_t = gate_t * h_{t-1} + value_t`` with ``h_{-1} = 0``.

    :param gate: ``[N, ..., T]`` CUDA tensor (float32 or float64)
    :param value: tensor of the same shape
    :return: ``[N, ..., T]`` tensor of accumulated values; differentiable in both arguments.
    """
    return Scan.apply(gate, value)


def _require_cuda(t: torch.Tensor) -> None:
    if t.device.type != "cuda":
        raise RuntimeError(
            f"scanscam_b200.scan needs CUDA tensors (got a tensor on '{t.device}'); this build has no CPU path")
    if not cuda.has_cuda_ops:
        cuda._ext()  # raises with the reason the extension is unavailable


class Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        _require_cuda(gate)
        if is_transpose_contig(gate) and is_transpose_contig(value):
            output = cuda.transposed_linear_scan_forward(gate.mT, value.mT, _CHANNELS_PER_BLOCK).mT
        else:
            output = cuda.blocked_linear_scan_forward(gate, value)
        ctx.save_for_backward(gate, output)
        return output

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        gate, output = ctx.saved_tensors
        _require_cuda(output_grad)
        if is_transpose_contig(gate) and is_transpose_contig(output):
            grads = cuda.transposed_linear_scan_backward(
                gate.mT, output.mT, output_grad.mT.contiguous(), _CHANNELS_PER_BLOCK)
            return grads[0].mT, grads[1].mT
        return cuda.blocked_linear_scan_backward(gate, output, output_grad)
