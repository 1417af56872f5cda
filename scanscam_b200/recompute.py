"""``scan_recompute(gate, value)``: the same result and gradients as ``scan``, keeping ``(gate,
value)`` for the backward instead of ``(gate, output)``.

The reference's ``Scan.forward`` saves its output for the backward (scanscam/op.py:36), so a
caller that does not otherwise need ``h`` after the layer still pays 4 bytes per element of
activation memory for it.  Here the backward rebuilds ``h``: for float32 rows of 32 * 2^k <= 4096
steps one kernel does that on the fly at the traffic of the ordinary backward; every other case
runs the forward kernel again into a temporary that lives only for the duration of the backward.
This is an addition: the reference has no counterpart.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch

from . import cuda
from .fused import sweep_row_16bit
from .op import _CHANNELS_PER_BLOCK, _require_cuda, is_transpose_contig


def _in_kernel(*tensors: torch.Tensor) -> bool:
    t0 = tensors[0]
    if t0.dim() < 2 or not all(t.is_contiguous() and t.data_ptr() % 16 == 0 for t in tensors):
        return False
    return t0.dtype == torch.float32 or (t0.dtype in (torch.bfloat16, torch.float16) and sweep_row_16bit(t0.shape[-1]))


class ScanRecompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        _require_cuda(gate)
        ctx.transposed = is_transpose_contig(gate) and is_transpose_contig(value)
        if ctx.transposed:
            output = cuda.transposed_linear_scan_forward(gate.mT, value.mT, _CHANNELS_PER_BLOCK).mT
        else:
            output = cuda.blocked_linear_scan_forward(gate, value)
        ctx.save_for_backward(gate, value)
        return output

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        gate, value = ctx.saved_tensors
        _require_cuda(output_grad)
        if ctx.transposed:
            output = cuda.transposed_linear_scan_forward(gate.mT, value.mT, _CHANNELS_PER_BLOCK)
            grads = cuda.transposed_linear_scan_backward(gate.mT, output, output_grad.mT.contiguous(), _CHANNELS_PER_BLOCK)
            return grads[0].mT, grads[1].mT
        grad = output_grad.contiguous()
        if _in_kernel(gate, value, grad):
            steps = gate.shape[-1]
            grad_gate, grad_value = torch.empty_like(gate), torch.empty_like(gate)
            cuda._ext().scan_backward_recompute(gate.reshape(-1, steps), value.reshape(-1, steps), grad.reshape(-1, steps),
                                                grad_gate.view(-1, steps), grad_value.view(-1, steps))
            return grad_gate, grad_value
        output = cuda.blocked_linear_scan_forward(gate, value)
        return cuda.blocked_linear_scan_backward(gate, output, output_grad)


def scan_recompute(gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """``scan(gate, value)`` whose backward does not need the output kept alive.

    :param gate: ``[N, ..., T]`` CUDA tensor (float32 or float64)
    :param value: tensor of the same shape
    """
    return ScanRecompute.apply(gate, value)
