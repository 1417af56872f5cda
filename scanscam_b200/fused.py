"""Scan with the gate's sigmoid fused in: ``h_t = sigmoid(z_t) * h_{t-1} + b_t``.

The reference operator takes ready-made gates (scanscam/op.py:13-21); its users compute
``gate = sigmoid(logits)`` in a separate elementwise pass before it and multiply by
``gate * (1 - gate)`` after its backward.  Taking the logits directly removes one read and one
write of a full tensor from each direction (20 -> 12 bytes per element forward, 32 -> 20
backward).  The fused kernels cover float32 tensors whose last axis is a multiple of 4 and
bfloat16 / float16 tensors whose last axis is 64 * 2^k <= 8192 or a larger multiple of 4096; other inputs are served by
``scan(torch.sigmoid(logits), value)``, i.e. the same operator unfused.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch

from . import cuda
from .op import is_transpose_contig, scan


def sweep_row_16bit(steps: int) -> bool:
    """Row lengths the 16-bit kernels take with the row inside one span: 64 * 2^k up to 8192."""
    return steps % 64 == 0 and steps <= 8192 and (steps // 64) & (steps // 64 - 1) == 0


def fused_row_16bit(steps: int) -> bool:
    """Row lengths the fused-sigmoid 16-bit kernels take: the above, or whole 4096-step spans."""
    return sweep_row_16bit(steps) or (steps > 8192 and steps % 4096 == 0)


def _fusable(*tensors: torch.Tensor) -> bool:
    t0 = tensors[0]
    if t0.device.type != "cuda" or t0.dim() < 2 or any(t.data_ptr() % 16 for t in tensors):
        return False
    if t0.dtype == torch.float32:
        return t0.shape[-1] % 4 == 0
    return t0.dtype in (torch.bfloat16, torch.float16) and fused_row_16bit(t0.shape[-1])


class ScanSigmoidGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, gate_logits: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        assert gate_logits.shape == value.shape and gate_logits.dim() >= 2
        steps = gate_logits.shape[-1]
        z = gate_logits.reshape(-1, steps).contiguous()
        b = value.reshape(-1, steps).contiguous()
        out = torch.empty_like(z)
        cuda._ext().scan_sigmoid_forward(z, b, out)
        ctx.save_for_backward(z, out)
        ctx.full_shape = gate_logits.shape
        return out.reshape(gate_logits.shape)

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        z, out = ctx.saved_tensors
        g = output_grad.reshape(z.shape).contiguous()
        grad_logits, grad_value = torch.empty_like(z), torch.empty_like(z)
        cuda._ext().scan_sigmoid_backward(z, out, g, grad_logits, grad_value)
        return grad_logits.reshape(ctx.full_shape), grad_value.reshape(ctx.full_shape)


def _fusable_channels_last(*tensors: torch.Tensor) -> bool:
    """Inputs viewed as ``[N, C, T]`` but dense in ``[N, T, C]`` order, with a channel count the
    streaming kernels take (a multiple of 4 for float32, of 8 for the 16-bit types)."""
    t0 = tensors[0]
    if t0.device.type != "cuda" or not all(is_transpose_contig(t) and t.data_ptr() % 16 == 0 for t in tensors):
        return False
    channels = t0.shape[1]
    if t0.dtype == torch.float32:
        return channels % 4 == 0
    return t0.dtype in (torch.bfloat16, torch.float16) and channels % 8 == 0


class ScanSigmoidGateChannelsLast(torch.autograd.Function):
    """The same operator for channels-last inputs; tensors are handled as dense ``[N, T, C]``."""

    @staticmethod
    def forward(ctx: Any, gate_logits: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        z, b = gate_logits.mT, value.mT
        out = torch.empty_like(z)
        cuda._ext().transposed_scan_sigmoid(z, b, out)
        ctx.save_for_backward(z, out)
        return out.mT

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        z, out = ctx.saved_tensors
        g = output_grad.mT.contiguous()
        grad_logits, grad_value = torch.empty_like(z), torch.empty_like(z)
        cuda._ext().transposed_scan_sigmoid_backward(z, out, g, grad_logits, grad_value)
        return grad_logits.mT, grad_value.mT


def scan_sigmoid_gate(gate_logits: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """``scan(sigmoid(gate_logits), value)`` over the last axis, differentiable in both arguments.

    :param gate_logits: ``[N, ..., T]`` CUDA tensor of pre-activation gates
    :param value: tensor of the same shape
    """
    if gate_logits.device.type != "cuda":
        raise RuntimeError("scanscam_b200.scan_sigmoid_gate needs CUDA tensors; this build has no CPU path")
    if gate_logits.is_contiguous() and value.is_contiguous() and _fusable(gate_logits, value):
        return ScanSigmoidGate.apply(gate_logits, value)
    if gate_logits.shape == value.shape and _fusable_channels_last(gate_logits, value):
        return ScanSigmoidGateChannelsLast.apply(gate_logits, value)
    return scan(torch.sigmoid(gate_logits), value)
