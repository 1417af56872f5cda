"""Host-buffer entry point: scan forward + backward on tensors that live in (pinned) host memory.

The reference has no such call -- its users move tensors themselves and call ``scan`` -- but a
caller whose data sits on the host pays for PCIe in both directions, and because rows are
independent that traffic can overlap with the kernels.  :class:`HostScanPipeline` splits the
rows into chunks and keeps three CUDA streams busy: host->device copies of chunk i+1, the
forward and fused backward kernels of chunk i, and device->host copies of chunk i-1.  The
numeric work is the same extension calls as ``scanscam_b200.scan``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import cuda


class HostScanPipeline:
    """Reusable pipeline for ``[rows, T]`` float32 problems of a fixed shape.

    Device staging buffers (``slots`` x 6 tensors of one chunk) are allocated once, here.
    """

    def __init__(self, rows: int, steps: int, chunks: int = 8, slots: int = 3,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32):
        if not torch.cuda.is_available():
            raise RuntimeError("HostScanPipeline needs a CUDA device; this build has no CPU path")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rows, self.steps = rows, steps
        self.chunk_rows = max(1, -(-rows // max(1, chunks)))
        self.n_chunks = -(-rows // self.chunk_rows)
        self.slots = max(2, slots)
        shape = (self.chunk_rows, steps)
        self._buf = [[torch.empty(shape, dtype=dtype, device=self.device) for _ in range(6)]
                     for _ in range(self.slots)]
        self._s_in = torch.cuda.Stream(self.device)
        self._s_run = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)

    def run(self, gate: torch.Tensor, value: torch.Tensor, out_grad: torch.Tensor,
            out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """gate, value, out_grad: CPU ``[rows, T]`` (pinned for full speed).  Returns CPU tensors
        ``(h, grad_gate, grad_value)``; pass ``out`` to reuse pinned result buffers.  The call
        returns after the current stream has been made to wait for the last copy; synchronise
        that stream (or the device) before reading the results on the host."""
        ext = cuda._ext()
        for t in (gate, value, out_grad):
            assert t.device.type == "cpu" and t.shape == (self.rows, self.steps) and t.is_contiguous()
        if out is None:
            out = tuple(torch.empty_like(gate).pin_memory() for _ in range(3))
        caller = torch.cuda.current_stream(self.device)
        for s in (self._s_in, self._s_run, self._s_out):
            s.wait_stream(caller)
        ran = [None] * self.n_chunks      # kernels of chunk i done (inputs of its slot are free)
        drained = [None] * self.n_chunks  # outputs of chunk i copied out (its slot is free)
        for i in range(self.n_chunks):
            lo = i * self.chunk_rows
            hi = min(self.rows, lo + self.chunk_rows)
            n = hi - lo
            a, b, g, h, ga, gb = (t[:n] for t in self._buf[i % self.slots])
            if i >= self.slots:
                self._s_in.wait_event(ran[i - self.slots])
            with torch.cuda.stream(self._s_in):
                a.copy_(gate[lo:hi], non_blocking=True)
                b.copy_(value[lo:hi], non_blocking=True)
                g.copy_(out_grad[lo:hi], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self._s_in)
            self._s_run.wait_event(loaded)
            if i >= self.slots:
                self._s_run.wait_event(drained[i - self.slots])
            with torch.cuda.stream(self._s_run):
                ext.blocked_linear_scan(a, b, h)
                ext.blocked_linear_scan_backward(a, h, g, ga, gb)
                ran[i] = torch.cuda.Event()
                ran[i].record(self._s_run)
            self._s_out.wait_event(ran[i])
            with torch.cuda.stream(self._s_out):
                out[0][lo:hi].copy_(h, non_blocking=True)
                out[1][lo:hi].copy_(ga, non_blocking=True)
                out[2][lo:hi].copy_(gb, non_blocking=True)
                drained[i] = torch.cuda.Event()
                drained[i].record(self._s_out)
        caller.wait_stream(self._s_out)
        caller.wait_stream(self._s_run)
        caller.wait_stream(self._s_in)
        return out


def scan_forward_backward_host(gate: torch.Tensor, value: torch.Tensor, out_grad: torch.Tensor,
                               chunks: int = 8) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One-shot convenience wrapper: ``[N, ..., T]`` CPU tensors in, ``(h, grad_gate, grad_value)``
    CPU tensors out (synchronised)."""
    assert gate.shape == value.shape == out_grad.shape and gate.dim() >= 2
    steps = gate.shape[-1]
    flat = [t.reshape(-1, steps).contiguous() for t in (gate, value, out_grad)]
    pipe = HostScanPipeline(flat[0].shape[0], steps, chunks=chunks, dtype=gate.dtype)
    res = pipe.run(*flat)
    torch.cuda.synchronize(pipe.device)
    return tuple(r.reshape(gate.shape) for r in res)
