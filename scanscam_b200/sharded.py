"""Sequence-parallel scan: one long sequence split along T across the ranks of a process group.

The reference never splits a sequence (one CUDA block walks a whole row,
src/scanscam_cuda.cu:154-167); this module is the multi-GPU extension of the same operator.
Rank ``s`` of ``G`` holds the contiguous slice ``[..., s*T/G : (s+1)*T/G]`` of gate and value.

Forward, per rank:
  1. map      -- per row, the shard's affine map ``(A, B)``: ``h_end = A*h_start + B``.  It is
                 folded from the shard's LAST step backwards and the walk stops once the product of
                 the gates walked so far has dropped to ``|A| <= cut`` (what lies further left can
                 then change ``B`` by at most ``cut`` relative to the largest value of the scan).
                 Gates in (0, 1) cost a few thousand steps per row; rows whose product does not
                 vanish are walked in full, so any gates are handled.         (8 bytes per row out)
  2. exchange -- ``all_gather`` of those ``[rows, 2]`` pairs (the only collective; a few KB)
  3. carry    -- fold the maps of the shards to the left into ``h_in`` for this shard
  4. scan     -- the ordinary forward kernel started from ``h_in``: the prefix fix-up happens
                 inside the scan kernel, at the first element of each row, not in a pass of its own
Backward mirrors it from the right with the reverse recurrence ``c_t = a_t*(g_t + c_{t+1})``
(its map is folded from the shard's FIRST step forwards); the ``h`` just left of the shard, needed
for ``grad_gate`` at the shard's first step, is the forward's ``h_in``.

Bytes moved per element and direction: the scan's 12 / 20 plus 8 x (walked fraction of the shard).

The numeric work is delegated to an *ops* object so the exchange logic can be exercised on CPU
process groups (gloo) with stand-in ops supplied by the tests; the default ops call the CUDA
extension and nothing else.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist

from . import cuda

#: Default early-termination threshold of the shard maps: error at most 2^-40 (9e-13) of the
#: largest scan value, far below fp32 rounding.  0.0 stops only at an exactly-zero product.
DEFAULT_CUT = 2.0 ** -40


class CudaShardOps:
    """Local kernels of the sharded scan, backed by the CUDA extension (float32, ``[rows, T]``)."""

    @staticmethod
    def map_forward(gate: torch.Tensor, value: torch.Tensor, cut: float = DEFAULT_CUT,
                    walked: Optional[torch.Tensor] = None) -> torch.Tensor:
        agg = torch.empty(gate.shape[0], 2, dtype=gate.dtype, device=gate.device)
        cuda._ext().shard_map_forward(gate, value, agg, cut, walked)
        return agg

    @staticmethod
    def map_backward(gate: torch.Tensor, out_grad: torch.Tensor, cut: float = DEFAULT_CUT,
                     walked: Optional[torch.Tensor] = None) -> torch.Tensor:
        agg = torch.empty(gate.shape[0], 2, dtype=gate.dtype, device=gate.device)
        cuda._ext().shard_map_backward(gate, out_grad, agg, cut, walked)
        return agg

    @staticmethod
    def reduce_forward(gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        """The full fold of the shard (many CTAs per row through scratch): for a few very long
        rows whose gate products do not vanish."""
        agg = torch.empty(gate.shape[0], 2, dtype=gate.dtype, device=gate.device)
        cuda._ext().shard_reduce_forward(gate, value, agg)
        return agg

    @staticmethod
    def reduce_backward(gate: torch.Tensor, out_grad: torch.Tensor) -> torch.Tensor:
        agg = torch.empty(gate.shape[0], 2, dtype=gate.dtype, device=gate.device)
        cuda._ext().shard_reduce_backward(gate, out_grad, agg)
        return agg

    @staticmethod
    def carry(aggs: torch.Tensor, shard: int, reverse: bool) -> torch.Tensor:
        out = torch.empty(aggs.shape[1], dtype=aggs.dtype, device=aggs.device)
        cuda._ext().shard_carry(aggs, shard, reverse, out)
        return out

    @staticmethod
    def scan_forward(gate: torch.Tensor, value: torch.Tensor, h_in: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(gate)
        cuda._ext().scan_forward_ex(gate, value, out, h_in, 0)
        return out

    @staticmethod
    def scan_backward(gate, output, out_grad, c_in, h_prev) -> Tuple[torch.Tensor, torch.Tensor]:
        grad_gate, grad_value = torch.empty_like(gate), torch.empty_like(gate)
        cuda._ext().scan_backward_ex(gate, output, out_grad, grad_gate, grad_value, c_in, h_prev, 0)
        return grad_gate, grad_value


def _gather_maps(agg: torch.Tensor, group) -> torch.Tensor:
    """all_gather of the per-row maps -> ``[world, rows, 2]`` (identity for a single rank)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return agg.unsqueeze(0).contiguous()
    gathered = torch.empty((world * agg.shape[0],) + tuple(agg.shape[1:]), dtype=agg.dtype, device=agg.device)
    dist.all_gather_into_tensor(gathered, agg.contiguous(), group=group)
    return gathered.view((world,) + tuple(agg.shape))


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def sharded_scan_forward(gate: torch.Tensor, value: torch.Tensor, group=None, ops: Any = CudaShardOps,
                         cut: float = DEFAULT_CUT, walked: Optional[torch.Tensor] = None
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward of this rank's T-slice. ``gate``/``value``: ``[rows, T_local]`` contiguous.

    Returns ``(h_local, h_in)`` where ``h_in`` (``[rows]``) is h just before the slice.  ``cut``:
    see the module docstring.  ``walked``: optional one-element int64 tensor on the inputs' device
    that accumulates how many elements per tensor the map pass read.
    """
    assert gate.shape == value.shape and gate.dim() == 2
    gate, value = gate.contiguous(), value.contiguous()
    maps = _gather_maps(ops.map_forward(gate, value, cut, walked), group)
    h_in = ops.carry(maps, _rank(group), False)
    return ops.scan_forward(gate, value, h_in), h_in


def sharded_scan_backward(gate: torch.Tensor, output: torch.Tensor, out_grad: torch.Tensor,
                          h_in: torch.Tensor, group=None, ops: Any = CudaShardOps,
                          cut: float = DEFAULT_CUT, walked: Optional[torch.Tensor] = None
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Backward of this rank's T-slice; ``h_in`` is what :func:`sharded_scan_forward` returned."""
    assert gate.shape == output.shape == out_grad.shape and gate.dim() == 2
    gate, output, out_grad = gate.contiguous(), output.contiguous(), out_grad.contiguous()
    maps = _gather_maps(ops.map_backward(gate, out_grad, cut, walked), group)
    c_in = ops.carry(maps, _rank(group), True)
    return ops.scan_backward(gate, output, out_grad, c_in, h_in)


class ShardedScan(torch.autograd.Function):
    """Autograd Function over the local slice; gradients stay sharded like the inputs."""

    @staticmethod
    def forward(ctx: Any, gate: torch.Tensor, value: torch.Tensor, group, ops, cut: float) -> torch.Tensor:
        rows_shape = gate.shape
        g2, v2 = gate.reshape(-1, rows_shape[-1]), value.reshape(-1, rows_shape[-1])
        out, h_in = sharded_scan_forward(g2, v2, group, ops, cut)
        ctx.save_for_backward(g2, out, h_in)
        ctx.group, ctx.ops, ctx.rows_shape, ctx.cut = group, ops, rows_shape, cut
        return out.reshape(rows_shape)

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor):
        gate, out, h_in = ctx.saved_tensors
        gg, gv = sharded_scan_backward(gate, out, output_grad.reshape(gate.shape), h_in, ctx.group, ctx.ops, ctx.cut)
        return gg.reshape(ctx.rows_shape), gv.reshape(ctx.rows_shape), None, None, None


def scan_sequence_parallel(gate: torch.Tensor, value: torch.Tensor, group: Optional[Any] = None,
                           ops: Any = CudaShardOps, cut: float = DEFAULT_CUT) -> torch.Tensor:
    """``scan`` for a sequence sharded along its last axis over ``group`` (default: the world).

    Every rank passes its own ``[N, ..., T_local]`` slice (slices in rank order form the full
    sequence) and receives the matching slice of the result.
    """
    assert gate.shape == value.shape and gate.dim() >= 2
    return ShardedScan.apply(gate, value, group, ops, cut)
