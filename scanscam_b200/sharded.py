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

Steps 1-3 also exist without the collective library (:class:`PeerCarryExchange`): the map kernel
stores its result into every rank's buffer through peer memory and the carry kernel waits for it.

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


class PeerCarryExchange:
    """The exchange step without a collective: every rank's map kernel stores its ``[rows, 2]`` result
    straight into every other rank's buffer over NVLink, and the carry kernel waits for them
    (``ssb_shard_map_publish_f32`` / ``ssb_shard_carry_peer_f32``).  Two kernel launches per
    direction before the scan instead of map, all-gather, carry.

    Needs one process per GPU on one node and peer access between the GPUs; each rank allocates its
    buffer with ``ssb_peer_buffer_create`` and maps the others' from their CUDA IPC handles, sent once,
    here, through the process group, with its own device current (``ssb_peer_buffer_open``).  ``PeerCarryExchange.create`` returns ``None`` where that
    is not possible (the callers then keep the collective path).  All ranks must make the same
    sequence of forward / backward calls with an exchange object: the epochs are counted locally.
    """

    def __init__(self, rows: int, group=None, device: Optional[torch.device] = None):
        from . import _native

        ct = _native.ctypes
        self.lib = _native.load()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows = int(rows)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        nbytes = self.lib.ssb_peer_exchange_bytes(self.world, self.rows)
        if nbytes == 0:
            raise ValueError(f"peer exchange supports 1..8 ranks and at least one row (world={self.world}, rows={rows})")
        self._own = ct.c_void_p()
        self._mapped = []
        handle = ct.create_string_buffer(64)
        problem = None  # every rank walks through the same collectives whatever goes wrong locally
        with torch.cuda.device(self.device):  # allocate, and map the peers' buffers, with THIS rank's device current
            if self.lib.ssb_peer_buffer_create(nbytes, ct.byref(self._own), handle) != _native.OK:
                problem = self.lib.ssb_last_error().decode()
            pointers = [self._own.value] * self.world
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, (handle.raw if problem is None else None, self.device.index), group=group)
                if problem is None and any(raw is None for raw, _ in handles):
                    problem = "another rank could not allocate its exchange buffer"
                if problem is None and len({dev for _, dev in handles}) != self.world:
                    problem = "two ranks share one GPU: the peer exchange needs one process per GPU"
                for r, (raw, _) in enumerate(handles):
                    if problem is None and r != self.rank:
                        p = ct.c_void_p()
                        if self.lib.ssb_peer_buffer_open(raw, ct.byref(p)) != _native.OK:
                            problem = self.lib.ssb_last_error().decode()
                        else:
                            self._mapped.append(p)
                            pointers[r] = p.value
                agree = torch.tensor([0 if problem is None else 1], device=self.device)
                dist.all_reduce(agree, op=dist.ReduceOp.MAX, group=group)  # also: every buffer is zeroed and mapped everywhere
                if int(agree.item()) != 0 and problem is None:
                    problem = "another rank could not map the exchange buffers"
        if problem is not None:
            self.close()
            raise RuntimeError(f"peer exchange set-up failed: {problem}")
        self.struct = _native.PeerExchangeStruct()
        self.struct.world, self.struct.rank, self.struct.rows = self.world, self.rank, self.rows
        for r, p in enumerate(pointers):
            self.struct.buffers[r] = p
        self.epoch = [0, 0]  # forward, backward
        self._check = _native.check
        self._byref = ct.byref

    def close(self) -> None:
        """Unmaps the peers' buffers and frees the own one.  Collective in effect: call it on every
        rank, after the last step has completed everywhere (e.g. behind a barrier)."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._mapped:
                self.lib.ssb_peer_buffer_close(p)
            self._mapped = []
            if self._own is not None and self._own.value:
                self.lib.ssb_peer_buffer_destroy(self._own)
            self._own = None

    @classmethod
    def create(cls, rows: int, group=None, device: Optional[torch.device] = None) -> Optional["PeerCarryExchange"]:
        """An exchange for ``rows`` rows, or None when this job cannot use peer memory (more than 8
        ranks, fewer visible GPUs than ranks, no peer access, IPC refused).  Collective: call it on
        every rank of the group."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        ok = torch.cuda.is_available() and world <= 8
        if ok and world > 1:
            me = torch.cuda.current_device()
            ok = all(torch.cuda.can_device_access_peer(me, d) for d in range(torch.cuda.device_count()) if d != me)
        if world > 1:  # all ranks or none: the constructor is collective
            agree = torch.tensor([1 if ok else 0], device="cuda")
            dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=group)
            ok = int(agree.item()) == 1
        if not ok:
            return None
        try:
            ex = cls(rows, group, device)  # raises on every rank or on none
        except RuntimeError:
            ex = None
        return ex

    def publish_map(self, gate: torch.Tensor, other: torch.Tensor, backward: bool, cut: float,
                    walked: Optional[torch.Tensor] = None) -> None:
        assert gate.shape == other.shape and gate.shape[0] == self.rows and gate.dtype == torch.float32
        d = 1 if backward else 0
        self.epoch[d] += 1
        stream = torch.cuda.current_stream(gate.device).cuda_stream
        self._check(self.lib.ssb_shard_map_publish_f32(gate.data_ptr(), other.data_ptr(), self.rows, gate.shape[1], cut, d,
                                                       self._byref(self.struct), self.epoch[d],
                                                       None if walked is None else walked.data_ptr(), stream))

    def carry(self, backward: bool) -> torch.Tensor:
        d = 1 if backward else 0
        out = torch.empty(self.rows, dtype=torch.float32, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self.lib.ssb_shard_carry_peer_f32(self._byref(self.struct), self.epoch[d], d, out.data_ptr(), stream))
        return out

    @staticmethod
    def usable_for(gate: torch.Tensor) -> bool:
        """The publishing map kernel takes 16-byte aligned fp32 rows of a multiple of 4 steps."""
        return gate.dtype == torch.float32 and gate.shape[1] % 4 == 0 and gate.data_ptr() % 16 == 0


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
                         cut: float = DEFAULT_CUT, walked: Optional[torch.Tensor] = None,
                         exchange: Optional["PeerCarryExchange"] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward of this rank's T-slice. ``gate``/``value``: ``[rows, T_local]`` contiguous.

    Returns ``(h_local, h_in)`` where ``h_in`` (``[rows]``) is h just before the slice.  ``cut``:
    see the module docstring.  ``walked``: optional one-element int64 tensor on the inputs' device
    that accumulates how many elements per tensor the map pass read.  ``exchange``: a
    :class:`PeerCarryExchange` made for this group and row count replaces the all-gather by peer
    stores (every rank has to pass one, or none).
    """
    assert gate.shape == value.shape and gate.dim() == 2
    gate, value = gate.contiguous(), value.contiguous()
    if exchange is not None and exchange.usable_for(gate) and value.data_ptr() % 16 == 0:
        exchange.publish_map(gate, value, False, cut, walked)
        h_in = exchange.carry(False)
    else:
        maps = _gather_maps(ops.map_forward(gate, value, cut, walked), group)
        h_in = ops.carry(maps, _rank(group), False)
    return ops.scan_forward(gate, value, h_in), h_in


def sharded_scan_backward(gate: torch.Tensor, output: torch.Tensor, out_grad: torch.Tensor,
                          h_in: torch.Tensor, group=None, ops: Any = CudaShardOps,
                          cut: float = DEFAULT_CUT, walked: Optional[torch.Tensor] = None,
                          exchange: Optional["PeerCarryExchange"] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Backward of this rank's T-slice; ``h_in`` is what :func:`sharded_scan_forward` returned."""
    assert gate.shape == output.shape == out_grad.shape and gate.dim() == 2
    gate, output, out_grad = gate.contiguous(), output.contiguous(), out_grad.contiguous()
    if exchange is not None and exchange.usable_for(gate) and out_grad.data_ptr() % 16 == 0:
        exchange.publish_map(gate, out_grad, True, cut, walked)
        c_in = exchange.carry(True)
    else:
        maps = _gather_maps(ops.map_backward(gate, out_grad, cut, walked), group)
        c_in = ops.carry(maps, _rank(group), True)
    return ops.scan_backward(gate, output, out_grad, c_in, h_in)


class ShardedScan(torch.autograd.Function):
    """Autograd Function over the local slice; gradients stay sharded like the inputs."""

    @staticmethod
    def forward(ctx: Any, gate: torch.Tensor, value: torch.Tensor, group, ops, cut: float, exchange) -> torch.Tensor:
        rows_shape = gate.shape
        g2, v2 = gate.reshape(-1, rows_shape[-1]), value.reshape(-1, rows_shape[-1])
        out, h_in = sharded_scan_forward(g2, v2, group, ops, cut, exchange=exchange)
        ctx.save_for_backward(g2, out, h_in)
        ctx.group, ctx.ops, ctx.rows_shape, ctx.cut, ctx.exchange = group, ops, rows_shape, cut, exchange
        return out.reshape(rows_shape)

    @staticmethod
    def backward(ctx: Any, output_grad: torch.Tensor):
        gate, out, h_in = ctx.saved_tensors
        gg, gv = sharded_scan_backward(gate, out, output_grad.reshape(gate.shape), h_in, ctx.group, ctx.ops, ctx.cut,
                                       exchange=ctx.exchange)
        return gg.reshape(ctx.rows_shape), gv.reshape(ctx.rows_shape), None, None, None, None


def scan_sequence_parallel(gate: torch.Tensor, value: torch.Tensor, group: Optional[Any] = None,
                           ops: Any = CudaShardOps, cut: float = DEFAULT_CUT,
                           exchange: Optional[PeerCarryExchange] = None) -> torch.Tensor:
    """``scan`` for a sequence sharded along its last axis over ``group`` (default: the world).

    Every rank passes its own ``[N, ..., T_local]`` slice (slices in rank order form the full
    sequence) and receives the matching slice of the result.
    """
    assert gate.shape == value.shape and gate.dim() >= 2
    return ShardedScan.apply(gate, value, group, ops, cut, exchange)
