"""Seeded synthetic workloads: the five benchmark configurations of the gated linear scan.

The reference measures on no dataset (its tests draw ``torch.randn`` on the fly,
scanscam/cuda_test.py:26-31), so every workload here is synthetic: shapes and gate
distributions follow the benchmark configurations, values are drawn on the CPU from
``torch.Generator().manual_seed(seed)`` in the fixed order *gate noise, value, upstream
gradient* and then copied to the device, so a CPU checker and the kernels see identical bits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    shape: Tuple[int, int, int]  # [B, C, T], scanned over T
    gates: str                   # gate distribution, see make_inputs
    sharding: str                # how it partitions across GPUs: "rows" or "T"
    note: str

    @property
    def rows(self) -> int:
        return self.shape[0] * self.shape[1]

    @property
    def steps(self) -> int:
        return self.shape[2]

    @property
    def elements(self) -> int:
        return self.rows * self.steps


WORKLOADS = {
    "cfg1": Workload("cfg1", (4, 256, 1024), "sigmoid2", "rows", "CPU-runnable reference case; fits in L2"),
    "cfg2": Workload("cfg2", (8, 2048, 4096), "sigmoid2", "rows", "training-size layer (headline)"),
    "cfg3": Workload("cfg3", (1, 1024, 1048576), "nearunit", "T", "long-context stress, near-unit gates"),
    "cfg4": Workload("cfg4", (64, 8192, 512), "sigmoid0", "rows", "wide, short sequences"),
    "cfg2q": Workload("cfg2q", (2, 2048, 4096), "sigmoid2", "rows", "a quarter of cfg2: small case for profiler captures"),
    "cfg3q": Workload("cfg3q", (1, 64, 262144), "nearunit", "T", "64 long rows: small case of cfg3 for profiler captures"),
    "cfg5": Workload("cfg5", (16, 4096, 2048), "resets", "rows", "mixed gates with exact zeros"),
}


def make_inputs(gates: str, shape, seed: int = 0, dtype: torch.dtype = torch.float32,
                rows: Optional[slice] = None):
    """Returns CPU tensors ``(gate, value, out_grad)`` of ``shape``.

    gates: ``sigmoid2`` a = sigmoid(N(0,1)+2) (median 0.88) | ``sigmoid0`` a = sigmoid(N(0,1)) |
    ``nearunit`` a ~ U(0.99, 1), value ~ 0.1*N(0,1) | ``resets`` a = U(0,1) with exact zeros
    w.p. 0.1 | ``randn`` a ~ N(0,1) (the reference's test inputs: negative and >1 gates) |
    ``ones`` a = 1 (a plain cumulative sum: the gate product never vanishes).
    """
    gen = torch.Generator().manual_seed(seed)

    def randn():
        return torch.randn(shape, generator=gen, dtype=dtype)

    def rand():
        return torch.rand(shape, generator=gen, dtype=dtype)

    if gates == "sigmoid2":
        a = torch.sigmoid_(randn().add_(2.0))
        b = randn()
    elif gates == "sigmoid0":
        a = torch.sigmoid_(randn())
        b = randn()
    elif gates == "nearunit":
        a = rand().mul_(0.01).add_(0.99)
        b = randn().mul_(0.1)
    elif gates == "resets":
        a = rand()
        a.mul_((rand() >= 0.1).to(dtype))
        b = randn()
    elif gates == "randn":
        a = randn()
        b = randn()
    elif gates == "ones":
        a = torch.ones(shape, dtype=dtype)
        b = randn()
    else:
        raise ValueError(f"unknown gate distribution {gates!r}")
    g = randn()
    return a, b, g


def workload_inputs(name: str, seed: int = 0):
    """CPU tensors ``(gate, value, out_grad)`` of a named configuration, shaped ``[B, C, T]``."""
    w = WORKLOADS[name]
    return make_inputs(w.gates, w.shape, seed)
