#!/usr/bin/env python
"""Benchmark of the gated linear scan (fwd + fused bwd) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One *step* is one forward scan plus one fused backward over the workload, i.e. two kernel
launches per GPU.  The default workload is the headline configuration, tensors [8, 2048, 4096]
fp32 scanned over T (16 384 rows of 4096 steps, 268 MB per tensor).

With N > 1 (launched under torch.distributed.run) the rows of that ONE workload are split over the
ranks -- rows are independent, so there is no collective on the data path -- and `value` is the
workload's elements over the slowest rank's time (strong scaling: at N = 8 a rank holds 2048 rows
and a step lasts ~40 us).  A rank's tensors are then comparable to the 126 MB L2, so the timed
steps rotate over several independent buffer sets and no step re-reads what the previous one
left in L2.  The same line carries two more measurements of the N-rank job: `weak` (every rank
runs the whole workload) and `t_sharded` (the long-context configuration, [1, 1024, 2^20], split
along T over the ranks through the sequence-parallel path with its NCCL all-gather of per-shard
carries, checked against the unsharded kernels on a row sample).

Rank 0 prints ONE JSON line.  `value` is Gelem/s with inputs resident in HBM, timed with CUDA
events on the launching stream; `e2e` is the same metric through the public Python operator
with pinned HOST buffers and both directions of PCIe traffic inside the timed region;
`roofline` describes the dominant kernel (the backward, 20 algorithmic bytes per element)
against the measured HBM copy peak; `cpu_baseline` is the reference's own CPU implementation
(compiled from its sources into oracle/_ref) or, if that is absent, the C restatement in
oracle/, timed on this host.

`--impl reference` times that CPU implementation alone, on as many host cores as the process
may use (independent row slices of the same seeded tensors, one process per core), and prints a
line of the same shape.  `--pcie-probe` measures plain pinned-memory copies instead (host to
device, device to host, both at once; one cudaMemcpyAsync per chunk) on every rank at the same
time and prints one JSON line per rank: the ceiling of `e2e`.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

METRIC = "scan Gelem/s fwd+bwd fp32"
L2_BYTES = 126 << 20
# DRAM traffic of the backward kernel as ncu counted it: a small record that the profiling step
# rewrites whenever the kernel changes (see the file itself for the command and the commit).
TRAFFIC_RECORD = os.path.join(REPO, "profiles", "bwd_kernel_dram_traffic.json")
# world sizes at which the peer-memory exchange of the T-sharded path has run on real B200s (tests and
# this bench); at other sizes the default run leaves it out rather than try it first inside the
# measurement every other number of the line depends on
PEER_EXCHANGE_WORLDS = frozenset({2, 4, 8})


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--workload", default="cfg2")
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--scaling", default="auto", choices=["auto", "strong", "weak"],
                   help="rows-sharded workloads on N > 1 ranks: split the one workload (strong, the default) or "
                        "give every rank the whole of it (weak)")
    p.add_argument("--emulate-gpus", type=int, default=1,
                   help="on ONE GPU, run the slice of the workload that a rank of an N-rank strong-scaling job would hold")
    p.add_argument("--variant", type=int, default=0, help="kernel family/tuning id passed to the C-ABI (0 = auto)")
    p.add_argument("--variant-bwd", type=int, default=0, help="as --variant, for the backward only (0 = same as --variant)")
    p.add_argument("--storage", default="f32", choices=["f32", "bf16", "f16"],
                   help="element type of the tensors in HBM (arithmetic is fp32 either way); the headline metric is f32")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--e2e-steps", type=int, default=5)
    p.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of as one CUDA graph")
    p.add_argument("--min-region-ms", type=float, default=500.0,
                   help="when K steps take less than this, the K-step region is repeated and the median reported")
    p.add_argument("--no-t-sharded", action="store_true", help="N > 1: skip the T-sharded long-context measurement")
    p.add_argument("--no-weak", action="store_true", help="N > 1: skip the weak-scaling measurement")
    p.add_argument("--ts-steps", type=int, default=20, help="timed steps of the T-sharded measurement")
    p.add_argument("--peer-exchange", default="auto", choices=["auto", "on", "off"],
                   help="T-sharded measurement: also time the shard maps exchanged through peer memory (auto: at the "
                        "world sizes this exchange has been run at on B200s: 2, 4 and 8)")
    p.add_argument("--cut", type=float, default=None, help="early-termination threshold of the shard maps (default: the library's)")
    p.add_argument("--sets", type=int, default=0,
                   help="independent buffer sets the timed steps rotate over (0 = as many as keep the L2 from serving re-reads; "
                        "1 = one set, i.e. L2-resident when the workload fits)")
    p.add_argument("--pcie-probe", action="store_true")
    return p.parse_args()


def workload_string(w):
    """Names the workload; identical in both arms."""
    return f"{w.name} {list(w.shape)} fp32 fwd+bwd, gates {w.gates}, seed 0"


def common_config(w, world):
    return {
        "workload": workload_string(w),
        "sharding": ("one sequence set split along T over the ranks" if w.sharding == "T" and world > 1
                     else "rows (batch x channel) split over the ranks, no collective"),
        "l2": "no flush: every pass streams tensors that exceed the last-level cache, or rotates over buffer sets that do",
    }


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) in a thread."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost",
               0x100: "display_clock_setting"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self, how: str):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "how": "NVML unavailable"}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples), "how": how}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if local_index < len(ids) and ids[local_index].isdigit():
            return int(ids[local_index])
    return local_index


def usable_cores():
    return sorted(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else list(range(os.cpu_count() or 1))


def bind_rank_to_cores(local_rank: int, local_world: int):
    """Gives each rank of a node its own slice of the usable cores, before it allocates or touches
    any host buffer, so that pinned pages are first touched -- and copy threads run -- on cores no
    other rank is using.  Returns the slice (None when there is nothing to split)."""
    cores = usable_cores()
    if local_world <= 1 or len(cores) < 2 * local_world or not hasattr(os, "sched_setaffinity"):
        return None
    per = len(cores) // local_world
    mine = cores[local_rank * per:(local_rank + 1) * per]
    try:
        os.sched_setaffinity(0, mine)
    except OSError:
        return None
    return mine


# --------------------------------------------------------------------------------------------
# CPU baseline (the reference's own CPU path, or the C restatement)
# --------------------------------------------------------------------------------------------
def cpu_impl():
    """Returns (kind, fwd, bwd) working on torch CPU tensors [rows, T]."""
    import oracle

    if oracle.reference_available():
        return "reference", oracle.reference_forward, oracle.reference_backward
    import torch

    def fwd(a, b):
        return torch.from_numpy(oracle.scan_forward(a.numpy(), b.numpy()))

    def bwd(a, h, g):
        ga, gb = oracle.scan_backward(a.numpy(), h.numpy(), g.numpy())
        return torch.from_numpy(ga), torch.from_numpy(gb)

    return "port", fwd, bwd


def time_cpu_single(a, b, g, reps: int = 2):
    """Single-core fwd+bwd over the given rows; returns (Gelem/s, kind)."""
    kind, fwd, bwd = cpu_impl()
    n = a.numel()
    h = fwd(a[:256], b[:256])  # warm-up (page in code and allocator)
    bwd(a[:256], h, g[:256])
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        h = fwd(a, b)
        bwd(a, h, g)
        times.append(time.perf_counter() - t0)
    return n / statistics.median(times) / 1e9, kind


def _cpu_worker(core, a, b, g, n_steps, warmup, barrier):
    import torch

    torch.set_num_threads(1)
    if core is not None and hasattr(os, "sched_setaffinity"):
        try:
            os.sched_setaffinity(0, {core})
        except OSError:
            pass
    _, fwd, bwd = cpu_impl()
    for _ in range(warmup + n_steps):
        barrier.wait()
        h = fwd(a, b)
        bwd(a, h, g)
        barrier.wait()


def run_reference_arm(args, workload):
    """The reference's CPU implementation on all usable host cores.  The workload's seeded tensors
    (the ones the GPU arm's rank 0 uses) are generated once, the rows are split into one contiguous
    slice per core, and a step is one forward + backward over ALL rows."""
    import multiprocessing as mp

    import torch

    from scanscam_b200.workloads import workload_inputs

    torch.set_num_threads(1)  # no thread pool in the parent: the workers are forked from it
    kind, _, _ = cpu_impl()
    cores = usable_cores()
    procs = max(1, min(len(cores), 64, workload.rows))
    a, b, g = (x.reshape(workload.rows, workload.steps) for x in workload_inputs(workload.name, seed=0))
    bounds = [workload.rows * i // procs for i in range(procs + 1)]
    ctx = mp.get_context("fork")
    barrier = ctx.Barrier(procs + 1)
    workers = [ctx.Process(target=_cpu_worker,
                           args=(cores[r] if len(cores) >= procs else None, a[bounds[r]:bounds[r + 1]],
                                 b[bounds[r]:bounds[r + 1]], g[bounds[r]:bounds[r + 1]], args.steps, args.warmup, barrier))
               for r in range(procs)]
    for w in workers:
        w.start()
    for _ in range(args.warmup):
        barrier.wait()
        barrier.wait()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        barrier.wait()
        barrier.wait()
    elapsed = time.perf_counter() - t0
    for w in workers:
        w.join()
    value = workload.elements * args.steps / elapsed / 1e9
    sample = (f"all {workload.rows} rows x T={workload.steps} per step, {workload.rows // procs}-"
              f"{-(-workload.rows // procs)} rows on each of {procs} processes (one per usable core)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "Gelem/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.scaling == "weak" else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": common_config(workload, args.gpus),
        "timed": "host wall clock around the K steps, CPU only",
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": procs, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def measured_peak():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


def kernel_source_digest():
    """Digest of the kernel sources the traffic record has to match."""
    h = hashlib.sha256()
    csrc = os.path.join(REPO, "scanscam_b200", "csrc")
    for name in ("scan_tma_flat.cuh", "scan_tma.cuh", "scan_common.cuh"):
        with open(os.path.join(csrc, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def recorded_traffic(workload_name: str, n_elems: int):
    """(bytes per launch or None, note): the ncu DRAM-traffic record scaled to this launch, if it was
    taken on this workload's kernel and the kernel sources have not changed since."""
    try:
        with open(TRAFFIC_RECORD) as f:
            rec = json.load(f)
    except Exception:
        return None, "no ncu traffic record (profiles/bwd_kernel_dram_traffic.json)"
    if workload_name not in rec.get("valid_for", []):
        return None, f"the ncu traffic record covers {rec.get('valid_for')}, not this workload"
    if rec.get("kernel_source_digest") != kernel_source_digest():
        return None, "kernel sources changed since the ncu traffic record was taken: capture it again"
    return rec["dram_bytes_per_elem"] * n_elems, rec.get("source", "")


class RowsProblem:
    """`sets` independent copies of a [rows, T] problem on the device plus the two launch closures."""

    def __init__(self, lib, native, torch, a_cpu, b_cpu, g_cpu, storage, sets, variant, variant_bwd):
        self.lib, self.native, self.torch = lib, native, torch
        self.rows, self.T = a_cpu.shape
        self.n = self.rows * self.T
        self.storage = storage
        dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[storage]
        self.elem = torch.empty((), dtype=dt).element_size()
        self.sets = []
        for _ in range(sets):
            a, b, g = (x.cuda().to(dt) for x in (a_cpu, b_cpu, g_cpu))
            self.sets.append((a, b, g, torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)))
        rows, T = self.rows, self.T
        if storage == "f32":
            # Kernel choice and scratch exactly as the PyTorch extension does it: ask the library, give it
            # the workspace it wants (allocated once here, outside the timed region, and reused).
            self.v_fwd = variant or lib.ssb_scan_recommend(rows, T, 0, 1, 1)
            self.v_bwd = variant_bwd or variant or lib.ssb_scan_recommend(rows, T, 1, 1, 1)
            self.ws_bytes = max(lib.ssb_scan_workspace_bytes(rows, T, self.v_fwd),
                                lib.ssb_scan_workspace_bytes(rows, T, self.v_bwd))
        else:  # 16-bit storage, fp32 arithmetic: the library picks the kernel, no workspace
            self.v_fwd = self.v_bwd = self.ws_bytes = 0
        self.ws = torch.empty(max(self.ws_bytes, 1), dtype=torch.uint8, device="cuda")
        self.ws_ptr = self.ws.data_ptr() if self.ws_bytes else None

    def fwd(self, stream, k=0):
        a, b, g, h, ga, gb = self.sets[k % len(self.sets)]
        lib, check = self.lib, self.native.check
        if self.storage == "f32":
            check(lib.ssb_scan_fwd_f32_ex(a.data_ptr(), b.data_ptr(), h.data_ptr(), self.rows, self.T, None, self.v_fwd,
                                          self.ws_ptr, self.ws_bytes, stream))
        else:
            check(getattr(lib, f"ssb_scan_fwd_{self.storage}")(a.data_ptr(), b.data_ptr(), h.data_ptr(), self.rows, self.T,
                                                              None, stream))

    def bwd(self, stream, k=0):
        a, b, g, h, ga, gb = self.sets[k % len(self.sets)]
        lib, check = self.lib, self.native.check
        if self.storage == "f32":
            check(lib.ssb_scan_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), self.rows,
                                          self.T, None, None, self.v_bwd, self.ws_ptr, self.ws_bytes, stream))
        else:
            check(getattr(lib, f"ssb_scan_bwd_{self.storage}")(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(),
                                                              gb.data_ptr(), self.rows, self.T, None, None, stream))

    def step(self, stream, k=0):
        self.fwd(stream, k)
        self.bwd(stream, k)


class Timer:
    """Times K-step regions on the device: barrier + synchronize on both sides, CUDA events on the
    launching stream, maximum over the ranks."""

    def __init__(self, torch, dist, world):
        self.torch, self.dist, self.world = torch, dist, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device="cuda", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]

    def region_ms(self, run):
        """One region: `run()` enqueues the K steps."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record(self.stream)
        run()
        e1.record(self.stream)
        self.barrier()
        return e0.elapsed_time(e1)

    def measure(self, run, min_region_ms, max_repeats=200):
        """Runs the region once; if it is shorter than `min_region_ms`, repeats it until that much
        device time has been covered.  Returns (median region ms over the repeats, each the max over
        ranks; number of repeats)."""
        first = self.max_over_ranks([self.region_ms(run)])[0]
        repeats = 1
        if first < min_region_ms:
            repeats = int(min(max_repeats, max(3, math.ceil(min_region_ms / max(first, 1e-3)))))
        local = [first] + [self.region_ms(run) for _ in range(repeats - 1)]
        per_repeat = self.max_over_ranks(local) if repeats > 1 else [first]
        return statistics.median(per_repeat), repeats


def capture_graph(torch, stream, problem, steps):
    """The K steps recorded once into a CUDA graph (the kernels take raw pointers and a stream, so
    they capture like any other launch).  Returns the graph or None."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                cap = torch.cuda.current_stream().cuda_stream
                for k in range(steps):
                    problem.step(cap, k)
        stream.wait_stream(side)
        graph.replay()  # one untimed replay: instantiation and upload happen here
        torch.cuda.synchronize()
        return graph
    except Exception as exc:  # pragma: no cover - depends on driver/torch support
        print(f"bench.py: CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
        return None


def measure_rows(args, torch, timer, problem, steps, min_region_ms, use_graph=True):
    """(ms per step, repeats, launch description) of K steps of a rows problem."""
    st = timer.stream.cuda_stream
    for k in range(max(args.warmup, 3)):
        problem.step(st, k)
    timer.barrier()
    graph = capture_graph(torch, timer.stream, problem, steps) if use_graph else None

    def run():
        if graph is not None:
            graph.replay()
        else:
            for k in range(steps):
                problem.step(st, k)

    ms, repeats = timer.measure(run, min_region_ms)
    return ms / steps, repeats, ("one CUDA graph of K x (forward, backward)" if graph is not None else "K x 2 stream launches")


def measure_t_sharded(args, torch, dist, timer, lib, native, workloads, world, rank):
    """cfg3 split along T over the ranks through scanscam_b200.sharded (NCCL all-gather of the shard
    maps); returns the `t_sharded` record (rank 0) after checking a row sample against the unsharded
    kernels."""
    from scanscam_b200 import sharded

    w = workloads.WORKLOADS["cfg3"]
    rows, T = w.rows, w.steps
    if T % world:
        return {"skipped": f"T={T} is not divisible by {world} ranks"}
    T_local = T // world
    cut = sharded.DEFAULT_CUT if args.cut is None else args.cut
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
    a = torch.rand(rows, T_local, generator=gen, device="cuda").mul_(0.01).add_(0.99)  # cfg3's gates: U(0.99, 1)
    b = torch.randn(rows, T_local, generator=gen, device="cuda").mul_(0.1)
    g = torch.randn(rows, T_local, generator=gen, device="cuda")
    walked = torch.zeros(1, dtype=torch.int64, device="cuda")
    steps = max(1, args.ts_steps)
    idx = torch.arange(3, rows, rows // 8, device="cuda")[:8]
    n_local = rows * T_local

    def measure(exchange):
        """(ms per step, elements walked by the map kernels in one step, max error on the row sample)."""
        out = {}

        def step(count=None):
            h, h_in = sharded.sharded_scan_forward(a, b, cut=cut, walked=count, exchange=exchange)
            ga, gb = sharded.sharded_scan_backward(a, h, g, h_in, cut=cut, walked=count, exchange=exchange)
            out["h"], out["ga"], out["gb"] = h, ga, gb

        timer.barrier()
        for _ in range(3):
            step()
        ms = timer.max_over_ranks([timer.region_ms(lambda: [step() for _ in range(steps)])])[0] / steps
        walked.zero_()
        step(walked)
        torch.cuda.synchronize()
        walked_all = timer.max_over_ranks([float(walked.item())])[0]  # per tensor, forward + backward, slowest rank
        # a row sample against the unsharded kernels on rank 0
        sample = [x[idx].contiguous() for x in (a, b, g, out["h"], out["ga"], out["gb"])]
        gathered = []
        for x in sample:
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            gathered.append(torch.cat(parts, dim=1))
        max_err = None
        if rank == 0:
            fa, fb, fg, sh, sga, sgb = gathered
            r, st = fa.shape[0], timer.stream.cuda_stream
            h1, ga1, gb1 = torch.empty_like(fa), torch.empty_like(fa), torch.empty_like(fa)
            native.check(lib.ssb_scan_fwd_f32(fa.data_ptr(), fb.data_ptr(), h1.data_ptr(), r, T, None, st))
            native.check(lib.ssb_scan_bwd_f32(fa.data_ptr(), h1.data_ptr(), fg.data_ptr(), ga1.data_ptr(), gb1.data_ptr(), r, T,
                                              None, None, st))
            torch.cuda.synchronize()
            max_err = max(float((x - y).abs().max() / y.abs().max()) for x, y in ((sh, h1), (sga, ga1), (sgb, gb1)))
        return ms, walked_all, max_err

    ms, walked_all, max_err = measure(None)
    # the same steps with the maps exchanged through peer memory instead of NCCL, where the box allows it
    peer = {"unavailable": "peer memory exchange could not be set up (GPUs not all visible, no peer access, or IPC refused)"}
    want_peer = args.peer_exchange == "on" or (args.peer_exchange == "auto" and world in PEER_EXCHANGE_WORLDS)
    if not want_peer:
        peer = {"skipped": f"--peer-exchange {args.peer_exchange}: measured by default only at world sizes {sorted(PEER_EXCHANGE_WORLDS)}, "
                           "where it has been run on B200s; --peer-exchange on forces it"}
    try:
        exchange = sharded.PeerCarryExchange.create(rows) if want_peer else None
        if exchange is not None:
            p_ms, _, p_err = measure(exchange)
            peer = {"value": rows * T / (p_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": p_ms,
                    "max_err_vs_unsharded": p_err, "launches_per_step_per_rank": 6,
                    "what": "map kernels store into every rank's buffer over NVLink and raise a flag; the carry kernels wait "
                            "(bounded) for all ranks' flags: no collective call"}
            timer.barrier()
            exchange.close()
    except Exception as exc:
        peer = {"failed": f"{type(exc).__name__}: {exc}"}
    del a, b, g
    torch.cuda.empty_cache()
    return {
        "workload": f"cfg3 {list(w.shape)} fp32 fwd+bwd, gates {w.gates}, T split over {world} ranks",
        "value": rows * T / (ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": ms, "steps": steps,
        "bytes_moved_per_elem": 32.0 + 8.0 * walked_all / n_local,
        "map_walk": {"cut": cut, "elements_per_row_and_direction": walked_all / rows / 2, "shard_length": T_local},
        "collective": "2 x NCCL all_gather of [rows, 2] fp32 per step",
        "max_err_vs_unsharded": max_err, "checked": "8 rows x full T: h, grad_gate, grad_value against ssb_scan_fwd/bwd_f32 on one GPU",
        "launches_per_step_per_rank": 6, "peer_exchange": peer,
    }


def pcie_probe(args):
    """Plain pinned-memory copies on every rank at once; one JSON line per rank."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cores = bind_rank_to_cores(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", world)))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n_bytes, chunk = 1 << 30, 64 << 20
    host_in = torch.empty(n_bytes, dtype=torch.uint8).pin_memory()
    host_out = torch.empty(n_bytes, dtype=torch.uint8).pin_memory()
    host_in.fill_(1)
    host_out.fill_(2)
    dev_in = torch.empty(n_bytes, dtype=torch.uint8, device="cuda")
    dev_out = torch.ones(n_bytes, dtype=torch.uint8, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def h2d():
        with torch.cuda.stream(s_in):
            for o in range(0, n_bytes, chunk):
                dev_in[o:o + chunk].copy_(host_in[o:o + chunk], non_blocking=True)

    def d2h():
        with torch.cuda.stream(s_out):
            for o in range(0, n_bytes, chunk):
                host_out[o:o + chunk].copy_(dev_out[o:o + chunk], non_blocking=True)

    def timed(fns, reps=4):
        best = float("inf")
        for _ in range(reps):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for f in fns:
                f()
            torch.cuda.synchronize()
            best = min(best, time.perf_counter() - t0)
        return n_bytes / best / 1e9

    res = {"rank": rank, "world": world, "gpu": physical_gpu_index(local_rank), "cores": cores,
           "bytes": n_bytes, "chunk_bytes": chunk,
           "h2d_gbs": timed([h2d]), "d2h_gbs": timed([d2h]), "both_gbs_per_direction": timed([h2d, d2h])}
    # which NUMA node the pinned pages sit on, where the kernel says (first page of each buffer)
    try:
        with open("/proc/self/numa_maps") as f:
            res["numa_nodes_seen"] = sorted({tok.split("=")[0] for line in f for tok in line.split() if tok.startswith("N") and "=" in tok})
    except Exception:
        res["numa_nodes_seen"] = None
    for r in range(world):
        if world > 1:
            dist.barrier()
        if r == rank:
            print(json.dumps({"pcie_probe": res}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_gpu_arm(args, workload):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # before anything allocates host memory: this rank's own cores (first touch of pinned pages, copy threads)
    cores = bind_rank_to_cores(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", world)))

    import torch
    import torch.distributed as dist

    from scanscam_b200 import _native, build, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build.build_library()
    lib = _native.load()  # raises when the native library is missing
    timer = Timer(torch, dist, world)
    t_sharded_main = workload.sharding == "T" and world > 1
    rows, T = workload.rows, workload.steps
    emulate = max(1, args.emulate_gpus) if world == 1 else 1
    parts = world * emulate  # how many slices the workload's rows are cut into
    strong = (not t_sharded_main) and parts > 1 and args.scaling != "weak"
    if args.storage != "f32" and t_sharded_main:
        raise SystemExit("bench.py: --storage bf16/f16 is measured on the row-sharded workloads only")

    line = {
        "metric": METRIC, "unit": "Gelem/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "vs_baseline": None,
        "dtype": "f32" if args.storage == "f32" else f"f32 arithmetic on {args.storage} tensors", "data": "synthetic",
        "config": common_config(workload, world),
    }
    if max(args.warmup, 3) != args.warmup:
        line["warmup_run"] = max(args.warmup, 3)
    if emulate > 1:
        line["emulated_world"] = emulate
    sampler = ClockSampler(physical_gpu_index(local_rank))

    if t_sharded_main:
        # ---- the sequence-parallel path as the main measurement (--workload cfg3 --gpus N) -----
        assert T % world == 0
        from scanscam_b200 import sharded

        T_local = T // world
        cut = sharded.DEFAULT_CUT if args.cut is None else args.cut
        a_cpu, b_cpu, g_cpu = workloads.make_inputs(workload.gates, (rows, T_local), seed=rank)  # this rank's T-slice
        a, b, g = a_cpu.cuda(), b_cpu.cuda(), g_cpu.cuda()
        del a_cpu, b_cpu, g_cpu

        def step():
            hh, h_in = sharded.sharded_scan_forward(a, b, cut=cut)
            sharded.sharded_scan_backward(a, hh, g, h_in, cut=cut)

        for _ in range(max(args.warmup, 3)):
            step()
        sampler.start()
        total_ms, repeats = timer.measure(lambda: [step() for _ in range(args.steps)], args.min_region_ms)
        sampler.stop()
        ms_per_step = total_ms / args.steps
        line.update({"value": rows * T / (ms_per_step * 1e-3) / 1e9, "ms_per_step": ms_per_step, "scaling": "strong",
                     "repeats": repeats, "launch": "per step: 2 x (map kernel, NCCL all_gather, carry kernel, scan kernel)",
                     "gpu_launches": 6 * args.steps * world,
                     "clocks": sampler.summary("NVML samples every 20 ms during the timed region")})
        _check_status(lib, _native)
        if rank == 0:
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
        return

    # ---- rows-sharded workloads ------------------------------------------------------------
    full_cpu = tuple(x.reshape(rows, T) for x in workloads.workload_inputs(workload.name, seed=0))
    if strong:
        slice_id = rank if world > 1 else 0
        lo, hi = rows * slice_id // parts, rows * (slice_id + 1) // parts
        mine_cpu = tuple(x[lo:hi].contiguous() for x in full_cpu)
    else:
        mine_cpu = full_cpu
    rows_local = mine_cpu[0].shape[0]
    n_local = rows_local * T
    elem = 4 if args.storage == "f32" else 2
    working_set = 6 * n_local * elem
    sets = args.sets or (1 if working_set >= 8 * L2_BYTES else min(8, max(4, math.ceil(8 * L2_BYTES / working_set))))
    problem = RowsProblem(lib, _native, torch, *mine_cpu, args.storage, sets, args.variant, args.variant_bwd)
    sampler.start()
    ms_per_step, repeats, launch = measure_rows(args, torch, timer, problem, args.steps, args.min_region_ms,
                                                use_graph=not args.no_graph)
    sampler.stop()
    total_elems = n_local * world if not strong else (workload.elements if world > 1 else n_local)
    value = total_elems / (ms_per_step * 1e-3) / 1e9
    line.update({
        "value": value, "ms_per_step": ms_per_step, "scaling": "weak" if args.scaling == "weak" else "strong",
        "repeats": repeats, "launch": launch,
        "per_gpu": {"rows": rows_local, "elements": n_local, "working_set_bytes": working_set, "buffer_sets": sets,
                    "l2": (f"{sets} independent buffer sets in rotation ({sets * working_set >> 20} MiB) so that no step re-reads "
                           "what the previous one left in the 126 MB L2") if sets > 1 else
                          ("one buffer set: every pass streams far more than the 126 MB L2" if working_set > 2 * L2_BYTES else
                           "one buffer set that fits the 126 MB L2: an L2-resident measurement")},
        "kernels": {"forward": problem.v_fwd, "backward": problem.v_bwd, "workspace_bytes": problem.ws_bytes},
        "gpu_launches": 2 * args.steps * world,
        "clocks": sampler.summary("NVML samples every 20 ms during the timed region" +
                                  (f" ({repeats} repeats of the K-step region)" if repeats > 1 else "")),
    })
    if cores is not None:
        line["host_cores_per_rank"] = len(cores)

    # ---- per-kernel durations for the roofline: K steps again, an event after every launch
    # (kept out of the region above, where the extra event records would cost ~1 %) -----
    st = timer.stream.cuda_stream
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    timer.barrier()
    ev[0].record(timer.stream)
    for i in range(args.steps):
        problem.fwd(st, i)
        ev[2 * i + 1].record(timer.stream)
        problem.bwd(st, i)
        ev[2 * i + 2].record(timer.stream)
    timer.barrier()
    fwd_ms = sum(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps))
    bwd_ms = sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps))
    fwd_total, bwd_total = timer.max_over_ranks([fwd_ms, bwd_ms])
    _check_status(lib, _native)

    # ---- N > 1: the same job measured the other two ways -------------------------------------
    weak = t_sharded = None
    if world > 1 and strong and not args.no_weak and args.storage == "f32":
        whole = RowsProblem(lib, _native, torch, *full_cpu, args.storage, 1, args.variant, args.variant_bwd)
        w_steps = min(args.steps, 50)
        w_ms, w_rep, _ = measure_rows(args, torch, timer, whole, w_steps, min(args.min_region_ms, 100.0),
                                      use_graph=not args.no_graph)
        weak = {"value": workload.elements * world / (w_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": w_ms,
                "steps": w_steps, "repeats": w_rep, "what": "every rank runs the whole workload on its own copy"}
        del whole
        torch.cuda.empty_cache()

    # ---- end to end through the public operator, host buffers -------------------------------
    e2e = None
    if not args.no_e2e and args.storage == "f32":
        e2e = measure_e2e(args, torch, timer, problem, mine_cpu, total_elems, world)

    if world > 1 and not args.no_t_sharded and args.storage == "f32":
        del problem
        torch.cuda.empty_cache()
        try:
            t_sharded = measure_t_sharded(args, torch, dist, timer, lib, _native, workloads, world, rank)
        except Exception as exc:  # the main measurement stands; say what happened
            t_sharded = {"failed": f"{type(exc).__name__}: {exc}"}
        try:  # a bounded wait that ran out in the sharded steps is reported in their record, not raised
            _check_status(lib, _native)
        except Exception as exc:
            t_sharded["device_status"] = str(exc)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    bwd_avg_s = bwd_total / args.steps * 1e-3
    fwd_avg_s = fwd_total / args.steps * 1e-3
    bytes_fwd, bytes_bwd = 3 * elem, 5 * elem  # per element: read a, b + write h | read a, h, g + write both gradients
    achieved = bytes_bwd * n_local / bwd_avg_s / 1e9
    traffic, traffic_note = recorded_traffic(workload.name, n_local) if elem == 4 else (None, "no ncu record for 16-bit storage")
    both = (bytes_fwd + bytes_bwd) * n_local / (fwd_avg_s + bwd_avg_s) / 1e9
    line["roofline"] = {
        "bound": "hbm", "kernel": "fused backward (reads a, h, g; writes grad_a, grad_b)",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
        "traffic": traffic, "traffic_source": traffic_note,
        "algorithmic_bytes_per_launch": bytes_bwd * n_local, "avg_launch_ms": bwd_avg_s * 1e3,
        "forward": {"achieved": bytes_fwd * n_local / fwd_avg_s / 1e9, "frac": bytes_fwd * n_local / fwd_avg_s / 1e9 / peak,
                    "avg_launch_ms": fwd_avg_s * 1e3},
        "fwd_plus_bwd": {"achieved": both, "frac_of_measured": both / peak, "frac_of_8TBps": both / 8000.0},
    }
    if e2e is not None:
        line["e2e"] = e2e
    if weak is not None:
        line["weak"] = weak
    if t_sharded is not None:
        line["t_sharded"] = t_sharded
    if world == 1 and emulate == 1 and not args.no_cpu_baseline and args.storage == "f32":
        a_cpu, b_cpu, g_cpu = mine_cpu
        sample_rows = rows_local if n_local <= (1 << 26) else max(1, (1 << 26) // T)
        v, kind = time_cpu_single(a_cpu[:sample_rows], b_cpu[:sample_rows], g_cpu[:sample_rows])
        line["cpu_baseline"] = {"value": v, "unit": "Gelem/s", "cores": 1, "kind": kind,
                                "sample": f"{sample_rows} of {rows_local} rows x T={T}, median of 2 passes, "
                                          f"single thread (the reference's CPU path has no threading)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _check_status(lib, native):
    detail = native.ctypes.c_int(0)
    native.check(lib.ssb_device_status(native.ctypes.byref(detail)))


def measure_e2e(args, torch, timer, problem, mine_cpu, total_elems, world):
    """The same metric through scanscam_b200.host.HostScanPipeline: pinned host tensors in, results
    in pinned host tensors, every step copies its inputs in and its results out."""
    from scanscam_b200.host import HostScanPipeline

    rows_local, T = mine_cpu[0].shape
    n_local = rows_local * T
    pin = [x.pin_memory() for x in mine_cpu]
    outs = tuple(torch.empty_like(x).pin_memory() for x in mine_cpu)
    # chunks of at least ~16 MB per tensor keep both copy engines streaming; at most 16 chunks
    chunks = int(min(16, max(2, n_local * 4 // (16 << 20))))
    pipe = HostScanPipeline(rows_local, T, chunks=chunks)
    stream = timer.stream

    def e2e_step():
        pipe.run(pin[0], pin[1], pin[2], outs)

    e2e_step()
    steps = max(1, args.e2e_steps)
    e2e_ms = timer.max_over_ranks([timer.region_ms(lambda: [e2e_step() for _ in range(steps)])])[0] / steps
    # spot-check the host results of the last step against the device-resident run
    torch.cuda.synchronize()
    problem.fwd(stream.cuda_stream, 0)
    torch.cuda.synchronize()
    assert torch.allclose(outs[0][:64], problem.sets[0][3][:64].float().cpu(), rtol=1e-5, atol=1e-6), \
        "end-to-end pipeline result differs from the resident run"

    # the link's own ceiling for this traffic: the same bytes, both directions at once, no kernels
    dev = [torch.empty_like(x, device="cuda") for x in mine_cpu]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copies_only():
        s_in.wait_stream(stream)
        s_out.wait_stream(stream)
        with torch.cuda.stream(s_in):
            for d, h in zip(dev, pin):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            for d, h in zip(dev, outs):
                h.copy_(d, non_blocking=True)
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)

    copies_only()
    link_ms = timer.max_over_ranks([timer.region_ms(lambda: [copies_only() for _ in range(3)])])[0] / 3
    return {"value": total_elems / (e2e_ms * 1e-3) / 1e9, "unit": "Gelem/s",
            "h2d_bytes_per_step": 3 * 4 * n_local, "d2h_bytes_per_step": 3 * 4 * n_local,
            "ms_per_step": e2e_ms, "steps": steps,
            "link_ceiling": {"value": total_elems / (link_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": link_ms,
                             "gbs_per_direction": 3 * 4 * n_local / (link_ms * 1e-3) / 1e9,
                             "what": "the step's host-to-device and device-to-host bytes copied at the same time from and to "
                                     "the same pinned buffers, no kernels: what the PCIe link allows for this metric"},
            "api": f"scanscam_b200.host.HostScanPipeline.run(gate, value, grad): pinned host tensors in, "
                   f"h / grad_gate / grad_value written to pinned host tensors; {pipe.n_chunks} row chunks, copies in both "
                   "directions overlapped with the kernels on three streams"}


def main():
    args = parse_args()
    if args.pcie_probe:
        pcie_probe(args)
        return
    from scanscam_b200.workloads import WORKLOADS

    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference_arm(args, workload)
        return
    run_gpu_arm(args, workload)


if __name__ == "__main__":
    main()
