#!/usr/bin/env python
"""Benchmark of the gated linear scan (fwd + fused bwd) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One *step* is one forward scan plus one fused backward over the whole workload, i.e. two kernel
launches per GPU.  The default workload is the headline configuration, tensors [8, 2048, 4096]
fp32 scanned over T (16 384 rows of 4096 steps, 268 MB per tensor, so every pass streams far
more than the 126 MB L2).  With N > 1 (launched under torch.distributed.run) every rank runs the
same per-GPU workload on its own rows -- rows are independent, so there is no collective on the
data path -- and the value is total elements over the slowest rank's time (weak scaling).  The
`cfg3` workload (one long sequence per row) is instead split along T across the ranks and uses
the sequence-parallel path with its NCCL all-gather of per-shard carries.

Rank 0 prints ONE JSON line.  `value` is Gelem/s with inputs resident in HBM, timed with CUDA
events on the launching stream; `e2e` is the same metric through the public Python operator
with pinned HOST buffers and both directions of PCIe traffic inside the timed region;
`roofline` describes the dominant kernel (the backward, 20 algorithmic bytes per element)
against the measured HBM copy peak; `cpu_baseline` is the reference's own CPU implementation
(compiled from its sources into oracle/_ref) or, if that is absent, the C restatement in
oracle/, timed on this host.

`--impl reference` times that CPU implementation alone, on as many host cores as the process
may use (independent row slices, one process per core), and prints a line of the same shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

METRIC = "scan Gelem/s fwd+bwd fp32"
BYTES_FWD, BYTES_BWD = 12, 20  # algorithmic bytes per element: read a,b write h | read a,h,g write ga,gb

# DRAM traffic per element of the backward kernel measured with ncu on the full cfg2 launch
# (dram__bytes_read.sum + dram__bytes_write.sum = 805.4 MB + 493.2 MB over 67 108 864 elements; the
# reads equal the algorithmic 12 B/element, the writes fall short of 8 B/element because the last
# ~40 MB of results are still in L2 when the kernel ends).  See profiles/tma_flat_kernels_cfg2.md.
NCU_BWD_TRAFFIC_BYTES_PER_ELEM = 19.35


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--workload", default="cfg2")
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--variant", type=int, default=0, help="kernel family/tuning id passed to the C-ABI (0 = auto)")
    p.add_argument("--variant-bwd", type=int, default=0, help="as --variant, for the backward only (0 = same as --variant)")
    p.add_argument("--storage", default="f32", choices=["f32", "bf16", "f16"],
                   help="element type of the tensors in HBM (arithmetic is fp32 either way); the headline metric is f32")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--e2e-steps", type=int, default=5)
    p.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of as one CUDA graph")
    return p.parse_args()


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


def _cpu_worker(rank, rows, steps_T, n_steps, warmup, barrier, gates):
    import torch

    torch.set_num_threads(1)
    from scanscam_b200.workloads import make_inputs

    _, fwd, bwd = cpu_impl()
    a, b, g = make_inputs(gates, (rows, steps_T), seed=100 + rank)
    for _ in range(warmup + n_steps):
        barrier.wait()
        h = fwd(a, b)
        bwd(a, h, g)
        barrier.wait()


def run_reference_arm(args, workload):
    """The reference's CPU implementation on all usable host cores: independent row slices, one
    process per core; a step processes `sample_rows` rows of the workload."""
    import multiprocessing as mp

    kind, _, _ = cpu_impl()
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    procs = max(1, min(cores, 64))
    rows_each = max(1, min(512, workload.rows // procs))
    sample_rows = rows_each * procs
    ctx = mp.get_context("fork")
    barrier = ctx.Barrier(procs + 1)
    workers = [ctx.Process(target=_cpu_worker, args=(r, rows_each, workload.steps, args.steps, args.warmup, barrier,
                                                     workload.gates)) for r in range(procs)]
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
    elems = sample_rows * workload.steps
    value = elems * args.steps / elapsed / 1e9
    sample = (f"{sample_rows} of {workload.rows} rows x T={workload.steps} per step "
              f"({rows_each} rows on each of {procs} processes)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "Gelem/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{workload.name} {list(workload.shape)} fp32 fwd+bwd, gates {workload.gates}",
                   "timed": "host wall clock, CPU only"},
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
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def run_gpu_arm(args, workload):
    import torch
    import torch.distributed as dist

    from scanscam_b200 import _native, build, workloads
    import scanscam_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build.build_library()
    lib = _native.load()  # raises when the native library is missing
    t_sharded = workload.sharding == "T" and world > 1

    rows, T = workload.rows, workload.steps
    if t_sharded:
        assert T % world == 0
        T_local = T // world
        full = workloads.make_inputs(workload.gates, (rows, T_local), seed=rank)  # this rank's T-slice
        a_cpu, b_cpu, g_cpu = full
    else:
        T_local = T
        a_cpu, b_cpu, g_cpu = (x.reshape(rows, T) for x in workloads.workload_inputs(workload.name, seed=rank))
    storage = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.storage]
    elem = torch.empty((), dtype=storage).element_size()
    if args.storage != "f32" and t_sharded:
        raise SystemExit("bench.py: --storage bf16/f16 is measured on the row-sharded workloads only")
    a, b, g = (x.cuda().to(storage) for x in (a_cpu, b_cpu, g_cpu))
    h = torch.empty_like(a)
    ga, gb = torch.empty_like(a), torch.empty_like(a)
    stream = torch.cuda.current_stream()
    st = stream.cuda_stream
    n_local = rows * T_local

    if t_sharded:
        from scanscam_b200 import sharded

        def step():
            hh, h_in = sharded.sharded_scan_forward(a, b)
            sharded.sharded_scan_backward(a, hh, g, h_in)

        launches_per_step = 8
    else:
        # Kernel choice and scratch exactly as the PyTorch extension does it: ask the library, give it
        # the workspace it wants (allocated once here, outside the timed region, and reused).
        v_fwd = args.variant or lib.ssb_scan_recommend(rows, T_local, 0, 1, 1)
        v_bwd = args.variant_bwd or args.variant or lib.ssb_scan_recommend(rows, T_local, 1, 1, 1)
        ws_bytes = max(lib.ssb_scan_workspace_bytes(rows, T_local, v_fwd),
                       lib.ssb_scan_workspace_bytes(rows, T_local, v_bwd))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
        ws_ptr = ws.data_ptr() if ws_bytes else None

        if args.storage == "f32":
            def fwd(s=st):
                _native.check(lib.ssb_scan_fwd_f32_ex(a.data_ptr(), b.data_ptr(), h.data_ptr(), rows, T_local, None,
                                                      v_fwd, ws_ptr, ws_bytes, s))

            def bwd(s=st):
                _native.check(lib.ssb_scan_bwd_f32_ex(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(),
                                                      gb.data_ptr(), rows, T_local, None, None, v_bwd, ws_ptr, ws_bytes, s))
        else:  # 16-bit storage, fp32 arithmetic: the library picks the kernel, no workspace
            fwd16, bwd16 = getattr(lib, f"ssb_scan_fwd_{args.storage}"), getattr(lib, f"ssb_scan_bwd_{args.storage}")
            v_fwd = v_bwd = ws_bytes = 0

            def fwd(s=st):
                _native.check(fwd16(a.data_ptr(), b.data_ptr(), h.data_ptr(), rows, T_local, None, s))

            def bwd(s=st):
                _native.check(bwd16(a.data_ptr(), h.data_ptr(), g.data_ptr(), ga.data_ptr(), gb.data_ptr(), rows, T_local,
                                    None, None, s))

        def step():
            fwd()
            bwd()

        launches_per_step = 2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- timed region: exactly K steps between barrier+synchronize, device-timed --------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    # The K steps are recorded once into a CUDA graph and replayed as one launch (the kernels take
    # raw pointers and a stream, so they capture like any other launch); with --no-graph, or when
    # capture is not possible (the T-sharded path calls NCCL and allocates), they are launched one by one.
    graph = None
    if not args.no_graph and not t_sharded:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    cap = torch.cuda.current_stream().cuda_stream
                    for _ in range(args.steps):
                        fwd(cap)
                        bwd(cap)
            stream.wait_stream(side)
            graph.replay()  # one untimed replay: instantiation and upload happen here
            torch.cuda.synchronize()
        except Exception as exc:  # pragma: no cover - depends on driver/torch support
            print(f"bench.py: CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
            graph = None
    sampler.start()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record(stream)
    if graph is not None:
        graph.replay()
    else:
        for _ in range(args.steps):
            step()
    t_end.record(stream)
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    sampler_how = "NVML samples every 20 ms during the timed region"
    if total_ms < 600.0:
        # too short for a meaningful clock record: keep sampling over a further 0.6 s of the same steps
        t_stop = time.perf_counter() + 0.6
        while time.perf_counter() < t_stop:
            for _ in range(20):
                step()
            torch.cuda.synchronize()
        sampler_how = "NVML samples every 20 ms during the timed region and a 0.6 s continuation of the same steps"
    sampler.stop()

    # ---- per-kernel durations for the roofline: the same K steps again, an event after every
    # launch (kept out of the region above, where the extra event records would cost ~1 %) -----
    fwd_ms, bwd_ms = [0.0], [0.0]
    if not t_sharded:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
        barrier()
        ev[0].record(stream)
        for i in range(args.steps):
            fwd()
            ev[2 * i + 1].record(stream)
            bwd()
            ev[2 * i + 2].record(stream)
        barrier()
        fwd_ms = [ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps)]
        bwd_ms = [ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)]

    detail = _native.ctypes.c_int(0)
    _native.check(lib.ssb_device_status(_native.ctypes.byref(detail)))

    t = torch.tensor([total_ms, sum(fwd_ms), sum(bwd_ms)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_total, bwd_total = (float(x) for x in t.cpu())
    ms_per_step = total_ms / args.steps
    value = n_local * world / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public operator, host buffers -------------------------------
    e2e = None
    if not args.no_e2e and not t_sharded and args.storage == "f32":
        from scanscam_b200.host import HostScanPipeline

        pin = [x.pin_memory() for x in (a_cpu, b_cpu, g_cpu)]
        outs = tuple(torch.empty_like(x).pin_memory() for x in (a_cpu, b_cpu, g_cpu))
        pipe = HostScanPipeline(rows, T_local, chunks=16)

        def e2e_step():
            pipe.run(pin[0], pin[1], pin[2], outs)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record(stream)
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.cpu()) / args.e2e_steps
        # spot-check the host results of the last step against the device-resident run
        torch.cuda.synchronize()
        fwd()
        torch.cuda.synchronize()
        assert torch.equal(outs[0][:64], h[:64].cpu()), "end-to-end pipeline result differs from the resident run"
        e2e = {"value": n_local * world / (e2e_ms * 1e-3) / 1e9, "unit": "Gelem/s",
               "h2d_bytes_per_step": 3 * 4 * n_local, "d2h_bytes_per_step": 3 * 4 * n_local,
               "ms_per_step": e2e_ms, "steps": args.e2e_steps,
               "api": "scanscam_b200.host.HostScanPipeline.run(gate, value, grad): pinned host tensors in, "
                      "h / grad_gate / grad_value written to pinned host tensors; 16 row chunks, copies in both "
                      "directions overlapped with the kernels on three streams"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    bwd_avg_s = bwd_total / args.steps * 1e-3
    fwd_avg_s = fwd_total / args.steps * 1e-3
    line = {
        "metric": METRIC, "value": value, "unit": "Gelem/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if t_sharded else "weak",
        "vs_baseline": None, "dtype": "f32" if args.storage == "f32" else f"f32 arithmetic on {args.storage} tensors",
        "data": "synthetic",
        "config": {
            "workload": (f"{workload.name} {list(workload.shape)} fp32 fwd+bwd, one sequence set split along T over all ranks"
                         if t_sharded else
                         f"{workload.name} {list(workload.shape)} {args.storage} fwd+bwd per GPU, gates {workload.gates}, seed = rank"),
            "sharding": ("T split across ranks, NCCL all-gather of per-shard carries" if t_sharded
                         else "rows (batch x channel) per rank, no collective"),
            "l2": "no flush: each pass streams 0.8-1.3 GB, far more than the 126 MB L2",
            "variant": args.variant,
            "launch": "one CUDA graph of K x (forward, backward)" if graph is not None else "K x 2 stream launches",
            "kernels": (None if t_sharded else {"forward": v_fwd, "backward": v_bwd, "workspace_bytes": ws_bytes}),
        },
        "gpu_launches": launches_per_step * args.steps * world,
        "clocks": sampler.summary(sampler_how),
    }
    if not t_sharded:
        BYTES_FWD, BYTES_BWD = 3 * elem, 5 * elem  # per element: read a, b + write h | read a, h, g + write both gradients
        achieved = BYTES_BWD * n_local / bwd_avg_s / 1e9
        line["roofline"] = {
            "bound": "hbm", "kernel": "fused backward (reads a, h, g; writes grad_a, grad_b)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
            "traffic": (NCU_BWD_TRAFFIC_BYTES_PER_ELEM * n_local if NCU_BWD_TRAFFIC_BYTES_PER_ELEM and elem == 4 else None),
            "algorithmic_bytes_per_launch": BYTES_BWD * n_local, "avg_launch_ms": bwd_avg_s * 1e3,
            "forward": {"achieved": BYTES_FWD * n_local / fwd_avg_s / 1e9,
                        "frac": BYTES_FWD * n_local / fwd_avg_s / 1e9 / peak, "avg_launch_ms": fwd_avg_s * 1e3},
            "fwd_plus_bwd": {"achieved": (BYTES_FWD + BYTES_BWD) * n_local / (fwd_avg_s + bwd_avg_s) / 1e9,
                             "frac_of_measured": (BYTES_FWD + BYTES_BWD) * n_local / (fwd_avg_s + bwd_avg_s) / 1e9 / peak,
                             "frac_of_8TBps": (BYTES_FWD + BYTES_BWD) * n_local / (fwd_avg_s + bwd_avg_s) / 1e9 / 8000.0},
        }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline and args.storage == "f32":
        sample_rows = rows if rows * T_local <= (1 << 26) else max(1, (1 << 26) // T_local)
        v, kind = time_cpu_single(a_cpu[:sample_rows], b_cpu[:sample_rows], g_cpu[:sample_rows])
        line["cpu_baseline"] = {"value": v, "unit": "Gelem/s", "cores": 1, "kind": kind,
                                "sample": f"{sample_rows} of {rows} rows x T={T_local}, median of 2 passes, "
                                          f"single thread (the reference's CPU path has no threading)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    from scanscam_b200.workloads import WORKLOADS

    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference_arm(args, workload)
        return
    run_gpu_arm(args, workload)


if __name__ == "__main__":
    main()
