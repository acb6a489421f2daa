"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl qx|reference]

One GPU (the headline): the 4-bit block GEMV at FFN-up shape -- M=1, K=4096 f32
activations ~N(0,1), N=14336 x K=4096 q4_0 weights (33 MB) -- measured as achieved HBM
GB/s: algorithmic bytes (packed weights + activations read + outputs written) / time. A
step is one GEMV call. The weights fit in L2, so the timed loop rotates over several
distinct weight copies whose total size exceeds L2 (stated in `config`).

N > 1 GPUs (one process per GPU): the batched q8_0 decode GEMV at the large FFN shape --
N=28672 x K=8192 (240 MB) -- under STRONG scaling: the weight rows are split N ways, every
rank streams its shard and all ranks end up with the full output. A step is one sharded
GEMV including the exchange of the output slices (fused into the kernel: peer stores over
NVLink + a wait kernel). `value` is the M=1 case; the M sweep, the kernel without the
exchange, an NCCL all-gather leg and the one-GPU time of the whole matrix are in `extra`.

Prints ONE JSON line (rank 0). `value` is timed with inputs resident in HBM, `e2e` through
host buffers (host<->device copies inside the timed region), `cpu_baseline` is the
reference's CPU path on this host's cores on a bounded sample, `roofline` relates the step
to the measured HBM copy bandwidth. Whatever --steps is, the timed region lasts at least
50 ms: the block of K steps is repeated (`config.timed_repeats`) and averaged.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "decode GEMV achieved HBM GB/s"
WORKLOAD_1GPU = "cfg1_q4_0_gemv"
WORKLOAD_SHARDED = "cfg3_q8_0_batched"
GRAPH_CHUNK = 100
MIN_TIMED_MS = 50.0
FORMAT_NAMES = {0: "q8_0", 1: "q4_0"}


def load_workloads():
    return entry._load_file(entry.PKG_NAME + ".workloads", os.path.join(entry.PKG_DIR, "workloads.py"))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return float(data["hbm_gbs"]), float(data.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons through NVML (read-only) while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int, period_s: float = 0.004):
        super().__init__(daemon=True)
        self.period = period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _one(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
        try:
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        for bit, name in self.REASONS.items():
            if mask & bit:
                self.reasons.add(name)

    def run(self):
        if not self.ok:
            return
        while not self._halt.is_set():
            try:
                self._one()
            except Exception:
                break
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join()
        if self.ok and not self.samples:
            try:
                self._one()
            except Exception:
                pass
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's own implementation on the host cores
# ---------------------------------------------------------------------------------------

def host_cpu():
    """(model string, logical CPUs, physical cores) of this host."""
    model, cores = "unknown", set()
    try:
        physical = core = None
        with open("/proc/cpuinfo") as f:
            for line in f:
                key, _, value = line.partition(":")
                key, value = key.strip(), value.strip()
                if key == "model name" and model == "unknown":
                    model = value
                elif key == "physical id":
                    physical = value
                elif key == "core id":
                    core = value
                elif not key and physical is not None and core is not None:
                    cores.add((physical, core))
                    physical = core = None
        if physical is not None and core is not None:
            cores.add((physical, core))
    except OSError:
        pass
    logical = os.cpu_count() or 1
    try:
        logical = min(logical, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        pass
    physical_cores = len(cores) if cores else max(1, logical // 2)
    return model, logical, max(1, min(physical_cores, logical))


def cpu_engine(threads: int):
    """(kind, engine, threads, variants): the built reference library when present, else the
    oracle port (single-threaded)."""
    oracle_mod = entry.load_oracle()
    if oracle_mod.Reference.available():
        ref = oracle_mod.Reference()
        ref.set_num_threads(threads)
        return "reference", ref, threads, ref.variants()
    return "port", oracle_mod.Oracle(), 1, {}


def cpu_gemv_call(kind, engine, fmt, packed, x, rows, k):
    if kind == "reference":
        return lambda: engine.qgemv(fmt, packed, x, rows, k)
    return lambda: engine.qgemv(fmt, packed, x, rows, k, 0)


def cpu_time_stats(call, budget_s: float = 6.0):
    """Timing discipline of the reference's own bench harness
    (benchmarks/harness/timing.cpp:19-83): warm-up of at least 3 calls AND 50 ms, then up to
    20 samples of batched calls, each sample at least 2 ms; median / p20 / p80 / CV of the
    per-call time. `budget_s` bounds the sampling (fewer samples for slow calls, at least 3)."""
    t0 = time.perf_counter()
    warm = 0
    while warm < 3 or time.perf_counter() - t0 < 0.05:
        call()
        warm += 1
    per_call = (time.perf_counter() - t0) / warm
    batch = max(1, min(4096, int(np.ceil(0.002 / max(per_call, 1e-9)))))
    samples = int(max(3, min(20, budget_s / max(per_call * batch, 1e-9))))
    times = []
    for _ in range(samples):
        s0 = time.perf_counter()
        for _ in range(batch):
            call()
        times.append((time.perf_counter() - s0) / batch)
    times.sort()
    median = statistics.median(times)
    pick = lambda q: times[min(len(times) - 1, int(q * len(times)))]  # noqa: E731
    cv = statistics.pstdev(times) / statistics.fmean(times) if len(times) > 1 else 0.0
    return {"median_s": median, "p20_s": pick(0.2), "p80_s": pick(0.8), "cv": cv,
            "samples": len(times), "calls_per_sample": batch, "warmup_calls": warm}


def reference_workload(wl, gpus: int):
    name = WORKLOAD_1GPU if gpus <= 1 else WORKLOAD_SHARDED
    c = wl.CONFIGS[name]
    return name, c["fmt"], c["n"], c["k"], c


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = load_workloads()
    name, fmt, n, k, c = reference_workload(wl, args.gpus)
    packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    x = wl.activations_f32(1, k, seed=0)[0].copy()
    model, logical, physical = host_cpu()
    kind, engine, threads, variants = cpu_engine(physical)

    # bound the run to about two minutes: shrink the per-step row sample if needed
    full = cpu_gemv_call(kind, engine, fmt, packed, x, n, k)
    t0 = time.perf_counter()
    warm = 0
    while warm < 3 or time.perf_counter() - t0 < 0.05:  # the pool's threads spin up here
        full()
        warm += 1
    per_call = (time.perf_counter() - t0) / warm
    rows = n
    total_steps = args.steps + args.warmup
    if per_call * total_steps > 120.0:
        rows = int(max(32 * threads, min(n, n * 120.0 / (per_call * total_steps))))
        rows -= rows % 32
        rows = max(rows, 32)
    call = cpu_gemv_call(kind, engine, fmt, packed, x, rows, k)
    for _ in range(args.warmup):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    elapsed = time.perf_counter() - t0
    step_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, rows, k)
    value = step_bytes * args.steps / elapsed / 1e9
    stats = cpu_time_stats(call, budget_s=4.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus <= 1 else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "m": 1, "n": n, "k": k, "format": FORMAT_NAMES[fmt],
                   "rows_per_step": rows, "variants": variants},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
                         "cpu_model": model, "logical_cpus": logical, "physical_cores": physical,
                         "sample": f"{args.steps} calls of the reference qgemv over {rows} of {n} rows "
                                   f"after {warm}+{args.warmup} warm-up calls (>= 50 ms)",
                         "harness_stats": {
                             "median_gbs": step_bytes / stats["median_s"] / 1e9,
                             "p20_ms": stats["p20_s"] * 1e3, "median_ms": stats["median_s"] * 1e3,
                             "p80_ms": stats["p80_s"] * 1e3, "cv": stats["cv"],
                             "samples": stats["samples"], "calls_per_sample": stats["calls_per_sample"]}},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def cpu_baseline(wl, c):
    """The reference's CPU GEMV on the headline workload: T = physical cores and T = 1."""
    fmt, n, k = c["fmt"], c["n"], c["k"]
    packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    x = wl.activations_f32(1, k, seed=0)[0].copy()
    model, logical, physical = host_cpu()
    step_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, n, k)
    kind, engine, threads, variants = cpu_engine(physical)
    many = cpu_time_stats(cpu_gemv_call(kind, engine, fmt, packed, x, n, k), budget_s=8.0)
    out = {"value": step_bytes / many["median_s"] / 1e9, "unit": "GB/s", "cores": threads,
           "kind": kind, "cpu_model": model, "logical_cpus": logical, "physical_cores": physical,
           "ms_per_call": many["median_s"] * 1e3, "p20_ms": many["p20_s"] * 1e3,
           "p80_ms": many["p80_s"] * 1e3, "cv": many["cv"],
           "sample": f"median of {many['samples']} samples x {many['calls_per_sample']} full-size qgemv "
                     f"calls ({n}x{k} {FORMAT_NAMES[fmt]}) after {many['warmup_calls']} warm-up calls (>= 50 ms)",
           "variants": variants}
    if kind == "reference":
        engine.set_num_threads(1)
        one = cpu_time_stats(cpu_gemv_call(kind, engine, fmt, packed, x, n, k), budget_s=4.0)
        out["single_thread"] = {"value": step_bytes / one["median_s"] / 1e9, "unit": "GB/s",
                                "ms_per_call": one["median_s"] * 1e3, "cv": one["cv"],
                                "samples": one["samples"]}
        engine.set_num_threads(threads)
    return out


# ---------------------------------------------------------------------------------------
# GPU arm, shared helpers
# ---------------------------------------------------------------------------------------

_cudart = None


def cudart():
    global _cudart
    if _cudart is None:
        _cudart = ctypes.CDLL("libcudart.so.12")
        _cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _cudart.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                            ctypes.c_int, ctypes.c_void_p]
    return _cudart


def _device_floats(torch, address: int, count: int):
    """`count` floats at a raw device address, copied into a torch tensor."""
    out = torch.empty(count, dtype=torch.float32, device="cuda")
    if cudart().cudaMemcpy(out.data_ptr(), address, count * 4, 3) != 0:  # device to device
        raise RuntimeError("cudaMemcpy failed")
    return out


class TimedBlock:
    """K steps as CUDA graphs (a chunk replayed q times plus a remainder graph), so that the
    host's launch cost stays out of the timed region; falls back to plain launches when
    capture is refused. A K below GRAPH_CHUNK is captured `group` blocks to a graph (a graph
    of a decode loop holds hundreds of kernels; a kernel at the head of a graph cannot
    overlap with the one in front of it), and run() then runs that many blocks."""

    def __init__(self, torch, step, steps: int, period: int, allow_graph: bool = True):
        self.torch, self.step, self.block_steps = torch, step, steps
        self.group = max(1, GRAPH_CHUNK // steps) if allow_graph else 1
        if self.group > 1 and (self.group * steps) % 2:
            self.group += 1   # keep every run an even number of steps
        steps = steps * self.group
        self.steps = steps    # steps per run()
        chunk = min(steps, GRAPH_CHUNK)
        if chunk >= period:
            chunk -= chunk % period
        self.chunk = max(1, chunk)
        self.reps, self.rem = divmod(steps, self.chunk)
        self.graph_chunk = self.graph_rem = None
        # two plain steps first: a call shape that is new to the library's default workspace
        # grows it (an allocation), which must not happen inside a capture. (Two, because the
        # fused all-gather alternates between two result buffers step by step and every
        # block of steps here is kept even.)
        for i in range(2):
            step(i)
        torch.cuda.synchronize()
        if allow_graph:
            try:
                self.graph_chunk = self._capture(0, self.chunk)
                if self.rem:
                    self.graph_rem = self._capture(self.reps * self.chunk, self.rem)
            except Exception as exc:  # fall back to plain launches
                print(f"bench: graph capture failed ({exc!r}); timing plain launches", file=sys.stderr)
                self.graph_chunk = self.graph_rem = None
                torch.cuda.synchronize()
        self.blocks_per_run = self.group

    def _capture(self, first: int, count: int):
        graph = self.torch.cuda.CUDAGraph()
        with self.torch.cuda.graph(graph):
            for i in range(first, first + count):
                self.step(i)
        graph.replay()
        self.torch.cuda.synchronize()
        return graph

    @property
    def graphed(self):
        return self.graph_chunk is not None

    def run(self):
        if self.graph_chunk is not None:
            for _ in range(self.reps):
                self.graph_chunk.replay()
            if self.graph_rem is not None:
                self.graph_rem.replay()
        else:
            for i in range(self.steps):
                self.step(i)


def time_block(torch, dist, block: TimedBlock, world: int):
    """(ms per step, blocks of K steps timed, ms): the block of K steps repeated until the
    region lasts at least MIN_TIMED_MS, between barriers and synchronisations, CUDA events,
    max over ranks."""
    def region(repeats):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(repeats):
            block.run()
        stop.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms
    probe = region(1)
    repeats = max(1, int(np.ceil(1.1 * MIN_TIMED_MS / max(probe, 1e-6))))
    if world > 1:  # every rank must run the same number of repeats
        t = torch.tensor([repeats], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        repeats = int(t.item())
    total = region(repeats)
    return total / (repeats * block.steps), repeats * block.blocks_per_run, total


# ---------------------------------------------------------------------------------------
# GPU arm, one GPU: the headline
# ---------------------------------------------------------------------------------------

def run_single(args):
    import torch

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    qx = entry.load_package()
    wl = load_workloads()
    c = wl.CONFIGS[WORKLOAD_1GPU]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    step_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, n, k)
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    info = qx.device_info()

    # distinct weight copies whose total size exceeds L2, rotated step by step
    copies = max(2, -(-2 * info["l2_bytes"] // (n * (k // 32) * 18)))
    handles = []
    for i in range(copies):
        packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=i)
        h = qx.PackedWeights()
        qx.check(h.prepare(fmt, packed, n, k), "qx_weights_prepare")
        handles.append(h)
    x_host = wl.activations_f32(1, k, seed=0)
    x_dev = torch.from_numpy(x_host).cuda()
    y_dev = torch.zeros(n, device="cuda")

    def step(i):
        qx.check(handles[i % copies].qgemm_dev(x_dev, y_dev, 1, n), "qx_qgemm_prepacked_dev")

    launches0 = qx.launch_count()
    step(0)
    launches_per_step = qx.launch_count() - launches0
    torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    block = TimedBlock(torch, step, args.steps, copies, allow_graph=not args.no_graph)
    ms_per_step, repeats, total_ms = time_block(torch, None, block, 1)
    clocks = sampler.stop()
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # One launch that cannot overlap its neighbours (what a caller sees when other kernels
    # sit between GEMVs): an unrelated 64 MB fill runs between consecutive GEMVs in a graph;
    # the time of the same graph without the GEMVs is subtracted.
    filler = torch.empty(16 << 20, dtype=torch.float32, device="cuda")
    pairs = 2 * copies
    t_pairs = _time_calls(torch, lambda i: (filler.fill_(1.0), step(i)), pairs)
    t_fill = _time_calls(torch, lambda i: filler.fill_(1.0), pairs)
    isolated_us = (t_pairs - t_fill) * 1e6
    del filler

    # end to end through the host-pointer entry point: pinned x in, pinned y out, every step
    x_pin = torch.from_numpy(x_host).pin_memory()
    y_pin = torch.zeros(n).pin_memory()
    e2e_steps = max(300, min(args.steps, 2000))
    for i in range(10):
        qx.check(handles[i % copies].qgemm_prepacked_ptr(x_pin.data_ptr(), y_pin.data_ptr(), 1), "e2e")
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        qx.check(handles[i % copies].qgemm_prepacked_ptr(x_pin.data_ptr(), y_pin.data_ptr(), 1), "e2e")
    e2e_s = time.perf_counter() - t0
    e2e_value = step_bytes * e2e_steps / e2e_s / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_1GPU, "m": 1, "n": n, "k": k, "format": FORMAT_NAMES[fmt],
                   "sharding": "none", "exchange": "none",
                   "l2_policy": f"rotates {copies} distinct weight copies "
                                f"({copies * n * (k // 32) * 18 / 1e6:.0f} MB > L2 {info['l2_bytes'] / 1e6:.0f} MB)",
                   "cuda_graph": block.graphed, "timed_repeats": repeats,
                   "timed_region_ms": total_ms, "variants": qx.variants()},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * k,
                "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
                "note": "qx_qgemm_prepacked per step on a handle prepared once (the counterpart of "
                        "CpuPackedWeights): x copied from pinned host memory, y written by the "
                        "kernel into the caller's pinned host buffer, then one stream "
                        "synchronisation. The literal qgemv(packed_host, ...) entry re-uploads the "
                        "33 MB of weights per call and is not what this number measures"},
        "gpu_launches": launches_per_step * args.steps * repeats,
        "roofline": {"bound": "hbm", "achieved": value, "peak": hbm_peak, "unit": "GB/s",
                     "frac": value / hbm_peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                                       "from an ncu capture of this workload, not measured by this run",
                     "peak_source": f"{peak_kind} HBM copy bandwidth",
                     "frac_of_nominal_8TBs": value / 8000.0,
                     "isolated_launch_us": isolated_us,
                     "isolated_frac": step_bytes / (isolated_us * 1e-6) / 1e9 / hbm_peak,
                     "note": "achieved = algorithmic bytes / step time over back-to-back, "
                             "graph-replayed steps (launch gaps included); isolated_launch_us = one "
                             "launch between synchronisations"},
    }
    if not args.no_extra:
        line["cpu_baseline"] = cpu_baseline(wl, c)
        try:
            line["extra"] = extra_measurements(qx, wl, torch, hbm_peak, bf16_peak)
        except Exception as exc:  # the headline line must still be printed
            line["extra"] = {"error": repr(exc)}
    emit(line)


# ---------------------------------------------------------------------------------------
# GPU arm, N > 1: the sharded decode configuration under strong scaling
# ---------------------------------------------------------------------------------------

def run_sharded(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    qx = entry.load_package()
    wl = load_workloads()
    sharded = entry._load_file(entry.PKG_NAME + ".sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
    c = wl.CONFIGS[WORKLOAD_SHARDED]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    sweep = tuple(c["m_sweep"])
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    info = qx.device_info()
    begin, rows = sharded.shard_rows(n, world, rank)
    if rows * world != n:
        raise SystemExit(f"bench: {n} rows do not split evenly over {world} ranks")
    block_bytes = 34 if fmt == 0 else 18
    shard_bytes = rows * (k // 32) * block_bytes

    # The whole matrix (seed 0) on every rank: the unsharded GEMV is the reference of the
    # self-check and the one-GPU time of the strong-scaling figure. Copy 0 of the shard is
    # this rank's row range of it; further copies (other seeds) only keep the timed loop out
    # of L2.
    packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    full = qx.PackedWeights()
    qx.check(full.prepare(fmt, packed, n, k), "prepare full")
    copies = max(2, -(-2 * info["l2_bytes"] // shard_bytes))
    handles = []
    for i in range(copies):
        h = qx.PackedWeights()
        if i == 0:
            qx.check(h.prepare(fmt, packed, n, k, begin, rows), "prepare shard")
        else:
            other = wl.packed_blocks(fmt, rows, k, c["d_lo"], c["d_hi"], seed=1000 * rank + i)
            qx.check(h.prepare(fmt, other, rows, k), "prepare shard copy")
        handles.append(h)
    del packed
    xs = {m: torch.from_numpy(wl.activations_f32(m, k, seed=m)).cuda() for m in sweep}

    # the exchange fused into the GEMV; NCCL only if the peer mapping cannot be set up
    gathers, exchange = {}, "peer stores fused into the GEMV epilogue + wait kernel"
    healthy = 1
    try:
        for m in sweep:
            gathers[m] = sharded.PushAllGather(qx, rows, m)
    except Exception as exc:
        print(f"bench: fused all-gather unavailable ({exc!r}); using NCCL", file=sys.stderr)
        healthy = 0
    flags = torch.tensor([healthy], device="cuda")
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    fused = int(flags.item()) == 1
    if not fused:
        gathers, exchange = {}, "nccl all_gather_into_tensor"

    def gathered_matches(m, steps_to_check):
        """Runs `steps_to_check` steps on the true shard and compares every rank's slice of the
        gathered result with the unsharded GEMV, bit for bit."""
        want = torch.zeros((m, n), device="cuda")
        qx.check(full.qgemm_dev(xs[m], want, m, n), "unsharded gemv")
        torch.cuda.synchronize()
        ok = True
        for _ in range(steps_to_check):
            ptr = gathers[m].step(handles[0], xs[m], m)
            torch.cuda.synchronize()
            got = _device_floats(torch, ptr, world * m * rows).view(world, m, rows)
            for r in range(world):
                ok = ok and torch.equal(got[r].view(torch.int32),
                                        want[:, r * rows:(r + 1) * rows].contiguous().view(torch.int32))
        return ok

    selfcheck = {"ok": None}
    if fused:
        checks = {}
        try:
            for m in (1, sweep[-1]):
                checks[f"m{m}_both_parities_all_slices_bit_equal"] = gathered_matches(m, 2)
            checks["no_wait_gave_up"] = qx.lib.qx_check_device_errors() == qx.OK
        except Exception as exc:
            print(f"bench: self-check raised {exc!r}", file=sys.stderr)
            checks["exception"] = False
        selfcheck = dict(checks)
        mine = torch.tensor([1 if all(checks.values()) else 0], device="cuda")
        dist.all_reduce(mine, op=dist.ReduceOp.MIN)
        selfcheck["ok"] = bool(int(mine.item()))
        selfcheck["ranks"] = world

    y_full = torch.zeros((1, n), device="cuda")
    y_local = torch.zeros((1, rows), device="cuda")

    def step_m(m):
        if fused:
            return lambda i: gathers[m].step(handles[i % copies], xs[m], m)

        def nccl_step(i):
            qx.check(handles[i % copies].qgemm_dev(xs[1], y_local, 1, rows), "gemv")
            dist.all_gather_into_tensor(y_full.view(-1), y_local.view(-1))
        return nccl_step

    step = step_m(1)
    launches0 = qx.launch_count()
    step(0)
    launches_per_step = qx.launch_count() - launches0
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    period = copies if copies % 2 == 0 else 2 * copies  # result buffers alternate step by step
    block = TimedBlock(torch, step, args.steps + (args.steps % 2 if fused else 0), period,
                       allow_graph=fused and not args.no_graph)
    ms_per_step, repeats, total_ms = time_block(torch, dist, block, world)
    clocks = sampler.stop()
    full_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, n, k)
    value = full_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- explanatory figures -------------------------------------------------------------
    def per_step_us(fn, count, use_graph=True):
        blk = TimedBlock(torch, fn, count, period, allow_graph=use_graph and not args.no_graph)
        ms, _, _ = time_block(torch, dist, blk, world)
        return ms * 1e3

    extra = {}
    try:
        y_shard = {m: torch.zeros((m, rows), device="cuda") for m in sweep}
        y_whole = {m: torch.zeros((m, n), device="cuda") for m in sweep}
        sweep_out = {}
        for m in sweep:
            count = 2 * period
            local_us = per_step_us(lambda i, m=m: qx.check(
                handles[i % copies].qgemm_dev(xs[m], y_shard[m], m, rows), "gemv"), count)
            one_gpu_us = per_step_us(lambda i, m=m: qx.check(
                full.qgemm_dev(xs[m], y_whole[m], m, n), "gemv"), 4)
            entry_m = {"one_gpu_whole_matrix_us": one_gpu_us, "shard_kernel_only_us": local_us,
                       "efficiency_kernel_only": one_gpu_us / (world * local_us)}
            if fused:
                step_us = ms_per_step * 1e3 if m == 1 else per_step_us(step_m(m), count)
                entry_m.update({"sharded_step_us": step_us,
                                "efficiency_with_exchange": one_gpu_us / (world * step_us),
                                "aggregate_gbs": wl.algorithmic_bytes_qgemv(fmt, m, n, k) / step_us / 1e3})
            sweep_out[f"m{m}"] = entry_m
        extra["strong_scaling"] = {"definition": "t(1 GPU, whole matrix) / (N * t(N))", "m_sweep": sweep_out}
        # the stated comparison: NCCL all-gather of the output slices after the shard's GEMV
        def nccl_leg(i):
            qx.check(handles[i % copies].qgemm_dev(xs[1], y_local, 1, rows), "gemv")
            dist.all_gather_into_tensor(y_full.view(-1), y_local.view(-1))
        for i in range(5):
            nccl_leg(i)
        extra["nccl_all_gather_leg"] = {"m": 1, "step_us": per_step_us(nccl_leg, 2 * period, use_graph=False),
                                        "launch": "eager (not captured in a graph)"}
    except Exception as exc:
        extra["error"] = repr(exc)
    try:
        extra["sharded_prefill_cfg4"] = _sharded_prefill(qx, wl, torch, dist, world, rank, bf16_peak)
    except Exception as exc:
        extra["sharded_prefill_cfg4"] = {"error": repr(exc)}

    # ---- end to end: host x in, gathered y out, every step ----------------------------------
    x_pin = torch.from_numpy(wl.activations_f32(1, k, seed=1)).pin_memory()
    y_pin = torch.zeros(n).pin_memory()
    x_stage = torch.zeros((1, k), device="cuda")
    stream = torch.cuda.current_stream()

    def e2e_step(i):
        x_stage.copy_(x_pin, non_blocking=True)
        if fused:
            ptr = gathers[1].step(handles[i % copies], x_stage, 1)
            cudart().cudaMemcpyAsync(y_pin.data_ptr(), ptr, 4 * n, 2, stream.cuda_stream)
        else:
            qx.check(handles[i % copies].qgemm_dev(x_stage, y_local, 1, rows), "gemv")
            dist.all_gather_into_tensor(y_full.view(-1), y_local.view(-1))
            y_pin.copy_(y_full.view(-1), non_blocking=True)
        stream.synchronize()

    e2e_steps = max(300, min(args.steps, 1000))
    e2e_steps += e2e_steps % 2
    for i in range(10):
        e2e_step(i)
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = full_bytes * e2e_steps / float(t.item()) / 1e9

    if fused:  # once more after all the timed loops: the gathered result is still right
        after = gathered_matches(1, 2) and qx.lib.qx_check_device_errors() == qx.OK
        mine = torch.tensor([1 if after else 0], device="cuda")
        dist.all_reduce(mine, op=dist.ReduceOp.MIN)
        selfcheck["after_timed_loops_ok"] = bool(int(mine.item()))
        selfcheck["ok"] = bool(selfcheck["ok"] and selfcheck["after_timed_loops_ok"])

    if rank == 0:
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_SHARDED, "m": 1, "n": n, "k": k,
                       "format": FORMAT_NAMES[fmt], "sharding": f"rows /{world} ({rows} per rank)",
                       "exchange": exchange,
                       "l2_policy": f"rotates {copies} distinct shard copies "
                                    f"({copies * shard_bytes / 1e6:.0f} MB > L2 {info['l2_bytes'] / 1e6:.0f} MB)",
                       "cuda_graph": block.graphed, "timed_repeats": repeats,
                       "timed_region_ms": total_ms, "variants": qx.variants()},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * k,
                    "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
                    "note": "per step on every rank: x from pinned host memory to the GPU, the "
                            "sharded GEMV with the exchange, the gathered 28672 results back to "
                            "pinned host memory, one stream synchronisation (max over ranks)"},
            "gpu_launches": launches_per_step * block.block_steps * repeats,
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": hbm_peak, "unit": "GB/s",
                         "frac": per_gpu / hbm_peak, "traffic": None,
                         "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "note": "per GPU: (algorithmic bytes of the whole matrix / N) / step time, "
                                 "exchange included"},
            "selfcheck": selfcheck,
            "extra": extra,
        }
        emit(line)
    dist.destroy_process_group()


def _sharded_prefill(qx, wl, torch, dist, world, rank, bf16_peak):
    """cfg4 (4-bit prefill GEMM, bf16 activations) with the weight rows sharded over the ranks:
    M cut into chunks of 256 tokens, the NCCL all-gather of a chunk on a second stream under
    the GEMM of the next (ShardedPrefill). Eager launches, CUDA events around 3 calls, max over
    ranks. The f32 output is 235 MB, so the exchange moves (N-1)/N of that into every GPU."""
    sharded = entry._load_file(entry.PKG_NAME + ".sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
    c = wl.CONFIGS["cfg4_q4_0_prefill"]
    fmt, m, n, k = c["fmt"], c["m"], c["n"], c["k"]
    begin, rows = sharded.shard_rows(n, world, rank)
    blocks = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    shard = qx.PackedWeights()
    qx.check(shard.prepare(fmt, blocks, n, k, begin, rows), "prepare shard")
    del blocks
    xb = torch.from_numpy(wl.to_bf16_bits(wl.activations_f32(m, k, seed=0)).view(np.int16)).cuda()

    def compute(x_chunk, out):
        qx.check(shard.qgemm_bf16_dev(x_chunk, out, x_chunk.shape[0]), "sharded prefill GEMM")

    layer = sharded.ShardedPrefill(n, k, compute, chunk_rows=256, device="cuda")
    local = torch.empty((m, rows), device="cuda")

    def timed(fn, calls=3):
        fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(calls):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / calls], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_exchange = timed(lambda: layer.forward(xb))
    ms_kernel = timed(lambda: compute(xb, local))
    flops = wl.flops_gemm(m, n, k) if hasattr(wl, "flops_gemm") else 2.0 * m * n * k
    shard.reset()
    return {"m": m, "n": n, "k": k, "rows_per_rank": rows, "chunk_rows": 256,
            "ms_with_exchange": ms_exchange, "ms_shard_gemm_only": ms_kernel,
            "aggregate_tflops": flops / (ms_exchange * 1e-3) / 1e12,
            "frac_of_measured_bf16_per_gpu": flops / world / (ms_exchange * 1e-3) / 1e12 / bf16_peak,
            "exchange": "NCCL all_gather_into_tensor per chunk on a second stream",
            "output_layout": "[chunk][rank][256 tokens][rows_per_rank] f32"}


def _time_calls(torch, fn, iters, warm=3):
    """Seconds per call of fn(i): `iters` calls captured in one CUDA graph (no host launch
    cost in the timed region), replayed once untimed and three times timed (mean)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (3 * iters) * 1e-3


# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_decode_kernel launch on the
# headline workload from an ncu capture (algorithmic bytes: 33 103 872; the 57 KB of outputs
# had not left L2 when the capture ended)
NCU_DRAM_BYTES_PER_LAUNCH = 33078528

EXTRA_CASES = ("cfg2_w8a8_gemm", "cfg0_q8_0_gemv", "cfg3_q8_0_batched", "cfg4_q4_0_prefill",
               "w8a32_gemm", "fused_decode", "lowbit_w4a8", "canonical_projection")


def extra_measurements(qx, wl, torch, hbm_peak, bf16_peak, only=None):
    """The other benchmark configurations on one GPU (not the headline; explanatory). `only`
    names a single one of EXTRA_CASES (profiling runs)."""
    out = {}
    if only in (None, "cfg2_w8a8_gemm"):
        out.update(_extra_cfg2(qx, wl, torch))
    if only in (None, "cfg0_q8_0_gemv"):
        out.update(_extra_cfg0(qx, wl, torch, hbm_peak))
    if only in (None, "cfg3_q8_0_batched"):
        out.update(_extra_cfg3(qx, wl, torch, hbm_peak))
    if only in (None, "cfg4_q4_0_prefill"):
        out.update(_extra_cfg4(qx, wl, torch, bf16_peak))
    if only in (None, "w8a32_gemm"):
        out.update(_extra_w8a32(qx, wl, torch, hbm_peak))
    if only in (None, "fused_decode"):
        out.update(_extra_fused(qx, wl, torch, hbm_peak))
    if only in (None, "lowbit_w4a8"):
        out.update(_extra_lowbit(qx, wl, torch, hbm_peak))
    if only in (None, "canonical_projection"):
        out.update(_extra_canonical(qx, wl, torch, hbm_peak))
    return out


def _extra_cfg2(qx, wl, torch):
    out = {}
    # cfg2: W8A8 prefill GEMM, TOPS (three weight copies = 176 MB, rotated, so W comes from HBM)
    c = wl.CONFIGS["cfg2_w8a8_gemm"]
    m, n, k = c["m"], c["n"], c["k"]
    w, x, ws, xs = wl.w8a8_inputs(m, n, k, seed=0)
    w_copies = [torch.from_numpy(w).cuda() for _ in range(3)]
    xd, wsd, xsd = (torch.from_numpy(a).cuda() for a in (x, ws, xs))
    y = torch.zeros((m, n), device="cuda")
    sec = _time_calls(torch, lambda i: qx.check(
        qx.int8_gemm_dev(w_copies[i % 3], xd, wsd, xsd, y, m, n, k), "int8"), 30)
    out["cfg2_w8a8_gemm"] = {"tops": 2.0 * m * n * k / sec / 1e12, "us": sec * 1e6,
                             "frac_of_nominal_4500_tops": 2.0 * m * n * k / sec / 4.5e15,
                             "peak_note": "4500 TOPS is the nominal dense int8 figure; no measured "
                                          "int8 peak exists for this pool",
                             "variant": qx.variants()["int8_gemm"]}
    return out


def _extra_cfg0(qx, wl, torch, hbm_peak):
    out = {}
    # cfg0: q8_0 GEMV 4096x4096 (16 rotating copies = 285 MB > L2)
    c = wl.CONFIGS["cfg0_q8_0_gemv"]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    handles = []
    for i in range(16):
        h = qx.PackedWeights()
        qx.check(h.prepare(fmt, wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=i), n, k), "prep")
        handles.append(h)
    xd = torch.from_numpy(wl.activations_f32(1, k)).cuda()
    yd = torch.zeros(n, device="cuda")
    sec = _time_calls(torch, lambda i: qx.check(handles[i % 16].qgemm_dev(xd, yd, 1, n), "gemv"), 160)
    gbs = wl.algorithmic_bytes_qgemv(fmt, 1, n, k) / sec / 1e9
    out["cfg0_q8_0_gemv"] = {"gbs": gbs, "us": sec * 1e6, "frac_of_measured_hbm": gbs / hbm_peak}
    for h in handles:
        h.reset()
    return out


def _extra_cfg3(qx, wl, torch, hbm_peak):
    out = {}
    # cfg3: batched q8_0 GEMV, two copies of the 240 MB weights alternate (> L2), M sweep
    c = wl.CONFIGS["cfg3_q8_0_batched"]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    pair = []
    for i in range(2):
        h = qx.PackedWeights()
        qx.check(h.prepare(fmt, wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=i), n, k), "prep")
        pair.append(h)
    sweep = {}
    for m in c["m_sweep"]:
        xd = torch.from_numpy(wl.activations_f32(m, k)).cuda()
        yd = torch.zeros((m, n), device="cuda")
        sec = _time_calls(torch, lambda i: qx.check(pair[i % 2].qgemm_dev(xd, yd, m, n), "gemm"), 10, 2)
        gbs = wl.algorithmic_bytes_qgemv(fmt, m, n, k) / sec / 1e9
        sweep[f"m{m}"] = {"gbs": gbs, "us": sec * 1e6, "frac_of_measured_hbm": gbs / hbm_peak}
    out["cfg3_q8_0_batched"] = sweep
    for h in pair:
        h.reset()
    return out


def _extra_cfg4(qx, wl, torch, bf16_peak):
    out = {}
    # cfg4: 4-bit prefill GEMM, q4_0 weights x bf16 activations (operands far larger than L2)
    c = wl.CONFIGS["cfg4_q4_0_prefill"]
    fmt, n, k, m = c["fmt"], c["n"], c["k"], c["m"]
    h = qx.PackedWeights()
    qx.check(h.prepare(fmt, wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0), n, k), "prep")
    xb = wl.to_bf16_bits(wl.activations_f32(m, k, seed=4))
    xd = torch.from_numpy(xb.view(np.int16)).cuda()
    yd = torch.zeros((m, n), device="cuda")
    sec = _time_calls(torch, lambda i: qx.check(h.qgemm_bf16_dev(xd, yd, m), "prefill"), 5, 1)
    tflops = 2.0 * m * n * k / sec / 1e12
    out["cfg4_q4_0_prefill"] = {"tflops": tflops, "ms": sec * 1e3,
                                "frac_of_measured_bf16": tflops / bf16_peak if bf16_peak else None,
                                "note": "includes the activation staging pre-pass"}
    h.reset()
    return out


def _extra_w8a32(qx, wl, torch, hbm_peak):
    """Weight-only int8 GEMM at the reference bench's own shapes
    (benchmarks/cases/colibri_ops.cpp:466-478). Algorithmic bytes: W (int8) + scales + X + Y."""
    out = {}
    for m, n, k in ((4, 1024, 1408), (16, 4096, 4096)):
        rng = np.random.default_rng(m)
        copies = 8 if n * k < (1 << 24) else 10
        ws = [torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).cuda() for _ in range(copies)]
        scale = torch.from_numpy(rng.uniform(0.001, 0.01, n).astype(np.float32)).cuda()
        xd = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda()
        yd = torch.zeros((m, n), device="cuda")
        sec = _time_calls(torch, lambda i: qx.check(
            qx.qgemm_w8a32_dev(ws[i % copies], scale, xd, yd, m, n, k), "w8a32"), 4 * copies)
        nbytes = n * k + 4 * n + 4 * m * k + 4 * m * n
        out[f"m{m}_n{n}_k{k}"] = {"us": sec * 1e6, "gbs": nbytes / sec / 1e9,
                                  "frac_of_measured_hbm": nbytes / sec / 1e9 / hbm_peak,
                                  "weights_in_l2": bool(n * k * copies < 120e6)}
    return {"w8a32_gemm": out}


def _extra_fused(qx, wl, torch, hbm_peak):
    """The fused decode projections at the headline shape: up + gate (2 x 14336 x 4096 q4_0,
    66 MB) in ONE launch, with and without the activation, and the activation-quantising
    GEMV (qgemv_w8a8) on the headline matrix. Weight copies rotate (> L2)."""
    c = wl.CONFIGS["cfg1_q4_0_gemv"]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    copies = 5
    fused, single = [], []
    for i in range(copies):
        parts = [wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=10 * i + s) for s in (1, 2)]
        h = qx.PackedWeights()
        qx.check(h.prepare_fused(fmt, parts, [n, n], k), "prepare_fused")
        fused.append(h)
    for i in range(9):
        h = qx.PackedWeights()
        qx.check(h.prepare(fmt, wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=100 + i), n, k), "prep")
        single.append(h)
    xd = torch.from_numpy(wl.activations_f32(1, k)).cuda()
    up, gate = torch.zeros((1, n), device="cuda"), torch.zeros((1, n), device="cuda")
    out, scratch = torch.zeros(n, device="cuda"), torch.zeros(2 * n, device="cuda")
    yd = torch.zeros(n, device="cuda")
    nbytes = 2 * n * (k // 32) * 18 + 4 * k + 8 * n
    sec = _time_calls(torch, lambda i: qx.check(fused[i % copies].qgemm_fused_dev(xd, [up, gate], 1), "fused"), 40)
    sec_act = _time_calls(torch, lambda i: qx.check(
        fused[i % copies].up_gate_activation_dev(xd[0], out, scratch, True), "act"), 40)
    sec_w8a8 = _time_calls(torch, lambda i: qx.check(single[i % 9].qgemv_w8a8_dev(xd[0], yd), "w8a8"), 90)
    one = wl.algorithmic_bytes_qgemv(fmt, 1, n, k)
    result = {"fused_decode": {
        "up_gate_q4_0_14336x4096": {"us": sec * 1e6, "gbs": nbytes / sec / 1e9,
                                    "frac_of_measured_hbm": nbytes / sec / 1e9 / hbm_peak,
                                    "launches": 1, "bytes": nbytes},
        "up_gate_activation_q4_0_14336x4096": {"us": sec_act * 1e6, "gbs": nbytes / sec_act / 1e9,
                                               "frac_of_measured_hbm": nbytes / sec_act / 1e9 / hbm_peak,
                                               "launches": 2},
        "qgemv_w8a8_q4_0_14336x4096": {"us": sec_w8a8 * 1e6, "gbs": one / sec_w8a8 / 1e9,
                                       "frac_of_measured_hbm": one / sec_w8a8 / 1e9 / hbm_peak}}}
    for h in fused + single:
        h.reset()
    return result


def _extra_lowbit(qx, wl, torch, hbm_peak):
    """W4A8 over compact int4 rows (lowbit_gemm_w8a8) at decode batches; algorithmic bytes:
    packed weights + scales + activations + outputs."""
    import ctypes as C
    out = {}
    for m, n, k in ((1, 4096, 4096), (4, 14336, 4096), (16, 4096, 4096)):
        rng = np.random.default_rng(m + n)
        copies = max(2, int(280e6 // (n * k // 2)))
        ws = [torch.from_numpy(rng.integers(0, 256, n * k // 2, dtype=np.uint8)).cuda() for _ in range(copies)]
        scale = torch.from_numpy(rng.uniform(0.001, 0.01, n).astype(np.float32)).cuda()
        xd = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda()
        yd = torch.zeros((m, n), device="cuda")
        scratch = torch.zeros(qx.lib.qx_lowbit_w8a8_scratch_bytes(m, k), dtype=torch.uint8, device="cuda")

        def call(i):
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)  # the capturing stream
            qx.check(qx.lib.qx_lowbit_gemm_w8a8_dev(C.c_void_p(ws[i % copies].data_ptr()), C.c_void_p(scale.data_ptr()),
                                                    C.c_void_p(xd.data_ptr()), C.c_void_p(yd.data_ptr()),
                                                    C.c_void_p(scratch.data_ptr()), m, n, k, stream), "w4a8")
        sec = _time_calls(torch, call, 4 * copies)
        nbytes = n * k // 2 + 4 * n + 4 * m * k + 4 * m * n
        out[f"m{m}_n{n}_k{k}"] = {"us": sec * 1e6, "gbs": nbytes / sec / 1e9,
                                  "frac_of_measured_hbm": nbytes / sec / 1e9 / hbm_peak, "launches": 2}
    return {"lowbit_w4a8": out}


def _extra_canonical(qx, wl, torch, hbm_peak):
    """Canonical prepared projections (kInt8Symmetric with channel scales, kInt4Symmetric and
    kUInt4Affine with groups of 128) with bf16 activations and outputs, bias and SiLU, at decode
    batches.
    Algorithmic bytes: codes + scales + X + bias + Y. Weight copies rotate (> L2)."""
    out = {}
    for layout, group, m, n, k in ((qx.INT8_SYMMETRIC, 0, 1, 4096, 4096), (qx.INT8_SYMMETRIC, 0, 1, 14336, 4096),
                                   (qx.INT8_SYMMETRIC, 0, 8, 4096, 4096), (qx.INT4_SYMMETRIC, 128, 1, 14336, 4096),
                                   (qx.INT4_SYMMETRIC, 128, 8, 4096, 4096), (qx.UINT4_AFFINE, 128, 1, 14336, 4096),
                                   (qx.INT8_SYMMETRIC, 0, 512, 14336, 4096)):
        rng = np.random.default_rng(n + m)
        code_bytes = n * k if layout == qx.INT8_SYMMETRIC else n * k // 2
        groups = 1 if group == 0 else k // group
        copies = max(3, int(300e6 // code_bytes)) if m < 32 else 2
        handles = []
        for _ in range(copies):
            data = rng.integers(0, 256, code_bytes, dtype=np.uint8)
            scales = rng.uniform(0.001, 0.01, n * groups).astype(np.float32)
            zeros = (rng.integers(0, 16, n * groups).astype(np.float32)
                     if layout == qx.UINT4_AFFINE else None)
            h = qx.CanonicalWeights()
            mode = qx.SCALE_CHANNEL if group == 0 else qx.SCALE_GROUP
            qx.check(h.prepare(qx.canonical_view(layout, mode, n, k, group or k, data, scales,
                                                 zeros=zeros)), "prepare")
            handles.append(h)
        xd = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda().to(torch.bfloat16)
        bias = torch.from_numpy(rng.standard_normal(n, dtype=np.float32)).cuda()
        yd = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        sec = _time_calls(torch, lambda i: qx.check(
            handles[i % copies].qgemm_storage_dev(xd, qx.BF16, yd, qx.BF16, m, bias=bias,
                                                  activation=qx.ACT_SILU), "canonical"),
            4 * copies if m < 32 else 4)
        nbytes = (code_bytes + 4 * n * groups * (2 if layout == qx.UINT4_AFFINE else 1) + 2 * m * k +
                  4 * n + 2 * m * n)
        name = {qx.INT8_SYMMETRIC: "int8", qx.INT4_SYMMETRIC: "int4g128",
                qx.UINT4_AFFINE: "uint4affine_g128"}[layout] + f"_m{m}_n{n}_k{k}"
        out[name] = {"us": sec * 1e6, "gbs": nbytes / sec / 1e9,
                     "frac_of_measured_hbm": nbytes / sec / 1e9 / hbm_peak,
                     # the digits of the activations, then the projection; from five tokens on
                     # row digits, the W8A8 tensor-core GEMM on the digit planes and the combine per 256 tokens
                     "launches": 2 if (m < 5 or layout != qx.INT8_SYMMETRIC) else 3 * ((m + 255) // 256)}
        if m >= 32:
            out[name]["tops"] = 2.0 * m * n * k / sec / 1e12
        for h in handles:
            h.reset()
    return {"canonical_projection": out}


_RESULT_FD = None


def emit(line: dict):
    """The one JSON line of the run, on the process's original standard output."""
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text)


def main():
    # Libraries loaded below (NCCL among them) write banners to standard output: everything
    # except the result line goes to standard error.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20000)
    parser.add_argument("--warmup", type=int, default=200)
    parser.add_argument("--impl", default="qx", choices=["qx", "reference"])
    parser.add_argument("--no-extra", action="store_true",
                        help="skip the non-headline configurations and the CPU baseline (profiling runs)")
    parser.add_argument("--no-graph", action="store_true", help="launch every step eagerly")
    parser.add_argument("--extra-only", choices=EXTRA_CASES, default=None,
                        help="run just this non-headline configuration and print its figures "
                             "(profiling runs)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "qx" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.extra_only is not None:
        import torch
        torch.cuda.set_device(0)
        hbm_peak, bf16_peak, _ = measured_peaks()
        emit(extra_measurements(entry.load_package(), load_workloads(), torch, hbm_peak, bf16_peak,
                                only=args.extra_only))
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_sharded(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
