"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl qx|reference]

Headline workload (N = 1): the 4-bit block GEMV at FFN-up shape -- M=1, K=4096 f32
activations ~N(0,1), N=14336 x K=4096 q4_0 weights (33 MB) -- measured as achieved HBM
GB/s: algorithmic bytes (packed weights + activations read + outputs written) / time.
A step is one GEMV call. The weights fit in L2, so the timed loop rotates over several
distinct weight copies whose total size exceeds L2 (stated in `config`). With N > 1 every
rank holds one such shard of an (N*14336) x 4096 matrix (weak scaling), computes its
output slice and all ranks exchange slices (all-gather), as the sharded configurations of
this path do.

Prints ONE JSON line (rank 0). `value` is timed with inputs resident in HBM, `e2e` through
the host-pointer C entry point with pinned host buffers (host<->device copies inside the
timed region), `cpu_baseline` is the reference's CPU path on this host's cores on a
bounded sample, `roofline` relates the step to the measured HBM copy bandwidth.
"""

from __future__ import annotations

import argparse
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
WORKLOAD = "cfg1_q4_0_gemv"
GRAPH_CHUNK = 100


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

def cpu_engine():
    """(kind, call, threads): the built reference library when present, else the oracle port."""
    oracle_mod = entry.load_oracle()
    threads = os.cpu_count() or 1
    if oracle_mod.Reference.available():
        ref = oracle_mod.Reference()
        ref.set_num_threads(threads)
        return "reference", ref, threads, ref.variants()
    return "port", oracle_mod.Oracle(), 1, {}


def time_cpu_gemv(engine_kind, engine, fmt, packed, x, n, k, budget_s, max_calls):
    """Median seconds per call of the CPU GEMV over rows [0, n); at least 3 calls."""
    def call():
        if engine_kind == "reference":
            return engine.qgemv(fmt, packed, x, n, k)
        return engine.qgemv(fmt, packed, x, n, k, 0)
    call()
    times, start = [], time.perf_counter()
    while len(times) < max_calls and (len(times) < 3 or time.perf_counter() - start < budget_s):
        t0 = time.perf_counter()
        call()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = load_workloads()
    c = wl.CONFIGS[WORKLOAD]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    x = wl.activations_f32(1, k, seed=0)[0].copy()
    kind, engine, threads, variants = cpu_engine()

    def call(rows):
        if kind == "reference":
            engine.qgemv(fmt, packed, x, rows, k)
        else:
            engine.qgemv(fmt, packed, x, rows, k, 0)
    # bound the run to about two minutes: shrink the per-step row sample if needed
    call(n)
    t0 = time.perf_counter()
    for _ in range(3):
        call(n)
    per_call = (time.perf_counter() - t0) / 3
    rows = n
    total_steps = args.steps + args.warmup
    if per_call * total_steps > 120.0:
        rows = int(max(32 * threads, min(n, n * 120.0 / (per_call * total_steps))))
        rows -= rows % 32
        rows = max(rows, 32)
    for _ in range(args.warmup):
        call(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call(rows)
    elapsed = time.perf_counter() - t0
    step_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, rows, k)
    value = step_bytes * args.steps / elapsed / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": 1, "n": n, "k": k, "format": "q4_0",
                   "rows_per_step": rows, "variants": variants},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": f"{args.steps} calls of the reference qgemv over {rows} of {n} rows"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

def run_qx_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    qx = entry.load_package()
    wl = load_workloads()
    c = wl.CONFIGS[WORKLOAD]
    fmt, n, k = c["fmt"], c["n"], c["k"]
    step_bytes = wl.algorithmic_bytes_qgemv(fmt, 1, n, k)
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    info = qx.device_info()

    # distinct weight copies whose total size exceeds L2, rotated step by step
    copies = max(2, -(-2 * info["l2_bytes"] // (n * (k // 32) * 18)))
    handles = []
    for i in range(copies):
        packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=rank * 1000 + i)
        h = qx.PackedWeights()
        qx.check(h.prepare(fmt, packed, n, k), "qx_weights_prepare")
        handles.append(h)
    x_host = wl.activations_f32(1, k, seed=0)
    x_dev = torch.from_numpy(x_host).cuda()
    y_full = torch.zeros(world * n, device="cuda")
    y_local = y_full[rank * n:(rank + 1) * n]

    # Sharded runs: every rank streams its own shard and the output slices are exchanged. The
    # exchange is fused into the GEMV (peer stores from its epilogue + a wait kernel); if the
    # peer mapping cannot be set up, NCCL's all-gather takes its place.
    gather, exchange = None, "none"
    if world > 1:
        try:
            sharded = entry._load_file(entry.PKG_NAME + ".sharded", os.path.join(entry.PKG_DIR, "sharded.py"))
            gather = sharded.PushAllGather(qx, n, 1)
            exchange = "peer stores fused into the GEMV epilogue + wait kernel"
        except Exception as exc:
            print(f"bench: fused all-gather unavailable ({exc!r}); using NCCL", file=sys.stderr)
            gather, exchange = None, "nccl all_gather_into_tensor"
        healthy = 1 if gather is not None else 0
        if gather is not None:
            # two trial steps: this rank's slice of the gathered result must equal its own GEMV
            # bit for bit, and no kernel may have given up a wait (a tiny host-pointer call
            # reports that)
            try:
                want = torch.zeros(n, device="cuda")
                for trial in range(2):
                    qx.check(handles[trial].qgemm_dev(x_dev, want, 1, n), "trial gemv")
                    got_ptr = gather.step(handles[trial], x_dev, 1)
                    torch.cuda.synchronize()
                    got = _device_floats(torch, got_ptr + 4 * rank * n, n)
                    if not torch.equal(got.view(torch.int32), want.view(torch.int32)):
                        healthy = 0
                tiny = wl.packed_blocks(fmt, 32, 32, c["d_lo"], c["d_hi"], seed=1)
                status, _ = qx.qgemv(fmt, tiny, wl.activations_f32(1, 32)[0], 32, 32)
                if status != qx.OK:
                    healthy = 0
            except Exception as exc:
                print(f"bench: fused all-gather trial failed ({exc!r}); using NCCL", file=sys.stderr)
                healthy = 0
        flags = torch.tensor([healthy], device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)  # all ranks take the same path
        if int(flags.item()) == 0:
            gather, exchange = None, "nccl all_gather_into_tensor"

    def step(i):
        if gather is not None:
            gather.step(handles[i % copies], x_dev, 1)
            return
        qx.check(handles[i % copies].qgemm_dev(x_dev, y_local, 1, n), "qx_qgemm_prepacked_dev")
        if world > 1:
            dist.all_gather_into_tensor(y_full, y_local)

    launches0 = qx.launch_count()
    step(0)
    launches_per_step = qx.launch_count() - launches0
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    graph = None
    chunk = GRAPH_CHUNK - GRAPH_CHUNK % copies or copies
    chunk -= chunk % 2  # fused all-gather: the result buffers alternate step by step
    if (world == 1 or gather is not None) and args.steps >= chunk and chunk > 0 and not args.no_graph:
        # The steps are captured once and replayed, so the host's launch cost stays out of the
        # timed region. Sharded runs that fall back to NCCL launch step by step: a graph that
        # also held the NCCL all-gathers did not make progress on two GPUs (both ranks stopped
        # inside the first replay), so that combination is not used.
        try:
            captured = torch.cuda.CUDAGraph()
            with torch.cuda.graph(captured):
                for i in range(chunk):
                    step(i)
            captured.replay()
            torch.cuda.synchronize()
            graph = captured
        except Exception as exc:  # fall back to plain launches
            print(f"bench: graph capture failed ({exc!r}); timing plain launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    done = 0
    if graph is not None:
        while done + chunk <= args.steps:
            graph.replay()
            done += chunk
    for i in range(done, args.steps):
        step(i)
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    value = step_bytes * world * args.steps / (elapsed_ms * 1e-3) / 1e9

    # end to end through the host-pointer entry point: pinned x in, pinned y out, every step
    x_pin = torch.from_numpy(x_host).pin_memory()
    y_pin = torch.zeros(n).pin_memory()
    e2e_steps = max(10, min(args.steps, 2000))
    for i in range(3):
        qx.check(handles[i % copies].qgemm_prepacked_ptr(x_pin.data_ptr(), y_pin.data_ptr(), 1), "e2e")
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        qx.check(handles[i % copies].qgemm_prepacked_ptr(x_pin.data_ptr(), y_pin.data_ptr(), 1), "e2e")
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = step_bytes * world * e2e_steps / e2e_s / 1e9

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    per_launch_gbs = step_bytes * args.steps / (elapsed_ms * 1e-3) / 1e9  # this rank's GPU
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": 1, "n": n, "k": k, "format": "q4_0",
                   "sharding": f"rows x{world}" if world > 1 else "none", "exchange": exchange,
                   "l2_policy": f"rotates {copies} distinct weight copies "
                                f"({copies * n * (k // 32) * 18 / 1e6:.0f} MB > L2 {info['l2_bytes'] / 1e6:.0f} MB)",
                   "cuda_graph": graph is not None, "variants": qx.variants()},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * k,
                "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
                "note": "host-pointer C entry point per step: x copied from pinned host memory, y "
                        "written by the kernel into the caller's pinned host buffer, then one "
                        "stream synchronisation"},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_launch_gbs, "peak": hbm_peak, "unit": "GB/s",
                     "frac": per_launch_gbs / hbm_peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                     "peak_source": f"{peak_kind} HBM copy bandwidth",
                     "frac_of_nominal_8TBs": per_launch_gbs / 8000.0,
                     "note": "achieved = algorithmic bytes / whole step time (one kernel per "
                             "step; launch gaps included)"},
    }
    if world == 1 and not args.no_extra:
        line["cpu_baseline"] = cpu_baseline(wl, c)
        try:
            line["extra"] = extra_measurements(qx, wl, torch, hbm_peak, bf16_peak)
        except Exception as exc:  # the headline line must still be printed
            line["extra"] = {"error": repr(exc)}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(wl, c):
    fmt, n, k = c["fmt"], c["n"], c["k"]
    packed = wl.packed_blocks(fmt, n, k, c["d_lo"], c["d_hi"], seed=0)
    x = wl.activations_f32(1, k, seed=0)[0].copy()
    kind, engine, threads, variants = cpu_engine()
    seconds, calls = time_cpu_gemv(kind, engine, fmt, packed, x, n, k, budget_s=10.0, max_calls=4000)
    return {"value": wl.algorithmic_bytes_qgemv(fmt, 1, n, k) / seconds / 1e9, "unit": "GB/s",
            "cores": threads, "kind": kind, "ms_per_call": seconds * 1e3,
            "sample": f"median of {calls} full-size qgemv calls ({n}x{k} q4_0)", "variants": variants}


def _device_floats(torch, address: int, count: int):
    """`count` floats at a raw device address, copied into a torch tensor."""
    import ctypes
    out = torch.empty(count, dtype=torch.float32, device="cuda")
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    if cudart.cudaMemcpy(out.data_ptr(), address, count * 4, 3) != 0:  # device to device
        raise RuntimeError("cudaMemcpy failed")
    return out


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


# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_tc_kernel launch on the headline
# workload, from the ncu capture summarised in profiles/gemv_tc_q4_0_cfg1.md (algorithmic
# bytes: 33 103 872)
NCU_DRAM_BYTES_PER_LAUNCH = 33167104

EXTRA_CASES = ("cfg2_w8a8_gemm", "cfg0_q8_0_gemv", "cfg3_q8_0_batched", "cfg4_q4_0_prefill")


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


def main():
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
        print(json.dumps(extra_measurements(entry.load_package(), load_workloads(), torch, hbm_peak,
                                            bf16_peak, only=args.extra_only)), flush=True)
    else:
        run_qx_arm(args)


if __name__ == "__main__":
    main()
