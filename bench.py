#!/usr/bin/env python
"""Benchmark of the hot path on B200: the fused pointwise chain (headline) and, in the same line, the
f32 matmul / bmm / MLP configurations.

    python bench.py --gpus N --steps K --warmup W            # this build (one rank per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores
    python bench.py --workload c3|c4|c5|c1|t1|copy           # one side workload alone (profiling aid)

Headline workload (N=1): `exp(2.0 * relu(x.mT + b)) - x.mT`, x f32 [8192,8192] ~N(0,1) read through a
transposed view, b f32 [8192] ~N(0,0.1) broadcast, scalar 2.0 -- a five-op chain run as ONE kernel.
A step builds the chain through the public `torch_rs` surface and forces its execution.  With N ranks
every rank runs the same-sized shard of an N-times larger batch (weak scaling, no data-path collective).
Algorithmic bytes per step and GPU: 8 B per element (x read once, result written once) + b
= 8*8192*8192 + 4*8192 = 536,903,680 B.

`extra` carries the rest: c1 relu(x+y) and t1 x.mT+y (the staged-tile kernel class) as further pointwise figures,
the streaming kernels of a backward pass, the host-link copy ceiling, and the metric's other half, each with its
own roofline, clock record, end-to-end figure and (at N=1) CPU baseline: c3 matmul 4096^3, c4 bmm 64x1024^3 + bias
+ relu (batches sharded over the ranks), c5 two-layer MLP forward+backward on 65,536 rows (rows sharded over the ranks, NCCL all-reduce of the
W1/W2/b1 gradients inside the step) -- those three strong-scaled: the total work is fixed as N grows.
Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "pytorch-rs_b200"))
sys.path.insert(0, ROOT)

N_SIDE = 8192
ALGO_BYTES = 8 * N_SIDE * N_SIDE + 4 * N_SIDE
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
WORKLOAD_TEXT = ("exp(2.0*relu(x.mT+b))-x.mT, x f32 [8192,8192] via transposed view, b [8192] broadcast, scalar 2.0; "
                 "one pass of the whole chain per step, per GPU")
# dram__bytes_read.sum + dram__bytes_write.sum of one trs_pw launch on this workload, from an ncu
# capture of exactly this kernel and size (its summary is kept under profiles/); writes that are
# still dirty in L2 when the kernel ends are not counted.
NCU_DRAM_BYTES_PER_LAUNCH = 488058752
MIN_REGION_SECONDS = 0.3            # side workloads are timed for at least this long, so the clock record is taken under load
GEMM_ALGOS = {1: "simt_fp32", 2: "tcgen05_3xtf32", 3: "tcgen05_3xtf32_2cta"}
C5_FLOPS = 2 * 65536 * (2 * 4096 ** 2 + 3 * 4096 * 1024)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        peaks = json.load(open(path))
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


def make_inputs(seed, rows=N_SIDE):
    """Seeded synthetic inputs with the workload's shapes and distributions (NumPy default_rng)."""
    rng = np.random.default_rng(seed)
    xs = rng.standard_normal((rows, N_SIDE)).astype(np.float32)      # storage of x; the operand is xs.mT
    b = (0.1 * rng.standard_normal(rows)).astype(np.float32)
    return xs, b


class ClockSampler:
    """Samples SM clocks and clock-event reasons through NVML on a thread.  `mark(True/False)` brackets the timed
    regions, so the summary can tell samples taken inside them from those of the untimed post-roll."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []            # (MHz, inside a timed region)
        self.reasons = set()
        self.max_clock = None
        self.stop = threading.Event()
        self.thread = None
        self.nvml = None
        self.timed = False

    def _physical_index(self):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            parts = [p for p in visible.split(",") if p.strip()]
            if self.gpu_index < len(parts) and parts[self.gpu_index].strip().isdigit():
                return int(parts[self.gpu_index])
        return self.gpu_index

    def _run(self, handle):
        nv = self.nvml
        while not self.stop.is_set():
            try:
                inside = self.timed
                self.samples.append((nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM), inside))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def mark(self, timed):
        self.timed = timed

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_clock = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._run, args=(handle,), daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        timed = [mhz for mhz, inside in self.samples if inside]
        everything = [mhz for mhz, _ in self.samples]
        return {"sm_mhz": statistics.median(timed) if timed else (statistics.median(everything) if everything else None),
                "sm_mhz_all_samples": statistics.median(everything) if everything else None,
                "sm_mhz_min": min(timed) if timed else None, "sm_max_mhz": self.max_clock, "reasons": sorted(self.reasons),
                "samples_in_timed_region": len(timed), "samples": len(everything),
                "how": "NVML on a thread every ~2 ms; sm_mhz is the plain median of the samples taken inside the timed "
                       "region(s), sm_mhz_all_samples includes the untimed post-roll of the same steps where there is one"}


def cpu_chain(xs, b):
    """The same chain through the CPU checker, op by op as the reference engine runs it."""
    from oracle.ref import RefTensor
    x, bt = RefTensor.from_numpy(xs), RefTensor.from_numpy(b)
    return (2.0 * (x.mT + bt).relu()).exp() - x.mT


def headline_config(world):
    return {"workload": WORKLOAD_TEXT, "l2": "inputs+outputs 512 MiB per step, larger than the 126 MB L2",
            "parallelism": f"dp{world}", "algorithmic_bytes_per_step_per_gpu": ALGO_BYTES}


def reference_rows(total_steps):
    """Physical rows of x per step of the reference arm.  One full-size step takes about 6 s on one core: the whole
    workload while the run fits in ~2.5 minutes, else as many of its 8192 rows (a multiple of 256) as keep it near 2."""
    if total_steps * 6.0 <= 160:
        return N_SIDE
    return max(256, min(N_SIDE, int(N_SIDE * 120.0 / (total_steps * 6.0)) // 256 * 256))


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU algorithm for this chain (C++ restatement in oracle/, since
    no Rust toolchain exists to build the original) on the host cores; single-threaded, as the
    reference engine is."""
    if rank != 0:
        return
    from oracle import ref
    ref.build()
    rows = reference_rows(args.steps + args.warmup)
    xs, b = make_inputs(0, rows)
    bytes_per_step = 8 * rows * N_SIDE + 4 * rows
    for _ in range(args.warmup):
        cpu_chain(xs, b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_chain(xs, b)
    dt = time.perf_counter() - t0
    value = bytes_per_step * args.steps / dt / 1e9
    sample = f"{rows} of {N_SIDE} physical rows of x per step ({bytes_per_step} algorithmic bytes)"
    line = {
        "impl": "reference", "metric": "fused pointwise GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Bench:
    """Per-process state shared by the workloads: device, engine stream, rank plumbing."""

    def __init__(self, rank, world, local_rank):
        import torch_rs as torch
        from torch_rs import _host, distributed as tdist
        from torch_rs._device import Stream
        self.torch, self.tdist = torch, tdist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.shards = world          # how many shards the strong-scaled workloads are cut into (--shard-of overrides it)
        self.dev = f"cuda:{local_rank}"
        from torch_rs import _abi
        _abi.check(_abi.lib().trs_set_current_device(local_rank))      # pinned staging memory belongs to this rank's GPU context
        self.numa_node = tdist.bind_to_device_numa_node(local_rank)     # staging memory local to this GPU's PCIe root
        if world > 1:
            tdist.init_process_group("nccl")       # gloo control plane + the engine's own NCCL communicator
        raw = ctypes.c_void_p()
        _host.check(_host.lib().trsh_stream(local_rank, ctypes.byref(raw)))
        self.stream = Stream.__new__(Stream)
        self.stream.device, self.stream.handle = local_rank, raw   # the engine's own stream: events go where the kernels go
        self.hbm_peak, self.bf16_peak, self.peak_kind = measured_peaks()
        self.tensor_peak = self.bf16_peak / 6.0      # tf32 runs at half the bf16 rate; the split issues 3 MMAs per product

    def sync(self):
        self.torch.synchronize(self.local_rank)

    def barrier(self):
        self.sync()
        self.tdist.barrier()

    def max_over_ranks(self, value):
        if self.world == 1:
            return value
        return float(self.tdist.all_reduce_host(np.array([value], dtype=np.float64), op="max")[0])

    def region_ms(self, fn, steps):
        from torch_rs._device import Event
        e0, e1 = Event(), Event()
        e0.record(self.stream)
        for _ in range(steps):
            fn()
        e1.record(self.stream)
        e1.sync()
        return e0.elapsed_ms(e1)

    def time_side(self, step, warmup=3, min_steps=5):
        """Warm up, then one timed region of at least MIN_REGION_SECONDS (the same step count on every rank),
        bracketed by barrier + sync, clocks sampled inside it.  Returns (ms_per_step, steps, launches, clocks)."""
        from torch_rs._device import launch_count
        for _ in range(max(warmup, 3)):
            step()
        self.barrier()
        estimate = self.max_over_ranks(self.region_ms(step, 3) / 3)
        steps = int(max(min_steps, math.ceil(MIN_REGION_SECONDS * 1e3 / max(estimate, 1e-3))))
        self.barrier()
        launches0 = launch_count()
        with ClockSampler(self.local_rank) as clocks:
            clocks.mark(True)
            ms = self.region_ms(step, steps)
            clocks.mark(False)
        launches = launch_count() - launches0
        self.barrier()
        return self.max_over_ranks(ms) / steps, steps, launches, clocks.summary()

    def time_wall(self, step, steps, warmup=4):
        """End-to-end steps end with a device sync of their own; wall clock, max over ranks.  Four warm-up steps: the
        block cache gives an upload stream new memory rather than a block the compute stream is still using, so the
        pool of a slab loop keeps growing (cudaMalloc) for its first two or three steps."""
        for _ in range(warmup):
            step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        self.sync()
        return self.max_over_ranks((time.perf_counter() - t0) * 1e3) / steps

    def tensor_roofline(self, per_gpu_tflops, kernel):
        return {"bound": "tensor", "achieved": per_gpu_tflops, "peak": self.tensor_peak, "unit": "TFLOP/s",
                "frac": per_gpu_tflops / self.tensor_peak, "traffic": None, "kernel": kernel,
                "peak_source": f"of {self.peak_kind}: bf16_tflops / 6 (kind::tf32 runs at half the bf16 rate and the 3xTF32 "
                               "split issues 3 MMAs per product); useful flops only"}


def matmul_algo_name(torch_mod, a, b, c_shape):
    """The algorithm TRS_GEMM_AUTO picks for a @ b (read-only query, no launch)."""
    from torch_rs import _abi
    desc = _abi.GemmDesc()
    batched = len(c_shape) == 3
    desc.batch = c_shape[0] if batched else 1
    desc.m, desc.n, desc.k = c_shape[-2], c_shape[-1], a.shape[-1]
    desc.a, desc.b, desc.c = a._const_data_ptr(), b._const_data_ptr(), a._const_data_ptr()
    sa, sb = a.stride(), b.stride()
    desc.a_batch_stride = sa[0] if batched else 0
    desc.a_row_stride, desc.a_col_stride = sa[-2], sa[-1]
    desc.b_batch_stride = sb[0] if batched else 0
    desc.b_row_stride, desc.b_col_stride = sb[-2], sb[-1]
    desc.c_batch_stride, desc.c_row_stride = desc.m * desc.n, desc.n
    algo = ctypes.c_int32()
    _abi.check(_abi.lib().trs_matmul_select_algo(ctypes.byref(desc), ctypes.byref(algo)))
    return GEMM_ALGOS.get(algo.value, "unknown")


def matmul_error_over_bound(got, want64, k):
    """max |dC| / (1e-5 * sqrt(K) * max(|C|, rms C)): the path's stated matmul tolerance; <= 1 passes."""
    want64 = np.asarray(want64, dtype=np.float64)
    rms = float(np.sqrt(np.mean(want64 ** 2)))
    bound = 1e-5 * np.sqrt(k) * np.maximum(np.abs(want64), rms) + 1e-30
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - want64) / bound))


# ---- the headline: config 2 ---------------------------------------------------------------------------

def run_headline(bench, args):
    torch, dev, rank, world, local_rank = bench.torch, bench.dev, bench.rank, bench.world, bench.local_rank
    from torch_rs._device import launch_count
    xs, b = make_inputs(rank)
    x, bt = torch.tensor(xs, device=dev), torch.tensor(b, device=dev)
    held = [None]

    def step():
        held[0] = (torch.exp(2.0 * torch.relu(x.mT + bt)) - x.mT).materialize()

    # ---- device-resident throughput: 9 timed regions of exactly `steps` steps each ---------------
    for _ in range(max(args.warmup, 3)):
        step()
    regions = []
    launches = 0
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.regions):
            bench.barrier()
            launches0 = launch_count()
            clocks.mark(True)
            ms = bench.region_ms(step, args.steps)
            clocks.mark(False)
            launches = launch_count() - launches0
            bench.barrier()
            regions.append(bench.max_over_ranks(ms) / args.steps)
        post_roll_until = time.perf_counter() + 0.3        # same steps, untimed, so the sampler also sees sustained load
        while time.perf_counter() < post_roll_until:
            for _ in range(20):
                step()
            bench.sync()
    ms_per_step = statistics.median(regions)
    value = world * ALGO_BYTES / (ms_per_step * 1e-3) / 1e9

    # ---- parity spot check on this rank's result (checker on a slab of physical rows) ---------
    parity = None
    if rank == 0:
        from oracle import ref
        from oracle.ref import RefTensor
        rows = 64
        got = held[0].mT.numpy()[:rows]                        # physical rows of the result
        got_e = torch.exp(2.0 * torch.relu(x.mT + bt)).mT.numpy()[:rows]
        rx, rb = RefTensor.from_numpy(xs[:rows]), RefTensor.from_numpy(b[:rows])
        want_e = (2.0 * (rx.mT + rb).relu()).exp()
        want = (want_e - rx.mT).mT.logical()
        same = got_e.view(np.uint32) == want_e.mT.logical().view(np.uint32)
        parity = {"exp_term_max_ulp_vs_cpu": int(ref.ulp_distance(got_e, want_e.mT.logical()).max()), "tolerance_ulp": 2,
                  "result_bit_exact_where_exp_agrees": bool(np.array_equal(got[same].view(np.uint32), want[same].view(np.uint32))),
                  "exp_lanes_bit_exact_fraction": float(same.mean()), "rows_checked": rows}

    # ---- end to end: pinned host buffers in, result read back, every step -----------------------
    x_host, b_host = torch.pinned_empty(N_SIDE, N_SIDE), torch.pinned_empty(N_SIDE)
    out_host = torch.pinned_empty(N_SIDE, N_SIDE)
    x_host[...] = xs
    b_host[...] = b
    slabs = args.e2e_slabs                         # physical-row slabs: upload of slab i+1 overlaps read-back of slab i

    def step_e2e():
        rows = N_SIDE // slabs
        for i in range(slabs):
            sl = slice(i * rows, (i + 1) * rows)
            xd, bd = torch.tensor(x_host[sl], device=dev), torch.tensor(b_host[sl], device=dev)
            out = torch.exp(2.0 * torch.relu(xd.mT + bd)) - xd.mT
            out.mT.copy_to_host(out_host[sl], non_blocking=True)     # the result's storage order
        torch.synchronize(local_rank)              # every slab's result is in host memory

    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = bench.time_wall(step_e2e, e2e_steps)
    e2e_value = world * ALGO_BYTES / (e2e_ms * 1e-3) / 1e9
    e2e_same = None
    if rank == 0:       # the end-to-end result is the device-resident step's result, bit for bit (a pointwise chain has one rounding order)
        e2e_same = bool(np.array_equal(out_host[:8].view(np.uint32), held[0].mT.numpy()[:8].view(np.uint32)))
    for array in (x_host, b_host, out_host):
        torch.pinned_free(array)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            cpu_chain(xs, b)
            times.append(time.perf_counter() - t0)
        cpu_baseline = {"value": ALGO_BYTES / statistics.median(times) / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                        "sample": "the full workload, median of 3 runs", "host_cores": os.cpu_count()}
    achieved = ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
    return {
        "value": value, "ms_per_step": ms_per_step, "launches": launches, "clocks": clocks.summary(), "parity": parity,
        "timing": {"regions": len(regions), "steps_per_region": args.steps, "ms_per_step_median": ms_per_step,
                   "ms_per_step_min": min(regions), "ms_per_step_max": max(regions),
                   "how": "CUDA events on the engine's stream around each region, barrier + sync on both sides, max over ranks per region"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": bench.hbm_peak, "unit": "GB/s", "frac": achieved / bench.hbm_peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "peak_source": f"of {bench.peak_kind}", "kernel": "trs_pw (vector class)"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ALGO_BYTES // 2 + 2 * N_SIDE,
                "d2h_bytes_per_step": 4 * N_SIDE * N_SIDE, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "how": f"pinned host buffers; {slabs} row slabs per step so uploads, kernels and read-backs overlap",
                "numa_node": bench.numa_node, "result_equals_device_resident_step": e2e_same},
        "cpu_baseline": cpu_baseline,
    }


# ---- the backward pass's streaming kernels -------------------------------------------------------------

def run_backward_kernels(bench):
    """The kernels a backward pass runs besides GEMMs, each alone through the C ABI on 1 GiB operands (larger than
    L2), against the HBM roofline: the relu VJP as a fused chain (read the saved input and the upstream, write the
    gradient: 12 B per element), the column sum that un-broadcasts a bias gradient (db1 = sum over rows of dZ: 4 B per
    element), the full sum of a loss (4 B per element) and the in-place accumulation of a leaf gradient (12 B per
    element).  Per GPU, rank 0's figures."""
    from torch_rs import _abi
    from torch_rs._device import DeviceBuffer, Event, Stream
    lib = _abi.lib()
    dev = bench.local_rank
    rows, cols = 65536, 4096
    n = rows * cols
    stream = Stream(dev)
    z, g, out = DeviceBuffer(n, dev), DeviceBuffer(n, dev), DeviceBuffer(n, dev)
    small = DeviceBuffer(cols, dev)
    _abi.check(lib.trs_fill_f32(z.ptr, n, ctypes.c_float(0.5), stream.handle))
    _abi.check(lib.trs_fill_f32(g.ptr, n, ctypes.c_float(0.25), stream.handle))
    _abi.check(lib.trs_fill_f32(out.ptr, n, ctypes.c_float(0.0), stream.handle))
    prog = _abi.make_program(2, [("relu_vjp", 0, 1, 0)], [2])
    ins = (_abi.Operand * 2)(_abi.make_operand(z.ptr, 0, [rows, cols], [cols, 1]), _abi.make_operand(g.ptr, 0, [rows, cols], [cols, 1]))
    outs = (_abi.Operand * 1)(_abi.make_operand(out.ptr, 0, [rows, cols], [cols, 1]))
    whole = _abi.make_operand(z.ptr, 0, [rows, cols], [cols, 1])
    cases = {
        "relu_vjp_chain": (12 * n, lambda: _abi.check(lib.trs_pointwise(prog, ins, outs, stream.handle))),
        "column_sum_unbroadcast": (4 * n, lambda: _abi.check(lib.trs_unbroadcast_sum_f32(g.ptr, rows, cols, 0, small.ptr, stream.handle))),
        "full_sum": (4 * n, lambda: _abi.check(lib.trs_reduce_sum_f32(ctypes.byref(whole), small.ptr, stream.handle))),
        "leaf_gradient_accumulate": (12 * n, lambda: _abi.check(lib.trs_accumulate_f32(out.ptr, g.ptr, n, stream.handle))),
    }
    result = {"operand": "f32 [65536, 4096] (1 GiB) each", "peak_gbs": bench.hbm_peak, "peak_source": f"of {bench.peak_kind}"}
    for name, (nbytes, call) in cases.items():
        for _ in range(3):
            call()
        stream.sync()
        e0, e1 = Event(), Event()
        e0.record(stream)
        reps = 20
        for _ in range(reps):
            call()
        e1.record(stream)
        e1.sync()
        ms = e0.elapsed_ms(e1) / reps
        gbs = nbytes / (ms * 1e-3) / 1e9
        result[name] = {"GB/s": gbs, "ms": ms, "algorithmic_bytes": nbytes, "frac": gbs / bench.hbm_peak}
    return result


# ---- host <-> device copy ceiling ---------------------------------------------------------------------

def run_copy_ceiling(bench, mib=256, reps=5):
    """What the box's host link gives this rank: pinned-buffer copies of 256 MiB, host-to-device alone, device-to-host
    alone, and both at once on two streams (how the end-to-end steps use it); no kernel involved.  GB/s, all ranks
    copying at the same time, the slowest rank reported."""
    from torch_rs import _abi
    from torch_rs._device import DeviceBuffer, Event, PinnedBuffer, Stream
    lib = _abi.lib()
    count = mib * (1 << 20) // 4
    up, down = PinnedBuffer(count), PinnedBuffer(count)
    up.array[:] = 1.0
    d_in, d_out = DeviceBuffer(count, bench.local_rank), DeviceBuffer(count, bench.local_rank)
    s0, s1 = Stream(bench.local_rank), Stream(bench.local_rank)
    nbytes = count * 4

    def timed(h2d, d2h):
        bench.barrier()
        begin, end0, end1 = Event(), Event(), Event()
        begin.record(s0)
        _abi.check(lib.trs_stream_wait_event(s1.handle, begin.handle))
        for _ in range(reps):
            if h2d:
                _abi.check(lib.trs_memcpy_h2d(d_in.ptr, up.ptr, nbytes, s0.handle))
            if d2h:
                _abi.check(lib.trs_memcpy_d2h(down.ptr, d_out.ptr, nbytes, s1.handle))
        end0.record(s0)
        end1.record(s1)
        end0.sync()
        end1.sync()
        ms = max(begin.elapsed_ms(end0), begin.elapsed_ms(end1))
        return nbytes * reps / (bench.max_over_ranks(ms) * 1e-3) / 1e9

    timed(True, True)                                   # warm-up
    result = {"h2d_gbs": timed(True, False), "d2h_gbs": timed(False, True), "each_direction_when_both_gbs": timed(True, True),
              "mib_per_copy": mib, "copies": reps, "ranks_copying_at_once": bench.world,
              "how": "cudaMemcpyAsync between page-locked host buffers and device memory; CUDA events; slowest rank"}
    bench.barrier()
    return result


# ---- side workloads ---------------------------------------------------------------------------------------

def run_c1(bench):
    torch, dev = bench.torch, bench.dev
    n = 4096
    rng = np.random.default_rng(bench.rank)
    sets = [(torch.tensor(rng.uniform(-1, 1, (n, n)).astype(np.float32), device=dev),
             torch.tensor(rng.uniform(-1, 1, (n, n)).astype(np.float32), device=dev)) for _ in range(4)]
    it, held = [0], [None]

    def step():
        xa, ya = sets[it[0] % 4]
        it[0] += 1
        held[0] = torch.relu(xa + ya).materialize()
    ms, steps, launches, clocks = bench.time_side(step)
    per_gpu = 12 * n * n / (ms * 1e-3) / 1e9
    return {"workload": "relu(x + y), x,y f32 [4096,4096] contiguous ~U(-1,1), per GPU; 4 rotating operand sets (768 MiB) defeat L2",
            "metric": "fused pointwise GB/s", "value": per_gpu * bench.world, "unit": "GB/s", "scaling": "weak", "ms_per_step": ms,
            "steps": steps, "gpu_launches": launches, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": bench.hbm_peak, "unit": "GB/s", "frac": per_gpu / bench.hbm_peak,
                         "traffic": None, "peak_source": f"of {bench.peak_kind}", "kernel": "trs_pw (vector class)"}}


def run_t1(bench):
    torch, dev = bench.torch, bench.dev
    n = 8192
    rng = np.random.default_rng(bench.rank)
    xt = torch.tensor(rng.standard_normal((n, n), dtype=np.float32), device=dev)
    yt = torch.tensor(rng.standard_normal((n, n), dtype=np.float32), device=dev)
    held = [None]

    def step():
        held[0] = (xt.mT + yt).materialize()
    ms, steps, launches, clocks = bench.time_side(step)
    per_gpu = 12 * n * n / (ms * 1e-3) / 1e9
    return {"workload": "x.mT + y, x,y f32 [8192,8192] ~N(0,1): operand layouts disagree, staged through shared-memory tiles",
            "metric": "fused pointwise GB/s", "value": per_gpu * bench.world, "unit": "GB/s", "scaling": "weak", "ms_per_step": ms,
            "steps": steps, "gpu_launches": launches, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": bench.hbm_peak, "unit": "GB/s", "frac": per_gpu / bench.hbm_peak,
                         "traffic": None, "peak_source": f"of {bench.peak_kind}", "kernel": "trs_pw (tiled class)"}}


def run_c3(bench, args):
    """matmul(A, B) 4096^3.  N ranks: rows of A (and of C) sharded, B replicated, no collective."""
    torch, dev, rank, world = bench.torch, bench.dev, bench.rank, bench.world
    n = 4096
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((n, n)) / 64).astype(np.float32)
    b = (rng.standard_normal((n, n)) / 64).astype(np.float32)
    lo, hi = bench.tdist.shard_bounds(n, rank, bench.shards)
    A, B = torch.tensor(a[lo:hi], device=dev), torch.tensor(b, device=dev)
    held = [None]

    def step():
        held[0] = torch.matmul(A, B).materialize()
    step()
    first_ms = bench.region_ms(step, 1)                # operand images exist from the very first call on
    ms, steps, launches, clocks = bench.time_side(step)
    flops = 2 * n ** 3
    value = flops / (ms * 1e-3) / 1e12
    out = {"workload": "matmul(A, B), A,B f32 [4096,4096] ~N(0,1/64), precision highest; rows of A sharded over the ranks, B replicated",
           "metric": "f32 matmul TFLOP/s", "value": value, "unit": "TFLOP/s", "scaling": "strong", "ms_per_step": ms, "steps": steps,
           "gpu_launches": launches, "launches_per_step": launches / steps, "algo": matmul_algo_name(torch, A, B, (hi - lo, n)),
           "rows_per_gpu": hi - lo, "clocks": clocks, "roofline": bench.tensor_roofline(value / world, "gemm_tf32x3_pair_kernel"),
           "operands": "A and B stay resident across steps: their lo images are computed on first use and kept beside the storages "
                       "(storages are immutable), so a steady-state step is the GEMM alone",
           "second_call_ms": first_ms}
    # the same call with every operand prepared per call (images off): what a product of fresh operands costs
    torch.set_operand_image_cache(False)
    try:
        A2, B2 = torch.tensor(a[lo:hi], device=dev), torch.tensor(b, device=dev)

        def cold():
            held[0] = torch.matmul(A2, B2).materialize()
        cold_ms, _, cold_launches, _ = bench.time_side(cold)
    finally:
        torch.set_operand_image_cache(True)
    out["operands_prepared_per_call"] = {"ms_per_step": cold_ms, "value": flops / (cold_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                         "frac": flops / (cold_ms * 1e-3) / 1e12 / world / bench.tensor_peak}
    # parity: sampled rows in the reference's k-ascending order + float64 bound
    if rank == 0:
        from oracle.ref import RefTensor
        rows = np.random.default_rng(1).choice(hi - lo, 8, replace=False)
        got = held[0].numpy()[rows]
        want32 = RefTensor.from_numpy(a[lo:hi][rows]).matmul(RefTensor.from_numpy(b)).logical()
        want64 = a[lo:hi][rows].astype(np.float64) @ b.astype(np.float64)
        out["parity"] = {"rows_checked": 8, "error_over_bound_vs_cpu_f32_order": matmul_error_over_bound(got, want32, n),
                         "error_over_bound_vs_f64": matmul_error_over_bound(got, want64, n),
                         "bound": "1e-5*sqrt(K)*max(|C|, rms C); <= 1 passes"}
    # end to end: operands from pinned host memory, result back into pinned host memory, every step
    a_host, b_host, c_host = torch.pinned_empty(hi - lo, n), torch.pinned_empty(n, n), torch.pinned_empty(hi - lo, n)
    a_host[...] = a[lo:hi]
    b_host[...] = b

    upcoming = [(torch.tensor(a_host, device=dev), torch.tensor(b_host, device=dev))]

    def step_e2e():
        Ad, Bd = upcoming[0]
        product = torch.matmul(Ad, Bd).materialize()
        product.copy_to_host(c_host, non_blocking=True)       # ordered behind the product only: issued before the next upload
        upcoming[0] = (torch.tensor(a_host, device=dev), torch.tensor(b_host, device=dev))     # uploads under this product and its read-back
        torch.synchronize(bench.local_rank)
    e2e_ms = bench.time_wall(step_e2e, 5)
    upcoming.clear()
    e2e_same = None
    if rank == 0:       # same shapes, same tile plan, same rounding order as the resident product
        e2e_same = bool(np.array_equal(c_host[:4].view(np.uint32), held[0].numpy()[:4].view(np.uint32)))
    out["e2e"] = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": 5,
                  "result_equals_device_resident_step": e2e_same,
                  "h2d_bytes_per_step": 4 * ((hi - lo) * n + n * n), "d2h_bytes_per_step": 4 * (hi - lo) * n,
                  "how": "A shard and B uploaded from pinned host memory, operand images prepared, product, C read back, every step; the next "
                         "step's operands are uploaded (upload stream) while this step's product runs and its result is read back"}
    for array in (a_host, b_host, c_host):
        torch.pinned_free(array)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle.ref import RefTensor
        sample_rows = 1024
        ra, rb = RefTensor.from_numpy(a[:sample_rows]), RefTensor.from_numpy(b)
        t0 = time.perf_counter()
        ra.matmul(rb)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": 2 * sample_rows * n * n / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                               "host_cores": os.cpu_count(), "seconds": dt,
                               "sample": f"{sample_rows} of 4096 rows of A against all of B, one run (the reference's 4-row blocked "
                                         "kernel); per-row cost is uniform, so the rate is extrapolated to the whole product"}
    return out


def run_c4(bench, args):
    """relu(X @ W.mT + bias), 64 batches of 1024^3; batches sharded over the ranks, no collective."""
    torch, dev, rank, world = bench.torch, bench.dev, bench.rank, bench.world
    lo, hi = bench.tdist.shard_bounds(64, rank, bench.shards)
    nb = hi - lo
    rng = np.random.default_rng(rank)
    x = rng.standard_normal((nb, 1024, 1024), dtype=np.float32)
    w = (rng.standard_normal((nb, 1024, 1024), dtype=np.float32) / np.float32(32)).astype(np.float32)
    bias = np.random.default_rng(0).uniform(-0.1, 0.1, 1024).astype(np.float32)
    X, W, Bt = torch.tensor(x, device=dev), torch.tensor(w, device=dev), torch.tensor(bias, device=dev)
    held = [None]

    def step():
        held[0] = torch.relu(X @ W.mT + Bt).materialize()
    step()
    ms, steps, launches, clocks = bench.time_side(step)
    flops = 64 * 2 * 1024 ** 3
    value = flops / (ms * 1e-3) / 1e12
    out = {"workload": "relu(X @ W.mT + bias), X,W f32 [64,1024,1024], bias [1024]; bias+relu fused into the GEMM's store; "
                       "batches sharded over the ranks",
           "metric": "f32 bmm+bias+relu TFLOP/s", "value": value, "unit": "TFLOP/s", "scaling": "strong", "ms_per_step": ms, "steps": steps,
           "gpu_launches": launches, "launches_per_step": launches / steps, "algo": matmul_algo_name(torch, X, W.mT, (nb, 1024, 1024)),
           "batches_per_gpu": nb, "clocks": clocks, "roofline": bench.tensor_roofline(value / world, "gemm_tf32x3_pair_kernel"),
           "operands": "X and W stay resident across steps: lo images computed on first use and kept beside the storages"}
    torch.set_operand_image_cache(False)
    try:
        X2, W2 = torch.tensor(x, device=dev), torch.tensor(w, device=dev)

        def cold():
            held[0] = torch.relu(X2 @ W2.mT + Bt).materialize()
        cold_ms, _, _, _ = bench.time_side(cold)
        del X2, W2
    finally:
        torch.set_operand_image_cache(True)
    out["operands_prepared_per_call"] = {"ms_per_step": cold_ms, "value": flops / (cold_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                         "frac": flops / (cold_ms * 1e-3) / 1e12 / world / bench.tensor_peak}
    if rank == 0:
        from oracle.ref import RefTensor
        got = held[0].numpy()[0][:4]
        want = (RefTensor.from_numpy(x[0][:4]).matmul(RefTensor.from_numpy(w[0]).mT) + RefTensor(bias, [1024])).relu().logical()
        pre64 = x[0][:4].astype(np.float64) @ w[0].astype(np.float64).T + bias
        out["parity"] = {"rows_checked": 4, "error_over_bound_vs_cpu_f32_order": matmul_error_over_bound(got, want, 1024),
                         "error_over_bound_vs_f64": matmul_error_over_bound(got, np.maximum(pre64, 0), 1024),
                         "bound": "1e-5*sqrt(K)*max(|C|, rms C); <= 1 passes"}
    # end to end in slabs of batches: the read-back of slab i overlaps the upload of slab i+1
    slab = max(1, nb // 8)
    x_host, w_host, o_host = torch.pinned_empty(nb, 1024, 1024), torch.pinned_empty(nb, 1024, 1024), torch.pinned_empty(nb, 1024, 1024)
    x_host[...] = x
    w_host[...] = w

    def step_e2e():
        for i in range(0, nb, slab):
            sl = slice(i, min(nb, i + slab))
            Xd, Wd = torch.tensor(x_host[sl], device=dev), torch.tensor(w_host[sl], device=dev)
            torch.relu(Xd @ Wd.mT + Bt).copy_to_host(o_host[sl], non_blocking=True)
        torch.synchronize(bench.local_rank)
    e2e_ms = bench.time_wall(step_e2e, 3)
    e2e_error = None
    if rank == 0:
        # a slab of batches is a product of another size: its last round of tiles is cut along K differently, so it
        # rounds differently from the resident product of all batches; both must meet the tolerance
        pre64 = x[0][:4].astype(np.float64) @ w[0].astype(np.float64).T + bias
        e2e_error = matmul_error_over_bound(o_host[0][:4], np.maximum(pre64, 0), 1024)
    out["e2e"] = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": 3,
                  "result_error_over_bound_vs_f64": e2e_error,
                  "h2d_bytes_per_step": 8 * nb * 1024 * 1024, "d2h_bytes_per_step": 4 * nb * 1024 * 1024,
                  "how": f"X and W uploaded from pinned host memory and the result read back in slabs of {slab} batches, every step"}
    for array in (x_host, w_host, o_host):
        torch.pinned_free(array)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle.ref import RefTensor
        rb = RefTensor(bias, [1024])
        t0 = time.perf_counter()
        done = 0
        while done < 4 and (done == 0 or time.perf_counter() - t0 < 12.0):
            (RefTensor.from_numpy(x[done]).matmul(RefTensor.from_numpy(w[done]).mT) + rb).relu()
            done += 1
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": done * 2 * 1024 ** 3 / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                               "host_cores": os.cpu_count(), "seconds": dt,
                               "sample": f"{done} of 64 batches, each composed as the reference would (rank-2 matmul on W[i].mT -- its "
                                         "strided loop --, broadcast add, relu); batches cost the same, so the rate is extrapolated"}
    return out


def mlp_step(torch, X, w1, w2, b1):
    W1, W2, B1 = w1.detach().requires_grad_(), w2.detach().requires_grad_(), b1.detach().requires_grad_()
    loss = (torch.relu(X @ W1 + B1) @ W2).sum()
    loss.backward()
    return loss, (W2, B1, W1)           # the order the gradients become ready in


def run_c5(bench, args):
    """Two-layer MLP forward+backward on 65,536 rows; rows of X sharded over the ranks, W1/W2/b1 replicated, NCCL
    all-reduce of the three gradients inside the step (each one as soon as its kernel has finished)."""
    torch, dev, rank, world, tdist = bench.torch, bench.dev, bench.rank, bench.world, bench.tdist
    total_rows = 65536
    lo, hi = tdist.shard_bounds(total_rows, rank, bench.shards)
    rows = hi - lo
    x = np.random.default_rng(1000 + rank).standard_normal((rows, 4096), dtype=np.float32)
    shared = np.random.default_rng(0)
    w1_host = (shared.standard_normal((4096, 4096)) / 64).astype(np.float32)
    w2_host = (shared.standard_normal((4096, 1024)) / 64).astype(np.float32)
    X = torch.tensor(x, device=dev)
    w1, w2, b1 = torch.tensor(w1_host, device=dev), torch.tensor(w2_host, device=dev), torch.zeros(4096, device=dev)
    held = [None]

    def step():
        loss, params = mlp_step(torch, X, w1, w2, b1)
        tdist.all_reduce_gradients(params)
        held[0] = (loss, params)
    step()
    ms, steps, launches, clocks = bench.time_side(step, min_steps=4)
    value = C5_FLOPS / (ms * 1e-3) / 1e12
    out = {"workload": "2-layer MLP forward+backward, loss=(relu(X@W1+b1)@W2).sum(): X f32 [65536,4096], W1 [4096,4096], W2 [4096,1024], "
                       "b1 [4096]; rows of X sharded over the ranks, NCCL all-reduce of the W1/W2/b1 gradients inside the step",
           "metric": "MLP fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "scaling": "strong", "ms_per_step": ms, "steps": steps,
           "gpu_launches": launches, "launches_per_step": launches / steps, "rows_per_gpu": rows, "clocks": clocks,
           "algo": matmul_algo_name(torch, X, w1, (rows, 4096)),
           "roofline": bench.tensor_roofline(value / world, "gemm_tf32x3_pair_kernel (5 products per step)"),
           "collective": None if world == 1 else "all-reduce (sum) of dW2 16 MiB, db1 16 KiB, dW1 64 MiB through trs_comm_allreduce_sum_f32 "
                                                 "on a side stream; dW2's runs under the dH and dW1 products",
           "operands": "X, W1, W2 stay resident across steps (lo images kept beside the storages); H and dZ get theirs from the "
                       "epilogues that store them"}
    # ---- parity on a reduced-size step (2,048 rows in all, sharded like the timed step) -----------------
    # Sampled hidden units are followed through the step in float64.  relu' is discontinuous at 0 and a product of
    # another shape rounds Z differently, so the expected gradients take their relu decisions from the Z the device
    # itself produced (the reference VJP is a function of the saved Z, src/tensor.rs:4422-4432).  Every rank adds up
    # its own rows; the float64 partial sums are summed over the ranks on the host and compared with the
    # all-reduced device gradients, which checks the collective as well.
    small_rows = 2048
    xs_small = np.random.default_rng(7).standard_normal((small_rows, 4096), dtype=np.float32)
    slo, shi = tdist.shard_bounds(small_rows, rank, world)
    xs_mine = xs_small[slo:shi]
    W1, W2, B1 = w1.detach().requires_grad_(), w2.detach().requires_grad_(), b1.detach().requires_grad_()
    Zt = torch.tensor(xs_mine, device=dev) @ W1 + B1            # held: stored by the same kernel that stores relu(Z)
    (torch.relu(Zt) @ W2).sum().backward()
    tdist.all_reduce_gradients((W2, B1, W1))
    z_gpu = Zt.numpy()
    units = np.sort(np.random.default_rng(8).choice(4096, 16, replace=False))
    dh = w2_host.astype(np.float64).sum(axis=1)
    dz = (z_gpu[:, units] > 0) * dh[units]
    z_err = matmul_error_over_bound(z_gpu[:, units], xs_mine.astype(np.float64) @ w1_host[:, units].astype(np.float64), 4096)
    partial = np.concatenate([(xs_mine.astype(np.float64).T @ dz).reshape(-1), dz.sum(axis=0),
                              np.maximum(z_gpu[:, units], 0).sum(axis=0, dtype=np.float64)])
    summed = tdist.all_reduce_host(partial)
    worst_z = float(tdist.all_reduce_host(np.array([z_err]), op="max")[0])
    if rank == 0:
        want_dw1 = summed[: 4096 * 16].reshape(4096, 16)
        want_db1 = summed[4096 * 16: 4096 * 16 + 16]
        want_dw2 = np.repeat(summed[4096 * 16 + 16: 4096 * 16 + 32][:, None], 1024, axis=1)
        out["parity"] = {"rows": small_rows, "hidden_units_followed": 16, "ranks": world,
                         "bound": "1e-5*sqrt(K)*max(|G|, rms G), K = 4096 for Z and the row count for the gradients; <= 1 passes",
                         "Z_error_over_bound_vs_f64": worst_z,
                         "dW1_error_over_bound_vs_f64": matmul_error_over_bound(W1.grad.numpy()[:, units], want_dw1, small_rows),
                         "db1_error_over_bound_vs_f64": matmul_error_over_bound(B1.grad.numpy()[units], want_db1, small_rows),
                         "dW2_error_over_bound_vs_f64": matmul_error_over_bound(W2.grad.numpy()[units], want_dw2, small_rows),
                         "gradients": "all-reduced over the ranks" if world > 1 else "single GPU"}
    del W1, W2, B1, Zt
    # ---- end to end: this rank's rows of X from pinned host memory, gradients and loss back, every step ----
    x_host = torch.pinned_empty(rows, 4096)
    x_host[...] = x
    g_host = [torch.pinned_empty(4096, 1024), torch.pinned_empty(4096), torch.pinned_empty(4096, 4096)]

    # double-buffered input pipeline: the upload of the next batch is issued (on the engine's upload stream) before this
    # step's result is awaited, so it runs under this step's kernels; K timed steps contain K uploads
    upcoming = [torch.tensor(x_host, device=dev)]

    def step_e2e():
        loss, params = mlp_step(torch, upcoming[0], w1, w2, b1)
        tdist.all_reduce_gradients(params)
        for p, dst in zip(params, g_host):
            p.grad.copy_to_host(dst, non_blocking=True)       # ordered behind the gradients only: issued before the next upload
        upcoming[0] = torch.tensor(x_host, device=dev)
        held[0] = loss.item()
        torch.synchronize(bench.local_rank)
    e2e_ms = bench.time_wall(step_e2e, 3, warmup=2)
    out["e2e"] = {"value": C5_FLOPS / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": 3,
                  "h2d_bytes_per_step": 4 * rows * 4096, "d2h_bytes_per_step": 4 * (4096 * 1024 + 4096 + 4096 * 4096) + 4,
                  "how": "this rank's rows of X uploaded from pinned host memory every step (the weights stay on the device, as "
                         "parameters do), forward, backward, gradient all-reduce, the three gradients and the loss read back; the next "
                         "batch's upload is issued before the current step's loss is awaited (double buffering), so it overlaps the kernels"}
    upcoming.clear()
    torch.pinned_free(x_host)
    for array in g_host:
        torch.pinned_free(array)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle.ref import RefTensor
        n = 512
        rx, rw1, rw2 = RefTensor.from_numpy(x[:n]), RefTensor.from_numpy(w1_host), RefTensor.from_numpy(w2_host)
        t0 = time.perf_counter()
        Z = rx.matmul(rw1) + RefTensor(np.zeros(4096, dtype=np.float32), [4096])
        H = Z.relu()
        H.matmul(rw2).sum()
        dY = RefTensor.from_numpy(np.ones((n, 1024), dtype=np.float32))
        H.T.matmul(dY)
        dZ = RefTensor.from_numpy(Z.relu_vjp(dY.matmul(rw2.T).logical()))
        rx.T.matmul(dZ)
        dZ.logical().sum(axis=0)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": C5_FLOPS * (n / total_rows) / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                               "host_cores": os.cpu_count(), "seconds": dt,
                               "sample": f"{n} of 65,536 rows: forward, loss and the backward products composed from the reference's "
                                         "primitives (the transposed operands take its strided loop); cost is linear in the rows, so the "
                                         "rate is extrapolated"}
    return out


SIDE = {"c1": lambda bench, args: run_c1(bench), "t1": lambda bench, args: run_t1(bench), "c3": run_c3, "c4": run_c4, "c5": run_c5,
        "copy": lambda bench, args: run_copy_ceiling(bench), "bwd": lambda bench, args: run_backward_kernels(bench)}


def run_ours(args, rank, world, local_rank):
    bench = Bench(rank, world, local_rank)
    if args.shard_of:
        bench.shards = args.shard_of
    torch = bench.torch
    if args.workload != "c2":
        result = SIDE[args.workload](bench, args)
        bench.barrier()
        if world > 1:
            bench.tdist.destroy_process_group()
        if rank == 0:
            result.update({"n_gpus": world, "config": {"workload": result.pop("workload", args.workload), "parallelism": f"dp{world}"}})
            print(json.dumps(result), flush=True)
        return
    head = run_headline(bench, args)
    extra = {}
    if not args.no_extra:
        extra["copy"] = run_copy_ceiling(bench)
        if rank == 0:
            try:
                extra["backward_kernels"] = run_backward_kernels(bench)
            except Exception as err:                                  # noqa: BLE001 - reported, not swallowed
                extra["backward_kernels"] = {"error": f"{type(err).__name__}: {err}"[:600]}
        for name in ("c1", "t1", "c3", "c4", "c5"):
            # a side workload that fails must not take the headline with it: its entry then carries the error
            try:
                extra[name] = SIDE[name](bench, args)
                torch.synchronize(local_rank)
            except Exception as err:                                  # noqa: BLE001 - reported, not swallowed
                import traceback
                traceback.print_exc()
                extra[name] = {"error": f"{type(err).__name__}: {err}"[:600]}
    bench.barrier()
    if world > 1:
        bench.tdist.destroy_process_group()
    if rank != 0:
        return
    e2e = head["e2e"]
    if "copy" in extra:
        # what the host link allows for this step: its upload and its read-back run at the same time
        each = extra["copy"]["each_direction_when_both_gbs"]
        floor_ms = max(e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]) / (each * 1e9) * 1e3
        e2e["ceiling_gbs"] = world * ALGO_BYTES / (floor_ms * 1e-3) / 1e9
        e2e["frac"] = e2e["value"] / e2e["ceiling_gbs"]
        e2e["ceiling_how"] = ("algorithmic bytes / (larger of the step's upload and read-back bytes / the measured per-direction copy rate "
                              "with both directions busy, extra.copy)")
    line = {
        "metric": "fused pointwise GB/s", "value": head["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": headline_config(world),
        "roofline": head["roofline"], "e2e": e2e, "gpu_launches": head["launches"], "clocks": head["clocks"],
        "timing": head["timing"], "parity": head["parity"], "extra": extra,
    }
    if head["cpu_baseline"] is not None:
        line["cpu_baseline"] = head["cpu_baseline"]
    print(json.dumps(line), flush=True)


def main():
    global MIN_REGION_SECONDS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--regions", type=int, default=9, help="timed regions of `steps` steps each for the headline; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-slabs", type=int, default=8, help="row slabs per end-to-end step (must divide 8192)")
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "t1", "c3", "c4", "c5", "copy", "bwd"],
                    help="c2 (default) is the headline fused chain with every other configuration under `extra`; "
                         "any other value runs that workload alone")
    ap.add_argument("--min-seconds", type=float, default=MIN_REGION_SECONDS,
                    help="shortest timed region of a side workload (a profiler run wants it short)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="profiling aid for one GPU: size configs 3/4/5 as rank 0's shard of a job of this many ranks "
                         "(the aggregate figures of such a run mean nothing; the per-step time is one rank's)")
    ap.add_argument("--no-extra", action="store_true", help="headline only: skip the copy ceiling and configs 1, 3, 4, 5")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    MIN_REGION_SECONDS = args.min_seconds
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
