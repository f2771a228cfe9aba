#!/usr/bin/env python
"""Benchmark of the fused pointwise hot path (and, as extra figures, f32 matmul) on B200.

    python bench.py --gpus N --steps K --warmup W            # this build (one rank per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores

Workload (N=1): `exp(2.0 * relu(x.mT + b)) - x.mT`, x f32 [8192,8192] ~N(0,1) read through a
transposed view, b f32 [8192] ~N(0,0.1) broadcast, scalar 2.0 — a five-op chain run as ONE kernel.
A step builds the chain through the public `torch_rs` surface and forces its execution.
With N ranks every rank runs the same-sized shard of an N-times larger batch (weak scaling, no
data-path collective).  Prints ONE JSON line (rank 0).

Algorithmic bytes per step and GPU: 8 B per element (x read once, result written once) + b
= 8*8192*8192 + 4*8192 = 536,903,680 B.
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
sys.path.insert(0, os.path.join(ROOT, "pytorch-rs_b200"))
sys.path.insert(0, ROOT)

N_SIDE = 8192
ALGO_BYTES = 8 * N_SIDE * N_SIDE + 4 * N_SIDE
FALLBACK_HBM_GBS = 6650.0
WORKLOAD_TEXT = ("exp(2.0*relu(x.mT+b))-x.mT, x f32 [8192,8192] via transposed view, b [8192] broadcast, scalar 2.0; "
                 "one pass of the whole chain per step, per GPU")
# dram__bytes_read.sum + dram__bytes_write.sum of one trs_pw launch on this workload, from an ncu
# capture of exactly this kernel and size (its summary is kept under profiles/); writes that are
# still dirty in L2 when the kernel ends are not counted.
NCU_DRAM_BYTES_PER_LAUNCH = 484834304


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        peaks = json.load(open(path))
        return float(peaks["hbm_gbs"]), "measured", peaks
    except Exception:
        return FALLBACK_HBM_GBS, "fallback", {}


def make_inputs(seed, rows=N_SIDE):
    """Seeded synthetic inputs with the workload's shapes and distributions (NumPy default_rng)."""
    rng = np.random.default_rng(seed)
    xs = rng.standard_normal((rows, N_SIDE)).astype(np.float32)      # storage of x; the operand is xs.mT
    b = (0.1 * rng.standard_normal(rows)).astype(np.float32)
    return xs, b


class ClockSampler:
    """Samples SM clocks and clock-event reasons through NVML on a thread while the timed region (and
    an untimed post-roll of the same steps, so that a millisecond-long region still gets samples) runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.reasons = set()
        self.max_clock = None
        self.stop = threading.Event()
        self.thread = None
        self.nvml = None

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
                self.samples.append(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

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
        out = {"sm_mhz": None, "sm_max_mhz": self.max_clock, "reasons": sorted(self.reasons), "samples": len(self.samples),
               "how": "NVML on a thread every ~2 ms over the timed region plus an untimed post-roll of the same steps"}
        if self.samples:
            ordered = sorted(self.samples)
            out["sm_mhz"] = statistics.median(ordered[len(ordered) // 2:])      # upper half = under load
        return out


def cpu_chain(xs, b):
    """The same chain through the CPU checker, op by op as the reference engine runs it."""
    from oracle.ref import RefTensor
    x, bt = RefTensor.from_numpy(xs), RefTensor.from_numpy(b)
    return (2.0 * (x.mT + bt).relu()).exp() - x.mT


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU algorithm for this chain (C++ restatement in oracle/, since
    no Rust toolchain exists to build the original) on the host cores; single-threaded, as the
    reference engine is."""
    if rank != 0:
        return
    from oracle import ref
    ref.build()
    total_steps = args.steps + args.warmup
    rows = N_SIDE if total_steps * 5.0 <= 150 else 2048
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
        "config": {"workload": WORKLOAD_TEXT, "l2": "inputs+outputs 512 MiB per step, larger than the 126 MB L2",
                   "parallelism": f"dp{args.gpus}", "algorithmic_bytes_per_step_per_gpu": ALGO_BYTES, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_region(stream, fn, steps):
    from torch_rs._device import Event
    e0, e1 = Event(), Event()
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    e1.sync()
    return e0.elapsed_ms(e1)


def run_ours(args, rank, world, local_rank):
    import torch_rs as torch
    from torch_rs import _abi, _host
    from torch_rs._device import Stream, launch_count
    import ctypes

    dist = None
    if world > 1:
        import torch as pt                      # plumbing only: rendezvous, barrier, max over ranks
        import torch.distributed as dist
        pt.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=pt.device("cuda", local_rank))

    def barrier():
        torch.synchronize(local_rank)
        if dist is not None:
            dist.barrier()

    def max_over_ranks(value):
        if dist is None:
            return value
        import torch as pt
        t = pt.tensor([value], dtype=pt.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev = f"cuda:{local_rank}"
    from torch_rs import distributed as tdist
    numa_node = tdist.bind_to_device_numa_node(local_rank)     # staging memory local to this GPU's PCIe root
    raw = ctypes.c_void_p()
    _host.check(_host.lib().trsh_stream(local_rank, ctypes.byref(raw)))
    stream = Stream.__new__(Stream)
    stream.device, stream.handle = local_rank, raw           # the engine's own stream: events go where the kernels go

    xs, b = make_inputs(rank)
    x, bt = torch.tensor(xs, device=dev), torch.tensor(b, device=dev)
    held = [None]

    def step():
        held[0] = (torch.exp(2.0 * torch.relu(x.mT + bt)) - x.mT).materialize()

    # ---- device-resident throughput ---------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    launches0 = launch_count()
    with ClockSampler(local_rank) as clocks:
        ms = time_region(stream, step, args.steps)
        launches = launch_count() - launches0
        barrier()
        post_roll_until = time.perf_counter() + 0.4       # same steps, untimed, so the sampler sees load
        while time.perf_counter() < post_roll_until:
            for _ in range(20):
                step()
            torch.synchronize(local_rank)
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    value = world * ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
    clock_info = clocks.summary()

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

    E2E_SLABS = args.e2e_slabs                     # physical-row slabs: upload of slab i+1 overlaps read-back of slab i

    def step_e2e():
        rows = N_SIDE // E2E_SLABS
        for i in range(E2E_SLABS):
            sl = slice(i * rows, (i + 1) * rows)
            xd, bd = torch.tensor(x_host[sl], device=dev), torch.tensor(b_host[sl], device=dev)
            out = torch.exp(2.0 * torch.relu(xd.mT + bd)) - xd.mT
            out.mT.copy_to_host(out_host[sl], non_blocking=True)     # the result's storage order
        torch.synchronize(local_rank)              # every slab's result is in host memory

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    torch.synchronize(local_rank)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    e2e_value = world * ALGO_BYTES / (e2e_ms * 1e-3) / 1e9
    if rank == 0:
        assert np.array_equal(out_host[:8].view(np.uint32), held[0].mT.numpy()[:8].view(np.uint32))

    # ---- extra figures: contiguous relu(x+y) and f32 matmul 4096^3 (per GPU, rank 0) --------------
    extra = {}
    if rank == 0 and not args.no_extra:
        n1 = 4096
        rng = np.random.default_rng(0)
        sets = [(torch.tensor(rng.uniform(-1, 1, (n1, n1)).astype(np.float32), device=dev),
                 torch.tensor(rng.uniform(-1, 1, (n1, n1)).astype(np.float32), device=dev)) for _ in range(4)]
        it = [0]

        def c1():
            xa, ya = sets[it[0] % 4]
            it[0] += 1
            held[0] = torch.relu(xa + ya).materialize()
        for _ in range(5):
            c1()
        torch.synchronize(local_rank)
        c1_ms = time_region(stream, c1, 40) / 40
        extra["relu_add_4096"] = {"GB/s": 12 * n1 * n1 / (c1_ms * 1e-3) / 1e9, "ms": c1_ms,
                                  "note": "4 rotating operand sets (768 MiB) defeat L2"}
        a = torch.tensor((rng.standard_normal((n1, n1)) / 64).astype(np.float32), device=dev)
        bm = torch.tensor((rng.standard_normal((n1, n1)) / 64).astype(np.float32), device=dev)
        del sets

        def c3():
            held[0] = torch.matmul(a, bm).materialize()
        for _ in range(3):
            c3()
        torch.synchronize(local_rank)
        c3_ms = time_region(stream, c3, 10) / 10
        desc = _abi.GemmDesc()
        desc.batch, desc.m, desc.n, desc.k = 1, n1, n1, n1
        desc.a, desc.b, desc.c = a.data_ptr(), bm.data_ptr(), held[0].data_ptr()
        desc.a_row_stride, desc.a_col_stride, desc.b_row_stride, desc.b_col_stride, desc.c_row_stride = n1, 1, n1, 1, n1
        algo = ctypes.c_int32()
        _abi.lib().trs_matmul_select_algo(ctypes.byref(desc), ctypes.byref(algo))
        extra["matmul_4096"] = {"TFLOP/s": 2 * n1 ** 3 / (c3_ms * 1e-3) / 1e12, "ms": c3_ms,
                                "algo": {1: "simt_fp32", 2: "tcgen05_3xtf32"}.get(algo.value, str(algo.value))}

    # ---- CPU baseline (rank 0, N=1): the whole workload through the checker, single thread ---------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            cpu_chain(xs, b)
            times.append(time.perf_counter() - t0)
        cpu_baseline = {"value": ALGO_BYTES / statistics.median(times) / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                        "sample": "the full workload, median of 3 runs", "host_cores": os.cpu_count()}

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak, peak_kind, _ = measured_peaks()
    achieved = ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
    traffic = NCU_DRAM_BYTES_PER_LAUNCH
    line = {
        "metric": "fused pointwise GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT,
                   "l2": "inputs+outputs 512 MiB per step, larger than the 126 MB L2", "parallelism": f"dp{world}",
                   "algorithmic_bytes_per_step_per_gpu": ALGO_BYTES},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": f"of {peak_kind}", "kernel": "trs_pw (vector class)"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ALGO_BYTES // 2 + 2 * N_SIDE,
                "d2h_bytes_per_step": 4 * N_SIDE * N_SIDE, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "how": f"pinned host buffers; {E2E_SLABS} row slabs per step so uploads, kernels and read-backs overlap",
                "numa_node": numa_node},
        "gpu_launches": launches, "clocks": clock_info, "parity": parity, "extra": extra,
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line), flush=True)


WORKLOADS = {
    "c1": "relu(x + y), x,y f32 [4096,4096] contiguous ~U(-1,1); 4 rotating operand sets defeat L2",
    "t1": "x.mT + y, x,y f32 [8192,8192] ~N(0,1): operand layouts disagree, staged through shared-memory tiles",
    "c3": "matmul(A, B), f32 [4096,4096]^2 ~N(0,1/64), precision highest",
    "c4": "relu(X @ W.mT + bias), X,W f32 [64,1024,1024], bias [1024]; batches sharded over ranks",
    "c5": "2-layer MLP forward+backward, X f32 [65536,4096], W1 [4096,4096], W2 [4096,1024], b1 [4096]; "
          "rows of X sharded over ranks, NCCL all-reduce of the W1/W2/b1 gradients",
}


def run_side_workload(args, rank, world, local_rank):
    """The other BASELINE configs (not the headline line): same timing rules, one JSON line on rank 0."""
    import ctypes
    import torch_rs as torch
    from torch_rs import _host, distributed as tdist
    from torch_rs._device import Stream, launch_count
    if world > 1:
        tdist.init_process_group("nccl")
    dev = f"cuda:{local_rank}"
    raw = ctypes.c_void_p()
    _host.check(_host.lib().trsh_stream(local_rank, ctypes.byref(raw)))
    stream = Stream.__new__(Stream)
    stream.device, stream.handle = local_rank, raw
    rng = np.random.default_rng(rank)
    held = [None]
    name = args.workload
    hbm_peak, peak_kind, peaks = measured_peaks()
    tensor_peak = float(peaks.get("bf16_tflops", 1590.0)) / 6.0     # tf32 runs at half the bf16 rate; 3 MMAs per product
    if name == "c1":
        n = 4096
        sets = [(torch.tensor(rng.uniform(-1, 1, (n, n)).astype(np.float32), device=dev),
                 torch.tensor(rng.uniform(-1, 1, (n, n)).astype(np.float32), device=dev)) for _ in range(4)]
        it = [0]

        def step():
            xa, ya = sets[it[0] % 4]
            it[0] += 1
            held[0] = torch.relu(xa + ya).materialize()
        work, unit, metric, bound, peak = 12 * n * n * world, "GB/s", "fused pointwise GB/s", "hbm", hbm_peak
        scale, scaling = 1e9, "weak"
    elif name == "t1":
        n = 8192
        xt = torch.tensor(rng.standard_normal((n, n)).astype(np.float32), device=dev)
        yt = torch.tensor(rng.standard_normal((n, n)).astype(np.float32), device=dev)

        def step():
            held[0] = (xt.mT + yt).materialize()
        work, unit, metric, bound, peak = 12 * n * n * world, "GB/s", "fused pointwise GB/s", "hbm", hbm_peak
        scale, scaling = 1e9, "weak"
    elif name == "c3":
        n = 4096
        a = torch.tensor((rng.standard_normal((n, n)) / 64).astype(np.float32), device=dev)
        b = torch.tensor((rng.standard_normal((n, n)) / 64).astype(np.float32), device=dev)

        def step():
            held[0] = torch.matmul(a, b).materialize()
        work, unit, metric, bound, peak = 2 * n ** 3 * world, "TFLOP/s", "f32 matmul TFLOP/s", "tensor", tensor_peak
        scale, scaling = 1e12, "weak"
    elif name == "c4":
        lo, hi = tdist.shard_bounds(64, rank, world)
        nb = hi - lo
        X = torch.tensor(rng.standard_normal((nb, 1024, 1024)).astype(np.float32), device=dev)
        W = torch.tensor((rng.standard_normal((nb, 1024, 1024)) / 32).astype(np.float32), device=dev)
        bias = torch.tensor(rng.uniform(-0.1, 0.1, 1024).astype(np.float32), device=dev)

        def step():
            held[0] = torch.relu(X @ W.mT + bias).materialize()
        work, unit, metric, bound, peak = 64 * 2 * 1024 ** 3, "TFLOP/s", "f32 bmm+bias+relu TFLOP/s", "tensor", tensor_peak
        scale, scaling = 1e12, "strong"
    else:
        lo, hi = tdist.shard_bounds(65536, rank, world)
        X = torch.tensor(rng.standard_normal((hi - lo, 4096)).astype(np.float32), device=dev)
        shared = np.random.default_rng(0)
        w1 = torch.tensor((shared.standard_normal((4096, 4096)) / 64).astype(np.float32), device=dev)
        w2 = torch.tensor((shared.standard_normal((4096, 1024)) / 64).astype(np.float32), device=dev)
        b1 = torch.zeros(4096, device=dev)

        def step():
            W1, W2, B1 = w1.detach().requires_grad_(), w2.detach().requires_grad_(), b1.detach().requires_grad_()
            loss = (torch.relu(X @ W1 + B1) @ W2).sum()
            loss.backward()
            tdist.all_reduce_gradients((W1, W2, B1))
            held[0] = (loss, W1.grad, W2.grad, B1.grad)
        work, unit, metric, bound, peak = 2 * 65536 * (2 * 4096 ** 2 + 3 * 4096 * 1024), "TFLOP/s", "MLP fwd+bwd TFLOP/s", "tensor", tensor_peak
        scale, scaling = 1e12, "strong"

    for _ in range(max(args.warmup, 3)):
        step()
    torch.synchronize(local_rank)
    tdist.barrier()
    launches0 = launch_count()
    with ClockSampler(local_rank) as clocks:
        ms = time_region(stream, step, args.steps)
        launches = launch_count() - launches0
        torch.synchronize(local_rank)
    ms = float(tdist.all_reduce_host(np.array([ms]), op="max")[0])
    tdist.barrier()
    if world > 1:
        tdist.destroy_process_group()
    if rank != 0:
        return
    ms_per_step = ms / args.steps
    value = work / (ms_per_step * 1e-3) / scale
    per_gpu = value / world
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": WORKLOADS[name], "parallelism": f"dp{world}"},
            "roofline": {"bound": bound, "achieved": per_gpu, "peak": peak, "unit": unit, "frac": per_gpu / peak, "traffic": None,
                         "peak_source": f"of {peak_kind}" + (" (bf16_tflops / 6: tf32 at half rate, 3 MMAs per product)" if bound == "tensor" else "")},
            "gpu_launches": launches, "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-slabs", type=int, default=8, help="row slabs per end-to-end step (must divide 8192)")
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "t1", "c3", "c4", "c5"],
                    help="c2 (default) is the headline fused chain; the others are BASELINE's remaining configs")
    ap.add_argument("--no-extra", action="store_true", help="skip the relu(x+y) and matmul side figures")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    if args.workload != "c2":
        run_side_workload(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
