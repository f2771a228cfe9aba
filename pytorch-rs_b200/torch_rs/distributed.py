"""Data-parallel plumbing: one process per GPU, `torch.distributed` for rendezvous and collectives.

The reference has no distributed backend at all (every `torch.distributed.is_*_available()` is False,
python/torch_rs/distributed/distributed_c10d.py:39-74); its only multi-process convention is the
`LOCAL_RANK` environment variable (same file, 71-72), which is kept here.  The hot path shards by
rows / batches with no exchange step; the single collective is the sum of the MLP weight gradients:
NCCL all-reduces (over NVLink / NVSwitch) issued by the engine itself through the C ABI
(`trs_comm_*`) on a side stream, each one behind the kernel that produced that gradient, so the
exchange overlaps the rest of the backward pass.  `torch.distributed` (gloo) is the control plane
only: rendezvous, barriers, handing the communicator id to the ranks, small host-side reductions.
"""
from __future__ import annotations

import os

import numpy as np

from . import _device

_state = {"initialized": False, "backend": None, "streams": {}}


def get_node_local_rank(fallback_rank=None) -> int:
    if "LOCAL_RANK" in os.environ:
        return int(os.environ["LOCAL_RANK"])
    if fallback_rank is not None:
        return int(fallback_rank)
    raise RuntimeError("LOCAL_RANK is not set and no fallback rank was given")


def is_initialized() -> bool:
    return _state["initialized"]


def get_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def get_world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def init_process_group(backend: str | None = None) -> str:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.  `nccl` (the default
    when this rank has a CUDA device) adds the engine's NCCL communicator on device LOCAL_RANK for the
    data path; `gloo` is the control plane alone (used by the CPU tests of the host-side logic)."""
    import torch.distributed as dist
    if _state["initialized"]:
        return _state["backend"]
    if backend is None:
        backend = "nccl" if _device.device_count() > 0 else "gloo"
    if backend not in ("nccl", "gloo"):
        raise ValueError(f"unknown backend {backend!r}")
    if not dist.is_initialized():
        import datetime
        # control-plane operations are small; a rank that died is noticed within this time instead of the default half hour
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=float(os.environ.get("TRS_CONTROL_TIMEOUT_S", "600"))))
    _state.update(initialized=True, backend=backend)
    if backend == "nccl":
        from . import _abi
        _abi.check(_abi.lib().trs_set_current_device(get_node_local_rank(0)))    # this process works on its own GPU only
    if backend == "nccl" and get_world_size() > 1:
        import ctypes
        from . import _host
        ident = ctypes.create_string_buffer(128)
        if get_rank() == 0:
            _host.check(_host.lib().trsh_comm_unique_id(ident))
        box = [ident.raw]
        dist.broadcast_object_list(box, src=0)
        _host.check(_host.lib().trsh_comm_init(get_node_local_rank(0), get_world_size(), get_rank(), box[0]))
    return backend


def destroy_process_group() -> None:
    import torch.distributed as dist
    if _state["initialized"]:
        if _state["backend"] == "nccl":
            from . import _host
            _host.check(_host.lib().trsh_comm_destroy())
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
        _state.update(initialized=False, backend=None)


def barrier() -> None:
    import torch.distributed as dist
    if _state["initialized"]:
        dist.barrier()


def _parse_cpu_list(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_device_numa_node(device_index: int) -> int | None:
    """Pin this process to the CPUs of the NUMA node its GPU hangs off, so that page-locked staging
    buffers allocated afterwards are local to that GPU's PCIe root (host<->device copies of several
    ranks then stop contending for one socket's memory).  Returns the node, or None when unknown."""
    import ctypes
    from . import _abi
    buf = ctypes.create_string_buffer(32)
    if _abi.lib().trs_device_pci_bus_id(device_index, buf, 32) != 0:
        return None
    bus = buf.value.decode().lower()
    try:
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node >= 0:
            cpus = _parse_cpu_list(open(f"/sys/devices/system/node/node{node}/cpulist").read())
        else:
            # no NUMA information for the device (a virtualised host): the CPUs local to its PCIe root, if listed
            cpus = _parse_cpu_list(open(f"/sys/bus/pci/devices/{bus}/local_cpulist").read())
            if len(cpus) >= len(os.sched_getaffinity(0)):
                return None                      # "local" is every CPU: nothing to bind to
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError):
        return None


def shard_bounds(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous [begin, end) slab of `total` rows/batches for `rank`: the first `total % world`
    ranks get one extra, so slabs differ by at most one and cover everything exactly once."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def all_reduce_(tensor) -> None:
    """In-place sum of a contiguous CUDA tensor over all ranks, on the engine's exchange stream: it
    waits for the kernels that wrote `tensor`, and later engine work waits for it."""
    from . import _host
    if not _state["initialized"] or get_world_size() == 1:
        return
    if not tensor.is_contiguous():
        raise RuntimeError("all_reduce_ needs a contiguous tensor")
    _host.check(_host.lib().trsh_all_reduce(tensor._h))


def all_reduce_host(array: np.ndarray, op: str = "sum") -> np.ndarray:
    """Sum (or max) of a host array over all ranks; works on either backend."""
    import torch as pt
    import torch.distributed as dist
    if not _state["initialized"] or get_world_size() == 1:
        return array
    t = pt.from_numpy(np.ascontiguousarray(array).copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
    return t.numpy()


def all_reduce_gradients(parameters) -> None:
    """Sum `.grad` of every parameter over the ranks (data-parallel MLP step).  Each gradient's
    all-reduce starts on the exchange stream as soon as the kernel that produced it has finished, in
    the order given; the engine's compute stream resumes after the last one."""
    import ctypes
    from . import _host
    if not _state["initialized"] or get_world_size() == 1:
        return
    params = [p for p in parameters]
    handles = (ctypes.c_void_p * len(params))(*[p._h for p in params])
    _host.check(_host.lib().trsh_all_reduce_grads(handles, len(params)))
