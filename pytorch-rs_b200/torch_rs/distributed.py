"""Data-parallel plumbing: one process per GPU, `torch.distributed` for rendezvous and collectives.

The reference has no distributed backend at all (every `torch.distributed.is_*_available()` is False,
python/torch_rs/distributed/distributed_c10d.py:39-74); its only multi-process convention is the
`LOCAL_RANK` environment variable (same file, 71-72), which is kept here.  The hot path shards by
rows / batches with no exchange step; the single collective is the sum of the MLP weight gradients,
issued as NCCL all-reduces (over NVLink / NVSwitch) that are stream-ordered after the kernels that
produce the gradients.  PyTorch is used for the process group only; it never computes a result.
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
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.  `nccl` when this
    rank has a CUDA device, else `gloo` (used by the CPU tests of the host-side logic)."""
    import torch as pt
    import torch.distributed as dist
    if _state["initialized"]:
        return _state["backend"]
    if backend is None:
        backend = "nccl" if _device.device_count() > 0 else "gloo"
    kwargs = {}
    if backend == "nccl":
        local = get_node_local_rank(0)
        pt.cuda.set_device(local)
        kwargs["device_id"] = pt.device("cuda", local)
    dist.init_process_group(backend, **kwargs)
    _state.update(initialized=True, backend=backend)
    return backend


def destroy_process_group() -> None:
    import torch.distributed as dist
    if _state["initialized"]:
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
        if node < 0:
            return None
        cpus = _parse_cpu_list(open(f"/sys/devices/system/node/node{node}/cpulist").read())
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


class _DeviceSpan:
    """Exposes `count` float32 at a raw device address through __cuda_array_interface__ (zero copy)."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def all_reduce_(tensor) -> None:
    """In-place sum of a contiguous CUDA tensor over all ranks.  Enqueued behind the engine's stream
    (the collective waits for the kernels that wrote `tensor`; later engine work waits for it)."""
    import torch as pt
    import torch.distributed as dist
    if not _state["initialized"] or get_world_size() == 1:
        return
    if not tensor.is_contiguous():
        raise RuntimeError("all_reduce_ needs a contiguous tensor")
    index = tensor.device.index
    ptr = tensor.data_ptr()          # forces the value onto the device
    view = pt.as_tensor(_DeviceSpan(ptr, tensor.numel()), device=f"cuda:{index}")
    stream = _state["streams"].get(index)
    if stream is None:
        raw = _engine_cuda_stream(index)
        stream = _state["streams"][index] = pt.cuda.ExternalStream(raw, device=f"cuda:{index}")
    with pt.cuda.stream(stream):
        dist.all_reduce(view, op=dist.ReduceOp.SUM)


def _engine_cuda_stream(index: int) -> int:
    import ctypes
    from . import _abi, _host
    handle = ctypes.c_void_p()
    _host.check(_host.lib().trsh_stream(index, ctypes.byref(handle)))
    raw = ctypes.c_void_p()
    _abi.check(_abi.lib().trs_stream_handle(handle, ctypes.byref(raw)))
    return raw.value or 0


def all_reduce_host(array: np.ndarray, op: str = "sum") -> np.ndarray:
    """Sum (or max) of a host array over all ranks; works on either backend."""
    import torch as pt
    import torch.distributed as dist
    if not _state["initialized"] or get_world_size() == 1:
        return array
    t = pt.from_numpy(np.ascontiguousarray(array))
    if _state["backend"] == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
    return t.cpu().numpy()


def all_reduce_gradients(parameters) -> None:
    """Sum `.grad` of every parameter over the ranks (data-parallel MLP step)."""
    for p in parameters:
        g = p.grad
        if g is not None:
            all_reduce_(g)
