"""Device buffers, streams and events on top of the C ABI (no torch involved).

A ``DeviceBuffer`` is what the reference's ``Storage`` becomes on a CUDA device
(src/storage.rs:7-18): an immutable-after-fill block of float32 in HBM, freed when dropped.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _abi

_streams = {}


def device_count() -> int:
    n = ctypes.c_int32(0)
    status = _abi.lib().trs_device_count(ctypes.byref(n))
    if status != 0:
        return 0
    return n.value


def require_device(device: int = 0) -> None:
    """Fail loudly when the CUDA path cannot run (there is no CPU fallback for CUDA tensors)."""
    n = device_count()
    if device >= n:
        raise _abi.TrsError(6, f"CUDA device {device} requested but {n} available")


class Stream:
    def __init__(self, device: int = 0):
        self.device = device
        handle = ctypes.c_void_p()
        _abi.check(_abi.lib().trs_stream_create(device, ctypes.byref(handle)))
        self.handle = handle

    def sync(self):
        _abi.check(_abi.lib().trs_stream_sync(self.handle))

    def cuda_stream(self) -> int:
        raw = ctypes.c_void_p()
        _abi.check(_abi.lib().trs_stream_handle(self.handle, ctypes.byref(raw)))
        return raw.value or 0


def default_stream(device: int = 0) -> Stream:
    """One library stream per device; every op of the Python host is enqueued on it."""
    s = _streams.get(device)
    if s is None:
        require_device(device)
        s = _streams[device] = Stream(device)
    return s


class Event:
    def __init__(self):
        handle = ctypes.c_void_p()
        _abi.check(_abi.lib().trs_event_create(ctypes.byref(handle)))
        self.handle = handle

    def record(self, stream: Stream):
        _abi.check(_abi.lib().trs_event_record(self.handle, stream.handle))

    def sync(self):
        _abi.check(_abi.lib().trs_event_sync(self.handle))

    def elapsed_ms(self, later: "Event") -> float:
        ms = ctypes.c_float()
        _abi.check(_abi.lib().trs_event_elapsed_ms(self.handle, later.handle, ctypes.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            _abi.lib().trs_event_destroy(self.handle)
        except Exception:
            pass


class DeviceBuffer:
    """``count`` float32 elements of device memory from the library's cached allocator."""

    __slots__ = ("ptr", "count", "device", "__weakref__")

    def __init__(self, count: int, device: int = 0):
        self.count = int(count)
        self.device = device
        ptr = ctypes.c_void_p()
        _abi.check(_abi.lib().trs_malloc(device, max(self.count, 1) * 4, ctypes.byref(ptr)))
        self.ptr = ptr.value

    def __del__(self):
        ptr, self.ptr = getattr(self, "ptr", None), None
        if ptr:
            try:
                _abi.lib().trs_free(self.device, ptr)
            except Exception:
                pass

    @classmethod
    def from_numpy(cls, array, device: int = 0, stream: Stream | None = None) -> "DeviceBuffer":
        array = np.ascontiguousarray(array, dtype=np.float32).reshape(-1)
        buf = cls(array.size, device)
        stream = stream or default_stream(device)
        if array.size:
            _abi.check(_abi.lib().trs_memcpy_h2d(buf.ptr, array.ctypes.data, array.size * 4, stream.handle))
            stream.sync()          # the pageable source may be released by the caller
        return buf

    def to_numpy(self, stream: Stream | None = None) -> np.ndarray:
        out = np.empty(self.count, dtype=np.float32)
        stream = stream or default_stream(self.device)
        if self.count:
            _abi.check(_abi.lib().trs_memcpy_d2h(out.ctypes.data, self.ptr, self.count * 4, stream.handle))
        stream.sync()
        return out


_pinned_ranges = {}     # start address -> (end address, owner) of live page-locked buffers


def is_pinned(array) -> bool:
    """Whether a NumPy array's bytes lie entirely inside a live PinnedBuffer."""
    start = array.ctypes.data
    end = start + array.nbytes
    return any(lo <= start and end <= hi for lo, (hi, _) in _pinned_ranges.items())


class PinnedBuffer:
    """Page-locked host staging memory exposed as a NumPy array (for timed host<->device copies)."""

    def __init__(self, count: int):
        self.count = int(count)
        ptr = ctypes.c_void_p()
        _abi.check(_abi.lib().trs_malloc_host(max(self.count, 1) * 4, ctypes.byref(ptr)))
        self.ptr = ptr.value
        self.array = np.ctypeslib.as_array(ctypes.cast(self.ptr, ctypes.POINTER(ctypes.c_float)), shape=(self.count,))
        _pinned_ranges[self.ptr] = (self.ptr + max(self.count, 1) * 4, None)

    def __del__(self):
        ptr, self.ptr = getattr(self, "ptr", None), None
        if ptr:
            _pinned_ranges.pop(ptr, None)
            try:
                _abi.lib().trs_free_host(ptr)
            except Exception:
                pass


def launch_count() -> int:
    return int(_abi.lib().trs_kernel_launch_count())
