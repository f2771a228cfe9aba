"""B200-native execution path behind the pytorch-rs (`torch_rs`) operator surface.

`import torch_rs as torch` gives the subset of the reference namespace that the data-parallel hot
path touches (python/torch_rs/__init__.py:9-21, src/python_variable_functions.rs:32-63):
`tensor/zeros/ones/full(device="cuda")`, `add/sub/mul/multiply/relu/exp/matmul/permute/select/
transpose/sum`, `nn.functional.relu`, `autograd.backward`, `no_grad`, and
`get_float32_matmul_precision`.  Layers: `_abi` (kernel C ABI, libtrs_cuda.so), `_host` (C++ host
engine, libtrs_host.so), `tensor` (this surface).
"""
from __future__ import annotations

import contextlib
import ctypes

import numpy as np

from . import _abi, _device, _host  # noqa: F401
from .tensor import (Tensor, device, _device_index, _wrap, memory_format, preserve_format, contiguous_format,  # noqa: F401
                     channels_last, channels_last_3d)

float32 = "torch.float32"


def tensor(data, *, dtype=None, device=None, requires_grad=False) -> Tensor:
    """`torch.tensor(data, device="cuda[:N]")`: one bulk host-to-device copy of any array-like
    (the reference ingests buffers at src/python.rs:10329-10403)."""
    index = _device_index(device)
    array = np.asarray(data, dtype=np.float32, order="C")      # keeps rank 0 (ascontiguousarray would not)
    shape = (ctypes.c_int64 * max(array.ndim, 1))(*array.shape)
    out = ctypes.c_void_p()
    # Arrays that live in page-locked staging memory (torch_rs.pinned_empty) are copied without waiting.
    copy = _host.lib().trsh_from_pinned_host if _device.is_pinned(array) else _host.lib().trsh_from_host
    _host.check(copy(array.ctypes.data, array.ndim, shape, index, ctypes.byref(out)))
    t = _wrap(out)
    return t.requires_grad_(True) if requires_grad else t


def pinned_empty(*size) -> np.ndarray:
    """A float32 NumPy array in page-locked host memory, for overlapping host<->device copies."""
    size = _sizes(size)
    buf = _device.PinnedBuffer(int(np.prod(size)) if size else 1)
    _pinned_keep[buf.ptr] = buf          # stays page-locked until pinned_free(array)
    return buf.array.reshape(size)


def pinned_free(array) -> None:
    """Release a staging array from pinned_empty (no copy may still be in flight)."""
    _pinned_keep.pop(array.ctypes.data, None)


_pinned_keep = {}


def full(size, fill_value, *, dtype=None, device=None, requires_grad=False) -> Tensor:
    index = _device_index(device)
    size = tuple(size)
    shape = (ctypes.c_int64 * max(len(size), 1))(*size)
    out = ctypes.c_void_p()
    _host.check(_host.lib().trsh_full(len(size), shape, ctypes.c_float(fill_value), index, ctypes.byref(out)))
    t = _wrap(out)
    return t.requires_grad_(True) if requires_grad else t


def _sizes(size):
    return tuple(size[0]) if len(size) == 1 and isinstance(size[0], (tuple, list)) else tuple(size)


def zeros(*size, dtype=None, device=None, requires_grad=False) -> Tensor:
    return full(_sizes(size), 0.0, device=device, requires_grad=requires_grad)


def ones(*size, dtype=None, device=None, requires_grad=False) -> Tensor:
    return full(_sizes(size), 1.0, device=device, requires_grad=requires_grad)


def eye(n, m=None, *, dtype=None, device=None, requires_grad=False) -> Tensor:
    return tensor(np.eye(n, n if m is None else m, dtype=np.float32), device=device, requires_grad=requires_grad)


def equal(input, other) -> bool:
    return _tensor_arg(input, "equal").equal(other)


def reshape(input, shape):
    return _tensor_arg(input, "reshape").reshape(*shape)


def clone(input, *, memory_format=None):
    return _tensor_arg(input, "clone").clone(memory_format=memory_format)


def _tensor_arg(value, name):
    if not isinstance(value, Tensor):
        raise TypeError(f"{name}(): argument 'input' (position 1) must be Tensor, not {type(value).__name__}")
    return value


def relu(input):
    return _tensor_arg(input, "relu").relu()


def exp(input):
    return _tensor_arg(input, "exp").exp()


def neg(input):
    return _tensor_arg(input, "neg").neg()


def sin(input):
    return _tensor_arg(input, "sin").sin()


def sqrt(input):
    return _tensor_arg(input, "sqrt").sqrt()


def reciprocal(input):
    return _tensor_arg(input, "reciprocal").reciprocal()


def add(input, other):
    return _tensor_arg(input, "add") + other


def sub(input, other):
    return _tensor_arg(input, "sub") - other


def mul(input, other):
    return _tensor_arg(input, "mul") * other


multiply = mul


def div(input, other):
    return _tensor_arg(input, "div") / other


def matmul(input, other):
    return _tensor_arg(input, "matmul").matmul(other)


def permute(input, dims):
    return _tensor_arg(input, "permute").permute(*dims)


def transpose(input, dim0, dim1):
    return _tensor_arg(input, "transpose").transpose(dim0, dim1)


def select(input, dim, index):
    return _tensor_arg(input, "select").select(dim, index)


def sum(input):   # noqa: A001 - mirrors torch.sum
    return _tensor_arg(input, "sum").sum()


def get_float32_matmul_precision() -> str:
    """Always "highest" (python/torch_rs/__init__.py:81-85): matmul never drops below float32 accuracy."""
    return "highest"


def set_operand_image_cache(enabled: bool) -> None:
    """Tensor-core matmul operands are split into a TF32 `hi` part (read in place) and a `lo` image.  With the
    cache on (the default) the image of a storage is computed once, kept beside it and reused by every matmul
    that reads the storage -- a storage's values never change (src/storage.rs:7-18) -- and a matmul whose result
    feeds another matmul writes that result's image in its epilogue.  Off: every matmul prepares its operands
    itself.  Results are bit-identical either way."""
    _host.check(_host.lib().trsh_set_plane_cache(1 if enabled else 0))


def is_grad_enabled() -> bool:
    on = ctypes.c_int32()
    _host.check(_host.lib().trsh_is_grad_enabled(ctypes.byref(on)))
    return bool(on.value)


@contextlib.contextmanager
def no_grad():
    _host.check(_host.lib().trsh_set_grad_enabled(0))
    try:
        yield
    finally:
        _host.check(_host.lib().trsh_set_grad_enabled(1))


def synchronize(device=0):
    """Wait for everything enqueued on the engine's stream of that device."""
    _host.check(_host.lib().trsh_sync(_device_index(device) if not isinstance(device, int) else device))


class _Cuda:
    @staticmethod
    def is_available() -> bool:
        return _device.device_count() > 0

    @staticmethod
    def device_count() -> int:
        return _device.device_count()

    synchronize = staticmethod(synchronize)


cuda = _Cuda()

from . import autograd, nn  # noqa: E402,F401
