"""The `torch_rs` tensor surface for CUDA tensors.

Mirrors what the reference's PyO3 layer exposes for the hot path (src/python.rs:3848-3952,
4067-4133, 3495-3507; src/python_variable_functions.rs:32-63): operators, `relu`/`exp`/`matmul`/
`multiply`, the views `.T/.mT/permute/transpose/select`, `backward()` and `.grad`.  Each method is
one call into the C++ host engine (libtrs_host.so); no arithmetic happens in Python, and there is
no CPU fallback: every tensor here lives on a CUDA device.
"""
from __future__ import annotations

import ctypes
import numbers

import numpy as np

from . import _abi, _host

OPS = _abi.OPS


class device:
    """`torch.device` for the one device family this path serves (src/python_device.rs:81-127)."""

    def __init__(self, spec="cuda", index=None):
        if isinstance(spec, device):
            self.type, self.index = spec.type, spec.index
            return
        if isinstance(spec, int):
            spec, index = "cuda", spec
        text = str(spec)
        if ":" in text:
            text, idx = text.split(":", 1)
            index = int(idx)
        if text == "cpu":
            raise RuntimeError("CPU tensors are served by the reference's own engine; this package executes "
                               "tensors created with device='cuda' only and never falls back to the CPU")
        if text != "cuda":
            raise RuntimeError(f"Expected one of cpu, cuda device type at start of device string: {text}")
        self.type = "cuda"
        self.index = 0 if index is None else int(index)

    def __repr__(self):
        return f"device(type='cuda', index={self.index})"

    def __str__(self):
        return f"cuda:{self.index}"

    def __eq__(self, other):
        return isinstance(other, device) and (self.type, self.index) == (other.type, other.index)

    def __hash__(self):
        return hash((self.type, self.index))


class memory_format:
    """Memory-format descriptor (reference: PyMemoryFormat, src/python_memory_format.rs:14-52): four
    canonical instances, printed as ``torch.<name>``, compared by identity of the format."""
    _names = ("preserve_format", "contiguous_format", "channels_last", "channels_last_3d")

    def __init__(self, code: int):
        self._code = int(code)

    def __repr__(self):
        return "torch." + self._names[self._code]

    __str__ = __repr__

    def __eq__(self, other):
        return isinstance(other, memory_format) and other._code == self._code

    def __hash__(self):
        return hash(("memory_format", self._code))

    def __reduce__(self):
        return repr(self)


preserve_format = memory_format(0)
contiguous_format = memory_format(1)
channels_last = memory_format(2)
channels_last_3d = memory_format(3)


def _memory_format_code(value, op="contiguous") -> int:
    if not isinstance(value, memory_format):
        raise TypeError(f"{op}(): argument 'memory_format' must be torch.memory_format, not {type(value).__name__}")
    return value._code


def _device_index(dev) -> int:
    if dev is None:
        raise RuntimeError("pass device='cuda' (or 'cuda:N'): tensors without a CUDA device belong to the "
                           "reference's CPU engine, which this package does not replace")
    return device(dev).index


def _wrap(handle) -> "Tensor":
    t = Tensor.__new__(Tensor)
    t._h = handle
    return t


def _new_handle():
    return ctypes.c_void_p()


class Tensor:
    __slots__ = ("_h", "__weakref__")
    __array_priority__ = 1000

    def __init__(self, *args, **kwargs):
        raise TypeError("use torch_rs.tensor(data, device='cuda')")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _host.lib().trsh_release(h)
            except Exception:
                pass

    # ---- metadata ----------------------------------------------------------------------------
    def _layout(self):
        lib = _host.lib()
        rank = ctypes.c_int32()
        _host.check(lib.trsh_rank(self._h, ctypes.byref(rank)))
        n = max(rank.value, 1)
        shape, strides = (ctypes.c_int64 * n)(), (ctypes.c_int64 * n)()
        offset, numel = ctypes.c_int64(), ctypes.c_int64()
        _host.check(lib.trsh_layout(self._h, shape, strides, ctypes.byref(offset), ctypes.byref(numel)))
        return list(shape)[:rank.value], list(strides)[:rank.value], offset.value, numel.value

    def _flags(self):
        a, b, c, d = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        _host.check(_host.lib().trsh_flags(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(d)))
        return bool(a.value), bool(b.value), bool(c.value), bool(d.value)

    @property
    def shape(self):
        return tuple(self._layout()[0])

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    def stride(self, dim=None):
        strides = tuple(self._layout()[1])
        return strides if dim is None else strides[dim]

    def storage_offset(self):
        return self._layout()[2]

    def numel(self):
        return self._layout()[3]

    def dim(self):
        return len(self.shape)

    ndim = property(dim)

    @property
    def dtype(self):
        return "torch.float32"

    @property
    def device(self):
        idx = ctypes.c_int32()
        _host.check(_host.lib().trsh_device(self._h, ctypes.byref(idx)))
        return device("cuda", idx.value)

    is_cuda = True
    is_cpu = False

    @property
    def requires_grad(self):
        return self._flags()[0]

    @property
    def is_leaf(self):
        return self._flags()[1]

    def is_contiguous(self, memory_format=None):
        """is_contiguous_with_memory_format (src/tensor.rs:1004-1014); preserve_format queries like contiguous_format."""
        if memory_format is None:
            return self._flags()[2]
        result = ctypes.c_int32()
        _host.check(_host.lib().trsh_is_contiguous_format(self._h, _memory_format_code(memory_format, "is_contiguous"), ctypes.byref(result)))
        return bool(result.value)

    def is_pending(self):
        """True while this tensor's values are still a recorded, not yet executed, pointwise chain."""
        return self._flags()[3]

    def data_ptr(self):
        p = ctypes.c_void_p()
        _host.check(_host.lib().trsh_data_ptr(self._h, ctypes.byref(p)))
        return p.value or 0

    def _const_data_ptr(self):
        """Device address for read-only use (checks, descriptors); unlike `data_ptr()` it does not make the
        engine treat the storage as writable from outside."""
        p = ctypes.c_void_p()
        _host.check(_host.lib().trsh_const_data_ptr(self._h, ctypes.byref(p)))
        return p.value or 0

    def _has_operand_image(self):
        """Whether this tensor's storage carries a cached matmul operand image (see set_operand_image_cache)."""
        r = ctypes.c_int32()
        _host.check(_host.lib().trsh_has_operand_image(self._h, ctypes.byref(r)))
        return bool(r.value)

    def shares_storage_with(self, other):
        r = ctypes.c_int32()
        _host.check(_host.lib().trsh_shares_storage(self._h, other._h, ctypes.byref(r)))
        return bool(r.value)

    def _grad_fn_name(self):
        return _host.lib().trsh_grad_fn_name(self._h).decode()

    # ---- egress -----------------------------------------------------------------------------
    def numpy(self):
        shape, _, _, numel = self._layout()
        out = np.empty(numel, dtype=np.float32)
        _host.check(_host.lib().trsh_to_host(self._h, out.ctypes.data))
        return out.reshape(shape)

    def copy_to_host(self, out, non_blocking=False):
        """Write the values in logical order into a caller-provided float32 array.  With
        `non_blocking=True` and a page-locked array (`torch_rs.pinned_empty`) the call returns at once
        and the copy overlaps later uploads and kernels; the data is valid after `torch_rs.synchronize`."""
        if out.dtype != np.float32 or not out.flags.c_contiguous or out.size != self.numel():
            raise ValueError("copy_to_host needs a C-contiguous float32 array with numel elements")
        if non_blocking:
            from . import _device
            if not _device.is_pinned(out):
                raise ValueError("non_blocking copy_to_host needs an array from torch_rs.pinned_empty")
            _host.check(_host.lib().trsh_to_pinned_host_async(self._h, out.ctypes.data))
        else:
            _host.check(_host.lib().trsh_to_host(self._h, out.ctypes.data))
        return out

    def cpu(self):
        """Values in logical order as a NumPy array (CPU tensors themselves belong to the reference engine)."""
        return self.numpy()

    def __array__(self, dtype=None, copy=None):
        a = self.numpy()
        return a if dtype is None else a.astype(dtype)

    def __dlpack__(self, stream=None):
        """Zero-copy export; pending work is enqueued first and the engine's stream is drained, so the
        consumer may use the memory on any stream."""
        from . import _dlpack
        capsule = _dlpack.to_dlpack(self)
        _host.check(_host.lib().trsh_sync(self.device.index))
        return capsule

    def __dlpack_device__(self):
        return (2, self.device.index)          # kDLCUDA

    def tolist(self):
        return self.numpy().tolist()

    def item(self):
        v = ctypes.c_float()
        _host.check(_host.lib().trsh_item(self._h, ctypes.byref(v)))
        return v.value

    def __float__(self):
        return float(self.item())

    def __repr__(self):
        return f"tensor({self.numpy()!r}, device='{self.device}')"

    # ---- views --------------------------------------------------------------------------------
    def _view(self, fn, *args):
        out = _new_handle()
        _host.check(fn(self._h, *args, ctypes.byref(out)))
        return _wrap(out)

    def permute(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        arr = (ctypes.c_int64 * max(len(dims), 1))(*dims)
        return self._view(_host.lib().trsh_permute, len(dims), arr)

    def transpose(self, dim0, dim1):
        return self._view(_host.lib().trsh_transpose, dim0, dim1)

    @property
    def mT(self):
        return self._view(_host.lib().trsh_matrix_transpose)

    @property
    def T(self):
        return self._view(_host.lib().trsh_reverse_dims)

    def t(self):
        if self.dim() > 2:
            raise RuntimeError(f"t() expects a tensor with <= 2 dimensions, but self is {self.dim()}D")
        return self.T

    def select(self, dim, index):
        if dim not in (0, -self.dim()):
            raise RuntimeError("select(): only dim=0 is supported")     # as in the reference (src/python.rs:2172-2177)
        return self._view(_host.lib().trsh_select0, index)

    def __getitem__(self, index):
        if isinstance(index, numbers.Integral):
            return self._view(_host.lib().trsh_select0, int(index))
        raise TypeError("only integer indexing of the leading dimension is supported on CUDA tensors")

    def detach(self):
        return self._view(_host.lib().trsh_detach)

    def contiguous(self, memory_format=None):
        """try_contiguous (src/tensor.rs:1606-1675): self's storage when the layout already matches the format."""
        if memory_format is None:
            return self._view(_host.lib().trsh_contiguous)
        return self._view(_host.lib().trsh_contiguous_format, _memory_format_code(memory_format))

    def clone(self, memory_format=None):
        """try_clone_with_memory_format (src/tensor.rs:1533-1575); the default is preserve_format."""
        if memory_format is None:
            return self._view(_host.lib().trsh_clone)
        return self._view(_host.lib().trsh_clone_format, _memory_format_code(memory_format, "clone"))

    def _reshape(self, shape, view_only):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        arr = (ctypes.c_int64 * max(len(shape), 1))(*shape)
        return self._view(_host.lib().trsh_reshape, len(shape), arr, int(view_only))

    def reshape(self, *shape):
        return self._reshape(shape, False)

    def view(self, *shape):
        return self._reshape(shape, True)

    def flatten(self, start_dim=0, end_dim=-1):
        shape = list(self.shape)
        rank = max(len(shape), 1)
        start, end = start_dim % rank, end_dim % rank
        if start > end:
            raise RuntimeError("flatten() has invalid args: start_dim cannot come after end_dim")
        if not shape:
            return self.reshape(1)
        merged = 1
        for d in shape[start:end + 1]:
            merged *= d
        return self.reshape(*shape[:start], merged, *shape[end + 1:])

    def ravel(self):
        return self.contiguous().reshape(-1)

    def squeeze(self, dim=None):
        if dim is None:
            return self._view(_host.lib().trsh_squeeze, 1, 0)
        return self._view(_host.lib().trsh_squeeze, 0, int(dim))

    def unbind(self, dim=0):
        """Slices along the leading dimension (each one a `select(0, i)` view)."""
        if dim not in (0, -self.dim()) or self.dim() == 0:
            raise RuntimeError("unbind(): only dim=0 of a tensor with at least one dimension is supported")
        return tuple(self[i] for i in range(self.shape[0]))

    def equal(self, other):
        r = ctypes.c_int32()
        _host.check(_host.lib().trsh_equal(self._h, other._h, ctypes.byref(r)))
        return bool(r.value)

    # ---- pointwise ----------------------------------------------------------------------------
    def _unary(self, name):
        return self._view(_host.lib().trsh_unary, OPS[name])

    def relu(self):
        return self._unary("relu")

    def exp(self):
        return self._unary("exp")

    def neg(self):
        return self._unary("neg")

    __neg__ = neg

    def reciprocal(self):
        return self._unary("reciprocal")

    def sqrt(self):
        return self._unary("sqrt")

    def sin(self):
        return self._unary("sin")

    def _arith(self, other, name, reflected=False):
        lib = _host.lib()
        out = _new_handle()
        if isinstance(other, Tensor):
            l, r = (other, self) if reflected else (self, other)
            _host.check(lib.trsh_binary(l._h, r._h, OPS[name], ctypes.byref(out)))
        elif isinstance(other, numbers.Real):
            _host.check(lib.trsh_scalar(self._h, OPS[name], ctypes.c_float(float(other)), int(reflected), ctypes.byref(out)))
        else:
            return NotImplemented
        return _wrap(out)

    def __add__(self, other):
        return self._arith(other, "add")

    def __radd__(self, other):            # scalar + x == x.add_scalar(scalar) (src/python.rs:3873-3879)
        return self._arith(other, "add")

    def __sub__(self, other):
        return self._arith(other, "sub")

    def __rsub__(self, other):
        return self._arith(other, "sub", reflected=True)

    def __mul__(self, other):
        return self._arith(other, "mul")

    def __rmul__(self, other):            # 2.0 * x == x.mul_scalar(2.0) (src/python.rs:3901)
        return self._arith(other, "mul")

    def __truediv__(self, other):
        return self._arith(other, "div")

    def __rtruediv__(self, other):
        return self._arith(other, "div", reflected=True)

    add, sub, mul, multiply, div = __add__, __sub__, __mul__, __mul__, __truediv__

    # ---- contraction / reduction ----------------------------------------------------------------
    def matmul(self, other):
        if not isinstance(other, Tensor):
            raise TypeError("matmul(): argument 'other' must be Tensor")
        out = _new_handle()
        _host.check(_host.lib().trsh_matmul(self._h, other._h, ctypes.byref(out)))
        return _wrap(out)

    __matmul__ = matmul

    def sum(self):
        return self._view(_host.lib().trsh_sum)

    # ---- autograd -----------------------------------------------------------------------------
    def requires_grad_(self, requires_grad=True):
        out = _new_handle()
        _host.check(_host.lib().trsh_set_requires_grad(self._h, int(requires_grad), ctypes.byref(out)))
        old, self._h = self._h, out
        _host.lib().trsh_release(old)
        return self

    def backward(self):
        _host.check(_host.lib().trsh_backward(self._h))

    @property
    def grad(self):
        out = _new_handle()
        _host.check(_host.lib().trsh_grad(self._h, ctypes.byref(out)))
        return _wrap(out) if out.value else None

    # ---- execution control ----------------------------------------------------------------------
    def materialize(self):
        """Run the pending chain that produces this tensor (enqueue only; does not wait)."""
        _host.check(_host.lib().trsh_materialize(self._h))
        return self
