"""TEST INFRASTRUCTURE — NOT PRODUCT CODE.

ctypes front-end over ``oracle/libcpu_ref.so`` (the C++ restatement of the
pytorch-rs CPU engine, see ``oracle/cpu_ref.cpp``).  ``RefTensor`` carries a
NumPy storage plus shape/strides/offset in elements so tests can compose the
same chains the product runs and compare values *and* layout metadata.

Only tests, the smoke check and the bench's CPU-baseline leg may import this.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcpu_ref.so")

I64P = ctypes.POINTER(ctypes.c_int64)
F32P = ctypes.POINTER(ctypes.c_float)

UNARY = {"relu": 0, "exp": 1, "neg": 2, "sin": 3, "sqrt": 4, "reciprocal": 5, "copy": 6}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3}
SCALAR = {"add": 0, "sub": 1, "mul": 2, "div": 3, "rsub": 4, "rdiv": 5}
STATUS = {1: "ShapeMismatch", 2: "StrideCalculationOverflow", 3: "ElementCountOverflow",
          4: "MatmulRequiresMatrices", 5: "MatmulInnerDimensionMismatch", 6: "BadOp",
          8: "ContiguousMemoryFormatRankMismatch", 9: "ContiguousPreserveFormatUnsupported"}
MEMORY_FORMATS = {"preserve_format": 0, "contiguous_format": 1, "channels_last": 2, "channels_last_3d": 3}


class RefError(RuntimeError):
    def __init__(self, status):
        super().__init__(STATUS.get(status, str(status)))
        self.kind = STATUS.get(status, str(status))


def build(force: bool = False) -> str:
    """Compile the checker with the flags recorded in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "cpu_ref.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libcpu_ref.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.ref_sum.restype = ctypes.c_float
        _lib.ref_relu_value.restype = ctypes.c_float
        _lib.ref_relu_value.argtypes = [ctypes.c_float]
        _lib.ref_relu_backward_value.restype = ctypes.c_float
        _lib.ref_relu_backward_value.argtypes = [ctypes.c_float, ctypes.c_float]
    return _lib


def _i64(values):
    return (ctypes.c_int64 * max(len(values), 1))(*[int(v) for v in values])


def _fp(array):
    return array.ctypes.data_as(F32P)


def contiguous_strides(shape):
    strides, s = [0] * len(shape), 1
    for axis in range(len(shape) - 1, -1, -1):
        strides[axis] = s
        s *= max(shape[axis], 1)
    return strides


def _check(status):
    if status:
        raise RefError(status)


class RefTensor:
    """Storage (1-D float32 ndarray) + view metadata, mirroring the reference Tensor (src/tensor.rs:212-221)."""

    def __init__(self, storage, shape, strides=None, offset=0):
        self.storage = np.ascontiguousarray(storage, dtype=np.float32).reshape(-1)
        self.shape = [int(d) for d in shape]
        self.strides = [int(s) for s in (contiguous_strides(self.shape) if strides is None else strides)]
        self.offset = int(offset)

    # -- construction -----------------------------------------------------
    @classmethod
    def from_numpy(cls, array):
        array = np.asarray(array, dtype=np.float32, order="C")     # keeps rank 0
        return cls(array.reshape(-1), array.shape)

    @property
    def numel(self):
        n = 1
        for d in self.shape:
            n *= d
        return n

    # -- views (src/tensor.rs:1082-1215, 1850-1973) ---------------------------
    def permute(self, dims):
        return RefTensor(self.storage, [self.shape[d] for d in dims], [self.strides[d] for d in dims], self.offset)

    def transpose(self, a, b):
        dims = list(range(len(self.shape)))
        if dims:
            dims[a], dims[b] = dims[b], dims[a]
        return self.permute(dims)

    @property
    def mT(self):
        return self.transpose(-2, -1)

    @property
    def T(self):
        return self.permute(list(range(len(self.shape)))[::-1])

    def select0(self, index):
        if index < 0:
            index += self.shape[0]
        return RefTensor(self.storage, self.shape[1:], self.strides[1:], self.offset + index * self.strides[0])

    def reshape(self, shape):
        """View when the strides allow it, else a packed copy (tensor.rs:2032-2148)."""
        shape = list(shape)
        if -1 in shape:
            known = 1
            for d in shape:
                if d != -1:
                    known *= d
            shape[shape.index(-1)] = self.numel // known
        out = _i64([0] * len(shape))
        status = lib().ref_reshape_view_strides(len(self.shape), _i64(self.shape), _i64(self.strides), len(shape),
                                                _i64(shape), out)
        if status == 0:
            return RefTensor(self.storage, shape, list(out)[:len(shape)], self.offset)
        if status != 7:
            raise RefError(status)
        return RefTensor(self.logical().reshape(-1), shape)

    def view_strides(self, shape):
        out = _i64([0] * len(shape))
        status = lib().ref_reshape_view_strides(len(self.shape), _i64(self.shape), _i64(self.strides), len(shape),
                                                _i64(list(shape)), out)
        return list(out)[:len(shape)] if status == 0 else None

    def is_contiguous_in(self, memory_format="contiguous_format"):
        """is_contiguous_with_memory_format (src/tensor.rs:1004-1014)."""
        return bool(lib().ref_is_contiguous_in_format(MEMORY_FORMATS[memory_format], len(self.shape), _i64(self.shape), _i64(self.strides)))

    def contiguous(self, memory_format="contiguous_format"):
        """try_contiguous (src/tensor.rs:1606-1675): self when the layout already matches, else a packed copy."""
        fmt = MEMORY_FORMATS[memory_format]
        want = {2: 4, 3: 5}.get(fmt)
        if want is not None and len(self.shape) != want:
            raise RefError(8)
        if self.is_contiguous_in(memory_format):
            return self
        return self._copy_in_format(fmt, for_clone=0)

    def clone(self, memory_format="preserve_format"):
        """try_clone_with_memory_format (src/tensor.rs:1533-1575)."""
        return self._copy_in_format(MEMORY_FORMATS[memory_format], for_clone=1)

    def _copy_in_format(self, fmt, for_clone):
        out = _i64([0] * max(len(self.shape), 1))
        _check(lib().ref_memory_format_strides(fmt, for_clone, len(self.shape), _i64(self.shape), _i64(self.strides), out))
        strides = list(out)[:len(self.shape)]
        packed = np.zeros(self.numel, dtype=np.float32)
        if self.numel:
            dst = np.lib.stride_tricks.as_strided(packed, self.shape, [4 * s for s in strides])
            dst[...] = self.logical()
        return RefTensor(packed, self.shape, strides)

    # -- egress -----------------------------------------------------------------
    def logical(self):
        """Values in logical row-major order as an ndarray of ``shape``."""
        if self.numel == 0:
            return np.zeros(self.shape, dtype=np.float32)
        view = np.lib.stride_tricks.as_strided(self.storage[self.offset:], self.shape,
                                               [4 * s for s in self.strides], writeable=False)
        return np.array(view, dtype=np.float32, order="C")

    # -- pointwise ------------------------------------------------------------
    def unary(self, op):
        out = np.zeros(self.numel, dtype=np.float32)
        out_strides = _i64([0] * len(self.shape))
        _check(lib().ref_unary(UNARY[op], _fp(self.storage), ctypes.c_int64(self.offset), len(self.shape),
                               _i64(self.shape), _i64(self.strides), _fp(out), out_strides))
        return RefTensor(out, self.shape, list(out_strides)[:len(self.shape)])

    def relu(self):
        return self.unary("relu")

    def exp(self):
        return self.unary("exp")

    def neg(self):
        return self.unary("neg")

    def scalar(self, op, value):
        out = np.zeros(self.numel, dtype=np.float32)
        out_strides = _i64([0] * len(self.shape))
        _check(lib().ref_scalar(SCALAR[op], ctypes.c_float(value), _fp(self.storage), ctypes.c_int64(self.offset),
                                len(self.shape), _i64(self.shape), _i64(self.strides), _fp(out), out_strides))
        return RefTensor(out, self.shape, list(out_strides)[:len(self.shape)])

    def binary(self, op, other):
        rank = max(len(self.shape), len(other.shape))
        out_shape, out_strides = _i64([0] * rank), _i64([0] * rank)
        _check(lib().ref_binary_plan(len(self.shape), _i64(self.shape), _i64(self.strides), len(other.shape),
                                     _i64(other.shape), _i64(other.strides), out_shape, out_strides))
        shape = list(out_shape)[:rank]
        n = 1
        for d in shape:
            n *= d
        out = np.zeros(n, dtype=np.float32)
        _check(lib().ref_binary(BINARY[op], _fp(self.storage), ctypes.c_int64(self.offset), len(self.shape),
                                _i64(self.shape), _i64(self.strides), _fp(other.storage),
                                ctypes.c_int64(other.offset), len(other.shape), _i64(other.shape),
                                _i64(other.strides), _fp(out), out_shape, out_strides))
        return RefTensor(out, shape, list(out_strides)[:rank])

    def __add__(self, other):
        return self.binary("add", other) if isinstance(other, RefTensor) else self.scalar("add", other)

    def __sub__(self, other):
        return self.binary("sub", other) if isinstance(other, RefTensor) else self.scalar("sub", other)

    def __mul__(self, other):
        return self.binary("mul", other) if isinstance(other, RefTensor) else self.scalar("mul", other)

    def __rmul__(self, other):   # 2.0 * t == t.mul_scalar(2.0)  (src/python.rs:3901, tensor.rs:2274)
        return self.scalar("mul", other)

    def __radd__(self, other):
        return self.scalar("add", other)

    def __rsub__(self, other):
        return self.scalar("rsub", other)

    def __truediv__(self, other):
        return self.binary("div", other) if isinstance(other, RefTensor) else self.scalar("div", other)

    def __rtruediv__(self, other):
        return self.scalar("rdiv", other)

    # -- contraction / reduction ------------------------------------------------
    def matmul(self, other):
        if len(self.shape) != 2 or len(other.shape) != 2:
            raise RefError(4)
        out = np.zeros(self.shape[0] * other.shape[1], dtype=np.float32)
        _check(lib().ref_matmul(_fp(self.storage), ctypes.c_int64(self.offset), _i64(self.shape), _i64(self.strides),
                                _fp(other.storage), ctypes.c_int64(other.offset), _i64(other.shape),
                                _i64(other.strides), _fp(out)))
        return RefTensor(out, [self.shape[0], other.shape[1]])

    def sum(self):
        return float(lib().ref_sum(_fp(self.storage), ctypes.c_int64(self.offset), len(self.shape),
                                   _i64(self.shape), _i64(self.strides)))

    # -- backward pieces ----------------------------------------------------------
    def relu_vjp(self, upstream):
        """``self`` is the saved relu input; ``upstream`` a logical row-major ndarray."""
        upstream = np.ascontiguousarray(upstream, dtype=np.float32).reshape(-1)
        grad = np.zeros(self.numel, dtype=np.float32)
        lib().ref_relu_vjp(_fp(self.storage), ctypes.c_int64(self.offset), len(self.shape), _i64(self.shape),
                           _i64(self.strides), _fp(upstream), _fp(grad))
        return grad.reshape(self.shape)


def unbroadcast(upstream, out_shape, in_shape, other: RefTensor | None = None):
    """Reduce a logical-order upstream of ``out_shape`` onto ``in_shape`` (tensor.rs:3204-3228)."""
    upstream = np.ascontiguousarray(upstream, dtype=np.float32).reshape(-1)
    n = 1
    for d in in_shape:
        n *= d
    grad = np.zeros(n, dtype=np.float32)
    if other is None:
        lib().ref_unbroadcast(len(out_shape), _i64(out_shape), len(in_shape), _i64(in_shape), _fp(upstream),
                              None, ctypes.c_int64(0), 0, _i64([]), _i64([]), _fp(grad))
    else:
        lib().ref_unbroadcast(len(out_shape), _i64(out_shape), len(in_shape), _i64(in_shape), _fp(upstream),
                              _fp(other.storage), ctypes.c_int64(other.offset), len(other.shape),
                              _i64(other.shape), _i64(other.strides), _fp(grad))
    return grad.reshape(in_shape)


def permute_vjp(upstream, in_shape, dims):
    upstream = np.ascontiguousarray(upstream, dtype=np.float32).reshape(-1)
    grad = np.zeros(upstream.size, dtype=np.float32)
    lib().ref_permute_vjp(len(in_shape), _i64(in_shape), _i64(dims), _fp(upstream), _fp(grad))
    return grad.reshape(in_shape)


def unary_strides(shape, strides):
    out = _i64([0] * len(shape))
    _check(lib().ref_unary_strides(len(shape), _i64(shape), _i64(strides), out))
    return list(out)[:len(shape)]


def scalar_strides(shape, strides):
    out = _i64([0] * len(shape))
    _check(lib().ref_scalar_strides(len(shape), _i64(shape), _i64(strides), out))
    return list(out)[:len(shape)]


def binary_plan(lshape, lstrides, rshape, rstrides):
    rank = max(len(lshape), len(rshape))
    out_shape, out_strides = _i64([0] * rank), _i64([0] * rank)
    _check(lib().ref_binary_plan(len(lshape), _i64(lshape), _i64(lstrides), len(rshape), _i64(rshape),
                                 _i64(rstrides), out_shape, out_strides))
    return list(out_shape)[:rank], list(out_strides)[:rank]


def ulp_distance(a, b):
    """Element-wise distance in units in the last place between two float32 arrays (NaN pairs count as 0)."""
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    ai = a.view(np.int32).astype(np.int64)
    bi = b.view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, -(ai & 0x7FFFFFFF), ai)
    bi = np.where(bi < 0, -(bi & 0x7FFFFFFF), bi)
    d = np.abs(ai - bi)
    both_nan = np.isnan(a) & np.isnan(b)
    one_nan = np.isnan(a) ^ np.isnan(b)
    d = np.where(both_nan, 0, d)
    d = np.where(one_nan, np.iinfo(np.int64).max, d)
    return d


def same_bits_or_nan(a, b):
    """True where bit patterns agree, or both are NaN (payloads differ between x86 and the GPU)."""
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    return (a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))
