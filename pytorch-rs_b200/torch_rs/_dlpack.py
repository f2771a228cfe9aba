"""DLPack export (zero copy) of CUDA tensors: `Tensor.__dlpack__` / `__dlpack_device__`.

The reference offers `__array__` (a host copy, src/python.rs:3743-3756); on a CUDA device the
equivalent zero-copy hand-off to other libraries is the DLPack capsule.  The capsule keeps the
producing tensor alive until the consumer calls the deleter.
"""
from __future__ import annotations

import ctypes

K_DL_CUDA = 2
K_DL_FLOAT = 2


class DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("device", DLDevice), ("ndim", ctypes.c_int32), ("dtype", DLDataType),
                ("shape", ctypes.POINTER(ctypes.c_int64)), ("strides", ctypes.POINTER(ctypes.c_int64)),
                ("byte_offset", ctypes.c_uint64)]


class DLManagedTensor(ctypes.Structure):
    pass


_DELETER = ctypes.CFUNCTYPE(None, ctypes.POINTER(DLManagedTensor))
DLManagedTensor._fields_ = [("dl_tensor", DLTensor), ("manager_ctx", ctypes.c_void_p), ("deleter", _DELETER)]

_live = {}          # address of the managed struct -> everything that must outlive the capsule


@_DELETER
def _deleter(managed):
    _live.pop(ctypes.addressof(managed.contents), None)


_api = ctypes.PyDLL(None)          # CPython's C API with the GIL held, taking raw object pointers
_api.PyCapsule_New.restype = ctypes.py_object
_api.PyCapsule_New.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
_api.PyCapsule_IsValid.restype = ctypes.c_int
_api.PyCapsule_IsValid.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
_api.PyCapsule_GetPointer.restype = ctypes.c_void_p
_api.PyCapsule_GetPointer.argtypes = [ctypes.c_void_p, ctypes.c_char_p]


@ctypes.PYFUNCTYPE(None, ctypes.c_void_p)
def _capsule_destructor(capsule):
    # The capsule is being finalised (reference count 0), so it is only touched as a raw pointer.
    # One that was never consumed is still named "dltensor": release what it holds.
    if _api.PyCapsule_IsValid(capsule, b"dltensor"):
        _live.pop(_api.PyCapsule_GetPointer(capsule, b"dltensor"), None)


def to_dlpack(tensor):
    shape, strides, _, _ = tensor._layout()
    rank = len(shape)
    shape_arr = (ctypes.c_int64 * max(rank, 1))(*shape)
    stride_arr = (ctypes.c_int64 * max(rank, 1))(*strides)
    managed = DLManagedTensor()
    managed.dl_tensor.data = tensor.data_ptr()            # forces the value onto the device
    managed.dl_tensor.device = DLDevice(K_DL_CUDA, tensor.device.index)
    managed.dl_tensor.ndim = rank
    managed.dl_tensor.dtype = DLDataType(K_DL_FLOAT, 32, 1)
    managed.dl_tensor.shape = ctypes.cast(shape_arr, ctypes.POINTER(ctypes.c_int64))
    managed.dl_tensor.strides = ctypes.cast(stride_arr, ctypes.POINTER(ctypes.c_int64))
    managed.dl_tensor.byte_offset = 0
    managed.manager_ctx = None
    managed.deleter = _deleter
    address = ctypes.addressof(managed)
    _live[address] = (managed, shape_arr, stride_arr, tensor)
    return _api.PyCapsule_New(address, b"dltensor", ctypes.cast(_capsule_destructor, ctypes.c_void_p))
