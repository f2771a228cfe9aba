"""ctypes declarations for libtrs_host.so (include/trs_host.h): the C++ host engine that plays the
role of the reference's Rust `Tensor` core for CUDA tensors."""
from __future__ import annotations

import ctypes
import os

from . import _abi

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libtrs_host.so")
_LIB = None

H = ctypes.c_void_p
HP = ctypes.POINTER(ctypes.c_void_p)
I64P = ctypes.POINTER(ctypes.c_int64)
I32P = ctypes.POINTER(ctypes.c_int32)
F32P = ctypes.POINTER(ctypes.c_float)

_PROTOTYPES = {
    "trsh_from_host": [ctypes.c_void_p, ctypes.c_int32, I64P, ctypes.c_int32, HP],
    "trsh_from_pinned_host": [ctypes.c_void_p, ctypes.c_int32, I64P, ctypes.c_int32, HP],
    "trsh_full": [ctypes.c_int32, I64P, ctypes.c_float, ctypes.c_int32, HP],
    "trsh_to_host": [H, ctypes.c_void_p],
    "trsh_to_pinned_host_async": [H, ctypes.c_void_p],
    "trsh_item": [H, F32P],
    "trsh_release": [H],
    "trsh_rank": [H, I32P],
    "trsh_layout": [H, I64P, I64P, I64P, I64P],
    "trsh_device": [H, I32P],
    "trsh_flags": [H, I32P, I32P, I32P, I32P],
    "trsh_data_ptr": [H, HP],
    "trsh_const_data_ptr": [H, HP],
    "trsh_shares_storage": [H, H, I32P],
    "trsh_permute": [H, ctypes.c_int32, I64P, HP],
    "trsh_transpose": [H, ctypes.c_int64, ctypes.c_int64, HP],
    "trsh_matrix_transpose": [H, HP],
    "trsh_reverse_dims": [H, HP],
    "trsh_select0": [H, ctypes.c_int64, HP],
    "trsh_detach": [H, HP],
    "trsh_contiguous": [H, HP],
    "trsh_clone": [H, HP],
    "trsh_clone_format": [H, ctypes.c_int32, HP],
    "trsh_contiguous_format": [H, ctypes.c_int32, HP],
    "trsh_is_contiguous_format": [H, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)],
    "trsh_reshape": [H, ctypes.c_int32, I64P, ctypes.c_int32, HP],
    "trsh_equal": [H, H, I32P],
    "trsh_squeeze": [H, ctypes.c_int32, ctypes.c_int64, HP],
    "trsh_unary": [H, ctypes.c_int32, HP],
    "trsh_scalar": [H, ctypes.c_int32, ctypes.c_float, ctypes.c_int32, HP],
    "trsh_binary": [H, H, ctypes.c_int32, HP],
    "trsh_matmul": [H, H, HP],
    "trsh_sum": [H, HP],
    "trsh_set_requires_grad": [H, ctypes.c_int32, HP],
    "trsh_backward": [H],
    "trsh_grad": [H, HP],
    "trsh_set_grad_enabled": [ctypes.c_int32],
    "trsh_is_grad_enabled": [I32P],
    "trsh_plan_unary": [ctypes.c_int32, I64P, I64P, I64P],
    "trsh_plan_scalar": [ctypes.c_int32, I64P, I64P, I64P],
    "trsh_plan_memory_format": [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, I64P, I64P, I32P, I64P],
    "trsh_plan_binary": [ctypes.c_int32, I64P, I64P, ctypes.c_int32, I64P, I64P, I32P, I64P, I64P],
    "trsh_set_plane_cache": [ctypes.c_int32],
    "trsh_has_operand_image": [H, I32P],
    "trsh_comm_unique_id": [ctypes.c_char_p],
    "trsh_comm_init": [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_char_p],
    "trsh_comm_destroy": [],
    "trsh_comm_size": [I32P],
    "trsh_all_reduce_grads": [HP, ctypes.c_int32],
    "trsh_all_reduce": [H],
    "trsh_materialize": [H],
    "trsh_sync": [ctypes.c_int32],
    "trsh_stream": [ctypes.c_int32, HP],
}
_SPECIAL = {"trsh_last_error": ([], ctypes.c_char_p), "trsh_grad_fn_name": ([H], ctypes.c_char_p)}
EXPORTS = sorted(list(_PROTOTYPES) + list(_SPECIAL))

# error kind -> Python exception class, as the reference maps TensorError (src/python_tensor_errors.rs:8-49)
INDEX_ERRORS = {5, 6, 8, 17}


def lib():
    global _LIB
    if _LIB is None:
        _abi.lib()   # libtrs_cuda.so first (the engine links against it)
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build`")
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int32
        for name, (argtypes, restype) in _SPECIAL.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _LIB = handle
    return _LIB


def check(kind):
    if kind == 0:
        return
    message = lib().trsh_last_error().decode(errors="replace")
    if kind in INDEX_ERRORS:
        raise IndexError(message)
    raise RuntimeError(message)
