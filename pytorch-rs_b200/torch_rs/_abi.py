"""ctypes declarations for libtrs_cuda.so (the C ABI in include/trs_cuda.h).

This is the binding a reference maintainer would write as a Rust ``extern "C"`` block; here it
serves the Python host and the parity tests.  Loading never needs a GPU; compute entry points
return TRS_ERR_NO_DEVICE without one (there is no CPU fallback).
"""
from __future__ import annotations

import ctypes
import os

MAX_RANK, MAX_INPUTS, MAX_OUTPUTS, MAX_INSTRS = 8, 8, 4, 64

OPS = {"const": 0, "add": 1, "sub": 2, "mul": 3, "div": 4, "neg": 5, "relu": 6, "exp": 7, "relu_vjp": 8,
       "reciprocal": 9, "sqrt": 10, "sin": 11, "cos": 12, "copy": 13, "ne": 14}
EPILOGUES = {"none": 0, "bias": 1, "bias_relu": 2, "relu": 3, "relu_vjp": 4}
GEMM_ALGOS = {"auto": 0, "simt_fp32": 1, "tcgen05_3xtf32": 2, "tcgen05_3xtf32_2cta": 3}
STATUS_NAMES = {0: "ok", 1: "invalid argument", 2: "allocation failed", 3: "CUDA error", 4: "JIT error",
                5: "unsupported", 6: "no CUDA device", 7: "device status"}


class Operand(ctypes.Structure):
    _fields_ = [("base", ctypes.c_void_p), ("offset", ctypes.c_int64), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_RANK), ("stride", ctypes.c_int64 * MAX_RANK)]


class Instr(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("a", ctypes.c_int32), ("b", ctypes.c_int32), ("imm", ctypes.c_float)]


class Program(ctypes.Structure):
    _fields_ = [("n_inputs", ctypes.c_int32), ("n_instrs", ctypes.c_int32), ("n_outputs", ctypes.c_int32),
                ("outputs", ctypes.c_int32 * MAX_OUTPUTS), ("instrs", Instr * MAX_INSTRS)]


class GemmDesc(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int64), ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
                ("a", ctypes.c_void_p), ("a_batch_stride", ctypes.c_int64), ("a_row_stride", ctypes.c_int64),
                ("a_col_stride", ctypes.c_int64),
                ("b", ctypes.c_void_p), ("b_batch_stride", ctypes.c_int64), ("b_row_stride", ctypes.c_int64),
                ("b_col_stride", ctypes.c_int64),
                ("c", ctypes.c_void_p), ("c_batch_stride", ctypes.c_int64), ("c_row_stride", ctypes.c_int64),
                ("bias", ctypes.c_void_p), ("aux", ctypes.c_void_p), ("preact", ctypes.c_void_p),
                ("epilogue", ctypes.c_int32), ("algo", ctypes.c_int32)]


class GemmPlanes(ctypes.Structure):
    _fields_ = [("a_lo", ctypes.c_void_p), ("b_lo", ctypes.c_void_p), ("c_lo", ctypes.c_void_p),
                ("a_flag", ctypes.c_void_p), ("b_flag", ctypes.c_void_p), ("c_flag", ctypes.c_void_p)]


class TrsError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


_LIB = None
LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libtrs_cuda.so")

# name -> argtypes (restype is int32 status unless listed in _SPECIAL)
_PROTOTYPES = {
    "trs_device_count": [ctypes.POINTER(ctypes.c_int32)],
    "trs_set_current_device": [ctypes.c_int32],
    "trs_device_pci_bus_id": [ctypes.c_int32, ctypes.c_char_p, ctypes.c_int32],
    "trs_malloc": [ctypes.c_int32, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)],
    "trs_free": [ctypes.c_int32, ctypes.c_void_p],
    "trs_malloc_async": [ctypes.c_int32, ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)],
    "trs_free_async": [ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p],
    "trs_empty_cache": [ctypes.c_int32],
    "trs_memory_stats": [ctypes.c_int32, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)],
    "trs_malloc_host": [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)],
    "trs_free_host": [ctypes.c_void_p],
    "trs_stream_create": [ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)],
    "trs_stream_destroy": [ctypes.c_void_p],
    "trs_stream_sync": [ctypes.c_void_p],
    "trs_stream_device": [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)],
    "trs_stream_handle": [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)],
    "trs_device_sync": [ctypes.c_int32],
    "trs_event_create": [ctypes.POINTER(ctypes.c_void_p)],
    "trs_event_record": [ctypes.c_void_p, ctypes.c_void_p],
    "trs_event_sync": [ctypes.c_void_p],
    "trs_event_elapsed_ms": [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)],
    "trs_event_destroy": [ctypes.c_void_p],
    "trs_stream_wait_event": [ctypes.c_void_p, ctypes.c_void_p],
    "trs_memcpy_h2d": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p],
    "trs_memcpy_d2h": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p],
    "trs_memcpy_d2d": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p],
    "trs_pointwise": [ctypes.POINTER(Program), ctypes.POINTER(Operand), ctypes.POINTER(Operand), ctypes.c_void_p],
    "trs_pointwise_prepare": [ctypes.POINTER(Program), ctypes.POINTER(Operand), ctypes.POINTER(Operand),
                              ctypes.c_char_p],
    "trs_fill_f32": [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p],
    "trs_accumulate_f32": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p],
    "trs_reduce_sum_f32": [ctypes.POINTER(Operand), ctypes.c_void_p, ctypes.c_void_p],
    "trs_unbroadcast_sum_f32": [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p,
                                ctypes.c_void_p],
    "trs_colsum_f32_noalloc": [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p],
    "trs_matmul_f32": [ctypes.POINTER(GemmDesc), ctypes.c_void_p],
    "trs_matmul_select_algo": [ctypes.POINTER(GemmDesc), ctypes.POINTER(ctypes.c_int32)],
    "trs_matmul_f32_planes": [ctypes.POINTER(GemmDesc), ctypes.POINTER(GemmPlanes), ctypes.c_void_p],
    "trs_matmul_plan": [ctypes.POINTER(GemmDesc), ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32),
                        ctypes.POINTER(ctypes.c_int32)],
    "trs_split_lo_f32": [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p],
    "trs_colsum_noalloc_geometry": [ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(ctypes.c_int32),
                                    ctypes.POINTER(ctypes.c_int64)],
    "trs_comm_unique_id": [ctypes.c_char_p],
    "trs_comm_init_rank": [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)],
    "trs_comm_allreduce_sum_f32": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p],
    "trs_comm_info": [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32),
                      ctypes.POINTER(ctypes.c_int32)],
    "trs_comm_destroy": [ctypes.c_void_p],
    "trs_debug_wait_probe": [ctypes.c_void_p, ctypes.c_int64],
    "trs_jit_cache_size": [ctypes.POINTER(ctypes.c_int32)],
}
_SPECIAL = {
    "trs_status_string": ([ctypes.c_int32], ctypes.c_char_p),
    "trs_last_error_message": ([], ctypes.c_char_p),
    "trs_kernel_launch_count": ([], ctypes.c_int64),
}
EXPORTS = sorted(list(_PROTOTYPES) + list(_SPECIAL))


def lib():
    """Load libtrs_cuda.so; raises (never falls back) when the built library is missing."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build` "
                              "(there is no CPU fallback)")
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


def check(status):
    if status != 0:
        raise TrsError(status, lib().trs_last_error_message().decode(errors="replace"))


def make_operand(base, offset, shape, strides):
    op = Operand()
    op.base = base
    op.offset = offset
    op.rank = len(shape)
    for i, (d, s) in enumerate(zip(shape, strides)):
        op.shape[i] = d
        op.stride[i] = s
    return op


def make_program(n_inputs, instrs, outputs):
    """instrs: list of (op_name, a, b, imm); outputs: list of value indices."""
    prog = Program()
    prog.n_inputs = n_inputs
    prog.n_instrs = len(instrs)
    prog.n_outputs = len(outputs)
    for i, (op, a, b, imm) in enumerate(instrs):
        prog.instrs[i].op = OPS[op] if isinstance(op, str) else op
        prog.instrs[i].a = a
        prog.instrs[i].b = b
        prog.instrs[i].imm = imm
    for i, v in enumerate(outputs):
        prog.outputs[i] = v
    return prog
