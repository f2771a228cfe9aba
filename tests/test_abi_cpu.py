"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, validates
arguments, plans and specialises kernels (NVRTC needs no GPU) and refuses to compute without a device."""
import ctypes
import os
import re

import numpy as np
import pytest

from torch_rs import _abi

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "trs_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"^(?:int32_t|int64_t|const char\*)\s+(trs_[a-z0-9_]+)\s*\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_abi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_abi.EXPORTS) == names


def fake_operand(addr, shape, strides, offset=0):
    return _abi.make_operand(addr, offset, shape, strides)


def prepare(instrs, outputs, inputs, outs):
    prog = _abi.make_program(len(inputs), instrs, outputs)
    ins = (_abi.Operand * max(len(inputs), 1))(*inputs)
    os_ = (_abi.Operand * len(outs))(*outs)
    klass = ctypes.create_string_buffer(16)
    status = _abi.lib().trs_pointwise_prepare(prog, ins, os_, klass)
    return status, klass.value.decode()


C2 = [("add", 0, 1, 0), ("relu", 2, 0, 0), ("const", 0, 0, 2.0), ("mul", 3, 4, 0), ("exp", 5, 0, 0), ("sub", 6, 0, 0)]


def test_planner_picks_streaming_kernel_for_the_transposed_broadcast_chain():
    n = 8192
    x = fake_operand(0x10000000, [n, n], [1, n])
    b = fake_operand(0x30000000, [n], [1])
    out = fake_operand(0x50000000, [n, n], [1, n])
    status, klass = prepare(C2, [7], [x, b], [out])
    assert status == 0 and klass == "vector"


def test_planner_picks_tiled_kernel_when_layouts_disagree():
    n = 512
    x = fake_operand(0x10000000, [n, n], [1, n])
    y = fake_operand(0x30000000, [n, n], [n, 1])
    out = fake_operand(0x50000000, [n, n], [n, 1])
    status, klass = prepare([("add", 0, 1, 0)], [2], [x, y], [out])
    assert status == 0 and klass == "tiled"


@pytest.mark.parametrize("shape,strides", [([7], [1]), ([3, 5], [5, 1]), ([3, 5], [1, 3]), ([2, 3, 4], [1, 2, 6]),
                                            ([4, 6], [12, 2]), ([], []), ([2, 0, 3], [3, 3, 1])])
def test_every_layout_class_specialises(shape, strides):
    x = fake_operand(0x10000004, shape, strides)
    out = fake_operand(0x50000000, shape, strides)
    status, klass = prepare([("relu", 0, 0, 0), ("exp", 1, 0, 0), ("relu_vjp", 0, 2, 0)], [3], [x], [out])
    assert status == 0, _abi.lib().trs_last_error_message()
    assert klass in ("vector", "tiled", "empty")


def test_bad_programs_are_rejected_with_messages():
    x = fake_operand(0x10000000, [4], [1])
    out = fake_operand(0x50000000, [4], [1])
    status, _ = prepare([("add", 0, 5, 0)], [1], [x], [out])
    assert status == 1 and b"not defined" in _abi.lib().trs_last_error_message()
    status, _ = prepare([(99, 0, 0, 0)], [1], [x], [out])
    assert status == 1
    bad = fake_operand(0x10000000, [3], [1])
    status, _ = prepare([("relu", 0, 0, 0)], [1], [bad], [out])
    assert status == 1 and b"broadcastable" in _abi.lib().trs_last_error_message()


def test_status_strings_and_launch_counter():
    lib = _abi.lib()
    assert lib.trs_status_string(0) == b"ok"
    assert lib.trs_status_string(2) == b"allocation failed"
    assert lib.trs_kernel_launch_count() >= 0


def test_compute_without_a_device_fails_loudly():
    n = ctypes.c_int32(-1)
    status = _abi.lib().trs_device_count(ctypes.byref(n))
    if status == 0 and n.value > 0:
        pytest.skip("a CUDA device is present")
    handle = ctypes.c_void_p()
    assert _abi.lib().trs_stream_create(0, ctypes.byref(handle)) != 0
    desc = _abi.GemmDesc()
    assert _abi.lib().trs_matmul_f32(ctypes.byref(desc), None) != 0


def test_huge_contiguous_extent_is_split_for_32_bit_indexing():
    n = 3 * (1 << 30)                      # 3 Gi elements (12 GiB) in one contiguous run
    x = fake_operand(0x100000000, [n], [1])
    out = fake_operand(0x800000000, [n], [1])
    status, klass = prepare([("relu", 0, 0, 0)], [1], [x], [out])
    assert status == 0 and klass == "vector", _abi.lib().trs_last_error_message()
