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


def test_allocation_free_column_sum_never_plans_more_partials_than_its_array_holds():
    """The fixed 1 MiB array bounds chunks * cols.  A 148-SM GPU never asks for more, so the bound is exercised with
    a larger made-up SM count (no device needed: this is host arithmetic)."""
    lib = _abi.lib()
    limit = 262144
    chunks, per = ctypes.c_int32(), ctypes.c_int64()
    for sms, rows, cols in [(148, 65536, 4096), (1024, 1 << 20, 4096), (4096, 1 << 22, 100000), (1024, 1 << 20, limit),
                            (1024, 3, 7), (148, 1, 1)]:
        assert lib.trs_colsum_noalloc_geometry(sms, rows, cols, ctypes.byref(chunks), ctypes.byref(per)) == 0
        assert 1 <= chunks.value and chunks.value * cols <= limit
        assert (chunks.value - 1) * per.value < rows <= chunks.value * per.value      # the chunks cover every row once
    assert lib.trs_colsum_noalloc_geometry(1024, 1 << 20, 4096, ctypes.byref(chunks), ctypes.byref(per)) == 0
    assert chunks.value == limit // 4096                                                 # the bound is what decided here
    assert lib.trs_colsum_noalloc_geometry(148, 8, limit + 1, ctypes.byref(chunks), ctypes.byref(per)) == 1


def gemm_desc(m, n, k, a_strides, b_strides, batch=1, algo="auto", a=0x10000000, b=0x30000000):
    d = _abi.GemmDesc()
    d.batch, d.m, d.n, d.k = batch, m, n, k
    d.a, d.b, d.c = a, b, 0x50000000
    d.a_batch_stride, d.a_row_stride, d.a_col_stride = m * k, a_strides[0], a_strides[1]
    d.b_batch_stride, d.b_row_stride, d.b_col_stride = k * n, b_strides[0], b_strides[1]
    d.c_batch_stride, d.c_row_stride = m * n, n
    d.algo = _abi.GEMM_ALGOS[algo]
    return d


def test_matmul_plan_tells_which_operand_images_would_be_read():
    lib = _abi.lib()

    def plan(d):
        algo, a, b = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        assert lib.trs_matmul_plan(ctypes.byref(d), ctypes.byref(algo), ctypes.byref(a), ctypes.byref(b)) == 0
        return algo.value, a.value, b.value

    # plain A @ B, 4096^3: the pair kernel reads A K-major and B MN-major, both in place
    assert plan(gemm_desc(4096, 4096, 4096, (4096, 1), (4096, 1))) == (3, 1, 1)
    # X[65536, 4096] @ W1: each element of W1 is reused 65,536 times, so it is re-laid K-major once per call
    assert plan(gemm_desc(65536, 4096, 4096, (4096, 1), (4096, 1))) == (3, 1, 0)
    # X^T @ dZ (weight gradient): both operands row-contiguous, read MN-major in place
    assert plan(gemm_desc(4096, 4096, 65536, (1, 4096), (4096, 1))) == (3, 1, 1)
    # W.mT per batch (config 4): K-major on both sides
    assert plan(gemm_desc(1024, 1024, 1024, (1024, 1), (1, 1024), batch=64)) == (3, 1, 1)
    # unaligned base: the operand is re-laid, an image of it would not be read
    assert plan(gemm_desc(512, 512, 512, (512, 1), (1, 512), a=0x10000004)) == (3, 0, 1)
    # tiny product: the FP32 kernel, no images
    assert plan(gemm_desc(8, 8, 8, (8, 1), (8, 1))) == (1, 0, 0)


def test_collective_and_stream_ordered_entry_points_check_their_arguments():
    lib = _abi.lib()
    assert lib.trs_comm_allreduce_sum_f32(None, None, 0, None) == 1
    assert b"comm is NULL" in lib.trs_last_error_message()
    comm = ctypes.c_void_p()
    assert lib.trs_comm_init_rank(0, 2, 2, b"\0" * 128, ctypes.byref(comm)) == 1
    assert b"outside a job of 2 ranks" in lib.trs_last_error_message()
    assert lib.trs_comm_init_rank(0, 2, 0, None, ctypes.byref(comm)) == 1
    assert lib.trs_comm_destroy(None) == 0
    assert lib.trs_comm_info(None, None, None, None) == 1
    p = ctypes.c_void_p()
    assert lib.trs_malloc_async(0, 1024, None, ctypes.byref(p)) == 1           # a stream is required
    assert lib.trs_free_async(0, None, None) == 1
    assert lib.trs_debug_wait_probe(None, 1000) == 1
    assert lib.trs_split_lo_f32(None, 4, None, None, None) == 1


def test_compiled_chains_can_be_kept_on_disk(tmp_path):
    """TRS_JIT_CACHE_DIR: a second process reads the compiled chain back instead of compiling it (no GPU needed)."""
    import subprocess
    import sys
    import time
    script = (
        "import ctypes, sys, time; sys.path.insert(0, %r); from torch_rs import _abi\n"
        "prog = _abi.make_program(1, [('sin', 0, 0, 0), ('exp', 1, 0, 0), ('relu', 2, 0, 0)], [3])\n"
        "ins = (_abi.Operand * 1)(_abi.make_operand(0x10000000, 0, [77, 33], [33, 1]))\n"
        "outs = (_abi.Operand * 1)(_abi.make_operand(0x50000000, 0, [77, 33], [33, 1]))\n"
        "k = ctypes.create_string_buffer(16)\n"
        "t = time.perf_counter(); s = _abi.lib().trs_pointwise_prepare(prog, ins, outs, k); print(s, (time.perf_counter() - t) * 1e3)\n"
    ) % os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "pytorch-rs_b200")
    env = dict(os.environ, TRS_JIT_CACHE_DIR=str(tmp_path))
    first = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=120)
    assert first.returncode == 0 and first.stdout.split()[0] == "0", first.stderr
    files = [f for f in os.listdir(tmp_path) if f.endswith(".cubin")]
    assert len(files) == 1
    second = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=120)
    assert second.returncode == 0 and second.stdout.split()[0] == "0", second.stderr
    assert float(second.stdout.split()[1]) < 0.5 * float(first.stdout.split()[1])      # no compilation the second time
    # a damaged file is ignored and replaced
    path = os.path.join(tmp_path, files[0])
    open(path, "r+b").write(b"garbage!")
    third = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=120)
    assert third.returncode == 0 and third.stdout.split()[0] == "0", third.stderr
    assert open(path, "rb").read(8) != b"garbage!"
