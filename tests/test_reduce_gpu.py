"""GPU parity of the deterministic reductions, fill and accumulate through the C ABI.

The reference adds sequentially; the device uses a fixed tree, so sums agree to a relative tolerance
of 1e-6 * sqrt(n) of the sum of magnitudes, and repeated runs agree bit for bit.
"""
import ctypes

import numpy as np
import pytest

from oracle import ref
from oracle.ref import RefTensor
from torch_rs import _abi
from torch_rs._device import DeviceBuffer, default_stream

pytestmark = pytest.mark.gpu


def device_sum(t: RefTensor):
    stream = default_stream()
    buf = DeviceBuffer.from_numpy(t.storage)
    out = DeviceBuffer(1)
    op = _abi.make_operand(buf.ptr, t.offset, t.shape, t.strides)
    _abi.check(_abi.lib().trs_reduce_sum_f32(ctypes.byref(op), out.ptr, stream.handle))
    return out.to_numpy()[0]


@pytest.mark.parametrize("shape", [(3,), (1000,), (257, 129), (1 << 20,), (33, 65, 17)])
def test_sum_matches_sequential_reference_within_tolerance(shape):
    t = RefTensor.from_numpy(np.random.default_rng(0).standard_normal(shape).astype(np.float32))
    got, expected = device_sum(t), t.sum()
    n = t.numel
    assert abs(got - expected) <= 1e-6 * np.sqrt(n) * float(np.abs(t.storage).sum()) + 1e-30
    assert device_sum(t) == got      # deterministic


def test_sum_goldens_and_views():
    assert device_sum(RefTensor([1.0, 2.0, 3.0], [3])) == 6.0
    view = RefTensor(np.arange(24, dtype=np.float32), [2, 3, 4]).transpose(0, 2)
    assert device_sum(view) == 276.0
    sliced = RefTensor(np.arange(40, dtype=np.float32), [4, 5], [10, 2])
    assert device_sum(sliced) == float(sliced.logical().sum())
    assert abs(device_sum(RefTensor([], [0]))) == 0.0


@pytest.mark.parametrize("rows,cols", [(1000, 4096), (8192, 4096), (7, 5), (300, 130), (1, 64)])
def test_unbroadcast_column_and_row_sums(rows, cols):
    x = np.random.default_rng(1).standard_normal((rows, cols)).astype(np.float32)
    stream = default_stream()
    buf = DeviceBuffer.from_numpy(x)
    col, row = DeviceBuffer(cols), DeviceBuffer(rows)
    _abi.check(_abi.lib().trs_unbroadcast_sum_f32(buf.ptr, rows, cols, 0, col.ptr, stream.handle))
    _abi.check(_abi.lib().trs_unbroadcast_sum_f32(buf.ptr, rows, cols, 1, row.ptr, stream.handle))
    got_col, got_row = col.to_numpy()[:cols], row.to_numpy()[:rows]
    # checker: GradientAccumulator order (src/tensor.rs:3204-3228)
    exp_col = ref.unbroadcast(x, [rows, cols], [cols])
    exp_row = ref.unbroadcast(x, [rows, cols], [rows, 1]).reshape(-1)
    mag = np.abs(x)
    assert np.all(np.abs(got_col - exp_col) <= 1e-6 * np.sqrt(rows) * mag.sum(axis=0) + 1e-30)
    assert np.all(np.abs(got_row - exp_row) <= 1e-6 * np.sqrt(cols) * mag.sum(axis=1) + 1e-30)


def test_fill_and_accumulate_bit_exact():
    stream = default_stream()
    n = 100003
    a = np.random.default_rng(2).standard_normal(n).astype(np.float32)
    b = np.random.default_rng(3).standard_normal(n).astype(np.float32)
    da, db = DeviceBuffer.from_numpy(a), DeviceBuffer.from_numpy(b)
    _abi.check(_abi.lib().trs_accumulate_f32(da.ptr, db.ptr, n, stream.handle))
    assert np.array_equal(da.to_numpy()[:n].view(np.uint32), (a + b).view(np.uint32))
    _abi.check(_abi.lib().trs_fill_f32(da.ptr + 4, n - 1, ctypes.c_float(-0.0), stream.handle))   # unaligned start
    got = da.to_numpy()[:n]
    assert got[0] == (a + b)[0] and np.all(got[1:].view(np.uint32) == 0x80000000)
