"""The allocation-free column sum (`trs_colsum_f32_noalloc`) against the regular entry point.

Hosts that cannot allocate device memory when they call in (stream capture in progress, driver
callbacks, fixed memory pools) use the variant whose partial sums live in a fixed array inside the
library.  It must give what `trs_unbroadcast_sum_f32` gives, call after call, although every call
reuses the same scratch.  This file sorts last on purpose: a failure here cannot hide other results.
"""
import ctypes

import numpy as np
import pytest

from torch_rs import _abi
from torch_rs._device import DeviceBuffer, default_stream

pytestmark = pytest.mark.gpu


def both(x):
    rows, cols = x.shape
    stream = default_stream()
    src = DeviceBuffer.from_numpy(x)
    regular, fixed = DeviceBuffer(cols), DeviceBuffer(cols)
    _abi.check(_abi.lib().trs_unbroadcast_sum_f32(src.ptr, rows, cols, 0, regular.ptr, stream.handle))
    _abi.check(_abi.lib().trs_colsum_f32_noalloc(src.ptr, rows, cols, fixed.ptr, stream.handle))
    return regular.to_numpy()[:cols], fixed.to_numpy()[:cols]


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    rng = np.random.default_rng(0)
    first = rng.standard_normal((4096, 1024)).astype(np.float32)
    second = (100.0 * rng.standard_normal((777, 130))).astype(np.float32)     # other shape, other magnitudes
    for x in (first, second, first):
        regular, fixed = both(x)
        # same chunking when the partials fit: the same additions in the same order
        assert np.array_equal(regular.view(np.uint32), fixed.view(np.uint32))


def test_unaligned_and_wide_shapes_stay_within_the_reduction_tolerance():
    rng = np.random.default_rng(1)
    for shape in ((513, 1001), (64, 200000), (3, 5)):          # scalar-load path, widest accepted class, tiny
        x = rng.standard_normal(shape).astype(np.float32)
        regular, fixed = both(x)
        bound = 1e-6 * np.sqrt(shape[0]) * np.abs(x).sum(axis=0) + 1e-30
        assert np.all(np.abs(regular - fixed) <= bound)
        assert np.all(np.abs(fixed - x.astype(np.float64).sum(axis=0)) <= bound)


def test_too_many_columns_is_refused_with_a_message():
    stream = default_stream()
    buf, out = DeviceBuffer(16), DeviceBuffer(16)
    status = _abi.lib().trs_colsum_f32_noalloc(buf.ptr, 1, 262145, out.ptr, stream.handle)
    assert status == 5
    assert b"exceed the fixed scratch" in _abi.lib().trs_last_error_message()
    empty = DeviceBuffer(8)
    _abi.check(_abi.lib().trs_colsum_f32_noalloc(buf.ptr, 0, 8, empty.ptr, stream.handle))
    assert np.all(empty.to_numpy()[:8] == 0.0)
