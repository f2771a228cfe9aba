"""Prepared operand images of the tensor-core matmul (trs_gemm_planes), the stream-ordered block cache and the
bounded-wait report, through the C ABI and through the host engine that caches images per storage.

The images only move work (the lo part of the 3xTF32 split is computed once instead of per call): every result
here must be BIT-IDENTICAL to the same call without images.
"""
import ctypes

import numpy as np
import pytest

from oracle.ref import RefTensor
from tests.abi_harness import matmul_tolerance_ok
from torch_rs import _abi
from torch_rs._device import DeviceBuffer, Stream, default_stream

pytestmark = pytest.mark.gpu


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def lo_image(values):
    """tf32(a - trunc_tf32(a)) with round-to-nearest, ties away from zero (cvt.rna.tf32.f32); 0 for inf / NaN."""
    a = np.ascontiguousarray(values, dtype=np.float32)
    bits = a.view(np.uint32)
    hi = (bits & np.uint32(0xFFFFE000)).view(np.float32)
    finite = np.isfinite(a)
    rest = np.where(finite, a - np.where(finite, hi, 0), 0).astype(np.float32)
    lo_bits = (rest.view(np.uint32) + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return lo_bits.view(np.float32)


def split_on_device(buf, count, stream):
    lo = DeviceBuffer(count + 8)
    flag_ptr = lo.ptr + 4 * ((count + 3) // 4 * 4)          # the word behind the image
    _abi.check(_abi.lib().trs_split_lo_f32(buf.ptr, count, lo.ptr, flag_ptr, stream.handle))
    return lo, flag_ptr


def read_word(ptr, stream):
    out = np.zeros(1, dtype=np.uint32)
    _abi.check(_abi.lib().trs_memcpy_d2h(out.ctypes.data, ptr, 4, stream.handle))
    stream.sync()
    return int(out[0])


def test_split_lo_matches_the_definition_and_flags_nonfinite():
    stream = default_stream(0)
    a = rnd(0, 1 << 16)
    a[:8] = [0.0, -0.0, 1.0, -1.5, 3.0e38, -3.0e38, 1.0000001, 65504.125]
    buf = DeviceBuffer.from_numpy(a)
    lo, flag = split_on_device(buf, a.size, stream)
    got = lo.to_numpy()[: a.size]
    assert np.array_equal(got.view(np.uint32), lo_image(a).view(np.uint32))
    assert read_word(flag, stream) == 0
    a[100], a[2000] = np.inf, np.nan
    buf = DeviceBuffer.from_numpy(a)
    lo, flag = split_on_device(buf, a.size, stream)
    got = lo.to_numpy()[: a.size]
    assert got[100] == 0.0 and got[2000] == 0.0
    assert read_word(flag, stream) == 1
    # an odd, unaligned range takes the scalar path
    lo2 = DeviceBuffer(1001 + 8)
    _abi.check(_abi.lib().trs_split_lo_f32(buf.ptr + 4, 1001, lo2.ptr + 4, lo2.ptr + 4 * 1004, stream.handle))
    assert np.array_equal(lo2.to_numpy()[1:1002].view(np.uint32), lo_image(a[1:1002]).view(np.uint32))


def make_desc(a, b, abuf, bbuf, cbuf, algo, epilogue="none"):
    batched = len(a.shape) == 3
    desc = _abi.GemmDesc()
    desc.batch = a.shape[0] if batched else 1
    desc.m, desc.k, desc.n = a.shape[-2], a.shape[-1], b.shape[-1]
    desc.a = abuf.ptr + 4 * a.offset
    desc.a_batch_stride = a.strides[0] if batched else 0
    desc.a_row_stride, desc.a_col_stride = a.strides[-2], a.strides[-1]
    desc.b = bbuf.ptr + 4 * b.offset
    desc.b_batch_stride = b.strides[0] if batched else 0
    desc.b_row_stride, desc.b_col_stride = b.strides[-2], b.strides[-1]
    desc.c = cbuf.ptr
    desc.c_batch_stride, desc.c_row_stride = desc.m * desc.n, desc.n
    desc.epilogue = _abi.EPILOGUES[epilogue]
    desc.algo = _abi.GEMM_ALGOS[algo]
    return desc


CASES = [
    # name, A view builder, B view builder, algo, expect (a_used, b_used)
    ("kmajor_both_pair", lambda: RefTensor.from_numpy(rnd(1, 512, 1024)), lambda: RefTensor.from_numpy(rnd(2, 384, 1024, scale=1 / 32)).mT,
     "tcgen05_3xtf32_2cta", (1, 1)),
    ("kmajor_both_one_cta", lambda: RefTensor.from_numpy(rnd(3, 256, 520)), lambda: RefTensor.from_numpy(rnd(4, 256, 520, scale=1 / 32)).mT,
     "tcgen05_3xtf32", (1, 1)),
    ("plain_a_at_b_pair", lambda: RefTensor.from_numpy(rnd(5, 512, 256)), lambda: RefTensor.from_numpy(rnd(6, 256, 512, scale=1 / 16)),
     "tcgen05_3xtf32_2cta", (1, 1)),                      # B row-contiguous: read MN-major in place
    ("transposed_a_pair", lambda: RefTensor.from_numpy(rnd(7, 1024, 512)).mT, lambda: RefTensor.from_numpy(rnd(8, 1024, 256, scale=1 / 32)),
     "tcgen05_3xtf32_2cta", (1, 1)),                      # the weight-gradient shape X^T @ dZ
    ("batched_kmajor_pair", lambda: RefTensor.from_numpy(rnd(9, 3, 256, 256)), lambda: RefTensor.from_numpy(rnd(10, 3, 256, 256, scale=1 / 16)).mT,
     "tcgen05_3xtf32_2cta", (1, 1)),
    ("plain_b_one_cta_is_relaid", lambda: RefTensor.from_numpy(rnd(11, 256, 256)), lambda: RefTensor.from_numpy(rnd(12, 256, 256, scale=1 / 16)),
     "tcgen05_3xtf32", (1, 0)),
]


@pytest.mark.parametrize("name,make_a,make_b,algo,expect", CASES, ids=[c[0] for c in CASES])
def test_given_images_give_identical_bits(name, make_a, make_b, algo, expect):
    stream = default_stream(0)
    a, b = make_a(), make_b()
    abuf, bbuf = DeviceBuffer.from_numpy(a.storage), DeviceBuffer.from_numpy(b.storage)
    batch = a.shape[0] if len(a.shape) == 3 else 1
    numel = batch * a.shape[-2] * b.shape[-1]
    c0, c1 = DeviceBuffer(numel), DeviceBuffer(numel)
    desc = make_desc(a, b, abuf, bbuf, c0, algo)
    algo_out, au, bu = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    _abi.check(_abi.lib().trs_matmul_plan(ctypes.byref(desc), ctypes.byref(algo_out), ctypes.byref(au), ctypes.byref(bu)))
    assert (au.value, bu.value) == expect
    _abi.check(_abi.lib().trs_matmul_f32(ctypes.byref(desc), stream.handle))
    a_lo, a_flag = split_on_device(abuf, a.storage.size, stream)
    b_lo, b_flag = split_on_device(bbuf, b.storage.size, stream)
    planes = _abi.GemmPlanes()
    planes.a_lo, planes.a_flag = a_lo.ptr + 4 * a.offset, a_flag
    planes.b_lo, planes.b_flag = b_lo.ptr + 4 * b.offset, b_flag
    desc.c = c1.ptr
    launches = _abi.lib().trs_kernel_launch_count()
    _abi.check(_abi.lib().trs_matmul_f32_planes(ctypes.byref(desc), ctypes.byref(planes), stream.handle))
    # one launch less per operand whose image was taken (split + GEMM + gated recompute otherwise)
    assert _abi.lib().trs_kernel_launch_count() - launches == 4 - au.value - bu.value
    stream.sync()
    got0, got1 = c0.to_numpy()[:numel], c1.to_numpy()[:numel]
    assert np.array_equal(got0.view(np.uint32), got1.view(np.uint32))
    ok, worst = matmul_tolerance_ok(got1.reshape(-1), a.matmul(b).logical().reshape(-1) if batch == 1 else
                                    np.stack([a.select0(i).matmul(b.select0(i)).logical() for i in range(batch)]).reshape(-1), a.shape[-1])
    assert ok, worst


@pytest.mark.parametrize("algo", ["tcgen05_3xtf32", "tcgen05_3xtf32_2cta", "simt_fp32"])
def test_epilogue_writes_the_image_of_its_result(algo):
    stream = default_stream(0)
    m, n, k = 512, 384, 256
    a, b = RefTensor.from_numpy(rnd(20, m, k)), RefTensor.from_numpy(rnd(21, n, k, scale=1 / 16)).mT
    bias = rnd(22, n)
    abuf, bbuf, biasbuf = DeviceBuffer.from_numpy(a.storage), DeviceBuffer.from_numpy(b.storage), DeviceBuffer.from_numpy(bias)
    c, c_lo = DeviceBuffer(m * n), DeviceBuffer(m * n + 4)
    desc = make_desc(a, b, abuf, bbuf, c, algo, "bias_relu")
    desc.bias = biasbuf.ptr
    planes = _abi.GemmPlanes()
    planes.c_lo, planes.c_flag = c_lo.ptr, c_lo.ptr + 4 * m * n
    _abi.check(_abi.lib().trs_fill_f32(planes.c_flag, 1, ctypes.c_float(0.0), stream.handle))
    _abi.check(_abi.lib().trs_matmul_f32_planes(ctypes.byref(desc), ctypes.byref(planes), stream.handle))
    stream.sync()
    got = c.to_numpy()[: m * n]
    assert np.array_equal(c_lo.to_numpy()[: m * n].view(np.uint32), lo_image(got).view(np.uint32))
    assert read_word(planes.c_flag, stream) == 0
    # c_lo without c_flag is refused before anything runs
    planes.c_flag = None
    assert _abi.lib().trs_matmul_f32_planes(ctypes.byref(desc), ctypes.byref(planes), stream.handle) == 1


@pytest.mark.parametrize("algo", ["tcgen05_3xtf32", "tcgen05_3xtf32_2cta"])
def test_flag_of_a_given_image_triggers_the_exact_recompute(algo):
    stream = default_stream(0)
    m, n, k = 256, 256, 256
    av = rnd(30, m, k)
    av[3, 7], av[100, 9] = np.inf, np.nan
    a, b = RefTensor.from_numpy(av), RefTensor.from_numpy(rnd(31, n, k, scale=1 / 16)).mT
    abuf, bbuf = DeviceBuffer.from_numpy(a.storage), DeviceBuffer.from_numpy(b.storage)
    c_ref, c_tc, c_lo = DeviceBuffer(m * n), DeviceBuffer(m * n), DeviceBuffer(m * n + 4)
    desc = make_desc(a, b, abuf, bbuf, c_ref, "simt_fp32")
    _abi.check(_abi.lib().trs_matmul_f32(ctypes.byref(desc), stream.handle))
    a_lo, a_flag = split_on_device(abuf, av.size, stream)
    b_lo, b_flag = split_on_device(bbuf, b.storage.size, stream)
    assert read_word(a_flag, stream) == 1 and read_word(b_flag, stream) == 0
    desc = make_desc(a, b, abuf, bbuf, c_tc, algo)
    planes = _abi.GemmPlanes()
    planes.a_lo, planes.a_flag, planes.b_lo, planes.b_flag = a_lo.ptr, a_flag, b_lo.ptr, b_flag
    planes.c_lo, planes.c_flag = c_lo.ptr, c_lo.ptr + 4 * m * n
    _abi.check(_abi.lib().trs_fill_f32(planes.c_flag, 1, ctypes.c_float(0.0), stream.handle))
    _abi.check(_abi.lib().trs_matmul_f32_planes(ctypes.byref(desc), ctypes.byref(planes), stream.handle))
    stream.sync()
    want, got = c_ref.to_numpy()[: m * n], c_tc.to_numpy()[: m * n]
    assert np.array_equal(want.view(np.uint32), got.view(np.uint32))      # the recompute IS the exact-FP32 kernel
    assert np.isnan(got.reshape(m, n)[100]).all() and np.isinf(got.reshape(m, n)[3]).any()
    assert read_word(planes.c_flag, stream) == 1                            # and the result's image carries the mark on


def test_engine_caches_images_per_storage_and_results_do_not_change():
    import torch_rs as torch
    dev = "cuda:0"
    x, w = rnd(40, 512, 768), rnd(41, 768, 512, scale=1 / 32)
    torch.set_operand_image_cache(False)
    try:
        X, W = torch.tensor(x, device=dev), torch.tensor(w, device=dev)
        plain = (X @ W).numpy()
        assert not X._has_operand_image() and not W._has_operand_image()
    finally:
        torch.set_operand_image_cache(True)
    X, W = torch.tensor(x, device=dev), torch.tensor(w, device=dev)
    first = (X @ W).numpy()
    assert X._has_operand_image() and W._has_operand_image()
    launches = _abi.lib().trs_kernel_launch_count()
    second = (X @ W).numpy()
    # GEMM + gated recompute only (reading back a contiguous result launches nothing): no preparation pass
    assert _abi.lib().trs_kernel_launch_count() - launches == 2
    assert np.array_equal(plain.view(np.uint32), first.view(np.uint32))
    assert np.array_equal(plain.view(np.uint32), second.view(np.uint32))
    # the image serves the storage through a transposed view too (the backward products read X^T)
    launches = _abi.lib().trs_kernel_launch_count()
    g = rnd(42, 512, 512)
    G = torch.tensor(g, device=dev)
    (X.mT @ G).materialize()
    assert _abi.lib().trs_kernel_launch_count() - launches == 3          # G's image + GEMM + gated recompute


def test_image_is_not_reused_for_a_new_storage_at_the_same_address():
    import torch_rs as torch
    dev = "cuda:0"
    w = rnd(50, 384, 256, scale=1 / 16)
    W = torch.tensor(w, device=dev)
    x1 = rnd(51, 256, 384)
    X1 = torch.tensor(x1, device=dev)
    (X1 @ W).materialize()
    assert X1._has_operand_image()
    address = X1._const_data_ptr()
    torch.synchronize(0)
    del X1
    x2 = rnd(52, 256, 384) * 3.0
    X2 = torch.tensor(x2, device=dev)
    if X2._const_data_ptr() != address:
        pytest.skip("the cache handed out another block")
    assert not X2._has_operand_image()
    got = (X2 @ W).numpy()
    want = RefTensor.from_numpy(x2).matmul(RefTensor.from_numpy(w)).logical()
    ok, worst = matmul_tolerance_ok(got, want, 384)
    assert ok, worst
    stale = RefTensor.from_numpy(x1).matmul(RefTensor.from_numpy(w)).logical()
    assert not matmul_tolerance_ok(got, stale, 384)[0]


def test_mlp_step_prepares_each_operand_once():
    """relu(X @ W1 + b1) @ W2 forward + backward: H and dZ get their images from the epilogues that store them, X, W2
    and dY are split once although each is read by two products."""
    import torch_rs as torch
    dev = "cuda:0"
    rng = np.random.default_rng(60)
    xs = rng.standard_normal((1024, 512)).astype(np.float32)
    w1 = (rng.standard_normal((512, 768)) / 16).astype(np.float32)
    w2 = (rng.standard_normal((768, 256)) / 16).astype(np.float32)
    b1 = (0.1 * rng.standard_normal(768)).astype(np.float32)

    def step(cache):
        torch.set_operand_image_cache(cache)
        try:
            X = torch.tensor(xs, device=dev)
            W1, W2 = torch.tensor(w1, device=dev, requires_grad=True), torch.tensor(w2, device=dev, requires_grad=True)
            B1 = torch.tensor(b1, device=dev, requires_grad=True)
            before = _abi.lib().trs_kernel_launch_count()
            loss = (torch.relu(X @ W1 + B1) @ W2).sum()
            loss.backward()
            torch.synchronize(0)
            launches = _abi.lib().trs_kernel_launch_count() - before
            return loss.item(), [p.grad.numpy() for p in (W1, W2, B1)], launches
        finally:
            torch.set_operand_image_cache(True)

    loss0, grads0, launches0 = step(False)
    loss1, grads1, launches1 = step(True)
    assert loss0 == loss1
    for g0, g1 in zip(grads0, grads1):
        assert np.array_equal(g0.view(np.uint32), g1.view(np.uint32))
    assert launches1 < launches0


def test_scratch_is_not_shared_between_streams_in_flight():
    """Two streams of one device run tensor-core products (which take scratch from the block cache and hand it back
    at once) and sums back to back without any host synchronisation; each must see only its own scratch."""
    s0, s1 = Stream(0), Stream(0)
    m = n = k = 256
    sets = []
    for i, stream in enumerate((s0, s1)):
        # a column-major A and a row-major B are both re-laid into hi and lo planes by the one-CTA kernel: the largest scratch use
        a = RefTensor.from_numpy(rnd(70 + i, k, m)).mT
        bt = RefTensor.from_numpy(rnd(80 + i, k, n, scale=1 / 16))
        abuf, bbuf, cbuf = DeviceBuffer.from_numpy(a.storage), DeviceBuffer.from_numpy(bt.storage), DeviceBuffer(m * n)
        sets.append((a, bt, abuf, bbuf, cbuf, DeviceBuffer(1), stream))
    wants = []
    for a, b, abuf, bbuf, cbuf, sbuf, stream in sets:
        desc = make_desc(a, b, abuf, bbuf, cbuf, "tcgen05_3xtf32")
        _abi.check(_abi.lib().trs_matmul_f32(ctypes.byref(desc), stream.handle))
        stream.sync()
        wants.append(cbuf.to_numpy(stream)[: m * n].copy())
    for _ in range(20):
        for a, b, abuf, bbuf, cbuf, sbuf, stream in sets:
            desc = make_desc(a, b, abuf, bbuf, cbuf, "tcgen05_3xtf32")
            _abi.check(_abi.lib().trs_matmul_f32(ctypes.byref(desc), stream.handle))
            op = _abi.make_operand(cbuf.ptr, 0, [m, n], [n, 1])
            _abi.check(_abi.lib().trs_reduce_sum_f32(ctypes.byref(op), sbuf.ptr, stream.handle))
    for (a, b, abuf, bbuf, cbuf, sbuf, stream), want in zip(sets, wants):
        stream.sync()
        got = cbuf.to_numpy(stream)[: m * n]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        total = sbuf.to_numpy(stream)[0]
        assert abs(total - want.astype(np.float64).sum()) <= 1e-6 * np.sqrt(m * n) * np.abs(want).sum()


def test_stream_ordered_blocks_cross_streams_safely():
    lib = _abi.lib()
    s0, s1 = Stream(0), Stream(0)
    p = ctypes.c_void_p()
    _abi.check(lib.trs_malloc_async(0, 1 << 20, s0.handle, ctypes.byref(p)))
    _abi.check(lib.trs_fill_f32(p, 1 << 18, ctypes.c_float(3.0), s0.handle))
    first = p.value
    _abi.check(lib.trs_free_async(0, p, s0.handle))
    q = ctypes.c_void_p()
    _abi.check(lib.trs_malloc_async(0, 1 << 20, s1.handle, ctypes.byref(q)))      # may be the same block: s1 now waits for s0's fill
    _abi.check(lib.trs_fill_f32(q, 1 << 18, ctypes.c_float(5.0), s1.handle))
    out = np.zeros(1 << 18, dtype=np.float32)
    _abi.check(lib.trs_memcpy_d2h(out.ctypes.data, q, out.nbytes, s1.handle))
    s1.sync()
    assert (out == 5.0).all()
    assert lib.trs_free_async(0, q, s0.handle) == 0
    assert lib.trs_free_async(0, ctypes.c_void_p(first + 64), s0.handle) == 1      # not a block of the cache
    s0.sync()


def test_a_bounded_wait_that_runs_out_is_reported_once_and_the_device_stays_usable():
    lib = _abi.lib()
    stream = default_stream(0)
    stream.sync()
    _abi.check(lib.trs_debug_wait_probe(stream.handle, 20000))       # nothing ever arrives on the probe's barrier
    status = lib.trs_stream_sync(stream.handle)
    assert status == 7, lib.trs_last_error_message()
    assert b"bounded wait" in lib.trs_last_error_message()
    assert lib.trs_stream_sync(stream.handle) == 0                    # reported once, then clear
    assert lib.trs_debug_wait_probe(stream.handle, 10 ** 9) == 1      # absurd limits are refused
    a, b = RefTensor.from_numpy(rnd(90, 256, 256)), RefTensor.from_numpy(rnd(91, 256, 256, scale=1 / 16))
    from tests.abi_harness import run_matmul
    c, _ = run_matmul(a, b, algo="tcgen05_3xtf32_2cta")
    ok, worst = matmul_tolerance_ok(c, a.matmul(b).logical(), 256)
    assert ok, worst
