"""Helpers for the GPU parity tests: run a fused chain through the C ABI and through the CPU checker."""
import ctypes

import numpy as np

from oracle.ref import RefTensor
from torch_rs import _abi
from torch_rs._device import DeviceBuffer, default_stream


def run_pointwise(instrs, outputs, inputs, out_layouts, device=0):
    """inputs: RefTensors (host views); out_layouts: list of (shape, strides).  Returns output storages."""
    stream = default_stream(device)
    bufs = [DeviceBuffer.from_numpy(t.storage, device) for t in inputs]
    ins = (_abi.Operand * max(len(inputs), 1))()
    for i, (t, b) in enumerate(zip(inputs, bufs)):
        ins[i] = _abi.make_operand(b.ptr, t.offset, t.shape, t.strides)
    outs = (_abi.Operand * len(out_layouts))()
    out_bufs = []
    for i, (shape, strides) in enumerate(out_layouts):
        n = int(np.prod(shape)) if len(shape) else 1
        ob = DeviceBuffer(n, device)
        if n:
            _abi.check(_abi.lib().trs_fill_f32(ob.ptr, n, ctypes.c_float(np.nan), stream.handle))
        out_bufs.append(ob)
        outs[i] = _abi.make_operand(ob.ptr, 0, shape, strides)
    prog = _abi.make_program(len(inputs), instrs, outputs)
    _abi.check(_abi.lib().trs_pointwise(prog, ins, outs, stream.handle))
    stream.sync()
    return [ob.to_numpy()[: (int(np.prod(s)) if len(s) else 1)] for ob, (s, _) in zip(out_bufs, out_layouts)]


def assert_bits_equal(actual, expected, what=""):
    actual = np.ascontiguousarray(actual, dtype=np.float32).reshape(-1)
    expected = np.ascontiguousarray(expected, dtype=np.float32).reshape(-1)
    assert actual.shape == expected.shape, what
    ok = (actual.view(np.uint32) == expected.view(np.uint32)) | (np.isnan(actual) & np.isnan(expected))
    if not ok.all():
        bad = np.flatnonzero(~ok)[:5]
        raise AssertionError(f"{what}: {(~ok).sum()} of {ok.size} lanes differ; first {bad}: "
                             f"got {actual[bad]} expected {expected[bad]}")


def run_matmul(a: RefTensor, b: RefTensor, bias=None, epilogue="none", aux=None, want_preact=False, algo="auto",
               device=0):
    """a: [..., M, K] view, b: [..., K, N] view (rank 2 or 3, equal batch).  Returns (C, preact or None)."""
    stream = default_stream(device)
    batched = len(a.shape) == 3
    batch = a.shape[0] if batched else 1
    m, k = a.shape[-2], a.shape[-1]
    n = b.shape[-1]
    abuf, bbuf = DeviceBuffer.from_numpy(a.storage, device), DeviceBuffer.from_numpy(b.storage, device)
    cbuf = DeviceBuffer(batch * m * n, device)
    desc = _abi.GemmDesc()
    desc.batch, desc.m, desc.n, desc.k = batch, m, n, k
    desc.a = abuf.ptr + 4 * a.offset
    desc.a_batch_stride = a.strides[0] if batched else 0
    desc.a_row_stride, desc.a_col_stride = a.strides[-2], a.strides[-1]
    desc.b = bbuf.ptr + 4 * b.offset
    desc.b_batch_stride = b.strides[0] if batched else 0
    desc.b_row_stride, desc.b_col_stride = b.strides[-2], b.strides[-1]
    desc.c = cbuf.ptr
    desc.c_batch_stride, desc.c_row_stride = m * n, n
    keep = []
    if bias is not None:
        bb = DeviceBuffer.from_numpy(bias, device)
        keep.append(bb)
        desc.bias = bb.ptr
    if aux is not None:
        ab = DeviceBuffer.from_numpy(aux, device)
        keep.append(ab)
        desc.aux = ab.ptr
    pbuf = None
    if want_preact:
        pbuf = DeviceBuffer(batch * m * n, device)
        desc.preact = pbuf.ptr
    desc.epilogue = _abi.EPILOGUES[epilogue]
    desc.algo = _abi.GEMM_ALGOS[algo]
    _abi.check(_abi.lib().trs_matmul_f32(ctypes.byref(desc), stream.handle))
    stream.sync()
    shape = ([batch] if batched else []) + [m, n]
    c = cbuf.to_numpy()[: batch * m * n].reshape(shape)
    p = pbuf.to_numpy()[: batch * m * n].reshape(shape) if pbuf is not None else None
    return c, p


def matmul_tolerance_ok(got, ref64, k):
    """|dC| <= 1e-5 * sqrt(K) * max(|C_ref|, rms(C_ref)) element-wise (the path's stated matmul tolerance)."""
    ref64 = np.asarray(ref64, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref64 ** 2))) if ref64.size else 0.0
    bound = 1e-5 * np.sqrt(max(k, 1)) * np.maximum(np.abs(ref64), rms) + 1e-30
    err = np.abs(np.asarray(got, dtype=np.float64) - ref64)
    return bool((err <= bound).all()), float((err / bound).max()) if err.size else 0.0
