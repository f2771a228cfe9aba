"""The BASELINE configurations at their full sizes, through the `torch_rs` surface.

Pointwise configs are compared element for element with the CPU checker (it finishes in seconds).
The GEMM configs are too large for the single-threaded checker, so they are verified on sampled
rows computed by the checker in the reference's k-ascending order, against a float64 product for
the error bound, and through size-independent properties (linearity in the left operand, the
relu output being the exact reference relu of the pre-activation).
"""
import numpy as np
import pytest

import torch_rs as torch
from oracle import ref
from oracle.ref import RefTensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def within_matmul_tolerance(got, want64, k):
    want64 = np.asarray(want64, dtype=np.float64)
    rms = np.sqrt(np.mean(want64 ** 2))
    return np.all(np.abs(got - want64) <= 1e-5 * np.sqrt(k) * np.maximum(np.abs(want64), rms) + 1e-30)


def test_config1_relu_add_4096_bit_exact():
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    y = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    out = torch.relu(torch.tensor(x, device=DEV) + torch.tensor(y, device=DEV))
    want = (RefTensor.from_numpy(x) + RefTensor.from_numpy(y)).relu()
    assert list(out.stride()) == want.strides
    assert np.array_equal(out.numpy().view(np.uint32), want.logical().view(np.uint32))


def test_config2_transposed_broadcast_chain_8192_within_1_ulp():
    rng = np.random.default_rng(0)
    xs = rng.standard_normal((8192, 8192)).astype(np.float32)
    b = (0.1 * rng.standard_normal(8192)).astype(np.float32)
    x, bt = torch.tensor(xs, device=DEV), torch.tensor(b, device=DEV)
    e = torch.exp(2.0 * torch.relu(x.mT + bt))            # held: written by the same kernel as the result
    out = e - x.mT
    rx = RefTensor.from_numpy(xs)
    want_e = (2.0 * (rx.mT + RefTensor.from_numpy(b)).relu()).exp()
    want = want_e - rx.mT
    assert list(out.stride()) == want.strides == [1, 8192] and out.storage_offset() == 0
    got, got_e = out.mT.numpy(), e.mT.numpy()              # physical order, like the checker's storages
    # the path's stated tolerance on exp is 2 ulp from libm expf; the device exp keeps within 1, everywhere
    assert ref.ulp_distance(got_e, want_e.storage).max() <= 1
    # the subtraction is exact arithmetic on that value: wherever exp agrees bit for bit, so does the result,
    # and elsewhere the difference is the exp difference plus one rounding of the (smaller) result
    we, wr = want_e.storage.reshape(8192, 8192), want.storage.reshape(8192, 8192)
    same = got_e.view(np.uint32) == we.view(np.uint32)
    assert np.array_equal(got[same].view(np.uint32), wr[same].view(np.uint32))
    assert np.all(np.abs(got.astype(np.float64) - wr) <= np.spacing(np.abs(we)) + np.spacing(np.abs(wr)))
    # where relu clamps to zero the result is exactly 1 - x: those lanes must be bit-exact
    clamped = (xs + b[:, None]) <= 0
    assert np.array_equal(got[clamped].view(np.uint32), want.storage.reshape(8192, 8192)[clamped].view(np.uint32))


def test_config3_matmul_4096_sampled_rows_and_linearity():
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    b = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    A, B = torch.tensor(a, device=DEV), torch.tensor(b, device=DEV)
    c = torch.matmul(A, B).numpy()
    rows = rng.choice(4096, 48, replace=False)
    want32 = RefTensor.from_numpy(a[rows]).matmul(RefTensor.from_numpy(b)).logical()    # reference order, f32
    want64 = a[rows].astype(np.float64) @ b.astype(np.float64)
    assert within_matmul_tolerance(c[rows], want64, 4096)
    assert within_matmul_tolerance(c[rows], want32, 4096)
    # linearity: (2A) @ B == 2 (A @ B) exactly (scaling by 2 is exact in binary floating point)
    c2 = torch.matmul(A * 2.0, B).numpy()
    assert np.array_equal(c2.view(np.uint32), (2.0 * c).astype(np.float32).view(np.uint32))


def test_config4_batched_bias_relu_1024():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 1024, 1024)).astype(np.float32)
    w = (rng.standard_normal((64, 1024, 1024)) / 32).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, 1024).astype(np.float32)
    X, W, Bt = torch.tensor(x, device=DEV), torch.tensor(w, device=DEV), torch.tensor(bias, device=DEV)
    pre = X @ W.mT + Bt                       # held: becomes the pre-activation output of the same GEMM
    out = torch.relu(pre)
    got, got_pre = out.numpy(), pre.numpy()
    assert out.shape == (64, 1024, 1024) and out.is_contiguous()
    for i in (0, 31, 63):
        want64 = x[i].astype(np.float64) @ w[i].astype(np.float64).T + bias
        assert within_matmul_tolerance(got_pre[i], want64, 1024)
        rows = slice(100, 116)
        want32 = (RefTensor.from_numpy(x[i][rows]).matmul(RefTensor.from_numpy(w[i]).mT) + RefTensor(bias, [1024])).logical()
        assert within_matmul_tolerance(got_pre[i][rows], want32, 1024)
    # the activation is the exact reference relu of the pre-activation the kernel produced
    assert np.array_equal(got.view(np.uint32), RefTensor.from_numpy(got_pre).relu().logical().view(np.uint32))


def test_config5_mlp_step_one_eighth_batch():
    # 8,192 rows of X: the shard one GPU owns when the 65,536-row batch is split over 8 GPUs.
    rng = np.random.default_rng(0)
    bsz = 8192
    x = rng.standard_normal((bsz, 4096)).astype(np.float32)
    w1 = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    w2 = (rng.standard_normal((4096, 1024)) / 64).astype(np.float32)
    X = torch.tensor(x, device=DEV)
    W1, W2 = torch.tensor(w1, device=DEV, requires_grad=True), torch.tensor(w2, device=DEV, requires_grad=True)
    B1 = torch.zeros(4096, device=DEV, requires_grad=True)
    Z = X @ W1 + B1                                     # held: the pre-activation output of the first GEMM
    loss = (torch.relu(Z) @ W2).sum()
    loss.backward()
    z = x.astype(np.float64) @ w1.astype(np.float64)
    z_gpu = Z.numpy()
    assert within_matmul_tolerance(z_gpu, z, 4096)
    h = np.maximum(z, 0.0)
    dy = np.ones((bsz, 1024))
    dw2 = h.T @ dy
    # relu' is discontinuous at 0: elements of Z within rounding of 0 may fall on either side, so the
    # expected dZ uses the mask of the Z this run produced (the reference VJP is a function of the saved Z)
    dz = (dy @ w2.astype(np.float64).T) * (z_gpu > 0)
    assert within_matmul_tolerance(W2.grad.numpy(), dw2, bsz)
    assert within_matmul_tolerance(W1.grad.numpy(), x.astype(np.float64).T @ dz, bsz)
    assert within_matmul_tolerance(B1.grad.numpy(), dz.sum(axis=0), bsz)
    assert abs(loss.item() - (h @ w2.astype(np.float64)).sum()) <= 1e-4 * np.abs(h @ w2.astype(np.float64)).sum()


def test_config5_mlp_step_full_batch_on_one_gpu():
    """All 65,536 rows on one GPU (X 1 GiB, Z and H 1 GiB each; K = 65,536 in the weight-gradient products, where
    the 1e-5*sqrt(K) gate and the split's error are exercised).  A float64 product of the whole step would take
    minutes on the host, so 24 sampled hidden units are followed end to end instead: their column of Z, their
    column of dW1, their row of dW2 and their entry of db1 in float64, plus 16 rows of Z in the reference's own
    order, plus the loss from column sums."""
    rng = np.random.default_rng(0)
    bsz, d, h_dim, o = 65536, 4096, 4096, 1024
    x = rng.standard_normal((bsz, d), dtype=np.float32)
    w1 = (rng.standard_normal((d, h_dim)) / 64).astype(np.float32)
    w2 = (rng.standard_normal((h_dim, o)) / 64).astype(np.float32)
    X = torch.tensor(x, device=DEV)
    W1, W2 = torch.tensor(w1, device=DEV, requires_grad=True), torch.tensor(w2, device=DEV, requires_grad=True)
    B1 = torch.zeros(h_dim, device=DEV, requires_grad=True)
    Z = X @ W1 + B1                                     # held: the pre-activation output of the first GEMM
    loss = (torch.relu(Z) @ W2).sum()
    loss.backward()
    z_gpu = Z.numpy()
    units = np.sort(rng.choice(h_dim, 24, replace=False))
    chunks = [slice(i, i + 8192) for i in range(0, bsz, 8192)]
    w1u = w1[:, units].astype(np.float64)
    z64 = np.concatenate([x[c].astype(np.float64) @ w1u for c in chunks])
    assert within_matmul_tolerance(z_gpu[:, units], z64, d)
    rows = rng.choice(bsz, 16, replace=False)
    want32 = RefTensor.from_numpy(x[rows]).matmul(RefTensor.from_numpy(w1)).logical()      # reference k order, f32
    assert within_matmul_tolerance(z_gpu[rows], want32, d)
    # relu' is discontinuous at 0, so the expected dZ uses the sign of the Z this run produced (the reference VJP
    # is a function of the saved Z, src/tensor.rs:4422-4432); dY is all ones, so dH[r, c] = sum_o W2[c, o]
    dh = w2.astype(np.float64).sum(axis=1)
    dz = (z_gpu[:, units] > 0) * dh[units]
    dw1_units = sum(x[c].astype(np.float64).T @ dz[c] for c in chunks)
    assert within_matmul_tolerance(W1.grad.numpy()[:, units], dw1_units, bsz)
    assert within_matmul_tolerance(B1.grad.numpy()[units], dz.sum(axis=0), bsz)
    h_colsum = np.maximum(z_gpu, 0).sum(axis=0, dtype=np.float64)
    dw2_units = np.repeat(h_colsum[units][:, None], o, axis=1)
    assert within_matmul_tolerance(W2.grad.numpy()[units], dw2_units, bsz)
    assert abs(loss.item() - h_colsum @ dh) <= 1e-4 * (h_colsum @ np.abs(dh))
    # the weights were each read by two products and X by two: one image each, made once
    assert X._has_operand_image() and W2._has_operand_image()
