"""GPU parity of float32 matmul / bmm (+ fused epilogues) through the C ABI against the CPU checker.

Tolerance: |dC| <= 1e-5 * sqrt(K) * max(|C|, rms(C)); the reference's sequential k order
(src/tensor.rs:3945) cannot be bit-matched by a parallel GEMM.  Small exact-integer goldens from the
reference's tests must still come out exactly.
"""
import json
import os

import numpy as np
import pytest

from oracle.ref import RefTensor
from tests.abi_harness import matmul_tolerance_ok, run_matmul
from tests.test_oracle_golden import build_operand

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))
ALGOS = ["simt_fp32", "auto"]


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


@pytest.mark.parametrize("algo", ALGOS)
def test_reference_goldens_exact(algo):
    for case in GOLD["matmul"]["cases"]:
        a, b = build_operand(case["left"]), build_operand(case["right"])
        c, _ = run_matmul(a, b, algo=algo)
        assert c.reshape(-1).tolist() == case["expected"], case["source"]


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (130, 70, 33), (1, 1, 1), (5, 1024, 64), (512, 512, 1024)])
def test_contiguous_matches_checker(algo, m, n, k):
    a, b = RefTensor.from_numpy(rnd(0, m, k)), RefTensor.from_numpy(rnd(1, k, n, scale=1 / np.sqrt(k)))
    expected = a.matmul(b).logical()
    c, _ = run_matmul(a, b, algo=algo)
    ok, worst = matmul_tolerance_ok(c, expected, k)
    assert ok, f"worst error/bound {worst}"


@pytest.mark.parametrize("algo", ALGOS)
def test_transposed_and_offset_views(algo):
    m, n, k = 192, 160, 256
    at = RefTensor.from_numpy(rnd(2, k, m)).mT                  # A read through .mT (m contiguous)
    bt = RefTensor.from_numpy(rnd(3, 2, n, k)).select0(1).mT    # offset + transposed B (k contiguous)
    expected = at.matmul(bt).logical()
    c, _ = run_matmul(at, bt, algo=algo)
    ok, worst = matmul_tolerance_ok(c, expected, k)
    assert ok, worst


@pytest.mark.parametrize("algo", ALGOS)
def test_batched_bias_relu_epilogue_matches_composition(algo):
    # relu(X @ W.mT + bias) per batch == the reference primitives composed: matmul -> add(bias) -> relu.
    batch, m, n, k = 3, 128, 256, 128
    x = RefTensor.from_numpy(rnd(4, batch, m, k))
    w = RefTensor.from_numpy(rnd(5, batch, n, k, scale=1 / 32))
    bias = np.random.default_rng(6).uniform(-0.1, 0.1, n).astype(np.float32)
    c, pre = run_matmul(x, w.mT, bias=bias, epilogue="bias_relu", want_preact=True, algo=algo)
    for i in range(batch):
        z = x.select0(i).matmul(w.select0(i).mT) + RefTensor(bias, [n])
        ok, worst = matmul_tolerance_ok(pre[i], z.logical(), k)
        assert ok, worst
        # the activation is the exact reference relu of the pre-activation this kernel produced
        expect_act = RefTensor.from_numpy(pre[i]).relu().logical()
        assert np.array_equal(c[i].view(np.uint32), expect_act.view(np.uint32))


@pytest.mark.parametrize("algo", ALGOS)
def test_relu_vjp_epilogue(algo):
    m, n, k = 256, 128, 64
    dy, w2 = RefTensor.from_numpy(rnd(7, m, k)), RefTensor.from_numpy(rnd(8, n, k))
    z = rnd(9, m, n)
    c, _ = run_matmul(dy, w2.mT, epilogue="relu_vjp", aux=z, algo=algo)
    dh = dy.matmul(w2.mT).logical()
    mask = (z > 0) | np.isnan(z)
    ok, worst = matmul_tolerance_ok(c, np.where(mask, dh, 0.0), k)
    assert ok, worst
    assert np.all(c[~mask] == 0.0)


def test_empty_and_zero_inner():
    a, b = RefTensor(np.zeros(0, dtype=np.float32), [4, 0]), RefTensor(np.zeros(0, dtype=np.float32), [0, 3])
    c, _ = run_matmul(a, b)
    assert c.shape == (4, 3) and np.all(c == 0.0)
