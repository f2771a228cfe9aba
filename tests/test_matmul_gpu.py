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
ALGOS = ["simt_fp32", "tcgen05_3xtf32", "tcgen05_3xtf32_2cta", "auto"]
TC_ALGOS = ["tcgen05_3xtf32", "tcgen05_3xtf32_2cta"]


def run(a, b, algo, **kw):
    """run_matmul, skipping shapes the requested algorithm does not take."""
    from torch_rs._abi import TrsError
    try:
        return run_matmul(a, b, algo=algo, **kw)
    except TrsError as err:
        if err.status == 5:
            pytest.skip("shape not eligible for " + algo)
        raise


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


@pytest.mark.parametrize("algo", ALGOS)
def test_reference_goldens_exact(algo):
    for case in GOLD["matmul"]["cases"]:
        a, b = build_operand(case["left"]), build_operand(case["right"])
        c, _ = run(a, b, algo)
        assert c.reshape(-1).tolist() == case["expected"], case["source"]


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (130, 70, 33), (1, 1, 1), (5, 1024, 64), (512, 512, 1024)])
def test_contiguous_matches_checker(algo, m, n, k):
    a, b = RefTensor.from_numpy(rnd(0, m, k)), RefTensor.from_numpy(rnd(1, k, n, scale=1 / np.sqrt(k)))
    expected = a.matmul(b).logical()
    c, _ = run(a, b, algo)
    ok, worst = matmul_tolerance_ok(c, expected, k)
    assert ok, f"worst error/bound {worst}"


@pytest.mark.parametrize("algo", ALGOS)
def test_transposed_and_offset_views(algo):
    m, n, k = 192, 160, 256
    at = RefTensor.from_numpy(rnd(2, k, m)).mT                  # A read through .mT (m contiguous)
    bt = RefTensor.from_numpy(rnd(3, 2, n, k)).select0(1).mT    # offset + transposed B (k contiguous)
    expected = at.matmul(bt).logical()
    c, _ = run(at, bt, algo)
    ok, worst = matmul_tolerance_ok(c, expected, k)
    assert ok, worst


@pytest.mark.parametrize("algo", ALGOS)
def test_batched_bias_relu_epilogue_matches_composition(algo):
    # relu(X @ W.mT + bias) per batch == the reference primitives composed: matmul -> add(bias) -> relu.
    batch, m, n, k = 3, 128, 256, 128
    x = RefTensor.from_numpy(rnd(4, batch, m, k))
    w = RefTensor.from_numpy(rnd(5, batch, n, k, scale=1 / 32))
    bias = np.random.default_rng(6).uniform(-0.1, 0.1, n).astype(np.float32)
    c, pre = run(x, w.mT, algo, bias=bias, epilogue="bias_relu", want_preact=True)
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
    c, _ = run(dy, w2.mT, algo, epilogue="relu_vjp", aux=z)
    dh = dy.matmul(w2.mT).logical()
    mask = (z > 0) | np.isnan(z)
    ok, worst = matmul_tolerance_ok(c, np.where(mask, dh, 0.0), k)
    assert ok, worst
    assert np.all(c[~mask] == 0.0)


def test_empty_and_zero_inner():
    a, b = RefTensor(np.zeros(0, dtype=np.float32), [4, 0]), RefTensor(np.zeros(0, dtype=np.float32), [0, 3])
    c, _ = run_matmul(a, b)
    assert c.shape == (4, 3) and np.all(c == 0.0)


@pytest.mark.parametrize("m,n,k", [(128, 256, 32), (129, 257, 40), (300, 520, 100), (1024, 768, 2048), (64, 64, 4096),
                                   (1664, 3072, 256), (1700, 3000, 264),    # 156 tiles on 148 SMs: the split-K tail
                                   (2560, 2304, 256), (385, 300, 72)])      # 90 tile pairs on 74 SM pairs; a peer CTA wholly past M
@pytest.mark.parametrize("algo", TC_ALGOS)
def test_tensor_core_path_odd_shapes_and_k_tails(algo, m, n, k):
    a, b = RefTensor.from_numpy(rnd(20, m, k)), RefTensor.from_numpy(rnd(21, k, n, scale=1 / np.sqrt(k)))
    c, _ = run(a, b, algo)
    ok, worst = matmul_tolerance_ok(c, a.matmul(b).logical(), k)
    assert ok, f"worst error/bound {worst}"
    # tighter than the stated tolerance: the 3-product split keeps ~2^-21 relative accuracy per product
    ref64 = a.logical().astype(np.float64) @ b.logical().astype(np.float64)
    rms = np.sqrt(np.mean(ref64 ** 2))
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * rms


@pytest.mark.parametrize("algo", TC_ALGOS)
def test_tensor_core_path_keeps_inf_nan_classification(algo):
    # The reference's differential tests classify inf / NaN / sign of matmul results
    # (tests/test_matmul_reference.py:43-50); non-finite operands reroute to the exact-FP32 kernel.
    m, n, k = 128, 256, 64
    a, b = rnd(22, m, k), rnd(23, k, n)
    a[3, 5] = np.inf
    a[70, 9] = np.nan
    b[9, 200] = -np.inf
    ra, rb = RefTensor.from_numpy(a), RefTensor.from_numpy(b)
    c, _ = run(ra, rb, algo)
    want = ra.matmul(rb).logical()
    assert np.array_equal(np.isnan(c), np.isnan(want))
    assert np.array_equal(np.isinf(c), np.isinf(want))
    finite = np.isfinite(want)
    assert np.array_equal(np.sign(c[np.isinf(want)]), np.sign(want[np.isinf(want)]))
    assert np.allclose(c[finite], want[finite], rtol=1e-4, atol=1e-4)
    # both operands K-major (the right one through .mT): both are fed to the MMA as they lie in memory
    c2, _ = run(ra, RefTensor.from_numpy(np.ascontiguousarray(b.T)).mT, algo)
    assert np.array_equal(np.isnan(c2), np.isnan(want)) and np.array_equal(np.isinf(c2), np.isinf(want))
    assert np.allclose(c2[finite], want[finite], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("algo", TC_ALGOS)
def test_tensor_core_path_with_low_mantissa_bits_all_set(algo):
    # The K-major operand is fed to the MMA unsplit (the MMA drops the low 13 mantissa bits) and only the
    # remainder plane is prepared.  Operands whose low 13 bits are all ones are the worst case for that:
    # if the hardware rounded instead of truncating, every product would be off by about 2^-11.
    m, n, k = 256, 256, 512
    rng = np.random.default_rng(30)
    a = (rng.standard_normal((m, k)).astype(np.float32).view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    bt = (rng.standard_normal((n, k)).astype(np.float32).view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    ra, rb = RefTensor.from_numpy(a), RefTensor.from_numpy(bt).mT          # both operands K-major
    c, _ = run(ra, rb, algo)
    ref64 = a.astype(np.float64) @ bt.astype(np.float64).T
    rms = np.sqrt(np.mean(ref64 ** 2))
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * rms
    # and the same product with a transposed (pre-split) right operand agrees to the same bound
    c2, _ = run(ra, RefTensor.from_numpy(np.ascontiguousarray(bt.T)), algo)
    assert np.abs(c2 - ref64).max() <= 4e-6 * np.sqrt(k) * rms


def test_both_tensor_core_kernels_agree_within_the_split_error():
    # One CTA per 128x256 tile or a CTA pair per 256x256 tile.  With a row-major right operand the pair kernel
    # reads it MN-major as it lies (hi = truncation) while the one-CTA kernel reads re-laid planes (hi = rounding):
    # the two differ by the dropped lo*lo terms only.
    m, n, k = 512, 512, 384
    a, b = RefTensor.from_numpy(rnd(40, m, k)), RefTensor.from_numpy(rnd(41, k, n, scale=1 / np.sqrt(k)))
    c1, _ = run(a, b, "tcgen05_3xtf32")
    c2, _ = run(a, b, "tcgen05_3xtf32_2cta")
    ref64 = a.logical().astype(np.float64) @ b.logical().astype(np.float64)
    rms = np.sqrt(np.mean(ref64 ** 2))
    assert np.abs(c1 - ref64).max() <= 4e-6 * np.sqrt(k) * rms and np.abs(c2 - ref64).max() <= 4e-6 * np.sqrt(k) * rms
    assert np.abs(c1 - c2).max() <= 2e-6 * np.sqrt(k) * rms


@pytest.mark.parametrize("m,n,k", [(256, 256, 40), (512, 384, 1000), (2560, 2304, 288), (96, 4096, 64)])
def test_pair_kernel_reads_row_contiguous_operands_mn_major(m, n, k):
    # A through .mT (rows of A contiguous) and B row-major (columns of B contiguous): both MN-major for the MMA.
    at, b = RefTensor.from_numpy(rnd(60, k, m)).mT, RefTensor.from_numpy(rnd(61, k, n, scale=1 / np.sqrt(k)))
    c, _ = run(at, b, "tcgen05_3xtf32_2cta")
    ref64 = at.logical().astype(np.float64) @ b.logical().astype(np.float64)
    rms = np.sqrt(np.mean(ref64 ** 2))
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * rms
    ok, worst = matmul_tolerance_ok(c, at.matmul(b).logical(), k)
    assert ok, f"worst error/bound {worst}"
    # operands with all low mantissa bits set: the MN-major hi operand is truncated by the MMA like the K-major one
    hot = (rnd(62, k, m).view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    hb = (rnd(63, k, n, scale=1 / np.sqrt(k)).view(np.uint32) | np.uint32(0x1FFF)).view(np.float32)
    c, _ = run(RefTensor.from_numpy(hot).mT, RefTensor.from_numpy(hb), "tcgen05_3xtf32_2cta")
    ref64 = hot.astype(np.float64).T @ hb.astype(np.float64)
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(ref64 ** 2))


@pytest.mark.parametrize("m,n,k", [(256, 256, 32), (512, 768, 1024), (300, 500, 200), (2560, 2304, 288), (4, 1000, 96)])
def test_pair_kernel_with_two_k_major_operands(m, n, k):
    # A @ W.mT with both operands K-major: both are fed to the MMA as they lie in memory, only lo planes are prepared.
    a, wt = RefTensor.from_numpy(rnd(50, m, k)), RefTensor.from_numpy(rnd(51, n, k, scale=1 / np.sqrt(k)))
    c, _ = run(a, wt.mT, "tcgen05_3xtf32_2cta")
    ref64 = a.logical().astype(np.float64) @ wt.logical().astype(np.float64).T
    rms = np.sqrt(np.mean(ref64 ** 2))
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * rms
    # the one-CTA kernel accumulates the same products in the same order: identical bits as long as neither kernel
    # cuts its last round of tiles along K (a cut needs at least 8 K blocks of the kernel's stage depth)
    c1, _ = run(a, wt.mT, "tcgen05_3xtf32")
    if k <= 96:
        assert np.array_equal(c.view(np.uint32), c1.view(np.uint32))
    else:
        assert np.abs(c1 - ref64).max() <= 4e-6 * np.sqrt(k) * rms


@pytest.mark.parametrize("algo", TC_ALGOS)
def test_batched_products_with_row_contiguous_operands(algo):
    # bmm whose operands are unit-stride along their rows: X.mT [b, m, k] over X [b, k, m], and W [b, k, n] row-major.
    # The pair kernel reads both MN-major through a 4-D tensor map with the batch as its outer dimension.
    batch, m, n, k = 3, 256, 320, 96
    xt = RefTensor.from_numpy(rnd(70, batch, k, m))
    w = RefTensor.from_numpy(rnd(71, batch, k, n, scale=1 / np.sqrt(k)))
    c, _ = run(xt.mT, w, algo)
    assert c.shape == (batch, m, n)
    for i in range(batch):
        want64 = xt.logical()[i].astype(np.float64).T @ w.logical()[i].astype(np.float64)
        assert np.abs(c[i] - want64).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(want64 ** 2))
        ok, worst = matmul_tolerance_ok(c[i], xt.select0(i).mT.matmul(w.select0(i)).logical(), k)
        assert ok, worst


def test_split_k_tail_with_row_contiguous_operands():
    # 90 tile pairs on 74 SM pairs with 16 K blocks: the last 16 pairs are cut in two along K and added atomically,
    # with both operands read MN-major.
    m, n, k = 2560, 2304, 512
    at, b = RefTensor.from_numpy(rnd(72, k, m)).mT, RefTensor.from_numpy(rnd(73, k, n, scale=1 / np.sqrt(k)))
    c, _ = run(at, b, "tcgen05_3xtf32_2cta")
    ref64 = at.logical().astype(np.float64) @ b.logical().astype(np.float64)
    assert np.abs(c - ref64).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(ref64 ** 2))


def test_batched_product_over_several_rounds_of_tiles():
    # 32 batches of 1024 x 1024 outputs are 7 rounds of tile pairs on the persistent pair kernel; every batch must
    # come out as if done alone, with the fused bias + relu epilogue and its pre-activation output.
    batch, m, n, k = 32, 1024, 1024, 64
    x = rnd(80, batch, m, k)
    w = rnd(81, batch, n, k, scale=1 / np.sqrt(k))
    bias = np.random.default_rng(82).uniform(-0.1, 0.1, n).astype(np.float32)
    c, pre = run(RefTensor.from_numpy(x), RefTensor.from_numpy(w).mT, "tcgen05_3xtf32_2cta", bias=bias, epilogue="bias_relu",
                 want_preact=True)
    for i in range(batch):
        want64 = x[i].astype(np.float64) @ w[i].astype(np.float64).T + bias
        assert np.abs(pre[i] - want64).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(want64 ** 2)) + 1e-6, i
    assert np.array_equal(c.view(np.uint32), RefTensor.from_numpy(pre).relu().logical().view(np.uint32))
    # the same product in one piece by the one-CTA kernel: identical bits (same products, same k order)
    c1, pre1 = run(RefTensor.from_numpy(x), RefTensor.from_numpy(w).mT, "tcgen05_3xtf32", bias=bias, epilogue="bias_relu",
                   want_preact=True)
    assert np.array_equal(pre.view(np.uint32), pre1.view(np.uint32))
    # row-major right operand (MN-major tiles), batched
    wt = np.ascontiguousarray(np.swapaxes(w, 1, 2))
    c2, _ = run(RefTensor.from_numpy(x), RefTensor.from_numpy(wt), "tcgen05_3xtf32_2cta")
    for i in (0, 8, 9, 31):
        want64 = x[i].astype(np.float64) @ wt[i].astype(np.float64)
        assert np.abs(c2[i] - want64).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(want64 ** 2)), i


@pytest.mark.parametrize("algo", TC_ALGOS)
@pytest.mark.parametrize("batch,m,n,k,epilogue", [(1, 1024, 1024, 8192, "bias_relu"),    # fewer tiles than SMs, deep K: every tile is cut in four
                                                   (1, 1024, 1024, 4096, "relu_vjp"),     # ... in two
                                                   (1, 512, 4096, 4096, "none"),          # one eighth of a 4096^3 product
                                                   (2, 300, 700, 6200, "bias"),           # ragged edges inside cut tiles, K tail
                                                   (8, 1024, 1024, 1024, "bias_relu")])   # shallow K: stays uncut (the parts would be epilogue-bound)
def test_tiles_cut_along_k_keep_epilogues_and_are_deterministic(algo, batch, m, n, k, epilogue):
    """When the last round of tiles would leave SMs idle its tiles are cut along K; the part that finishes last adds
    the partial sums in part order and applies the epilogue.  The result must not depend on which part finishes
    last (two runs agree bit for bit) and must meet the same tolerance as an uncut product."""
    a = RefTensor.from_numpy(rnd(300, batch, m, k))
    b = RefTensor.from_numpy(rnd(301, batch, n, k, scale=1 / np.sqrt(k))).mT
    bias = rnd(302, n) if epilogue in ("bias", "bias_relu") else None
    aux = rnd(303, batch, m, n) if epilogue == "relu_vjp" else None
    want_pre = epilogue == "bias_relu"
    c1, p1 = run(a, b, algo, bias=bias, epilogue=epilogue, aux=aux, want_preact=want_pre)
    c2, p2 = run(a, b, algo, bias=bias, epilogue=epilogue, aux=aux, want_preact=want_pre)
    assert np.array_equal(c1.view(np.uint32), c2.view(np.uint32))
    a64 = a.storage.reshape(batch, m, k).astype(np.float64)
    b64 = b.storage.reshape(batch, n, k).astype(np.float64)
    pre = np.einsum("bmk,bnk->bmn", a64, b64)
    if bias is not None:
        pre = pre + bias
    if epilogue == "bias_relu":
        ok, worst = matmul_tolerance_ok(p1, pre, k)
        assert ok, worst
        assert np.array_equal(c1.view(np.uint32), RefTensor.from_numpy(p1).relu().logical().view(np.uint32))
        assert np.array_equal(p1.view(np.uint32), p2.view(np.uint32))
    elif epilogue == "relu_vjp":
        want = np.where(aux > 0, pre, 0.0)
        ok, worst = matmul_tolerance_ok(c1, want, k)
        assert ok, worst
        assert np.all(c1[aux <= 0] == 0.0)
    else:
        ok, worst = matmul_tolerance_ok(c1, pre, k)
        assert ok, worst
