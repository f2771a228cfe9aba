"""GPU parity through the `torch_rs` surface (Python -> C++ host engine -> C ABI kernels) against the
CPU checker: values, and the layout metadata (.shape/.stride()/.storage_offset()) of every result, the
way the reference's differential tests compare them (tests/test_operation_chains_reference.py:213-228)."""
import json
import os

import numpy as np
import pytest

import torch_rs as torch
from oracle import ref
from oracle.ref import RefTensor
from torch_rs._device import launch_count

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))
DEV = "cuda:0"


def hexf(items):
    return np.array([int(h, 16) for h in items], dtype=np.uint32).view(np.float32)


def bits(a):
    return [f"{b:08x}" for b in np.ascontiguousarray(a, dtype=np.float32).reshape(-1).view(np.uint32)]


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def check_same(t, r: RefTensor, exact=True, ulp=0):
    assert list(t.shape) == r.shape
    assert list(t.stride()) == r.strides, (t.stride(), r.strides)
    assert t.storage_offset() == r.offset
    got, want = t.numpy(), r.logical()
    if exact:
        assert ref.same_bits_or_nan(got, want).all()
    else:
        assert ref.ulp_distance(got, want).max() <= ulp


def test_relu_add_contiguous_is_one_kernel():
    x, y = np.random.default_rng(0).uniform(-1, 1, (300, 257)).astype(np.float32), np.random.default_rng(1).uniform(-1, 1, (300, 257)).astype(np.float32)
    tx, ty = torch.tensor(x, device=DEV), torch.tensor(y, device=DEV)
    before = launch_count()
    out = torch.relu(tx + ty)
    assert out.is_pending()
    out.materialize()
    assert launch_count() - before == 1
    assert not out.is_pending()
    check_same(out, (RefTensor.from_numpy(x) + RefTensor.from_numpy(y)).relu())
    assert not out.shares_storage_with(tx)


def test_transposed_broadcast_exp_chain_metadata_and_values():
    n, m = 160, 96
    xs, b = rnd(0, n, m), (0.1 * rnd(1, n)).astype(np.float32)
    x, bt = torch.tensor(xs, device=DEV), torch.tensor(b, device=DEV)
    before = launch_count()
    out = torch.exp(2.0 * torch.relu(x.mT + bt)) - x.mT
    assert out.stride() == x.mT.stride()          # the chain stays in x's physical order
    out.materialize()
    assert launch_count() - before == 1           # five ops, one kernel
    rx = RefTensor.from_numpy(xs)
    exp_term = (2.0 * (rx.mT + RefTensor.from_numpy(b)).relu()).exp()
    expected = exp_term - rx.mT
    assert list(out.stride()) == expected.strides and out.storage_offset() == 0
    got, want = out.numpy(), expected.logical()
    # exp is within 1 ulp of libm (checked on its own elsewhere); the final subtraction adds one rounding
    assert np.all(np.abs(got.astype(np.float64) - want) <= np.spacing(np.abs(exp_term.logical())) + np.spacing(np.abs(want)))


def test_every_intermediate_matches_when_held():
    xs = rnd(2, 64, 48)
    x = torch.tensor(xs, device=DEV)
    rx = RefTensor.from_numpy(xs)
    a = x.mT + 1.5
    b = a.relu()
    c = b * x.mT
    d = c - 0.25
    before = launch_count()
    d.materialize()
    assert launch_count() - before == 1           # held intermediates become extra outputs of the same kernel
    ra = rx.mT + 1.5
    rb = ra.relu()
    rc = rb * rx.mT
    rd = rc - 0.25
    for t, r in ((a, ra), (b, rb), (c, rc), (d, rd)):
        check_same(t, r)


def test_views_select_permute_T():
    base = rnd(3, 2, 6, 5)
    t = torch.tensor(base, device=DEV)
    r = RefTensor.from_numpy(base)
    v, rv = t.select(0, 1).T, r.select0(1).T
    assert v.storage_offset() == rv.offset and list(v.stride()) == rv.strides
    check_same(v.relu(), rv.relu())
    p, rp = t.permute(2, 0, 1), r.permute([2, 0, 1])
    row = rnd(4, 6)
    check_same(p * torch.tensor(row, device=DEV), rp * RefTensor.from_numpy(row))
    check_same(t[1] + t[0], r.select0(1) + r.select0(0))
    assert np.array_equal(torch.transpose(t, 0, 2).numpy(), base.transpose(2, 1, 0))


def test_layouts_disagree_uses_tiled_kernel_and_matches():
    a, b = rnd(5, 200, 120), rnd(6, 120, 200)
    out = torch.tensor(a, device=DEV).mT + torch.tensor(b, device=DEV)
    check_same(out, RefTensor.from_numpy(a).mT + RefTensor.from_numpy(b))


def test_broadcast_golden_and_errors():
    g = GOLD["broadcast_arithmetic"]
    left = torch.tensor(np.array(g["left"]["values"], dtype=np.float32).reshape(g["left"]["shape"]), device=DEV)
    right = torch.tensor(np.array(g["right"]["values"], dtype=np.float32).reshape(g["right"]["shape"]), device=DEV)
    assert (left + right).numpy().reshape(-1).tolist() == g["add"]
    assert (left - right).numpy().reshape(-1).tolist() == g["sub"]
    assert torch.multiply(left, right).numpy().reshape(-1).tolist() == g["mul"]
    assert (left / right).numpy().reshape(-1).tolist() == g["div"]
    with pytest.raises(RuntimeError, match=r"The size of tensor a \(0\) must match the size of tensor b \(2\) at non-singleton dimension 0"):
        torch.zeros(0, device=DEV) + torch.ones(2, device=DEV)
    empty = torch.zeros(2, 0, 3, device=DEV) + torch.ones(1, 1, 3, device=DEV)
    assert empty.shape == (2, 0, 3) and empty.numpy().size == 0


def test_matmul_goldens_errors_and_precision():
    assert torch.get_float32_matmul_precision() == "highest"
    a = torch.tensor(np.arange(1, 7, dtype=np.float32).reshape(2, 3), device=DEV)
    b = torch.tensor(np.arange(7, 13, dtype=np.float32).reshape(3, 2), device=DEV)
    out = torch.matmul(a, b)
    assert out.shape == (2, 2) and out.stride() == (2, 1)
    assert out.numpy().reshape(-1).tolist() == [58.0, 64.0, 139.0, 154.0]
    assert (a.T @ b.T).shape == (3, 3)
    with pytest.raises(RuntimeError, match=r"mat1 and mat2 shapes cannot be multiplied \(2x3 and 4x2\)"):
        torch.zeros(2, 3, device=DEV) @ torch.zeros(4, 2, device=DEV)
    with pytest.raises(RuntimeError, match="matmul currently requires two rank-2 tensors"):
        torch.zeros(3, device=DEV) @ torch.zeros(3, 2, device=DEV)
    assert not out.requires_grad


def test_batched_bias_relu_fuses_into_the_matmul():
    batch, m, n, k = 4, 96, 128, 64
    xs, ws = rnd(7, batch, m, k), rnd(8, batch, n, k, scale=1 / 8)
    bias = np.random.default_rng(9).uniform(-0.1, 0.1, n).astype(np.float32)
    x, w, bt = torch.tensor(xs, device=DEV), torch.tensor(ws, device=DEV), torch.tensor(bias, device=DEV)
    before = launch_count()
    out = torch.relu(x @ w.mT + bt).materialize()
    launches = launch_count() - before
    assert launches <= 3           # GEMM with the bias+relu epilogue (plus operand preparation for the tensor-core path)
    rx, rw = RefTensor.from_numpy(xs), RefTensor.from_numpy(ws)
    got = out.numpy()
    for i in range(batch):
        want = (rx.select0(i).matmul(rw.select0(i).mT) + RefTensor(bias, [n])).relu().logical().astype(np.float64)
        rms = np.sqrt(np.mean(want ** 2))
        assert np.all(np.abs(got[i] - want) <= 1e-5 * np.sqrt(k) * np.maximum(np.abs(want), rms) + 1e-30)


def test_autograd_goldens():
    a = GOLD["autograd"]
    x = torch.tensor(a["square_sum"]["x"], device=DEV, requires_grad=True)
    (x * x).sum().backward()
    assert x.grad.tolist() == a["square_sum"]["grad_first"]
    (x * x).sum().backward()
    assert x.grad.tolist() == a["square_sum"]["grad_second"]

    u = a["unbroadcast_both"]
    left = torch.tensor(np.array(u["left"]["values"], dtype=np.float32).reshape(u["left"]["shape"]), device=DEV, requires_grad=True)
    right = torch.tensor(np.array(u["right"]["values"], dtype=np.float32).reshape(u["right"]["shape"]), device=DEV, requires_grad=True)
    (left * right).sum().backward()
    assert left.grad.numpy().reshape(-1).tolist() == u["left_grad"]
    assert right.grad.numpy().reshape(-1).tolist() == u["right_grad"]

    r = a["rank_zero_view"]
    for scalar_on_left in (True, False):
        source = torch.tensor(np.array(r["source_values"], dtype=np.float32).reshape(r["source_shape"]), device=DEV, requires_grad=True)
        view = source[1].transpose(0, 1)
        scalar = torch.tensor(r["scalar"], device=DEV, requires_grad=True)
        out = scalar * view if scalar_on_left else view * scalar
        assert out.shape == (3, 2) and out.stride() == (1, 3)
        out.sum().backward()
        assert scalar.grad.numpy().reshape(-1).tolist() == r["scalar_grad"]
        assert source.grad.numpy().reshape(-1).tolist() == r["source_grad"]

    z = a["negative_zero_first"]
    left = torch.tensor([2.0], device=DEV, requires_grad=True)
    (left * torch.tensor([-0.0], device=DEV)).sum().backward()
    assert bits(left.grad.numpy()) == [z["same_count_bits"]]
    bl = torch.tensor(2.0, device=DEV, requires_grad=True)
    (bl * torch.tensor([-0.0, -0.0], device=DEV)).sum().backward()
    assert bits(bl.grad.numpy()) == [z["broadcast_bits"]]


def test_relu_vjp_golden_bits_and_graph_is_freed():
    g = GOLD["relu_vjp_bits"]
    leaf = torch.tensor(hexf(g["input"]), device=DEV, requires_grad=True)
    weights = torch.tensor(hexf(g["weights"]), device=DEV)
    out = torch.nn.functional.relu(leaf)
    assert out.requires_grad and not out.is_leaf and out._grad_fn_name() == "ReluBackward0"
    loss = (out * weights).sum()
    torch.autograd.backward(loss)
    assert bits(leaf.grad.numpy()) == g["expected_gradient"]
    with pytest.raises(RuntimeError, match="Trying to backward through the graph a second time"):
        loss.backward()
    with pytest.raises(RuntimeError, match="does not require grad"):
        weights.sum().backward()
    with torch.no_grad():
        assert not torch.relu(leaf).requires_grad


def test_exp_sub_add_backward_edges_exist_on_cuda():
    xs = rnd(10, 33, 17)
    x = torch.tensor(xs, device=DEV, requires_grad=True)
    y = torch.tensor(rnd(11, 17), device=DEV, requires_grad=True)
    loss = (torch.exp(x * 0.5) - (x + y)).sum()
    loss.backward()
    want_x = 0.5 * np.exp(0.5 * xs.astype(np.float64)) - 1.0
    assert np.allclose(x.grad.numpy(), want_x, rtol=2e-6, atol=1e-6)
    assert np.allclose(y.grad.numpy(), -33.0 * np.ones(17), rtol=1e-6)


def test_mlp_forward_backward_matches_composed_reference():
    # loss = (relu(X @ W1 + b1) @ W2).sum(): the reference primitives composed (matmul, add, relu, sum and
    # the VJPs of src/tensor.rs:3002-3107, 4422-4432) define the expected gradients.
    bsz, d, h, o = 256, 128, 192, 64
    xs, w1s, w2s = rnd(12, bsz, d), rnd(13, d, h, scale=1 / 8), rnd(14, h, o, scale=1 / 8)
    b1s = (0.1 * rnd(15, h)).astype(np.float32)
    X = torch.tensor(xs, device=DEV)
    W1, W2 = torch.tensor(w1s, device=DEV, requires_grad=True), torch.tensor(w2s, device=DEV, requires_grad=True)
    b1 = torch.tensor(b1s, device=DEV, requires_grad=True)
    loss = (torch.relu(X @ W1 + b1) @ W2).sum()
    loss.backward()
    rX, rW1, rW2 = RefTensor.from_numpy(xs), RefTensor.from_numpy(w1s), RefTensor.from_numpy(w2s)
    Z = rX.matmul(rW1) + RefTensor(b1s, [h])
    H = Z.relu()
    Y = H.matmul(rW2)
    dY = RefTensor.from_numpy(np.ones((bsz, o), dtype=np.float32))
    dW2 = H.T.matmul(dY).logical()
    dH = dY.matmul(rW2.T)
    dZ = RefTensor.from_numpy(Z.relu_vjp(dH.logical()))
    db1 = ref.unbroadcast(dZ.logical(), [bsz, h], [h])
    dW1 = rX.T.matmul(dZ).logical()

    def close(got, want, k):
        want = want.astype(np.float64)
        rms = np.sqrt(np.mean(want ** 2))
        return np.all(np.abs(got - want) <= 1e-5 * np.sqrt(k) * np.maximum(np.abs(want), rms) + 1e-30)

    assert close(W2.grad.numpy(), dW2, bsz)
    assert close(W1.grad.numpy(), dW1, bsz)
    assert close(b1.grad.numpy(), db1, bsz)
    assert abs(loss.item() - Y.sum()) <= 1e-5 * np.sqrt(bsz * o) * float(np.abs(Y.logical()).sum()) / (bsz * o) * 100
    assert W1.grad.is_contiguous() and W1.grad.shape == (d, h)


def test_item_tolist_and_scalar_forms():
    xs = rnd(16, 5, 3)
    x = torch.tensor(xs, device=DEV)
    rx = RefTensor.from_numpy(xs)
    check_same(1.5 - x, 1.5 - rx)
    check_same(2.0 / x.T, 2.0 / rx.T)
    check_same(x / 3.0, rx / 3.0)
    check_same(-x, rx.neg())
    assert x.sum().item() == pytest.approx(float(xs.sum()), rel=1e-5)
    with pytest.raises(RuntimeError, match="item requires one element, got 15"):
        x.item()
    with pytest.raises(IndexError, match="index 7 is out of bounds for dimension 0 with size 5"):
        x[7]


def test_pinned_upload_and_non_blocking_read_back():
    xs = rnd(17, 64, 96)
    staging = torch.pinned_empty(64, 96)
    staging[...] = xs
    result = torch.pinned_empty(96, 64)
    x = torch.tensor(staging, device=DEV)                 # asynchronous upload from page-locked memory
    out = torch.relu(x.mT * 2.0)
    out.copy_to_host(result, non_blocking=True)           # gathered to logical order, copied on the egress stream
    torch.synchronize(0)
    want = (RefTensor.from_numpy(xs).mT * 2.0).relu().logical()
    assert np.array_equal(result.view(np.uint32), want.view(np.uint32))
    with pytest.raises(ValueError, match="pinned_empty"):
        out.copy_to_host(np.empty((96, 64), dtype=np.float32), non_blocking=True)
    torch.pinned_free(staging)
    torch.pinned_free(result)


def test_concurrent_backward_passes_from_two_threads():
    # The reference runs whole backward passes under one lock and tests it with two racing threads
    # (tests/autograd.rs:128-173); here two Python threads share a leaf and each runs 20 backward passes.
    import threading
    x = torch.tensor(np.array([-2.0, 0.5, 3.0], dtype=np.float32), device=DEV, requires_grad=True)
    errors = []

    def worker():
        try:
            for _ in range(20):
                (x * x).sum().backward()
        except Exception as exc:            # pragma: no cover - reported below
            errors.append(exc)

    threads = [threading.Thread(target=worker) for _ in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    assert x.grad.tolist() == [-160.0, 40.0, 240.0]        # 40 accumulated passes of 2x


def test_refused_allocation_is_reported_like_the_reference():
    # AllocationFailed{elements} (src/tensor_error.rs): a request the device cannot satisfy is an error
    # message, not a crash, and the engine keeps working afterwards.
    with pytest.raises(RuntimeError, match=r"failed to allocate storage for 1099511627776 elements"):
        torch.zeros(1 << 20, 1 << 20, device=DEV)
    assert (torch.ones(4, device=DEV) + 1.0).tolist() == [2.0, 2.0, 2.0, 2.0]


def test_more_reference_goldens_on_the_device():
    g = GOLD["strided_relu_grads"]
    storage = np.concatenate([np.full(12, 9.0, dtype=np.float32), hexf(g["storage_tail_bits"])]).reshape(2, 3, 4)
    source = torch.tensor(storage, device=DEV, requires_grad=True)
    offset = source[1]
    out = offset.relu()
    assert out.requires_grad and out.shape == (3, 4) and out.stride() == (4, 1) and out.storage_offset() == 0
    out.sum().backward()
    strided = offset.transpose(0, 1)
    sout = strided.relu()
    assert sout.shape == (4, 3) and sout.stride() == (1, 4) and not sout.shares_storage_with(strided)
    weights = torch.tensor(np.arange(1, 13, dtype=np.float32).reshape(4, 3), device=DEV)
    (sout * weights).sum().backward()
    assert source.grad.numpy().reshape(-1).tolist() == [float(v) for v in g["expected_grad"]]

    d = GOLD["reflected_division"]
    view = torch.tensor([[1.0, 2.0]], device=DEV).transpose(0, 1)
    assert view.shape == (2, 1) and view.stride() == (1, 2)
    assert (view / 1.0).stride() == tuple(d["div_one_strides"])
    reflected = 1.0 / view
    assert reflected.stride() == tuple(d["reflected_strides"]) and reflected.numpy().reshape(-1).tolist() == d["reflected_values"]
    assert (1.0 / torch.zeros(1, 0, device=DEV).transpose(0, 1)).stride() == (1, 0)
    assert (1.0 / torch.zeros(1, 0, 1, device=DEV)).stride() == (0, 1, 0)
    assert (1.0 / torch.zeros(2, 0, 3, device=DEV).transpose(0, 2)).stride() == (2, 2, 1)
    import sys
    large = torch.zeros(2, 0, sys.maxsize, device=DEV)
    assert (1.0 / large).stride() == (0, 1, 0)
    assert large.transpose(0, 2).stride() == (1, sys.maxsize, sys.maxsize)
    with pytest.raises(RuntimeError, match="Stride calculation overflowed"):
        1.0 / large.transpose(0, 1)

    r = GOLD["reshape_view_strides"]
    v = torch.tensor(np.arange(24, dtype=np.float32).reshape(2, 3, 4), device=DEV).transpose(0, 2)
    for case in r["cases"]:
        out = v.reshape(*case["shape"])
        assert out.stride() == tuple(case["strides"]) and out.shares_storage_with(v) == case["shares"]

    # small matmuls run on the k-ascending FP32 kernel, so the reference's ordering golden holds exactly
    m = GOLD["matmul_ordering"]
    out = torch.tensor(hexf(m["left_bits"]).reshape(m["left_shape"]), device=DEV) @ torch.tensor(hexf(m["right_bits"]).reshape(m["right_shape"]), device=DEV)
    assert bits(out.numpy())[0] == m["first_element_bits"]


def test_dlpack_export_is_zero_copy_and_keeps_the_layout():
    pt = pytest.importorskip("torch")
    xs = rnd(18, 6, 10)
    view = torch.tensor(xs, device=DEV).T                  # [10,6], strides (1,10)
    out = view * 2.0                                                                             # pending until exported
    shared = pt.from_dlpack(out)
    assert shared.device.type == "cuda" and tuple(shared.shape) == (10, 6) and tuple(shared.stride()) == out.stride()
    assert shared.data_ptr() == out.data_ptr()
    assert np.array_equal(shared.cpu().numpy(), (xs.T * 2.0).astype(np.float32))
    del out                     # the capsule keeps the storage alive
    assert np.array_equal(shared.cpu().numpy(), (xs.T * 2.0).astype(np.float32))


# ---- transform VJPs: bits, accumulation over passes, freeing of value-dependent graphs ----------------------
# Same scheme as the reference's tests/test_transpose_backward.py:9-146: gradients with awkward bit patterns
# must arrive at the leaf untouched through t / transpose / permute of direct, offset and non-contiguous views.

_GRADIENT_BITS = np.array([0x00000000, 0x80000000, 0x3F800001, 0xBF000001, 0x41234567, 0xC1234567,
                           0x00800000, 0x80800000, 0x3EAAAAAB, 0xBEAAAAAB], dtype=np.uint32).view(np.float32)


def _patterned(shape):
    return np.resize(_GRADIENT_BITS, int(np.prod(shape))).reshape(shape).astype(np.float32)


def _rank_two_source(kind, rows, cols):
    """(leaf, rank-two view of it, function mapping a gradient of the view to the leaf's gradient)."""
    if kind == "direct":
        leaf = torch.zeros(rows, cols, device=DEV, requires_grad=True)
        return leaf, leaf, lambda g: g
    if kind == "offset":
        leaf = torch.zeros(2, rows, cols, device=DEV, requires_grad=True)

        def lift(g):
            out = np.zeros((2, rows, cols), dtype=np.float32)
            out[1] = g
            return out
        return leaf, leaf[1], lift
    if kind == "noncontiguous":
        leaf = torch.zeros(cols, rows, device=DEV, requires_grad=True)
        return leaf, leaf.transpose(0, 1), lambda g: np.ascontiguousarray(g.T)
    leaf = torch.zeros(cols, rows, 2, device=DEV, requires_grad=True)          # offset and non-contiguous

    def lift(g):
        out = np.zeros((cols, rows, 2), dtype=np.float32)
        out[:, :, 1] = g.T
        return out
    return leaf, leaf.transpose(0, 2)[1], lift


@pytest.mark.parametrize("kind,shape", [("direct", (1, 1)), ("direct", (1, 7)), ("direct", (7, 11)), ("offset", (5, 7)),
                                        ("noncontiguous", (5, 7)), ("offset noncontiguous", (5, 7))])
@pytest.mark.parametrize("op", ["t", "transpose", "permute"])
def test_rank_two_transform_backward_bits_accumulation_and_freeing(kind, shape, op):
    apply = {"t": lambda x: x.t(), "transpose": lambda x: torch.transpose(x, 0, 1), "permute": lambda x: x.permute(1, 0)}[op]
    leaf, source, lift = _rank_two_source(kind, *shape)
    transformed = apply(source)
    weights = _patterned(tuple(transformed.shape))
    loss = (transformed * torch.tensor(weights, device=DEV)).sum()
    once = lift(np.ascontiguousarray(weights.T))
    loss.backward()
    assert np.array_equal(leaf.grad.numpy().view(np.uint32), once.view(np.uint32))
    with pytest.raises(RuntimeError, match="backward through the graph a second time"):
        loss.backward()                                             # the product saved its operands; they are freed
    (apply(source) * torch.tensor(weights, device=DEV)).sum().backward()
    twice = once + once
    assert np.array_equal(leaf.grad.numpy().view(np.uint32), twice.view(np.uint32))
    reusable = apply(source).sum()                                  # no saved values: the graph survives a pass
    ones = lift(np.ones(tuple(source.shape), dtype=np.float32))
    for _ in range(2):
        reusable.backward()
        twice = twice + ones
        assert np.array_equal(leaf.grad.numpy().view(np.uint32), twice.view(np.uint32))


def test_rank_three_permutation_backward_bits():
    leaf = torch.zeros(2, 3, 5, device=DEV, requires_grad=True)
    weights = _patterned((5, 2, 3))
    loss = (leaf.permute(2, 0, 1) * torch.tensor(weights, device=DEV)).sum()
    once = np.ascontiguousarray(weights.transpose(1, 2, 0))
    loss.backward()
    assert np.array_equal(leaf.grad.numpy().view(np.uint32), once.view(np.uint32))
    with pytest.raises(RuntimeError, match="backward through the graph a second time"):
        loss.backward()
    (leaf.permute(2, 0, 1) * torch.tensor(weights, device=DEV)).sum().backward()
    assert np.array_equal(leaf.grad.numpy().view(np.uint32), (once + once).view(np.uint32))


def test_three_contributions_accumulate_in_the_reference_order():
    """((x*y1)*(x*y2))*x sends three gradient contributions to x.  The reference walks the graph in the reverse of
    a depth-first post-order (collect_topology, src/tensor.rs:2945-2994; run_backward 2895) and adds each
    contribution onto the sum so far (add_gradient 3302-3317), which fixes the order: first the outer product's
    right edge, then the inner right product's, then the inner left product's.  Float addition does not commute over
    three terms, so the bits pin the order."""
    rng = np.random.default_rng(77)
    xs, y1, y2 = (rng.standard_normal(4096).astype(np.float32) for _ in range(3))
    x = torch.tensor(xs, device=DEV, requires_grad=True)
    a, b = x * torch.tensor(y1, device=DEV), x * torch.tensor(y2, device=DEV)
    ((a * b) * x).sum().backward()
    av, bv = xs * y1, xs * y2
    c_outer = av * bv                      # upstream 1 * value of (a*b)
    c_b = (xs * av) * y2                   # through b = x*y2: upstream is x * a
    c_a = (xs * bv) * y1                   # through a = x*y1: upstream is x * b
    want = (c_outer + c_b) + c_a
    other_order = (c_outer + c_a) + c_b
    assert (want.view(np.uint32) != other_order.view(np.uint32)).any()      # the case does tell the orders apart
    assert np.array_equal(x.grad.numpy().view(np.uint32), want.view(np.uint32))


def test_values_derived_from_a_gradient_do_not_see_later_accumulation():
    """`x.grad` is accumulated in place by the next backward pass (src/storage.rs:85-100).  The reference computes
    clone() and every op on it at once; deferring them here must not let them observe the later values."""
    xs = rnd(5, 33, 7)
    x = torch.tensor(xs, device=DEV, requires_grad=True)
    (x * 2.0).sum().backward()
    g0, doubled, moved = x.grad.clone(), x.grad * 2.0, x.grad.mT.contiguous()
    (x * 3.0).sum().backward()
    assert np.array_equal(g0.numpy(), np.full_like(xs, 2.0))
    assert np.array_equal(doubled.numpy(), np.full_like(xs, 4.0))
    assert np.array_equal(moved.numpy(), np.full_like(xs.T, 2.0))
    assert np.array_equal(x.grad.numpy(), np.full_like(xs, 5.0))


def test_deep_chains_are_released_and_differentiated_without_recursion():
    """tests/autograd.rs:1059-1090 in the reference: a 20,000-op chain is differentiated and a 100,000-op chain that
    is never differentiated is dropped; neither may recurse once per op."""
    x = torch.tensor(np.array([1.5, -2.0], dtype=np.float32), device=DEV, requires_grad=True)
    y = x
    for _ in range(20000):
        y = y * 1.0
    y.sum().backward()
    assert x.grad.tolist() == [1.0, 1.0]
    z = x
    for _ in range(100000):
        z = z * 1.0
    detached = z.detach()
    del z
    assert detached.tolist() == [1.5, -2.0]


def test_pinned_uploads_on_their_own_stream_respect_recycled_blocks():
    """Uploads from page-locked memory run on an upload stream, beside the kernels.  A block that the compute stream
    has just given up (with kernels that read it still queued) may be handed to the next upload: the copy must wait
    for exactly those kernels, and kernels must wait for the copy they read."""
    n = 1 << 20
    stage = [torch.pinned_empty(n) for _ in range(6)]       # a source stays untouched until its copy has run
    outs = [torch.pinned_empty(n) for _ in range(6)]
    held = None
    for i in range(6):
        buf = stage[i]
        buf[...] = np.arange(n, dtype=np.float32) + i
        x = torch.tensor(buf, device=DEV)              # same size every time: the cache recycles the previous block
        y = (x * 2.0 + 1.0).relu()
        y.copy_to_host(outs[i], non_blocking=True)
        held = y                                         # x is dropped here with its readers still queued
        del x
    torch.synchronize(0)
    for i in range(6):
        assert np.array_equal(outs[i], (np.arange(n, dtype=np.float32) + i) * 2.0 + 1.0), i
    for array in stage + outs:
        torch.pinned_free(array)
