"""Seeded random operation chains through the `torch_rs` surface against the CPU checker.

In the spirit of the reference's differential chain test (tests/test_operation_chains_reference.py:
input kind -> view -> unary -> broadcast multiply -> unary -> sum -> backward, comparing values and
shape/stride/offset/requires_grad/is_leaf of every step), with the checker in place of PyTorch and
the expected gradients composed from the reference's VJPs (src/tensor.rs:3002-3300).
"""
import numpy as np
import pytest

import torch_rs as torch
from oracle import ref
from oracle.ref import RefTensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SEED = 0xB200
CHAINS = 48
RTOL, ATOL = 5e-6, 2e-6          # the reference's own chain tolerances (test_operation_chains_reference.py)

INPUT_KINDS = ("scalar", "empty", "offset", "transposed", "contiguous", "permuted")
UNARIES = ("neg", "relu", "sin", "exp")


def make_input(rng, kind):
    """Returns (leaf values, function building the input view from a leaf for either engine, shape)."""
    if kind == "scalar":
        return rng.standard_normal(()).astype(np.float32), (lambda t: t)
    if kind == "empty":
        return np.zeros((2, 0, 3), dtype=np.float32), (lambda t: t)
    if kind == "offset":
        return rng.standard_normal((2, 3, 4)).astype(np.float32), (lambda t: t[1] if not isinstance(t, RefTensor) else t.select0(1))
    if kind == "transposed":
        return rng.standard_normal((2, 3, 4)).astype(np.float32), (lambda t: t.transpose(0, 2))
    if kind == "permuted":
        return rng.standard_normal((5, 6, 7)).astype(np.float32), (lambda t: t.permute(2, 0, 1) if not isinstance(t, RefTensor) else t.permute([2, 0, 1]))
    return rng.standard_normal((33, 17)).astype(np.float32), (lambda t: t)


def multiplier_shape(rng, shape):
    if not shape:
        return (int(rng.integers(2, 5)),)
    out = [1 if d == 0 else d for d in shape]
    for axis, d in enumerate(shape):
        if d != 1 and rng.integers(0, 2):
            out[axis] = 1
    if rng.integers(0, 3) == 0:
        out = out[1:]                                   # lower rank: broadcast from the right
    return tuple(out)


def apply_unary(t, name):
    return getattr(t, name)() if not isinstance(t, RefTensor) else t.unary(name)


def unary_vjp(name, saved_in: RefTensor, out: RefTensor, g):
    if name == "neg":
        return -g
    if name == "relu":
        return saved_in.relu_vjp(g)
    if name == "sin":
        return (g * np.cos(saved_in.logical())).astype(np.float32)
    return (g * out.logical()).astype(np.float32)      # exp


def same_meta(t, r):
    assert list(t.shape) == r.shape and list(t.stride()) == r.strides and t.storage_offset() == r.offset, \
        (t.shape, t.stride(), r.shape, r.strides)


@pytest.mark.parametrize("index", range(CHAINS))
def test_random_chain(index):
    rng = np.random.default_rng([SEED, index])
    kind = INPUT_KINDS[index % len(INPUT_KINDS)]
    first, second = UNARIES[rng.integers(0, 4)], UNARIES[rng.integers(0, 4)]
    leaf_values, view = make_input(rng, kind)
    leaf = torch.tensor(leaf_values, device=DEV, requires_grad=True)
    rleaf = RefTensor.from_numpy(leaf_values)
    x, rx = view(leaf), view(rleaf)
    same_meta(x, rx)
    assert x.requires_grad and (kind in ("scalar", "empty", "contiguous") or not x.is_leaf)
    mshape = multiplier_shape(rng, tuple(rx.shape))
    mvals = rng.standard_normal(mshape).astype(np.float32)
    m_grad = bool(rng.integers(0, 2))
    m = torch.tensor(mvals, device=DEV, requires_grad=m_grad)
    rm = RefTensor.from_numpy(mvals)

    t1, r1 = apply_unary(x, first), apply_unary(rx, first)
    form = index % 3
    t2 = t1 * m if form == 0 else (torch.mul(t1, m) if form == 1 else torch.multiply(t1, m))
    r2 = r1 * rm
    t3, r3 = apply_unary(t2, second), apply_unary(r2, second)
    for t, r in ((t1, r1), (t2, r2), (t3, r3)):
        same_meta(t, r)
        assert t.requires_grad and not t.is_leaf
        assert np.allclose(t.numpy(), r.logical(), rtol=RTOL, atol=ATOL, equal_nan=True)
    if "sin" not in (first, second) and "exp" not in (first, second):
        assert ref.same_bits_or_nan(t3.numpy(), r3.logical()).all()      # add/mul/relu/neg chains are bit-exact

    loss = t3.sum()
    assert loss.shape == () and loss.requires_grad
    loss.backward()

    # expected gradients, composed from the reference VJPs in logical order
    g = np.ones(r3.shape, dtype=np.float32)                                 # Sum VJP
    g = unary_vjp(second, r2, r3, g)
    g_m = ref.unbroadcast(g, r2.shape, list(mshape), other=r1) if m_grad else None
    g = ref.unbroadcast(g, r2.shape, r1.shape, other=rm)                    # Multiply VJP, un-broadcast
    g = unary_vjp(first, rx, r1, g)
    if kind == "offset":
        full = np.zeros(leaf_values.shape, dtype=np.float32)
        full[1] = g
        g = full
    elif kind == "transposed":
        g = ref.permute_vjp(g, list(leaf_values.shape), [2, 1, 0])
    elif kind == "permuted":
        g = ref.permute_vjp(g, list(leaf_values.shape), [2, 0, 1])
    got = leaf.grad
    assert got is not None and got.shape == leaf_values.shape and got.is_contiguous()
    scale = max(1.0, float(np.abs(g).max()) if g.size else 1.0)
    assert np.allclose(got.numpy(), g, rtol=50 * RTOL, atol=50 * ATOL * scale, equal_nan=True)
    if m_grad:
        assert np.allclose(m.grad.numpy(), g_m, rtol=50 * RTOL, atol=50 * ATOL * max(1.0, float(np.abs(g_m).max()) if g_m.size else 1.0))
    else:
        assert m.grad is None
