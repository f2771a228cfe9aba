"""Materialising layout ops on the device — clone, contiguous, reshape / view, flatten, equal — against
the CPU checker's layout rules and the reference's goldens (tests/tensor_baseline.rs:1606-1631,
tests/autograd.rs:1122-1137)."""
import json
import os

import numpy as np
import pytest

import torch_rs as torch
from oracle.ref import RefTensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))


def rnd(seed, *shape):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def test_reference_goldens_for_clone_and_reshape_of_views():
    source = torch.tensor(np.arange(24, dtype=np.float32).reshape(2, 3, 4), device=DEV)
    view = source.transpose(0, 2)
    indexed = view[1]
    assert indexed.shape == (3, 2) and indexed.stride() == (4, 12) and indexed.storage_offset() == 1
    clone = indexed.clone()
    assert clone.stride() == (1, 3) and not clone.shares_storage_with(source)
    assert clone.numpy().reshape(-1).tolist() == [1.0, 13.0, 5.0, 17.0, 9.0, 21.0]
    same = view.reshape(4, 3, 2)
    assert same.stride() == view.stride() and same.shares_storage_with(view)
    flat = view.reshape(24)
    assert flat.stride() == (1,) and not flat.shares_storage_with(view)
    assert np.array_equal(flat.numpy(), view.numpy().reshape(-1))
    with pytest.raises(RuntimeError, match="view size is not compatible"):
        view.view(24)
    assert source.view(6, 4).shares_storage_with(source)


@pytest.mark.parametrize("seed", range(12))
def test_reshape_and_clone_layouts_match_the_checker(seed):
    rng = np.random.default_rng(seed)
    base = rnd(seed, 4, 6, 5)
    t, r = torch.tensor(base, device=DEV), RefTensor.from_numpy(base)
    perm = [int(p) for p in rng.permutation(3)]
    tv, rv = t.permute(*perm), r.permute(perm)
    if rng.integers(0, 2):
        tv, rv = tv[1], rv.select0(1)
    shape = list(rv.shape)
    targets = [[-1], [shape[0], -1], shape[::-1], shape + [1], [1] + shape]
    if len(shape) == 3:
        targets.append([shape[0] * shape[1], shape[2]])
    for target in targets:
        got, want = tv.reshape(*target), rv.reshape(target)
        assert list(got.shape) == want.shape and list(got.stride()) == want.strides and got.storage_offset() == want.offset
        assert got.shares_storage_with(tv) == (rv.view_strides(want.shape) is not None)
        assert np.array_equal(got.numpy().view(np.uint32), want.logical().view(np.uint32))
    c, rc = tv.clone(), rv.clone()
    assert list(c.stride()) == rc.strides and c.storage_offset() == 0
    assert np.array_equal(c.numpy(), rv.logical())
    packed = tv.contiguous()
    assert packed.is_contiguous() and np.array_equal(packed.numpy(), rv.logical())
    assert np.array_equal(tv.flatten().numpy(), rv.logical().reshape(-1))
    assert np.array_equal(tv.ravel().numpy(), rv.logical().reshape(-1))


def test_reshape_errors():
    t = torch.zeros(2, 3, device=DEV)
    with pytest.raises(RuntimeError, match=r"shape '\[4, 2\]' is invalid for input of size 6"):
        t.reshape(4, 2)
    with pytest.raises(RuntimeError, match="only one dimension can be inferred"):
        t.reshape(-1, -1)
    with pytest.raises(RuntimeError, match="ambiguous"):
        torch.zeros(0, device=DEV).reshape(0, -1)


def test_equal_follows_ieee_comparison():
    a = np.array([[1.0, -0.0, 3.5], [np.inf, 2.0, -7.0]], dtype=np.float32)
    ta = torch.tensor(a, device=DEV)
    assert torch.equal(ta, torch.tensor(a.copy(), device=DEV))
    b = a.copy()
    b[0, 1] = 0.0                                  # -0.0 == +0.0
    assert ta.equal(torch.tensor(b, device=DEV))
    b[1, 2] = -7.000001
    assert not ta.equal(torch.tensor(b, device=DEV))
    n = a.copy()
    n[0, 0] = np.nan
    tn = torch.tensor(n, device=DEV)
    assert not tn.equal(tn)                        # NaN equals nothing, itself included
    assert not ta.equal(torch.tensor(a.reshape(3, 2), device=DEV))
    assert ta.T.equal(torch.tensor(np.ascontiguousarray(a.T), device=DEV))     # logical values, not layout
    assert torch.zeros(0, 3, device=DEV).equal(torch.zeros(0, 3, device=DEV))
    assert torch.eye(3, device=DEV).numpy().tolist() == np.eye(3).tolist()


def test_gradients_flow_back_through_reshape_clone_and_contiguous():
    g = GOLD["autograd"]["transposed_reshape"]
    leaf = torch.tensor(np.array(g["leaf"], dtype=np.float32).reshape(g["leaf_shape"]), device=DEV, requires_grad=True)
    weights = torch.tensor(np.array(g["weights"], dtype=np.float32), device=DEV)
    copy = leaf.transpose(0, 1).reshape(6)          # not viewable: a packed copy
    assert copy.requires_grad and copy._grad_fn_name() == "ViewBackward0"
    (copy * weights).sum().backward()
    assert leaf.grad.numpy().reshape(-1).tolist() == g["grad"]

    leaf2 = torch.tensor(np.arange(1, 7, dtype=np.float32).reshape(1, 2, 3), device=DEV, requires_grad=True)
    packed = leaf2.permute(2, 0, 1).contiguous()     # [3,1,2]
    picked = packed.reshape(3, 2)[1].reshape(2, 1).clone()
    (picked * picked).sum().backward()
    # tests/autograd.rs:1098-1120 (the same mapping without its squeeze step): d/dx x^2 at elements 2 and 5
    assert leaf2.grad.numpy().reshape(-1).tolist() == [0.0, 4.0, 0.0, 0.0, 10.0, 0.0]


def test_squeeze_and_unbind_views_and_their_gradients():
    # the full mapping of tests/autograd.rs:1098-1120: permute -> contiguous -> squeeze -> index -> reshape -> clone
    leaf = torch.tensor(np.arange(1, 7, dtype=np.float32).reshape(1, 2, 3), device=DEV, requires_grad=True)
    packed = leaf.permute(2, 0, 1).contiguous()
    squeezed = packed.squeeze(1)
    assert squeezed.shape == (3, 2) and squeezed.requires_grad and squeezed.shares_storage_with(packed)
    cloned = squeezed[1].reshape(2, 1).clone()
    (cloned * cloned).sum().backward()
    assert leaf.grad.numpy().reshape(-1).tolist() == [0.0, 4.0, 0.0, 0.0, 10.0, 0.0]

    t = torch.tensor(rnd(1, 1, 4, 1, 5), device=DEV)
    assert t.squeeze().shape == (4, 5) and t.squeeze().stride() == (5, 1)
    assert t.squeeze(0).shape == (4, 1, 5) and t.squeeze(1).shape == (1, 4, 1, 5) and t.squeeze(-2).shape == (1, 4, 5)
    with pytest.raises(IndexError, match="Dimension out of range"):
        t.squeeze(4)

    w = torch.tensor(rnd(2, 3, 4), device=DEV, requires_grad=True)
    a, b, c = w.unbind(0)
    (a * 2.0 + c).sum().backward()
    want = np.zeros((3, 4), dtype=np.float32)
    want[0], want[2] = 2.0, 1.0
    assert np.array_equal(w.grad.numpy(), want)
