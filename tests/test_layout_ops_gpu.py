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


# ---- memory formats: clone / contiguous / is_contiguous with channels_last and channels_last_3d ---------------

FORMATS = {"preserve_format": torch.preserve_format, "contiguous_format": torch.contiguous_format,
           "channels_last": torch.channels_last, "channels_last_3d": torch.channels_last_3d}


def _bits(values):
    return np.array([int(h, 16) for h in values], dtype=np.uint32).view(np.float32)


def _format_source(case, patterns):
    values = _bits([patterns[i % len(patterns)] for i in range(case["count"])])
    if "outer_shape" in case:
        return torch.tensor(values.reshape(case["outer_shape"]), device=DEV)[case["select0"]]
    t = torch.tensor(values.reshape(case["shape"]), device=DEV)
    return t.transpose(*case["transpose"]) if "transpose" in case else t


def test_reference_goldens_for_channel_last_clones():
    m = GOLD["memory_format"]
    for key, fmt in (("clone_channels_last", "channels_last"), ("clone_channels_last_3d", "channels_last_3d")):
        for case in m[key]["cases"]:
            src = _format_source(case, m["bit_patterns"])
            out = src.clone(memory_format=FORMATS[fmt])
            assert list(out.stride()) == case["expected_strides"], (key, case["name"])
            assert out.shape == src.shape and out.storage_offset() == 0
            assert out.is_contiguous(memory_format=FORMATS[fmt]) and not out.shares_storage_with(src)
            # a copy moves bits: signed zeros, denormals, infinities and NaN payloads survive
            assert np.array_equal(out.numpy().view(np.uint32), src.numpy().view(np.uint32))
    err = m["clone_channels_last_3d"]["rank_error"]
    with pytest.raises(RuntimeError, match=err["message"]):
        torch.zeros(*err["shape"], device=DEV).clone(memory_format=torch.channels_last_3d)


def test_reference_goldens_for_contiguous_with_memory_format():
    c = GOLD["memory_format"]["contiguous"]
    src = torch.tensor(np.arange(24, dtype=np.float32).reshape(c["arange_shape"]), device=DEV)
    cl = src.contiguous(memory_format=torch.channels_last)
    assert list(cl.stride()) == c["channels_last_strides"] and cl.storage_offset() == 0
    assert cl.is_contiguous(memory_format=torch.channels_last) and not cl.is_contiguous() and not cl.shares_storage_with(src)
    assert cl.numpy().reshape(-1).tolist() == list(range(24))
    assert cl.contiguous(memory_format=torch.channels_last).shares_storage_with(cl)
    cloned = cl.clone()
    assert list(cloned.stride()) == c["channels_last_strides"] and not cloned.shares_storage_with(cl)
    row_major = cl.contiguous(memory_format=torch.contiguous_format)
    assert list(row_major.stride()) == c["row_major_strides"] and not row_major.shares_storage_with(cl)
    assert row_major.numpy().reshape(-1).tolist() == list(range(24))
    assert list((cl + 1.0).stride()) == c["add_scalar_strides"]
    assert cl.sum().item() == c["sum"]
    vol = torch.tensor(np.arange(48, dtype=np.float32).reshape(c["volume_shape"]), device=DEV)
    v3 = vol.contiguous(memory_format=torch.channels_last_3d)
    assert list(v3.stride()) == c["channels_last_3d_strides"] and v3.is_contiguous(memory_format=torch.channels_last_3d)
    assert v3.numpy().reshape(-1).tolist() == list(range(48)) and not v3.shares_storage_with(vol)
    single = torch.zeros(*c["singleton"]["shape"], device=DEV)
    kept = single.contiguous(memory_format=torch.channels_last)
    assert kept.shares_storage_with(single) and list(kept.stride()) == c["singleton"]["strides"]
    for case in c["empty_cases"]:
        out = torch.zeros(*case["shape"], device=DEV).contiguous(memory_format=torch.channels_last)
        assert list(out.stride()) == case["expected"] and out.is_contiguous(memory_format=torch.channels_last)
    out = torch.zeros(*c["empty_volume"]["shape"], device=DEV).contiguous(memory_format=torch.channels_last_3d)
    assert list(out.stride()) == c["empty_volume"]["expected"]
    with pytest.raises(RuntimeError, match=c["rank_error_message"]):
        torch.zeros(2, 3, device=DEV).contiguous(memory_format=torch.channels_last)
    with pytest.raises(RuntimeError, match="preserve memory format is unsupported by the contiguous operator"):
        src.mT.contiguous(memory_format=torch.preserve_format)
    with pytest.raises(TypeError, match="must be torch.memory_format, not str"):
        src.contiguous(memory_format="channels_last")


def test_memory_format_queries_match_reference_goldens():
    for case in GOLD["memory_format"]["queries"]["cases"]:
        count = int(np.prod(case["shape"]))
        # rebuild the strided view from a permutation of a contiguous tensor: order axes by descending stride
        order = sorted(range(len(case["shape"])), key=lambda a: (-case["strides"][a], a))
        base = torch.zeros(*[case["shape"][a] for a in order], device=DEV)
        inverse = [order.index(a) for a in range(len(order))]
        view = base.permute(*inverse)
        if count:                                              # for empty tensors the strides are not unique
            assert list(view.stride()) == case["strides"]
            for name, fmt in FORMATS.items():
                if name in case:
                    assert view.is_contiguous(memory_format=fmt) == case[name], (case, name)


def test_channel_last_clone_gradients_are_identity():
    for case in GOLD["memory_format"]["autograd_clone"]["cases"]:
        n = int(np.prod(case["shape"]))
        leaf = torch.tensor(np.arange(1, n + 1, dtype=np.float32).reshape(case["shape"]), device=DEV, requires_grad=True)
        src = leaf.transpose(*case["transpose"])
        cloned = src.clone(memory_format=FORMATS[case["format"]])
        assert list(cloned.stride()) == case["strides"] and cloned.requires_grad and not cloned.is_leaf
        del src
        cloned.sum().backward()
        assert np.array_equal(leaf.grad.numpy(), np.full(case["shape"], case["grad"], dtype=np.float32))
        with torch.no_grad():
            quiet = leaf.transpose(*case["transpose"]).clone(memory_format=FORMATS[case["format"]])
        assert list(quiet.stride()) == case["strides"] and not quiet.requires_grad and quiet.is_leaf


@pytest.mark.parametrize("seed", range(10))
def test_memory_format_copies_match_the_checker(seed):
    rng = np.random.default_rng(100 + seed)
    rank = 4 if seed % 2 == 0 else 5
    shape = [int(d) for d in rng.integers(1, 7, rank)]
    base = rnd(seed, *shape)
    perm = [int(p) for p in rng.permutation(rank)]
    t, r = torch.tensor(base, device=DEV).permute(*perm), RefTensor.from_numpy(base).permute(perm)
    fmt = "channels_last" if rank == 4 else "channels_last_3d"
    for name in ("preserve_format", "contiguous_format", fmt):
        got, want = t.clone(memory_format=FORMATS[name]), r.clone(name)
        assert list(got.stride()) == want.strides, (name, shape, perm)
        assert np.array_equal(got.numpy().view(np.uint32), want.logical().view(np.uint32))
        assert t.is_contiguous(memory_format=FORMATS[name]) == r.is_contiguous_in(name)
    for name in ("contiguous_format", fmt):
        got, want = t.contiguous(memory_format=FORMATS[name]), r.contiguous(name)
        assert list(got.stride()) == want.strides and got.shares_storage_with(t) == (want is r)
        assert np.array_equal(got.numpy().view(np.uint32), want.logical().view(np.uint32))
        # ops on the copy keep its layout (channel-last precedence of the output-stride rule)
        assert list(got.relu().stride()) == want.relu().strides


def test_channels_last_copy_of_a_large_tensor_runs_at_memory_speed_layout():
    # [N, C, H, W] = [8, 64, 56, 56] -> channel-last and back; both directions transpose C against H*W
    x = rnd(7, 8, 64, 56, 56)
    t = torch.tensor(x, device=DEV)
    cl = t.contiguous(memory_format=torch.channels_last)
    assert list(cl.stride()) == [64 * 56 * 56, 1, 56 * 64, 64]
    assert np.array_equal(cl.numpy(), x)
    back = cl.contiguous()
    assert back.is_contiguous() and np.array_equal(back.numpy(), x)
