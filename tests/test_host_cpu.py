"""CPU-side checks of the host engine library: exports, layout planner vs the checker, error strings."""
import ctypes
import os
import re

import pytest

from torch_rs import _host

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "trs_host.h")


def test_host_library_exports_every_declared_symbol():
    text = open(HEADER).read()
    names = sorted(set(re.findall(r"^(?:int32_t|const char\*)\s+(trsh_[a-z0-9_]+)\s*\(", text, flags=re.M)))
    lib = ctypes.CDLL(_host.LIB_PATH)
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_host.EXPORTS) == names


def test_cuda_tensor_creation_fails_loudly_without_a_device():
    import torch_rs as torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError, match="no CUDA device"):
        torch.tensor([1.0, 2.0], device="cuda")
    with pytest.raises(RuntimeError, match="never falls back to the CPU"):
        torch.tensor([1.0], device="cpu")
    with pytest.raises(RuntimeError, match="pass device='cuda'"):
        torch.zeros(3)


def _arr(values):
    return (ctypes.c_int64 * max(len(values), 1))(*values)


def _random_view(rng):
    """A random dense-or-sliced view: permuted contiguous base, optional singleton and step-2 axes."""
    rank = int(rng.integers(0, 5))
    base = [int(rng.choice([1, 2, 3, 4, 5])) for _ in range(rank)]
    strides, s = [0] * rank, 1
    for axis in range(rank - 1, -1, -1):
        step = int(rng.choice([1, 1, 1, 2]))
        strides[axis] = s * step
        s *= base[axis] * step
    perm = list(rng.permutation(rank)) if rank else []
    return [base[p] for p in perm], [strides[p] for p in perm]


def test_layout_planner_matches_the_checker_on_random_views():
    import numpy as np
    from oracle import ref
    lib = _host.lib()
    rng = np.random.default_rng(123)
    checked = 0
    for _ in range(3000):
        shape, strides = _random_view(rng)
        out = _arr([0] * len(shape))
        assert lib.trsh_plan_unary(len(shape), _arr(shape), _arr(strides), out) == 0
        assert list(out)[:len(shape)] == ref.unary_strides(shape, strides)
        assert lib.trsh_plan_scalar(len(shape), _arr(shape), _arr(strides), out) == 0
        assert list(out)[:len(shape)] == ref.scalar_strides(shape, strides)
        other_shape, other_strides = _random_view(rng)
        if rng.random() < 0.5:           # same-shape partner with another layout
            other_shape = list(shape)
            order = list(rng.permutation(len(shape)))
            other_strides, s = [0] * len(shape), 1
            for axis in order:
                other_strides[axis] = s
                s *= max(shape[axis], 1)
        rank = ctypes.c_int32()
        oshape, ostrides = _arr([0] * 8), _arr([0] * 8)
        status = lib.trsh_plan_binary(len(shape), _arr(shape), _arr(strides), len(other_shape), _arr(other_shape),
                                      _arr(other_strides), ctypes.byref(rank), oshape, ostrides)
        try:
            want_shape, want_strides = ref.binary_plan(shape, strides, other_shape, other_strides)
        except ref.RefError as err:
            assert err.kind == "ShapeMismatch" and status == 1
            continue
        assert status == 0
        assert list(oshape)[:rank.value] == want_shape and list(ostrides)[:rank.value] == want_strides
        checked += 1
    assert checked > 500


def test_layout_planner_reference_goldens():
    import json
    lib = _host.lib()
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))["strides"]
    g = gold["singleton_channels_last"]
    out = _arr([0] * 4)
    assert lib.trsh_plan_unary(4, _arr(g["view_shape"]), _arr(g["view_strides"]), out) == 0
    assert list(out) == g["expected"]
    for case in gold["empty_scalar_op"]["cases"]:
        n = len(case["shape"])
        strides, s = [0] * n, 1
        for axis in range(n - 1, -1, -1):
            strides[axis] = s
            s *= max(case["shape"][axis], 1)
        out = _arr([0] * n)
        assert lib.trsh_plan_scalar(n, _arr(case["shape"]), _arr(strides), out) == 0
        assert list(out)[:n] == case["expected"]
    rank = ctypes.c_int32()
    oshape, ostrides = _arr([0] * 8), _arr([0] * 8)
    status = lib.trsh_plan_binary(1, _arr([0]), _arr([1]), 1, _arr([2]), _arr([1]), ctypes.byref(rank), oshape, ostrides)
    assert status == 1
    assert b"The size of tensor a (0) must match the size of tensor b (2) at non-singleton dimension 0" in lib.trsh_last_error()


def test_layout_planner_remaining_reference_stride_goldens():
    """Every stride case the reference's own tests hold for this path, asserted on the host planner itself (the
    planner and the CPU checker's planner are translations of the same rules by the same hand, so comparing them
    with each other proves little; these vectors are the independent pin): dense views keep their strides through
    unary / scalar / same-layout binary / row-broadcast ops (tests/tensor_baseline.rs:1606-1658,
    tests/test_transpose.py:244-259), empty operands (tensor_baseline.rs:2189-2211), a rank-0 operand against a
    transposed view (tests/autograd.rs:190-218), reflected division (tests/test_transpose.py:288-313)."""
    import json
    lib = _host.lib()
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))

    def unary(shape, strides):
        out = _arr([0] * max(len(shape), 1))
        assert lib.trsh_plan_unary(len(shape), _arr(shape), _arr(strides), out) == 0
        return list(out)[:len(shape)]

    def scalar(shape, strides):
        out = _arr([0] * max(len(shape), 1))
        status = lib.trsh_plan_scalar(len(shape), _arr(shape), _arr(strides), out)
        return list(out)[:len(shape)] if status == 0 else status

    def binary(ls, lst, rs, rst):
        rank = ctypes.c_int32()
        oshape, ostrides = _arr([0] * 8), _arr([0] * 8)
        assert lib.trsh_plan_binary(len(ls), _arr(ls), _arr(lst), len(rs), _arr(rs), _arr(rst), ctypes.byref(rank), oshape, ostrides) == 0
        return list(oshape)[:rank.value], list(ostrides)[:rank.value]

    def contiguous(shape):
        strides, s = [0] * len(shape), 1
        for axis in range(len(shape) - 1, -1, -1):
            strides[axis] = s
            s *= max(shape[axis], 1)
        return strides

    g = gold["strides"]["unary_keeps_dense_view"]
    shape, strides = g["view_shape"], g["view_strides"]
    assert unary(shape, strides) == strides                                   # relu / sin / exp
    assert scalar(shape, strides) == strides                                  # view + 2.0
    assert binary(shape, strides, shape, strides) == (shape, strides)         # view + view
    assert binary(shape, strides, [2], [1]) == (shape, strides)               # view + row of two
    transposed = ([4, 3], [1, 4])                                            # the rank-2 slice of the same test
    assert unary(*transposed) == transposed[1]
    g = gold["strides"]["singleton_channels_last"]
    assert binary(g["view_shape"], g["view_strides"], g["view_shape"], g["view_strides"])[1] == g["expected"]
    for case in gold["strides"]["empty_binary"]["cases"]:
        assert binary(case["left"], contiguous(case["left"]), case["right"], contiguous(case["right"])) == (case["shape"], case["expected"])
    c = gold["strides"]["empty_binary"]["chained_relu_after_scalar"]
    after_scalar = scalar(c["shape"], contiguous(c["shape"]))
    assert after_scalar == c["scalar_strides"] and unary(c["shape"], after_scalar) == c["relu_strides"]
    g = gold["strides"]["rank_zero_mul_view"]
    assert binary(g["view_shape"], g["view_strides"], [], []) == (g["view_shape"], g["expected"])
    assert binary([], [], g["view_shape"], g["view_strides"]) == (g["view_shape"], g["expected"])

    # reflected division is planned as reciprocal (a unary op) followed by a scalar op (src/tensor.rs:2324-2363)
    d = gold["reflected_division"]
    view = d["view"]
    assert scalar(view["shape"], view["strides"]) == d["div_one_strides"]
    assert scalar(view["shape"], unary(view["shape"], view["strides"])) == d["reflected_strides"]
    for case in d["empty_cases"] + [d["large"]]:
        assert scalar(case["shape"], unary(case["shape"], case["strides"])) == case["expected"]
    e = d["extreme_transposed"]
    out = _arr([0] * 3)
    assert lib.trsh_plan_unary(3, _arr(e["shape"]), _arr(e["strides"]), out) == 11           # StrideCalculationOverflow


def test_layout_planner_extreme_empty_goldens():
    import json
    lib = _host.lib()
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))
    for case in gold["extreme_empty_strides"]["cases"]:
        n = len(case["shape"])
        out = _arr([0] * n)
        assert lib.trsh_plan_scalar(n, _arr(case["shape"]), _arr(case["strides"]), out) == 0
        assert list(out)[:n] == case["scalar_expected"]
        if "unary_error" in case:
            assert lib.trsh_plan_unary(n, _arr(case["shape"]), _arr(case["strides"]), out) == 11      # StrideCalculationOverflow


def test_memory_format_planner_matches_the_checker_and_the_reference_goldens():
    """clone(memory_format) / contiguous(memory_format) layout decisions: random rank-4/5 views against the
    CPU checker, plus the stride goldens of tests/tensor_baseline.rs:2476-2610, 2698-2770."""
    import json
    import os
    import numpy as np
    from oracle import ref
    lib = _host.lib()

    def plan(fmt, for_clone, shape, strides):
        out, copies = _arr([0] * max(len(shape), 1)), ctypes.c_int32()
        status = lib.trsh_plan_memory_format(fmt, for_clone, len(shape), _arr(shape), _arr(strides), ctypes.byref(copies), out)
        return status, bool(copies.value), list(out)[:len(shape)]

    rng = np.random.default_rng(321)
    for _ in range(2000):
        rank = int(rng.choice([3, 4, 5]))
        base = [int(rng.choice([0, 1, 1, 2, 3, 4])) if rng.random() < 0.9 else 1 for _ in range(rank)]
        strides, s = [0] * rank, 1
        for axis in range(rank - 1, -1, -1):
            step = int(rng.choice([1, 1, 1, 2]))
            strides[axis] = s * step
            s *= max(base[axis], 1) * step
        perm = list(rng.permutation(rank))
        shape, strides = [base[p] for p in perm], [strides[p] for p in perm]
        for name, fmt in ref.MEMORY_FORMATS.items():
            for for_clone in (1, 0):
                want = (ctypes.c_int64 * max(rank, 1))()
                want_status = ref.lib().ref_memory_format_strides(fmt, for_clone, rank, _arr(shape), _arr(strides), want)
                shares = (not for_clone) and want_status in (0, 9) and (fmt < 2 or rank == {2: 4, 3: 5}[fmt]) and bool(
                    ref.lib().ref_is_contiguous_in_format(fmt, rank, _arr(shape), _arr(strides)))
                status, copies, got = plan(fmt, for_clone, shape, strides)
                if shares:
                    assert status == 0 and not copies, (name, shape, strides)
                elif want_status == 0:
                    assert status == 0 and copies and got == list(want)[:rank], (name, for_clone, shape, strides)
                else:
                    assert status == {8: 25, 9: 24, 2: 11}[want_status], (name, for_clone, shape, strides, status, want_status)

    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))["memory_format"]["contiguous"]
    for case in gold["empty_cases"]:
        shape = case["shape"]
        assert plan(2, 0, shape, ref.contiguous_strides(shape)) == (0, True, case["expected"])
    shape = gold["empty_volume"]["shape"]
    assert plan(3, 0, shape, ref.contiguous_strides(shape)) == (0, True, gold["empty_volume"]["expected"])
    assert plan(2, 0, gold["singleton"]["shape"], gold["singleton"]["strides"])[:2] == (0, False)
    assert plan(2, 0, gold["arange_shape"], [12, 4, 2, 1]) == (0, True, gold["channels_last_strides"])
    assert plan(3, 1, [1, 2, 3, 4], [24, 12, 4, 1])[0] == 25          # ContiguousMemoryFormatRankMismatch
    assert "required rank 5 tensor to use channels_last_3d format" in lib.trsh_last_error().decode()
    assert plan(0, 0, [2, 3], [1, 2])[0] == 24                       # ContiguousPreserveFormatUnsupported
