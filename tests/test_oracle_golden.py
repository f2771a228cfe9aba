"""Pins the CPU checker (oracle/) against the golden vectors of the reference's own tests.

Each case names the reference test it comes from (see tests/golden/reference_vectors.json).
"""
import json
import math
import os

import numpy as np
import pytest

from oracle import ref
from oracle.ref import RefTensor

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))


def f32_from_hex(items):
    return np.array([int(h, 16) for h in items], dtype=np.uint32).view(np.float32)


def bits(array):
    return [f"{b:08x}" for b in np.ascontiguousarray(array, dtype=np.float32).reshape(-1).view(np.uint32)]


def build_operand(spec):
    if "values" in spec:
        t = RefTensor(np.array(spec["values"], dtype=np.float32), spec["shape"])
    else:
        start = spec["arange_from"]
        t = RefTensor(np.arange(start, start + spec["count"], dtype=np.float32), spec["shape"])
    if "select0" in spec:
        t = t.select0(spec["select0"])
    if "transpose" in spec:
        t = t.transpose(*spec["transpose"])
    return t


def test_relu_bits_offset_and_transposed_views():
    g = GOLD["relu_bits"]
    storage = np.concatenate([np.ones(12, dtype=np.float32), f32_from_hex(g["input"])])
    base = RefTensor(storage, g["base_shape"])
    view = base.select0(1)
    assert view.offset == 12
    out = view.relu()
    assert out.strides == view.strides and out.offset == 0
    assert bits(out.logical()) == g["expected"]
    strided = view.transpose(0, 1)
    assert strided.shape == [4, 3] and strided.strides == [1, 4]
    sout = strided.relu()
    assert sout.strides == strided.strides and sout.offset == 0
    assert bits(sout.logical()) == g["transposed_expected"]
    for zero in ("80000000", "00000000"):
        scalar = RefTensor(f32_from_hex([zero]), [])
        assert bits(scalar.relu().logical()) == [zero]


def test_relu_vjp_bits():
    g = GOLD["relu_vjp_bits"]
    leaf = RefTensor(f32_from_hex(g["input"]), [12])
    weights = f32_from_hex(g["weights"])
    # Sum VJP fills 1.0 (tensor.rs:3008-3013); Multiply VJP gives upstream*weights with the first
    # contribution stored (tensor.rs:3066-3077, 3220-3227); then the relu VJP.
    upstream = ref.unbroadcast(np.ones(12, dtype=np.float32), [12], [12], RefTensor(weights, [12]))
    grad = leaf.relu_vjp(upstream)
    assert bits(grad) == g["expected_gradient"]


def test_exp_ordinary_and_special():
    g = GOLD["exp_ordinary"]
    out = RefTensor(np.array(g["input"], dtype=np.float32), [2, 2, 3]).exp().logical().reshape(-1)
    atol = float(f32_from_hex([g["atol_bits"]])[0])
    for actual, expected in zip(out, g["expected"]):
        assert abs(float(actual) - expected) <= atol + g["rtol"] * abs(expected)
    s = GOLD["exp_special"]
    out = RefTensor(f32_from_hex(s["input_bits"]), [11]).exp().logical()
    for value, cls in zip(out, s["classes"]):
        b = int(np.float32(value).view(np.uint32))
        if cls == "one":
            assert b == 0x3F800000
        elif cls == "subnormal":
            assert 0 < b < 0x00800000
        elif cls == "pos_zero":
            assert b == 0
        elif cls == "finite":
            assert math.isfinite(float(value))
        elif cls == "pos_inf":
            assert b == 0x7F800000
        elif cls == "nan":
            assert math.isnan(float(value))


def test_broadcast_arithmetic_values():
    g = GOLD["broadcast_arithmetic"]
    left, right = build_operand(g["left"]), build_operand(g["right"])
    for op in ("add", "sub", "mul", "div"):
        out = left.binary(op, right)
        assert out.shape == g["shape"]
        assert out.logical().reshape(-1).tolist() == g[op]
    r = GOLD["rank_zero_arithmetic"]
    scalar, matrix = RefTensor([r["scalar"]], []), build_operand(r["matrix"])
    assert matrix.binary("add", scalar).logical().reshape(-1).tolist() == r["matrix_add_scalar"]
    assert scalar.binary("sub", matrix).logical().reshape(-1).tolist() == r["scalar_sub_matrix"]


def test_empty_broadcast_and_mismatch():
    g = GOLD["empty_broadcast"]
    for case in g["cases"]:
        left = RefTensor(np.zeros(int(np.prod(case["left"])), dtype=np.float32), case["left"])
        right = RefTensor(np.ones(int(np.prod(case["right"])), dtype=np.float32), case["right"])
        for op in ("add", "sub", "mul", "div"):
            assert left.binary(op, right).shape == case["shape"]
    with pytest.raises(ref.RefError) as err:
        RefTensor([], g["mismatch"]["left"]).binary("add", RefTensor([1, 1], g["mismatch"]["right"]))
    assert err.value.kind == "ShapeMismatch"


def test_sum():
    cases = GOLD["sum"]["cases"]
    assert RefTensor(cases[0]["values"], cases[0]["shape"]).sum() == cases[0]["expected"]
    t = RefTensor(np.arange(cases[1]["arange"], dtype=np.float32), cases[1]["shape"]).transpose(*cases[1]["transpose"])
    assert t.sum() == cases[1]["expected"]
    assert abs(RefTensor([], [0]).sum()) == 0.0


def test_matmul_known_results():
    for case in GOLD["matmul"]["cases"]:
        out = build_operand(case["left"]).matmul(build_operand(case["right"]))
        assert out.shape == case["shape"] and out.strides == ref.contiguous_strides(case["shape"])
        assert out.logical().reshape(-1).tolist() == case["expected"]
    for left, right in GOLD["matmul"]["inner_mismatch"]["pairs"]:
        with pytest.raises(ref.RefError) as err:
            RefTensor(np.zeros(int(np.prod(left))), left).matmul(RefTensor(np.zeros(int(np.prod(right))), right))
        assert err.value.kind == "MatmulInnerDimensionMismatch"


def test_matmul_blocked_path_equals_strided_loop_bits():
    # The reference's in-crate tests pin "fast path == fallback" bitwise (src/tensor.rs:4712-4886):
    # the 4-row blocked kernel must keep the k-ascending order of the strided loop.
    rng = np.random.default_rng(7)
    a = rng.standard_normal((9, 70)).astype(np.float32)
    b = rng.standard_normal((70, 64)).astype(np.float32)
    fast = RefTensor.from_numpy(a).matmul(RefTensor.from_numpy(b)).logical()
    bt = RefTensor.from_numpy(np.ascontiguousarray(b.T)).transpose(0, 1)      # same values, strided view
    slow = RefTensor.from_numpy(a).matmul(bt).logical()
    assert np.array_equal(fast.view(np.uint32), slow.view(np.uint32))
    expected = np.zeros((9, 64), dtype=np.float32)
    for k in range(70):
        expected += (a[:, k:k + 1] * b[k:k + 1, :]).astype(np.float32)
    assert np.array_equal(fast.view(np.uint32), expected.view(np.uint32))


def test_stride_rules():
    s = GOLD["strides"]
    g = s["unary_keeps_dense_view"]
    view = RefTensor(np.arange(24, dtype=np.float32), g["base_shape"]).transpose(*g["transpose"])
    assert view.shape == g["view_shape"] and view.strides == g["view_strides"]
    for op in ("relu", "sin", "exp"):
        out = view.unary(op)
        assert out.strides == view.strides and out.offset == 0
    row = RefTensor(g["broadcast_row"], [2])
    out = view.binary("add", row)
    assert out.strides == view.strides
    assert out.logical().reshape(-1)[:6].tolist() == g["broadcast_first6"]

    g = s["singleton_channels_last"]
    view = RefTensor(np.arange(4, dtype=np.float32), g["view_shape"], g["view_strides"])
    assert view.relu().strides == g["expected"]
    assert view.binary("add", view).strides == g["expected"]

    for case in s["empty_scalar_op"]["cases"]:
        t = RefTensor([], case["shape"])
        assert t.scalar("add", 1.0).strides == case["expected"]
    for case in s["empty_binary"]["cases"]:
        out = RefTensor([], case["left"]).binary("add", RefTensor(np.ones(int(np.prod(case["right"]))), case["right"]))
        assert out.shape == case["shape"] and out.strides == case["expected"]
    c = s["empty_binary"]["chained_relu_after_scalar"]
    chained = RefTensor([], c["shape"]).scalar("add", 1.0)
    assert chained.strides == c["scalar_strides"]
    assert chained.relu().strides == c["relu_strides"]

    g = s["rank_zero_mul_view"]
    view = RefTensor(np.arange(12, dtype=np.float32), g["view_shape"], g["view_strides"], offset=6)
    scalar = RefTensor([2.0], [])
    assert view.binary("mul", scalar).strides == g["expected"]
    assert scalar.binary("mul", view).strides == g["expected"]


def test_autograd_goldens_by_composition():
    a = GOLD["autograd"]
    x = np.array(a["square_sum"]["x"], dtype=np.float32)
    xt = RefTensor(x, [3])
    ones = np.ones(3, dtype=np.float32)
    # Multiply VJP with both operands the same leaf: left grad + right grad accumulate (tensor.rs:3302-3317).
    grad = ref.unbroadcast(ones, [3], [3], xt) + ref.unbroadcast(ones, [3], [3], xt)
    assert grad.tolist() == a["square_sum"]["grad_first"]
    assert (grad + grad).tolist() == a["square_sum"]["grad_second"]

    u = a["unbroadcast_both"]
    left, right = build_operand(u["left"]), build_operand(u["right"])
    ones = np.ones(6, dtype=np.float32)
    assert ref.unbroadcast(ones, [2, 3], [2, 1], right).reshape(-1).tolist() == u["left_grad"]
    assert ref.unbroadcast(ones, [2, 3], [1, 3], left).reshape(-1).tolist() == u["right_grad"]

    t = a["transposed_reshape"]
    upstream = np.array(t["weights"], dtype=np.float32)          # d/d(reshaped_copy) = weights
    grad = ref.permute_vjp(upstream, t["leaf_shape"], [1, 0])     # transpose(0,1) VJP
    assert grad.reshape(-1).tolist() == t["grad"]

    z = a["negative_zero_first"]
    g1 = ref.unbroadcast(np.ones(1, dtype=np.float32), [1], [1], RefTensor([-0.0], [1]))
    assert bits(g1) == [z["same_count_bits"]]
    g2 = ref.unbroadcast(np.ones(2, dtype=np.float32), [2], [], RefTensor([-0.0, -0.0], [2]))
    assert bits(g2) == [z["broadcast_bits"]]


def test_more_reference_goldens_strides_reshape_reflected_division_and_ordering():
    r = GOLD["reshape_view_strides"]
    view = RefTensor(np.arange(24, dtype=np.float32), r["base_shape"]).transpose(*r["transpose"])
    for case in r["cases"]:
        out = view.reshape(case["shape"])
        assert out.strides == case["strides"]
        assert (view.view_strides(case["shape"]) is not None) == case["shares"]
    s = GOLD["singleton_channels_last_reshape"]
    v = RefTensor(np.arange(4, dtype=np.float32), [1, 2, 2, 1], [4, 1, 2, 4])
    out = v.relu()
    assert out.strides == s["output_strides"]
    assert out.reshape(out.shape).strides == s["reshape_same_shape_strides"]

    d = GOLD["reflected_division"]
    view = RefTensor(d["view"]["values"], d["view"]["shape"], d["view"]["strides"])
    assert (view / 1.0).strides == d["div_one_strides"]
    reflected = 1.0 / view
    assert reflected.strides == d["reflected_strides"] and reflected.logical().reshape(-1).tolist() == d["reflected_values"]
    for case in d["empty_cases"] + [d["large"]]:
        assert (1.0 / RefTensor([], case["shape"], case["strides"])).strides == case["expected"]
    with pytest.raises(ref.RefError) as err:
        1.0 / RefTensor([], d["extreme_transposed"]["shape"], d["extreme_transposed"]["strides"])
    assert err.value.kind == d["extreme_transposed"]["error"]

    for case in GOLD["extreme_empty_strides"]["cases"]:
        assert ref.scalar_strides(case["shape"], case["strides"]) == case["scalar_expected"]
        if "unary_error" in case:
            with pytest.raises(ref.RefError) as err:
                ref.unary_strides(case["shape"], case["strides"])
            assert err.value.kind == case["unary_error"]

    m = GOLD["matmul_ordering"]
    out = RefTensor(f32_from_hex(m["left_bits"]), m["left_shape"]).matmul(RefTensor(f32_from_hex(m["right_bits"]), m["right_shape"]))
    assert bits(out.logical())[0] == m["first_element_bits"]


def test_strided_relu_gradients_golden_by_composition():
    g = GOLD["strided_relu_grads"]
    storage = np.concatenate([np.full(12, 9.0, dtype=np.float32), f32_from_hex(g["storage_tail_bits"])])
    source = RefTensor(storage, [2, 3, 4])
    offset = source.select0(1)
    grad = np.zeros((2, 3, 4), dtype=np.float32)
    grad[1] += offset.relu_vjp(np.ones((3, 4), dtype=np.float32))                      # relu(offset).sum()
    strided = offset.transpose(0, 1)
    weights = RefTensor(np.arange(1, 13, dtype=np.float32), [4, 3])
    upstream = ref.unbroadcast(np.ones(12, dtype=np.float32), [4, 3], [4, 3], weights)  # Multiply VJP
    g_strided = strided.relu_vjp(upstream)                                               # logical [4,3]
    grad[1] += ref.permute_vjp(g_strided, [3, 4], [1, 0])                                # transpose VJP
    assert grad.reshape(-1).tolist() == [float(v) for v in g["expected_grad"]]


def _memory_format_source(case, patterns):
    """Builds the source views of the reference's channel-last clone tests from their recipe."""
    values = f32_from_hex([patterns[i % len(patterns)] for i in range(case["count"])])
    if "outer_shape" in case:
        return RefTensor(values, case["outer_shape"]).select0(case["select0"])
    t = RefTensor(values, case["shape"])
    return t.transpose(*case["transpose"]) if "transpose" in case else t


def test_memory_format_goldens():
    m = GOLD["memory_format"]
    for case in m["queries"]["cases"]:
        t = RefTensor(np.zeros(max(int(np.prod(case["shape"])), 0), dtype=np.float32), case["shape"], case["strides"])
        for fmt in ref.MEMORY_FORMATS:
            if fmt in case:
                assert t.is_contiguous_in(fmt) == case[fmt], (case, fmt)
    for key, fmt in (("clone_channels_last", "channels_last"), ("clone_channels_last_3d", "channels_last_3d")):
        for case in m[key]["cases"]:
            src = _memory_format_source(case, m["bit_patterns"])
            out = src.clone(fmt)
            assert out.strides == case["expected_strides"], case["name"]
            assert out.is_contiguous_in(fmt) and out.shape == src.shape
            assert np.array_equal(out.logical().view(np.uint32), src.logical().view(np.uint32))   # NaN payloads survive a copy
    with pytest.raises(ref.RefError) as err:
        RefTensor(np.zeros(24, dtype=np.float32), m["clone_channels_last_3d"]["rank_error"]["shape"]).clone("channels_last_3d")
    assert err.value.kind == m["clone_channels_last_3d"]["rank_error"]["kind"]

    c = m["contiguous"]
    src = RefTensor(np.arange(24, dtype=np.float32), c["arange_shape"])
    cl = src.contiguous("channels_last")
    assert cl.strides == c["channels_last_strides"] and not cl.is_contiguous_in() and cl.is_contiguous_in("channels_last")
    assert cl.logical().reshape(-1).tolist() == src.logical().reshape(-1).tolist()
    assert cl.contiguous("channels_last") is cl                    # matching layout: storage is shared
    assert cl.clone().strides == c["channels_last_strides"]
    assert cl.contiguous().strides == c["row_major_strides"]
    assert (cl + 1.0).strides == c["add_scalar_strides"]
    assert float(cl.sum()) == c["sum"]
    vol = RefTensor(np.arange(48, dtype=np.float32), c["volume_shape"]).contiguous("channels_last_3d")
    assert vol.strides == c["channels_last_3d_strides"]
    single = RefTensor(np.zeros(40, dtype=np.float32), c["singleton"]["shape"])
    assert single.contiguous("channels_last") is single and single.strides == c["singleton"]["strides"]
    for case in c["empty_cases"]:
        assert RefTensor(np.zeros(0, dtype=np.float32), case["shape"]).contiguous("channels_last").strides == case["expected"]
    assert RefTensor(np.zeros(0, dtype=np.float32), c["empty_volume"]["shape"]).contiguous("channels_last_3d").strides == c["empty_volume"]["expected"]
    with pytest.raises(ref.RefError) as err:
        cl.mT.contiguous("preserve_format")
    assert err.value.kind == "ContiguousPreserveFormatUnsupported"
