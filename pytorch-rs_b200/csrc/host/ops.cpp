// The reference Tensor's op methods for CUDA tensors: layout planning as in the reference, a
// pending expression node (or a lazy matmul) instead of an element loop, and the tape entry.
#include <algorithm>

#include "autograd.h"
#include "engine.h"

namespace trsh {

static std::string shape_text(const std::vector<i64>& s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
    return t + "]";
}

// src/tensor.rs:1086-1148
TensorP permute(const TensorP& t, const std::vector<i64>& dims, int node_kind) {
    const size_t rank = t->v.shape.size();
    if (dims.size() != rank)
        throw Error(ErrKind::PermutationRankMismatch, "permute(sparse_coo): number of dimensions in the tensor input does not match the length of the desired ordering of dimensions i.e. input.dim() = " +
                                                          std::to_string(rank) + " is not equal to len(dims) = " + std::to_string(dims.size()));
    std::vector<bool> seen(rank, false);
    std::vector<i64> norm(rank);
    for (size_t i = 0; i < rank; ++i) {
        i64 d = dims[i] < 0 ? dims[i] + (i64)rank : dims[i];
        if (d < 0 || d >= (i64)rank)
            throw Error(ErrKind::PermutationDimensionOutOfRange, "Dimension out of range (expected to be in range of [-" + std::to_string(std::max<size_t>(rank, 1)) +
                                                                     ", " + std::to_string((i64)std::max<size_t>(rank, 1) - 1) + "], but got " + std::to_string(dims[i]) + ")");
        if (seen[d]) throw Error(ErrKind::DuplicatePermutationDimension, "permute(): duplicate dims are not allowed.");
        seen[d] = true;
        norm[i] = d;
    }
    View v{t->v.st, Shape(rank), Shape(rank), t->v.offset};
    for (size_t i = 0; i < rank; ++i) { v.shape[i] = t->v.shape[norm[i]]; v.strides[i] = t->v.strides[norm[i]]; }
    TensorP out = make_tensor(std::move(v));
    out->view_requires_grad = t->requires_grad();
    if (t->requires_grad() && grad_enabled())
        record(out, GK::Permute, node_kind == 1 ? "TransposeBackward0" : "PermuteBackward0", {t.get()}, {}, false, 0.f, norm);
    return out;
}

// select(0, index) / t[index] (src/tensor.rs:1850-1973)
TensorP select0(const TensorP& t, i64 index) {
    if (t->v.shape.empty())
        throw Error(ErrKind::InvalidScalarIndex, "invalid index of a 0-dim tensor. Use `tensor.item()` in Python or `tensor.item<T>()` in C++ to convert a 0-dim tensor to a number");
    const i64 size = t->v.shape[0];
    const i64 wrapped = index < 0 ? index + size : index;
    if (wrapped < 0 || wrapped >= size)
        throw Error(ErrKind::IndexOutOfBounds, "index " + std::to_string(index) + " is out of bounds for dimension 0 with size " + std::to_string(size));
    View v{t->v.st, Shape(t->v.shape.begin() + 1, t->v.shape.end()), Shape(t->v.strides.begin() + 1, t->v.strides.end()),
           t->v.offset + wrapped * t->v.strides[0]};
    TensorP out = make_tensor(std::move(v));
    out->view_requires_grad = t->requires_grad();
    if (t->requires_grad() && grad_enabled()) record(out, GK::Index, "SelectBackward0", {t.get()}, {}, false, 0.f, {}, wrapped);
    return out;
}

// relu / exp / neg / sin / sqrt / reciprocal (src/tensor.rs:2378-2410, 2294, 2348; unary_map 2737-2749)
TensorP unary(const TensorP& t, int op) {
    const Shape strides = unary_output_strides(t->v.shape, t->v.strides);
    TensorP out = pointwise_node(op, 0.f, {t->v}, t->v.shape, strides, t->device());
    if (t->requires_grad() && grad_enabled()) {
        switch (op) {
            case TRS_OP_RELU: record(out, GK::Relu, "ReluBackward0", {t.get()}, {t->v}, true); break;
            case TRS_OP_NEG: record(out, GK::Neg, "NegBackward0", {t.get()}, {}, false); break;
            case TRS_OP_EXP: record(out, GK::Exp, "ExpBackward0", {t.get()}, {out->v}, true); break;
            case TRS_OP_SIN: record(out, GK::Sin, "SinBackward0", {t.get()}, {t->v}, true); break;
            case TRS_OP_SQRT: record(out, GK::Sqrt, "SqrtBackward0", {t.get()}, {t->v}, true); break;
            case TRS_OP_RECIP:   // src/tensor.rs:2348-2353
                throw Error(ErrKind::InvalidArgument, "reciprocal(): autograd recording is not supported");
            default: break;
        }
    }
    return out;
}

// Tensor-scalar forms (src/tensor.rs:2254-2371).  op is ADD/SUB/MUL/DIV; `reflected` selects
// scalar - x and scalar / x.  The scalar is the closure's right operand except when reflected.
TensorP scalar_op(const TensorP& t, int op, float s, bool reflected) {
    const int device = t->device();
    if (reflected && op == TRS_OP_DIV) {
        // scalar_div: planned as reciprocal then scalar op; value is scalar * (1/x) (src/tensor.rs:2324-2363)
        const Shape recip = unary_output_strides(t->v.shape, t->v.strides);
        const Shape strides = scalar_output_strides(t->v.shape, recip);
        TensorP c = pointwise_node(TRS_OP_CONST, s, {}, t->v.shape, strides, device);
        TensorP r = pointwise_node(TRS_OP_RECIP, 0.f, {t->v}, t->v.shape, strides, device);
        // reciprocal op is 1.0 * (1/x); scalar * that keeps the reference's single multiply because 1.0 * y == y
        return pointwise_node(TRS_OP_MUL, 0.f, {c->v, r->v}, t->v.shape, strides, device);
    }
    const Shape strides = scalar_output_strides(t->v.shape, t->v.strides);
    TensorP c = pointwise_node(TRS_OP_CONST, s, {}, t->v.shape, strides, device);
    std::vector<View> args = reflected ? std::vector<View>{c->v, t->v} : std::vector<View>{t->v, c->v};
    TensorP out = pointwise_node(op, 0.f, std::move(args), t->v.shape, strides, device);
    if (t->requires_grad() && grad_enabled()) {
        if (op == TRS_OP_MUL) record(out, GK::MulScalar, "MulBackward0", {t.get()}, {}, true, s);
        else if (op == TRS_OP_ADD) record(out, GK::Identity, "AddBackward0", {t.get()}, {}, false);
        else if (op == TRS_OP_SUB && !reflected) record(out, GK::Identity, "SubBackward0", {t.get()}, {}, false);
        else if (op == TRS_OP_SUB && reflected) record(out, GK::Neg, "RsubBackward1", {t.get()}, {}, false);
    }
    return out;
}

// add / sub / mul / div with broadcasting (zip_map, src/tensor.rs:2535-2557)
TensorP binary(const TensorP& l, const TensorP& r, int op) {
    if (l->device() != r->device())
        throw Error(ErrKind::DeviceMismatch, "Expected all tensors to be on the same device, but found at least two devices, cuda:" +
                                                 std::to_string(l->device()) + " and cuda:" + std::to_string(r->device()) + "!");
    Shape shape, strides;
    binary_plan(l->v.shape, l->v.strides, r->v.shape, r->v.strides, &shape, &strides);
    TensorP out = pointwise_node(op, 0.f, {l->v, r->v}, shape, strides, l->device());
    if ((l->requires_grad() || r->requires_grad()) && grad_enabled()) {
        if (op == TRS_OP_MUL) {
            // each side's values are saved only when the other side has an edge (src/tensor.rs:2223-2225)
            View keep_l = r->meta ? l->v : View{};
            View keep_r = l->meta ? r->v : View{};
            record(out, GK::Mul, "MulBackward0", {l.get(), r.get()}, {keep_l, keep_r}, true);
        } else if (op == TRS_OP_ADD) {
            record(out, GK::Add, "AddBackward0", {l.get(), r.get()}, {}, false);
        } else if (op == TRS_OP_SUB) {
            record(out, GK::Sub, "SubBackward0", {l.get(), r.get()}, {}, false);
        }
    }
    return out;
}

// Rank-2 matmul (src/tensor.rs:2453-2533) extended to rank-3 batches with equal batch sizes.
TensorP matmul(const TensorP& l, const TensorP& r) {
    const Shape& a = l->v.shape;
    const Shape& b = r->v.shape;
    const bool ok_rank = (a.size() == 2 && b.size() == 2) || (a.size() == 3 && b.size() == 3);
    if (!ok_rank)
        throw Error(ErrKind::MatmulRequiresMatrices, "matmul currently requires two rank-2 tensors, got " + shape_text(a) + " and " + shape_text(b));
    if (l->device() != r->device())
        throw Error(ErrKind::DeviceMismatch, "Expected all tensors to be on the same device, but found at least two devices, cuda:" +
                                                 std::to_string(l->device()) + " and cuda:" + std::to_string(r->device()) + "!");
    const i64 m = a[a.size() - 2], k = a[a.size() - 1], k2 = b[b.size() - 2], n = b[b.size() - 1];
    if (k != k2) {
        if (a.size() == 2 && b.size() == 2)
            throw Error(ErrKind::MatmulInnerDimensionMismatch, "mat1 and mat2 shapes cannot be multiplied (" + std::to_string(m) + "x" + std::to_string(k) +
                                                                   " and " + std::to_string(k2) + "x" + std::to_string(n) + ")");
        throw Error(ErrKind::MatmulInnerDimensionMismatch, "matmul inner dimensions differ for " + shape_text(a) + " and " + shape_text(b));
    }
    Shape shape;
    if (a.size() == 3 || b.size() == 3) {
        const i64 ba = a.size() == 3 ? a[0] : b[0], bb = b.size() == 3 ? b[0] : a[0];
        if (ba != bb) throw Error(ErrKind::ShapeMismatch, "The size of tensor a (" + std::to_string(ba) + ") must match the size of tensor b (" + std::to_string(bb) + ") at non-singleton dimension 0");
        shape = {ba, m, n};
    } else {
        shape = {m, n};
    }
    auto node = std::make_shared<Node>();
    node->op = OP_MATMUL;
    node->args = {l->v, r->v};
    node->shape = shape;
    node->strides = contiguous_strides(shape);
    node->n_instr = 1;
    node->n_leaf = 1;
    auto st = std::make_shared<Storage>();
    st->device = l->device();
    st->count = element_count(shape);
    st->node = node;
    if (l->v.st->written_in_place || r->v.st->written_in_place) materialize(st);   // operands that may change are read now
    TensorP out = make_tensor(View{st, shape, node->strides, 0});
    if ((l->requires_grad() || r->requires_grad()) && grad_enabled())
        record(out, GK::Matmul, shape.size() == 3 ? "BmmBackward0" : "MmBackward0", {l.get(), r.get()},
               {r->meta ? l->v : View{}, l->meta ? r->v : View{}}, true);
    return out;
}

// try_clone_with_memory_format (src/tensor.rs:1517-1575): an independent copy at offset 0.  Preserve
// keeps dense strides and packs other views in the same dimension order; the explicit formats lay
// the copy out row-major or channel-last.
TensorP clone(const TensorP& t, MemoryFormat format) {
    Shape strides;
    memory_format_plan(t->v.shape, t->v.strides, format, true, &strides);
    TensorP out = pointwise_node(TRS_OP_COPY, 0.f, {t->v}, t->v.shape, strides, t->device());
    if (t->requires_grad() && grad_enabled()) record(out, GK::Copy, "CloneBackward0", {t.get()}, {}, false);
    return out;
}

// reshape / view (src/tensor.rs:2032-2189): a metadata-only alias when the strides can express the
// new shape, otherwise (reshape only) a packed copy.
TensorP reshape(const TensorP& t, const std::vector<i64>& requested, bool view_only) {
    // resolve_reshape_shape (src/tensor.rs:2057-2125)
    int inferred = -1;
    for (size_t i = 0; i < requested.size(); ++i) {
        if (requested[i] == -1) {
            if (inferred >= 0) throw Error(ErrKind::ReshapeInvalid, "only one dimension can be inferred");
            inferred = (int)i;
        } else if (requested[i] < 0) {
            throw Error(ErrKind::ReshapeInvalid, "invalid shape dimension " + std::to_string(requested[i]) + " at index " +
                                                     std::to_string(i) + " of shape " + shape_text(requested));
        }
    }
    Shape resolved(requested.begin(), requested.end());
    auto mismatch = [&]() {
        return Error(ErrKind::ReshapeInvalid, "shape '" + shape_text(requested) + "' is invalid for input of size " + std::to_string(t->numel));
    };
    if (inferred >= 0) {
        i64 known = 1;
        for (size_t i = 0; i < requested.size(); ++i) if ((int)i != inferred) known *= requested[i];
        if (known == 0) {
            if (t->numel == 0)
                throw Error(ErrKind::ReshapeInvalid, "cannot reshape tensor of 0 elements into shape " + shape_text(requested) +
                                                         " because the unspecified dimension size -1 can be any value and is ambiguous");
            throw mismatch();
        }
        if (t->numel % known != 0) throw mismatch();
        resolved[inferred] = t->numel / known;
    }
    if (element_count(resolved) != t->numel) throw mismatch();

    Shape strides;
    bool viewable;
    if (t->numel == 0) { viewable = true; strides = resolved == t->v.shape ? t->v.strides : contiguous_strides(resolved); }
    else viewable = reshape_view_strides(t->v.shape, t->v.strides, resolved, &strides);
    TensorP out;
    if (viewable) {
        out = make_tensor(View{t->v.st, resolved, strides, t->v.offset});
        out->view_requires_grad = t->requires_grad();
    } else {
        if (view_only)
            throw Error(ErrKind::ViewIncompatibleLayout, "view size is not compatible with input tensor's size and stride (at least one dimension "
                                                         "spans across two contiguous subspaces). Use .reshape(...) instead.");
        TensorP packed;
        {
            // the packing copy is not a tape node of its own: the reshape edge covers it
            const bool was = grad_enabled();
            if (was) set_grad_enabled(false);
            packed = contiguous(t);
            if (was) set_grad_enabled(true);
        }
        out = make_tensor(View{packed->v.st, resolved, contiguous_strides(resolved), 0});
    }
    if (t->requires_grad() && grad_enabled()) record(out, GK::Reshape, "ViewBackward0", {t.get()}, {}, false);
    return out;
}

// squeeze() / squeeze(dim) (src/tensor.rs:1305-1336): drop singleton dimensions, sharing storage; a
// chosen dimension whose size is not 1 gives an unchanged alias.  `dimension` == INT64_MIN means all.
TensorP squeeze(const TensorP& t, i64 dimension) {
    const size_t rank = t->v.shape.size();
    i64 axis = -1;
    if (dimension != INT64_MIN) {
        const i64 r = (i64)std::max<size_t>(rank, 1);
        if (dimension < -r || dimension >= r)
            throw Error(ErrKind::DimensionOutOfRange, "Dimension out of range (expected to be in range of [-" + std::to_string(r) + ", " +
                                                          std::to_string(r - 1) + "], but got " + std::to_string(dimension) + ")");
        axis = rank == 0 ? 0 : (dimension < 0 ? dimension + r : dimension);
    }
    View v{t->v.st, {}, {}, t->v.offset};
    for (size_t a = 0; a < rank; ++a) {
        const bool drop = t->v.shape[a] == 1 && (dimension == INT64_MIN || (i64)a == axis);
        if (drop) continue;
        v.shape.push_back(t->v.shape[a]);
        v.strides.push_back(t->v.strides[a]);
    }
    TensorP out = make_tensor(std::move(v));
    out->view_requires_grad = t->requires_grad();
    if (t->requires_grad() && grad_enabled())
        record(out, GK::Reshape, dimension == INT64_MIN ? "SqueezeBackward0" : "SqueezeBackward1", {t.get()}, {}, false);
    return out;
}

// Tensor equality (PartialEq, src/tensor.rs:286-293): same shape and every pair of logical values
// compares equal under IEEE rules (NaN equals nothing, -0.0 equals +0.0).
bool equal(const TensorP& a, const TensorP& b) {
    if (a->v.shape != b->v.shape || a->device() != b->device()) return false;
    if (a->numel == 0) return true;
    const bool was = grad_enabled();
    if (was) set_grad_enabled(false);
    TensorP differing = pointwise_node(TRS_OP_NE, 0.f, {a->v, b->v}, a->v.shape, contiguous_strides(a->v.shape), a->device());
    TensorP count = sum(differing);
    if (was) set_grad_enabled(true);
    return item(*count) == 0.0f;
}

// Tensor::sum (src/tensor.rs:2413-2431): all elements -> rank-0 tensor.
TensorP sum(const TensorP& t) {
    const int device = t->device();
    materialize(t->v.st);
    TensorP out = full({}, 0.0f, device);
    trs_operand op{};
    op.base = t->v.st->ptr;
    op.offset = t->v.offset;
    op.rank = (int32_t)t->v.shape.size();
    for (size_t i = 0; i < t->v.shape.size(); ++i) { op.shape[i] = t->v.shape[i]; op.stride[i] = t->v.strides[i]; }
    check_cuda(trs_reduce_sum_f32(&op, out->v.st->ptr, stream_for(device)), "sum");
    if (t->requires_grad() && grad_enabled()) record(out, GK::Sum, "SumBackward0", {t.get()}, {}, false);
    return out;
}

}  // namespace trsh
