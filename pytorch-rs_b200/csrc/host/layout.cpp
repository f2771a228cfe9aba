// Layout planning on the host: contiguity predicates, TensorIterator-compatible output strides
// and broadcast shapes.  These decide `.stride()` of every result exactly as the reference does
// (src/tensor.rs:2636-2656, 2751-2766, 3601-3693, 4249-4336) and therefore which device kernel
// class a chain gets; no element is touched here.
#include <algorithm>

#include "engine.h"

namespace trsh {

namespace {

i64 stride_product(i64 stride, i64 dim) {
    // checked_stride_product (src/tensor.rs:4374-4379)
    __int128 p = (__int128)stride * std::max<i64>(dim, 1);
    if (p > (__int128)INT64_MAX) throw Error(ErrKind::StrideCalculationOverflow, "Stride calculation overflowed");
    return (i64)p;
}

struct Operand {
    const Shape* shape;
    const Shape* strides;
};

// Stride (in bytes, wrapping) an operand has along an output axis once right-aligned and
// broadcast (src/tensor.rs:4112-4151).
i64 aligned_byte_stride(const Operand& op, size_t out_rank, size_t axis, i64 out_dim) {
    const size_t lead = out_rank - op.shape->size();
    if (axis < lead) return 0;
    const size_t a = axis - lead;
    const i64 stride = ((*op.shape)[a] == 1 && out_dim != 1) ? 0 : (*op.strides)[a];
    return (i64)((uint64_t)stride * 4u);
}

// src/tensor.rs:4314-4336: first operand with two non-zero strides decides; ties go by size.
int compare_axes(const Shape& shape, const std::vector<Operand>& ops, size_t a0, size_t a1) {
    for (const Operand& op : ops) {
        const i64 s0 = aligned_byte_stride(op, shape.size(), a0, shape[a0]);
        const i64 s1 = aligned_byte_stride(op, shape.size(), a1, shape[a1]);
        if (s0 == 0 || s1 == 0) continue;
        if (s0 < s1) return -1;
        if (s0 > s1 || shape[a0] > shape[a1]) return 1;
    }
    return 0;
}

// src/tensor.rs:4249-4312
Shape sorted_output_strides(const Shape& shape, const std::vector<Operand>& ops) {
    const size_t rank = shape.size();
    std::vector<size_t> perm(rank);
    for (size_t i = 0; i < rank; ++i) perm[i] = rank - 1 - i;
    for (size_t i = 1; i < rank; ++i) {
        size_t d1 = i;
        for (size_t d0 = i; d0-- > 0;) {
            const int c = compare_axes(shape, ops, perm[d0], perm[d1]);
            if (c > 0) { std::swap(perm[d0], perm[d1]); d1 = d0; }
            else if (c < 0) break;
        }
    }
    bool row_major = true;
    for (size_t i = 0; i < rank; ++i) row_major &= perm[i] == rank - 1 - i;
    if (row_major) return contiguous_strides(shape);

    std::vector<i64> bytes(rank, 0);
    i64 next = 4;
    for (size_t pos = 0; pos < rank; ++pos) {
        bytes[perm[pos]] = next;
        if (pos + 1 < rank) next = (i64)((uint64_t)next * (uint64_t)shape[perm[pos]]);
    }
    Shape out(rank, 0);
    for (size_t axis = rank; axis-- > 0;) {
        const i64 s = bytes[axis] / 4;
        if (s >= 0) out[axis] = s;
        else if (axis + 1 == rank) out[axis] = 1;
        else out[axis] = stride_product(out[axis + 1], shape[axis + 1]);
    }
    return out;
}

// layout_is_contiguous_in_order (src/tensor.rs:3765-3791): dense when walked in the given physical
// order (innermost axis first), size-1 axes skipped.
bool contiguous_in_order(const Shape& shape, const Shape& strides, const int* order, size_t rank) {
    if (shape.size() != rank) return false;
    bool empty = false;
    for (i64 d : shape) empty |= d == 0;
    uint64_t expected = 1;
    for (size_t pos = 0; pos < rank; ++pos) {
        const int axis = order[pos];
        if (shape[axis] == 1) continue;
        if ((uint64_t)strides[axis] != expected) return false;
        const __int128 next = (__int128)expected * (uint64_t)shape[axis];
        if (next > (__int128)UINT64_MAX && !empty) return false;
        expected = (uint64_t)next;                      // wraps only for empty tensors, as the reference allows
    }
    return true;
}

const int kChannelsLastOrder[4] = {1, 3, 2, 0};         // physical order C, W, H, N
const int kChannelsLast3dOrder[5] = {1, 4, 3, 2, 0};    // C, W, H, D, N

bool channels_last_contiguous(const Shape& shape, const Shape& strides) {
    // src/tensor.rs:3717-3719
    return contiguous_in_order(shape, strides, kChannelsLastOrder, 4);
}

// strides_in_physical_order (src/tensor.rs:4225-4247): a zero-sized physical dimension zeroes every later stride.
Shape strides_in_order(const Shape& shape, const int* order, size_t rank) {
    (void)contiguous_strides(shape);                     // the canonical strides must be representable too
    Shape out(rank, 0);
    i64 stride = 1;
    for (size_t pos = 0; pos < rank; ++pos) {
        out[order[pos]] = stride;
        if (pos + 1 < rank) {
            __int128 p = (__int128)stride * shape[order[pos]];
            if (p > (__int128)INT64_MAX) throw Error(ErrKind::StrideCalculationOverflow, "Stride calculation overflowed");
            stride = (i64)p;
        }
    }
    return out;
}

Shape channels_last_strides(const Shape& shape) {
    // src/tensor.rs:4211-4216
    return strides_in_order(shape, kChannelsLastOrder, 4);
}

}  // namespace

i64 element_count(const Shape& shape) {
    __int128 n = 1;
    for (i64 d : shape) {
        n *= d;
        if (n > (__int128)INT64_MAX) throw Error(ErrKind::ElementCountOverflow, "tensor element count overflowed usize");
    }
    return (i64)n;
}

Shape contiguous_strides(const Shape& shape) {
    // src/tensor.rs:4198-4209
    Shape out(shape.size(), 0);
    i64 stride = 1;
    for (size_t axis = shape.size(); axis-- > 0;) {
        out[axis] = stride;
        if (axis > 0) stride = stride_product(stride, shape[axis]);
    }
    return out;
}

bool layout_is_contiguous(const Shape& shape, const Shape& strides) {
    // src/tensor.rs:3695-3715
    for (i64 d : shape) if (d == 0) return true;
    i64 expected = 1;
    for (size_t axis = shape.size(); axis-- > 0;) {
        if (shape[axis] == 1) continue;
        if (strides[axis] != expected) return false;
        expected *= shape[axis];
    }
    return true;
}

bool is_non_overlapping_and_dense(const Shape& shape, const Shape& strides) {
    // src/tensor.rs:1019-1053
    for (i64 d : shape) if (d == 0) return true;
    size_t want = 0;
    for (i64 d : shape) want += d > 1;
    i64 expected = 1;
    for (size_t matched = 0; matched < want; ++matched) {
        int found = -1;
        for (size_t a = 0; a < shape.size(); ++a)
            if (shape[a] > 1 && strides[a] == expected) {
                if (found >= 0) return false;
                found = (int)a;
            }
        if (found < 0) return false;
        expected *= shape[found];
    }
    return true;
}

Shape unary_output_strides(const Shape& shape, const Shape& strides) {
    // src/tensor.rs:2751-2766
    if (layout_is_contiguous(shape, strides)) return contiguous_strides(shape);
    if (channels_last_contiguous(shape, strides)) return channels_last_strides(shape);
    if (is_non_overlapping_and_dense(shape, strides)) return strides;
    return sorted_output_strides(shape, {Operand{&shape, &strides}});
}

Shape scalar_output_strides(const Shape& shape, const Shape& strides) {
    // src/tensor.rs:2718-2727: tensor-scalar ops always use the sorted rule
    return sorted_output_strides(shape, {Operand{&shape, &strides}});
}

// compute_reshape_view_strides (src/tensor.rs:3996-4055): strides that let `new_shape` alias the same
// elements, or false when some new dimension would straddle two runs of the old layout.
bool reshape_view_strides(const Shape& shape, const Shape& strides, const Shape& new_shape, Shape* out) {
    if (shape.empty()) { *out = contiguous_strides(new_shape); return true; }
    out->assign(new_shape.size(), 0);
    size_t view_d = new_shape.size();
    i64 chunk_base = strides.back(), tensor_n = 1, view_n = 1;
    for (size_t d = shape.size(); d-- > 0;) {
        tensor_n *= shape[d];
        const bool ends = d == 0 || (shape[d - 1] != 1 && strides[d - 1] != tensor_n * chunk_base);
        if (!ends) continue;
        while (view_d > 0 && (view_n < tensor_n || new_shape[view_d - 1] == 1)) {
            --view_d;
            (*out)[view_d] = view_n * chunk_base;
            view_n *= new_shape[view_d];
        }
        if (view_n != tensor_n) return false;
        if (d > 0) { chunk_base = strides[d - 1]; tensor_n = 1; view_n = 1; }
    }
    return view_d == 0;
}

// clone() with the preserve format (src/tensor.rs:1555-1565)
Shape clone_strides(const Shape& shape, const Shape& strides) {
    if (is_non_overlapping_and_dense(shape, strides)) return strides;
    return sorted_output_strides(shape, {Operand{&shape, &strides}});
}

const char* memory_format_name(MemoryFormat f) {
    // Display for MemoryFormat (src/memory_format.rs:17-26)
    switch (f) {
        case MemoryFormat::Preserve: return "preserve_format";
        case MemoryFormat::Contiguous: return "contiguous_format";
        case MemoryFormat::ChannelsLast: return "channels_last";
        default: return "channels_last_3d";
    }
}

// is_contiguous_with_memory_format (src/tensor.rs:1004-1014): preserve queries like contiguous.
bool is_contiguous_in_format(const Shape& shape, const Shape& strides, MemoryFormat f) {
    switch (f) {
        case MemoryFormat::Preserve:
        case MemoryFormat::Contiguous: return layout_is_contiguous(shape, strides);
        case MemoryFormat::ChannelsLast: return contiguous_in_order(shape, strides, kChannelsLastOrder, 4);
        default: return contiguous_in_order(shape, strides, kChannelsLast3dOrder, 5);
    }
}

// Canonical strides of an explicit format (src/tensor.rs:1566-1568, 1659-1661); the caller has checked the rank.
Shape memory_format_strides(const Shape& shape, MemoryFormat f) {
    if (f == MemoryFormat::ChannelsLast) return strides_in_order(shape, kChannelsLastOrder, 4);
    if (f == MemoryFormat::ChannelsLast3d) return strides_in_order(shape, kChannelsLast3dOrder, 5);
    return contiguous_strides(shape);
}

// The rank a channel-last format needs, or -1 (src/tensor.rs:1539-1543).
int memory_format_rank(MemoryFormat f) {
    return f == MemoryFormat::ChannelsLast ? 4 : (f == MemoryFormat::ChannelsLast3d ? 5 : -1);
}

// Layout decision of clone(memory_format) (src/tensor.rs:1533-1575) and of contiguous(memory_format)
// (1606-1675).  Returns false when contiguous() keeps the tensor's own storage; otherwise `out`
// holds the strides of the packed copy.
bool memory_format_plan(const Shape& shape, const Shape& strides, MemoryFormat f, bool for_clone, Shape* out) {
    const int want = memory_format_rank(f);
    if (want >= 0 && (int)shape.size() != want) {
        if (for_clone) (void)contiguous_strides(shape);        // clone validates the destination metadata first (1545-1549)
        throw Error(ErrKind::ContiguousMemoryFormatRankMismatch,
                    "required rank " + std::to_string(want) + " tensor to use " + memory_format_name(f) + " format");
    }
    if (!for_clone) {
        if (is_contiguous_in_format(shape, strides, f)) return false;
        if (f == MemoryFormat::Preserve)
            throw Error(ErrKind::ContiguousPreserveFormatUnsupported, "preserve memory format is unsupported by the contiguous operator");
    }
    *out = f == MemoryFormat::Preserve ? clone_strides(shape, strides) : memory_format_strides(shape, f);
    return true;
}

static std::string shape_text(const Shape& s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
    return t + "]";
}

void binary_plan(const Shape& ls, const Shape& lst, const Shape& rs, const Shape& rst, Shape* shape, Shape* strides) {
    if (ls == rs) {
        // src/tensor.rs:2636-2656
        *shape = ls;
        if (layout_is_contiguous(ls, lst) && layout_is_contiguous(rs, rst)) *strides = contiguous_strides(ls);
        else if (channels_last_contiguous(ls, lst) && channels_last_contiguous(rs, rst)) *strides = channels_last_strides(ls);
        else if (is_non_overlapping_and_dense(ls, lst) && is_non_overlapping_and_dense(rs, rst) && lst == rst) *strides = lst;
        else *strides = sorted_output_strides(ls, {Operand{&ls, &lst}, Operand{&rs, &rst}});
        return;
    }
    // src/tensor.rs:3601-3646; message src/tensor_error.rs:217-233, 377-393
    const size_t rank = std::max(ls.size(), rs.size());
    Shape out(rank, 0);
    for (size_t t = 0; t < rank; ++t) {
        const size_t axis = rank - 1 - t;
        const i64 l = t < ls.size() ? ls[ls.size() - 1 - t] : 1;
        const i64 r = t < rs.size() ? rs[rs.size() - 1 - t] : 1;
        if (l != r && l != 1 && r != 1)
            throw Error(ErrKind::ShapeMismatch, "The size of tensor a (" + std::to_string(l) + ") must match the size of tensor b (" +
                                                    std::to_string(r) + ") at non-singleton dimension " + std::to_string(axis));
        out[axis] = l == r ? l : (l == 1 ? r : l);
    }
    (void)shape_text;
    (void)element_count(out);
    *shape = out;
    *strides = sorted_output_strides(out, {Operand{&ls, &lst}, Operand{&rs, &rst}});
}

}  // namespace trsh
