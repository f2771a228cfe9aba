// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of the pytorch-rs reference engine's pointwise / matmul /
// backward loops and of its TensorIterator-compatible layout rules, used only
// as the checker in tests, in the smoke check and as the timed CPU baseline.
// Nothing in the product path may link or call this file.
//
// The reference is Rust; no Rust toolchain exists where this is built, so the
// algorithm is restated in C++17 and compiled with
//   g++ -O3 -fno-fast-math -ffp-contract=off            (baseline x86-64)
// which mirrors the reference release profile (Cargo.toml:23-25: thin LTO, one
// codegen unit, no target-cpu, and Rust never contracts a*b+c into an FMA).
// Parity pin: this file is checked against the golden vectors held by the
// reference's own tests (tests/tensor_baseline.rs, tests/autograd.rs), which
// are transcribed in tests/golden/reference_vectors.json.
//
// Every function cites the reference source it follows (path:line inside the
// reference project).  All strides are in elements, non-negative.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

namespace {

using i64 = int64_t;
using u64 = uint64_t;
constexpr uint32_t SIGN = 0x80000000u;
constexpr i64 ISIZE_MAX = INT64_MAX;

enum Status : int {
    OK = 0,
    SHAPE_MISMATCH = 1,          // TensorError::ShapeMismatch
    STRIDE_OVERFLOW = 2,         // TensorError::StrideCalculationOverflow
    ELEMENT_OVERFLOW = 3,        // TensorError::ElementCountOverflow
    MATMUL_RANK = 4,             // TensorError::MatmulRequiresMatrices
    MATMUL_INNER = 5,            // TensorError::MatmulInnerDimensionMismatch
    BAD_OP = 6,
    FORMAT_RANK = 8,             // TensorError::ContiguousMemoryFormatRankMismatch
    PRESERVE_UNSUPPORTED = 9,    // TensorError::ContiguousPreserveFormatUnsupported
};

inline uint32_t bits(float v) { uint32_t b; std::memcpy(&b, &v, 4); return b; }
inline float from_bits(uint32_t b) { float v; std::memcpy(&v, &b, 4); return v; }

// ---- scalar kernels ------------------------------------------------------

// src/tensor.rs:4388-4390
inline float negate_value(float v) { return from_bits(bits(v) ^ SIGN); }

// src/tensor.rs:4392-4400.  Rust's f32::max returns the non-NaN operand, so
// relu(NaN) == +0.0; exact zeros keep their sign.
inline float relu_value(float v) {
    if ((bits(v) & ~SIGN) == 0) return v;
    return std::fmax(v, 0.0f);
}

// src/tensor.rs:4402-4414
inline float sqrt_value(float v) {
    uint32_t b = bits(v), mag = b & ~SIGN;
    bool is_nan = mag > 0x7f800000u;
    bool neg_nonzero = (b & SIGN) != 0 && mag != 0;
    if (neg_nonzero && !is_nan) return from_bits(0x7fc00000u);
    return std::sqrt(v);
}

// src/tensor.rs:4422-4432
inline float relu_backward_value(float input, float upstream) {
    uint32_t b = bits(input), mag = b & ~SIGN;
    bool is_nan = mag > 0x7f800000u;
    bool pos_nonzero = (b & SIGN) == 0 && mag != 0;
    return (is_nan || pos_nonzero) ? upstream : 0.0f;
}

enum UnaryOp { U_RELU = 0, U_EXP = 1, U_NEG = 2, U_SIN = 3, U_SQRT = 4, U_RECIP = 5, U_COPY = 6 };
enum BinaryOp { B_ADD = 0, B_SUB = 1, B_MUL = 2, B_DIV = 3 };
// Scalar forms (src/tensor.rs:2254-2371): the tensor value is always the left
// argument of the closure except for the two reflected forms.
enum ScalarOp { S_ADD = 0, S_SUB = 1, S_MUL = 2, S_DIV = 3, S_RSUB = 4, S_RDIV = 5 };

inline float apply_unary(int op, float v) {
    switch (op) {
        case U_RELU: return relu_value(v);               // tensor.rs:2378-2381
        case U_EXP: return ::expf(v);                     // tensor.rs:2398-2400 (f32::exp -> libm expf)
        case U_NEG: return negate_value(v);               // tensor.rs:2294-2297
        case U_SIN: return ::sinf(v);                     // tensor.rs:2388-2391
        case U_SQRT: return sqrt_value(v);                // tensor.rs:2407-2410
        case U_RECIP: return 1.0f * (1.0f / v);           // tensor.rs:2348-2355
        default: return v;
    }
}
inline float apply_binary(int op, float l, float r) {
    switch (op) {
        case B_ADD: return l + r;                         // tensor.rs:2197-2199
        case B_SUB: return l - r;                         // tensor.rs:2207-2209
        case B_MUL: return l * r;                         // tensor.rs:2217-2218
        default: return l / r;                            // tensor.rs:2245-2247
    }
}
inline float apply_scalar(int op, float v, float s) {
    switch (op) {
        case S_ADD: return v + s;                         // tensor.rs:2254-2257
        case S_SUB: return v - s;                         // tensor.rs:2264-2267
        case S_MUL: return v * s;                         // tensor.rs:2274-2275
        case S_DIV: return v / s;                         // tensor.rs:2304-2306
        case S_RSUB: return s - v;                        // tensor.rs:2313-2316
        default: return s * (1.0f / v);                   // tensor.rs:2357-2363
    }
}

// ---- layout rules ----------------------------------------------------------

struct View {
    const float* data;   // storage base
    i64 offset;
    std::vector<i64> shape, strides;
    i64 elements() const { i64 n = 1; for (i64 d : shape) n *= d; return n; }
};

// src/tensor.rs:4374-4379
bool checked_stride_product(i64 stride, i64 dim, i64* out) {
    i64 d = std::max<i64>(dim, 1);
    __int128 p = (__int128)stride * d;
    if (p > ISIZE_MAX) return false;
    *out = (i64)p;
    return true;
}

// src/tensor.rs:4198-4209
int contiguous_strides(const std::vector<i64>& shape, std::vector<i64>& out) {
    out.assign(shape.size(), 0);
    i64 stride = 1;
    for (int axis = (int)shape.size() - 1; axis >= 0; --axis) {
        out[axis] = stride;
        if (axis > 0 && !checked_stride_product(stride, shape[axis], &stride)) return STRIDE_OVERFLOW;
    }
    return OK;
}

// src/tensor.rs:4225-4247 (channels-last: order {1,3,2,0})
int strides_in_physical_order(const std::vector<i64>& shape, const int* order, std::vector<i64>& out) {
    std::vector<i64> tmp;
    if (int s = contiguous_strides(shape, tmp)) return s;
    out.assign(shape.size(), 0);
    i64 stride = 1;
    for (size_t pos = 0; pos < shape.size(); ++pos) {
        int axis = order[pos];
        out[axis] = stride;
        if (pos + 1 < shape.size()) {
            __int128 p = (__int128)stride * shape[axis];
            if (p > ISIZE_MAX) return STRIDE_OVERFLOW;
            stride = (i64)p;
        }
    }
    return OK;
}

// src/tensor.rs:3695-3715
bool layout_is_contiguous(const std::vector<i64>& shape, const std::vector<i64>& strides, i64 elements) {
    if (elements == 0) return true;
    i64 expected = 1;
    for (int axis = (int)shape.size() - 1; axis >= 0; --axis) {
        if (shape[axis] == 1) continue;
        if (strides[axis] != expected) return false;
        expected *= shape[axis];
    }
    return true;
}

// src/tensor.rs:3765-3791 with order {1,3,2,0} (3717-3719)
bool layout_is_channels_last_contiguous(const std::vector<i64>& shape, const std::vector<i64>& strides) {
    static const int order[4] = {1, 3, 2, 0};
    if (shape.size() != 4 || strides.size() != 4) return false;
    u64 expected = 1;
    for (int axis : order) {
        if (shape[axis] == 1) continue;
        if ((u64)strides[axis] != expected) return false;
        expected *= (u64)shape[axis];   // wraps only for empty tensors, as the reference allows
    }
    return true;
}

// src/tensor.rs:1019-1053
bool is_non_overlapping_and_dense(const std::vector<i64>& shape, const std::vector<i64>& strides, i64 elements) {
    if (elements == 0) return true;
    size_t dims = 0;
    for (i64 d : shape) dims += d > 1;
    size_t matched = 0;
    i64 expected = 1;
    while (matched < dims) {
        int found = -1;
        for (size_t a = 0; a < shape.size(); ++a) {
            if (shape[a] > 1 && strides[a] == expected) {
                if (found >= 0) return false;
                found = (int)a;
            }
        }
        if (found < 0) return false;
        expected *= shape[found];
        ++matched;
    }
    return true;
}

struct Layout { const std::vector<i64>* shape; const std::vector<i64>* strides; };

// src/tensor.rs:4112-4151 (byte strides as wrapping signed 64-bit)
i64 aligned_stride_bytes(const Layout& l, size_t out_rank, size_t out_axis, i64 out_dim) {
    size_t lead = out_rank - l.shape->size();
    if (out_axis < lead) return 0;
    size_t in_axis = out_axis - lead;
    i64 in_dim = (*l.shape)[in_axis];
    i64 stride = (in_dim == 1 && out_dim != 1) ? 0 : (*l.strides)[in_axis];
    return (i64)((u64)stride * 4u);
}

// src/tensor.rs:4314-4336
int compare_dims(const std::vector<i64>& shape, const std::vector<Layout>& ops, size_t d0, size_t d1) {
    for (const Layout& l : ops) {
        i64 s0 = aligned_stride_bytes(l, shape.size(), d0, shape[d0]);
        i64 s1 = aligned_stride_bytes(l, shape.size(), d1, shape[d1]);
        if (s0 == 0 || s1 == 0) continue;
        if (s0 < s1) return -1;
        if (s0 > s1 || shape[d0] > shape[d1]) return 1;
    }
    return 0;
}

// src/tensor.rs:4249-4312
int elementwise_output_strides(const std::vector<i64>& shape, const std::vector<Layout>& ops,
                               std::vector<i64>& out) {
    size_t rank = shape.size();
    std::vector<size_t> perm(rank);
    for (size_t i = 0; i < rank; ++i) perm[i] = rank - 1 - i;
    for (size_t index = 1; index < rank; ++index) {
        size_t d1 = index;
        for (size_t d0 = index; d0-- > 0;) {
            int c = compare_dims(shape, ops, perm[d0], perm[d1]);
            if (c > 0) { std::swap(perm[d0], perm[d1]); d1 = d0; }
            else if (c < 0) break;
        }
    }
    bool identity = true;
    for (size_t i = 0; i < rank; ++i) identity &= perm[i] == rank - 1 - i;
    if (identity) return contiguous_strides(shape, out);

    std::vector<i64> byte_strides(rank, 0);
    i64 next = 4;
    for (size_t pos = 0; pos < rank; ++pos) {
        size_t axis = perm[pos];
        byte_strides[axis] = next;
        if (pos + 1 < rank) next = (i64)((u64)next * (u64)shape[axis]);
    }
    out.assign(rank, 0);
    for (size_t axis = rank; axis-- > 0;) {
        i64 stride = byte_strides[axis] / 4;
        if (stride >= 0) out[axis] = stride;
        else if (axis + 1 == rank) out[axis] = 1;
        else if (!checked_stride_product(out[axis + 1], shape[axis + 1], &out[axis])) return STRIDE_OVERFLOW;
    }
    return OK;
}

// src/tensor.rs:2751-2766
int unary_output_strides(const View& v, std::vector<i64>& out) {
    i64 n = v.elements();
    if (layout_is_contiguous(v.shape, v.strides, n)) return contiguous_strides(v.shape, out);
    if (layout_is_channels_last_contiguous(v.shape, v.strides)) {
        static const int order[4] = {1, 3, 2, 0};
        return strides_in_physical_order(v.shape, order, out);
    }
    if (is_non_overlapping_and_dense(v.shape, v.strides, n)) { out = v.strides; return OK; }
    return elementwise_output_strides(v.shape, {Layout{&v.shape, &v.strides}}, out);
}

// src/tensor.rs:2636-2656
int same_shape_output_strides(const View& l, const View& r, std::vector<i64>& out) {
    i64 n = l.elements();
    if (layout_is_contiguous(l.shape, l.strides, n) && layout_is_contiguous(r.shape, r.strides, n))
        return contiguous_strides(l.shape, out);
    if (layout_is_channels_last_contiguous(l.shape, l.strides) &&
        layout_is_channels_last_contiguous(r.shape, r.strides)) {
        static const int order[4] = {1, 3, 2, 0};
        return strides_in_physical_order(l.shape, order, out);
    }
    if (is_non_overlapping_and_dense(l.shape, l.strides, n) &&
        is_non_overlapping_and_dense(r.shape, r.strides, n) && l.strides == r.strides) {
        out = l.strides;
        return OK;
    }
    return elementwise_output_strides(l.shape, {Layout{&l.shape, &l.strides}, Layout{&r.shape, &r.strides}}, out);
}

// src/tensor.rs:3601-3646 (shape check + result shape + output strides)
int broadcast_plan(const View& l, const View& r, std::vector<i64>& shape, std::vector<i64>& strides) {
    size_t rank = std::max(l.shape.size(), r.shape.size());
    shape.assign(rank, 0);
    for (size_t axis = 0; axis < rank; ++axis) {
        size_t ll = rank - l.shape.size(), rl = rank - r.shape.size();
        i64 ld = axis < ll ? 1 : l.shape[axis - ll];
        i64 rd = axis < rl ? 1 : r.shape[axis - rl];
        if (ld == rd) shape[axis] = ld;
        else if (ld == 1) shape[axis] = rd;
        else if (rd == 1) shape[axis] = ld;
        else return SHAPE_MISMATCH;
    }
    __int128 n = 1;
    for (i64 d : shape) { n *= d; if (n > (__int128)UINT64_MAX) return ELEMENT_OVERFLOW; }
    return elementwise_output_strides(shape, {Layout{&l.shape, &l.strides}, Layout{&r.shape, &r.strides}}, strides);
}

// ---- element loops -----------------------------------------------------------

// src/tensor.rs:3815-3841
inline i64 logical_offset(const std::vector<i64>& shape, const std::vector<i64>& strides, i64 base, i64 linear) {
    i64 rem = linear, off = base;
    for (int axis = (int)shape.size() - 1; axis >= 0; --axis) {
        i64 d = shape[axis];
        i64 c = rem % d;
        rem /= d;
        off += c * strides[axis];
    }
    return off;
}

// src/tensor.rs:1805-1838: contiguous slice stream, dense-physical stream, or
// logical-order scatter through the planned output strides.
template <class F>
void materialize_with_strides(const View& v, const std::vector<i64>& out_strides, float* out, F op) {
    i64 n = v.elements();
    if (n == 0) return;
    bool in_contig = layout_is_contiguous(v.shape, v.strides, n);
    if (layout_is_contiguous(v.shape, out_strides, n)) {
        if (in_contig) {
            const float* src = v.data + v.offset;
            for (i64 i = 0; i < n; ++i) out[i] = op(src[i]);
        } else {
            for (i64 i = 0; i < n; ++i) out[i] = op(v.data[logical_offset(v.shape, v.strides, v.offset, i)]);
        }
        return;
    }
    if (v.strides == out_strides && is_non_overlapping_and_dense(v.shape, v.strides, n)) {
        const float* src = v.data + v.offset;
        for (i64 i = 0; i < n; ++i) out[i] = op(src[i]);
        return;
    }
    for (i64 i = 0; i < n; ++i) {
        float value = in_contig ? v.data[v.offset + i] : v.data[logical_offset(v.shape, v.strides, v.offset, i)];
        out[logical_offset(v.shape, out_strides, 0, i)] = op(value);
    }
}

inline i64 aligned_step(const View& v, size_t rank, size_t axis, i64 out_dim) {
    size_t lead = rank - v.shape.size();
    if (axis < lead) return 0;
    size_t a = axis - lead;
    return (v.shape[a] == 1 && out_dim != 1) ? 0 : v.strides[a];
}

// src/tensor.rs:3546-3599: odometer over the logical output order; a
// non-contiguous output additionally decodes its offset per element.
template <class F>
void materialize_broadcast(const View& l, const View& r, const std::vector<i64>& shape,
                           const std::vector<i64>& strides, float* out, F op) {
    size_t rank = shape.size();
    i64 n = 1;
    for (i64 d : shape) n *= d;
    if (n == 0) return;
    std::vector<i64> ls(rank), rs(rank), lrew(rank), rrew(rank), coord(rank, 0);
    for (size_t a = 0; a < rank; ++a) {
        ls[a] = aligned_step(l, rank, a, shape[a]);
        rs[a] = aligned_step(r, rank, a, shape[a]);
        i64 rep = shape[a] > 0 ? shape[a] - 1 : 0;
        lrew[a] = ls[a] * rep;
        rrew[a] = rs[a] * rep;
    }
    bool contig_out = layout_is_contiguous(shape, strides, n);
    i64 lo = l.offset, ro = r.offset;
    for (i64 i = 0; i < n; ++i) {
        float value = op(l.data[lo], r.data[ro]);
        if (contig_out) out[i] = value;
        else out[logical_offset(shape, strides, 0, i)] = value;
        if (i + 1 == n) break;
        for (size_t a = rank; a-- > 0;) {
            if (++coord[a] < shape[a]) { lo += ls[a]; ro += rs[a]; break; }
            coord[a] = 0;
            lo -= lrew[a];
            ro -= rrew[a];
        }
    }
}

// src/tensor.rs:2535-2557 + 2629-2716 + 2559-2627.  One IEEE operation per
// element in every branch; the branches differ only in traversal order.
template <class F>
int zip_map(const View& l, const View& r, std::vector<i64>& shape, std::vector<i64>& strides, float* out,
            bool plan_only, F op) {
    if (l.shape == r.shape) {
        shape = l.shape;
        if (int s = same_shape_output_strides(l, r, strides)) return s;
        if (plan_only) return OK;
        i64 n = l.elements();
        if (n == 0) return OK;
        bool lc = layout_is_contiguous(l.shape, l.strides, n), rc = layout_is_contiguous(r.shape, r.strides, n);
        if (lc && rc) {
            const float *a = l.data + l.offset, *b = r.data + r.offset;
            for (i64 i = 0; i < n; ++i) out[i] = op(a[i], b[i]);
            return OK;
        }
        if (l.strides == strides && r.strides == strides && is_non_overlapping_and_dense(l.shape, l.strides, n)) {
            // tensor.rs:2675-2699 (the NaN-pair pre-scan only pins payloads; it is kept for timing fidelity)
            const float *a = l.data + l.offset, *b = r.data + r.offset;
            bool nan_pair = false;
            for (i64 i = 0; i < n; ++i) nan_pair |= (a[i] != a[i]) && (b[i] != b[i]);
            if (!nan_pair) {
                for (i64 i = 0; i < n; ++i) out[i] = op(a[i], b[i]);
                return OK;
            }
        }
        for (i64 i = 0; i < n; ++i) {
            float a = lc ? l.data[l.offset + i] : l.data[logical_offset(l.shape, l.strides, l.offset, i)];
            float b = rc ? r.data[r.offset + i] : r.data[logical_offset(r.shape, r.strides, r.offset, i)];
            out[logical_offset(shape, strides, 0, i)] = op(a, b);
        }
        return OK;
    }
    if (int s = broadcast_plan(l, r, shape, strides)) return s;
    if (plan_only) return OK;
    // tensor.rs:3454-3543 (contiguous trailing-vector / trailing-singleton
    // streams) and 2768-2789 (rank-zero operand) compute the same values as the
    // odometer; they are traversal shortcuts only.
    i64 ln = l.elements(), rn = r.elements();
    i64 n = 1;
    for (i64 d : shape) n *= d;
    if (n != 0 && layout_is_contiguous(shape, strides, n) && layout_is_contiguous(l.shape, l.strides, ln) &&
        layout_is_contiguous(r.shape, r.strides, rn)) {
        const View* broad = nullptr; const View* vec = nullptr; bool vec_left = false;
        if (l.shape.size() > 1 && r.shape.size() == 1 && l.shape.back() == r.shape[0]) { broad = &l; vec = &r; }
        else if (r.shape.size() > 1 && l.shape.size() == 1 && r.shape.back() == l.shape[0]) { broad = &r; vec = &l; vec_left = true; }
        if (broad) {
            i64 w = vec->shape[0];
            const float* bv = broad->data + broad->offset; const float* vv = vec->data + vec->offset;
            for (i64 row = 0; row < n / w; ++row)
                for (i64 c = 0; c < w; ++c)
                    out[row * w + c] = vec_left ? op(vv[c], bv[row * w + c]) : op(bv[row * w + c], vv[c]);
            return OK;
        }
    }
    materialize_broadcast(l, r, shape, strides, out, op);
    return OK;
}

View make_view(const float* data, i64 offset, int rank, const i64* shape, const i64* strides) {
    View v{data, offset, {}, {}};
    v.shape.assign(shape, shape + rank);
    v.strides.assign(strides, strides + rank);
    return v;
}

}  // namespace

extern "C" {

// Output strides of a unary op (tensor.rs:2751-2766).
int ref_unary_strides(int rank, const i64* shape, const i64* strides, i64* out_strides) {
    View v = make_view(nullptr, 0, rank, shape, strides);
    std::vector<i64> o;
    if (int s = unary_output_strides(v, o)) return s;
    std::copy(o.begin(), o.end(), out_strides);
    return OK;
}

// Output strides of a tensor-scalar op (tensor.rs:2718-2727: always the sorted rule).
int ref_scalar_strides(int rank, const i64* shape, const i64* strides, i64* out_strides) {
    View v = make_view(nullptr, 0, rank, shape, strides);
    std::vector<i64> o;
    if (int s = elementwise_output_strides(v.shape, {Layout{&v.shape, &v.strides}}, o)) return s;
    std::copy(o.begin(), o.end(), out_strides);
    return OK;
}

// Shape + strides of a binary op (tensor.rs:2535-2557).  out arrays hold max(lrank, rrank) entries.
int ref_binary_plan(int lrank, const i64* lshape, const i64* lstrides, int rrank, const i64* rshape,
                    const i64* rstrides, i64* out_shape, i64* out_strides) {
    View l = make_view(nullptr, 0, lrank, lshape, lstrides), r = make_view(nullptr, 0, rrank, rshape, rstrides);
    std::vector<i64> shape, strides;
    int s = zip_map(l, r, shape, strides, nullptr, true, [](float a, float) { return a; });
    if (s) return s;
    std::copy(shape.begin(), shape.end(), out_shape);
    std::copy(strides.begin(), strides.end(), out_strides);
    return OK;
}

// out receives numel(shape) floats laid out by out_strides at offset 0.
int ref_unary(int op, const float* data, i64 offset, int rank, const i64* shape, const i64* strides, float* out,
              i64* out_strides) {
    View v = make_view(data, offset, rank, shape, strides);
    std::vector<i64> o;
    if (int s = unary_output_strides(v, o)) return s;
    std::copy(o.begin(), o.end(), out_strides);
    materialize_with_strides(v, o, out, [op](float x) { return apply_unary(op, x); });
    return OK;
}

int ref_scalar(int op, float scalar, const float* data, i64 offset, int rank, const i64* shape, const i64* strides,
               float* out, i64* out_strides) {
    View v = make_view(data, offset, rank, shape, strides);
    std::vector<i64> o;
    if (op == S_RDIV) {
        // tensor.rs:2324-2340: planned as reciprocal (unary rule) then scalar rule.
        std::vector<i64> recip;
        if (int s = unary_output_strides(v, recip)) return s;
        if (int s = elementwise_output_strides(v.shape, {Layout{&v.shape, &recip}}, o)) return s;
    } else if (int s = elementwise_output_strides(v.shape, {Layout{&v.shape, &v.strides}}, o)) {
        return s;
    }
    std::copy(o.begin(), o.end(), out_strides);
    materialize_with_strides(v, o, out, [op, scalar](float x) { return apply_scalar(op, x, scalar); });
    return OK;
}

int ref_binary(int op, const float* ldata, i64 loffset, int lrank, const i64* lshape, const i64* lstrides,
               const float* rdata, i64 roffset, int rrank, const i64* rshape, const i64* rstrides, float* out,
               i64* out_shape, i64* out_strides) {
    View l = make_view(ldata, loffset, lrank, lshape, lstrides), r = make_view(rdata, roffset, rrank, rshape, rstrides);
    std::vector<i64> shape, strides;
    int s = zip_map(l, r, shape, strides, out, false, [op](float a, float b) { return apply_binary(op, a, b); });
    if (s) return s;
    std::copy(shape.begin(), shape.end(), out_shape);
    std::copy(strides.begin(), strides.end(), out_strides);
    return OK;
}

// Rank-2 matmul (tensor.rs:2453-2533): zero-filled output, k ascending, one
// multiply rounding and one add rounding per step; contiguous operands use the
// 4-row blocked sweep (3889-3966), others the strided loop (2478-2506).
int ref_matmul(const float* a, i64 aoff, const i64* ashape, const i64* astrides, const float* b, i64 boff,
               const i64* bshape, const i64* bstrides, float* out) {
    i64 rows = ashape[0], inner = ashape[1], columns = bshape[1];
    if (inner != bshape[0]) return MATMUL_INNER;
    i64 out_n = rows * columns;
    for (i64 i = 0; i < out_n; ++i) out[i] = 0.0f;
    if (out_n == 0 || inner == 0) return OK;
    std::vector<i64> as(ashape, ashape + 2), ast(astrides, astrides + 2), bs(bshape, bshape + 2), bst(bstrides, bstrides + 2);
    if (layout_is_contiguous(as, ast, rows * inner) && layout_is_contiguous(bs, bst, inner * columns)) {
        const float* left = a + aoff; const float* right = b + boff;
        i64 blocked = (rows >= 4 && inner * columns >= 4096) ? rows / 4 * 4 : 0;
        for (i64 r0 = 0; r0 < blocked; r0 += 4) {
            float *o0 = out + r0 * columns, *o1 = o0 + columns, *o2 = o1 + columns, *o3 = o2 + columns;
            const float* lt = left + r0 * inner;
            for (i64 k = 0; k < inner; ++k) {
                float l0 = lt[k], l1 = lt[inner + k], l2 = lt[2 * inner + k], l3 = lt[3 * inner + k];
                const float* rr = right + k * columns;
                for (i64 c = 0; c < columns; ++c) {
                    float rv = rr[c];
                    o0[c] += l0 * rv; o1[c] += l1 * rv; o2[c] += l2 * rv; o3[c] += l3 * rv;
                }
            }
        }
        for (i64 r = blocked; r < rows; ++r)
            for (i64 k = 0; k < inner; ++k) {
                float lv = left[r * inner + k];
                const float* rr = right + k * columns;
                for (i64 c = 0; c < columns; ++c) out[r * columns + c] += lv * rr[c];
            }
        return OK;
    }
    for (i64 r = 0; r < rows; ++r) {
        float* orow = out + r * columns;
        i64 lo = aoff + r * astrides[0];
        for (i64 k = 0; k < inner; ++k) {
            float lv = a[lo];
            i64 ro = boff + k * bstrides[0];
            for (i64 c = 0; c < columns; ++c) { orow[c] += lv * b[ro]; ro += bstrides[1]; }
            lo += astrides[1];
        }
    }
    return OK;
}

// Sequential sum in logical row-major order (tensor.rs:2413-2431).  Rust's f32
// Iterator::sum folds from -0.0 on the pinned 1.92 toolchain, so an empty sum is
// -0.0 (unpinned by the reference tests, which only check its magnitude).
float ref_sum(const float* data, i64 offset, int rank, const i64* shape, const i64* strides) {
    View v = make_view(data, offset, rank, shape, strides);
    i64 n = v.elements();
    float acc = -0.0f;
    bool contig = layout_is_contiguous(v.shape, v.strides, n);
    for (i64 i = 0; i < n; ++i)
        acc += contig ? data[offset + i] : data[logical_offset(v.shape, v.strides, offset, i)];
    return acc;
}

// relu VJP in logical order (tensor.rs:3161-3176): gradient is a flat logical
// row-major buffer with the saved input read through its view.
void ref_relu_vjp(const float* saved, i64 offset, int rank, const i64* shape, const i64* strides,
                  const float* upstream, float* gradient) {
    View v = make_view(saved, offset, rank, shape, strides);
    i64 n = v.elements();
    bool contig = layout_is_contiguous(v.shape, v.strides, n);
    for (i64 i = 0; i < n; ++i) {
        float x = contig ? saved[offset + i] : saved[logical_offset(v.shape, v.strides, offset, i)];
        gradient[i] = relu_backward_value(x, upstream[i]);
    }
}

// Un-broadcast accumulation (GradientAccumulator, tensor.rs:3204-3228, driven
// by the Multiply VJP loop 3057-3090): contributions arrive in logical output
// order; target index is the broadcast source position; the first contribution
// is stored rather than added when target and output have equal element counts.
// contribution[i] = upstream[i] * (other ? other_logical[i] : 1).
void ref_unbroadcast(int out_rank, const i64* out_shape, int in_rank, const i64* in_shape, const float* upstream,
                     const float* other_data, i64 other_offset, int other_rank, const i64* other_shape,
                     const i64* other_strides, float* gradient) {
    std::vector<i64> oshape(out_shape, out_shape + out_rank);
    i64 n = 1; for (i64 d : oshape) n *= d;
    i64 in_n = 1; for (int a = 0; a < in_rank; ++a) in_n *= in_shape[a];
    bool preserve_first = in_n == n;
    std::vector<char> init(in_n, !preserve_first);
    for (i64 i = 0; i < in_n; ++i) gradient[i] = 0.0f;
    std::vector<i64> in_contig(in_rank);
    { i64 s = 1; for (int a = in_rank - 1; a >= 0; --a) { in_contig[a] = s; s *= in_shape[a]; } }
    std::vector<i64> coord(out_rank);
    for (i64 i = 0; i < n; ++i) {
        i64 rem = i;
        for (int a = out_rank - 1; a >= 0; --a) { coord[a] = rem % oshape[a]; rem /= oshape[a]; }
        i64 idx = 0;
        for (int a = 0; a < in_rank; ++a) {
            int oa = a + (out_rank - in_rank);
            idx += (in_shape[a] == 1 ? 0 : coord[oa]) * in_contig[a];
        }
        float c = upstream[i];
        if (other_data) {
            i64 off = other_offset;
            for (int a = 0; a < other_rank; ++a) {
                int oa = a + (out_rank - other_rank);
                off += (other_shape[a] == 1 ? 0 : coord[oa]) * other_strides[a];
            }
            c = c * other_data[off];
        }
        if (init[idx]) gradient[idx] += c;
        else { gradient[idx] = c; init[idx] = 1; }
    }
}

// Permute VJP (tensor.rs:3248-3298): upstream is logical row-major over the
// permuted shape; gradient is logical row-major over the input shape.
void ref_permute_vjp(int rank, const i64* in_shape, const i64* dims, const float* upstream, float* gradient) {
    std::vector<i64> oshape(rank), istr(rank), coord(rank);
    for (int a = 0; a < rank; ++a) oshape[a] = in_shape[dims[a]];
    { i64 s = 1; for (int a = rank - 1; a >= 0; --a) { istr[a] = s; s *= in_shape[a]; } }
    i64 n = 1; for (int a = 0; a < rank; ++a) n *= in_shape[a];
    for (i64 i = 0; i < n; ++i) {
        i64 rem = i;
        for (int a = rank - 1; a >= 0; --a) { coord[a] = rem % oshape[a]; rem /= oshape[a]; }
        i64 idx = 0;
        for (int a = 0; a < rank; ++a) idx += coord[a] * istr[dims[a]];
        gradient[idx] = upstream[i];
    }
}

// In-place leaf gradient accumulation (storage.rs:85-100).
void ref_accumulate(float* grad, const float* contribution, i64 n) {
    for (i64 i = 0; i < n; ++i) grad[i] += contribution[i];
}

// Strides of a metadata-only reshape, or status 7 when the layout cannot be viewed that way
// (compute_reshape_view_strides, tensor.rs:3996-4055; empty tensors 2152-2164 are not covered here).
int ref_reshape_view_strides(int rank, const i64* shape, const i64* strides, int new_rank, const i64* new_shape,
                             i64* out_strides) {
    if (rank == 0) {
        std::vector<i64> ns(new_shape, new_shape + new_rank), o;
        if (int s = contiguous_strides(ns, o)) return s;
        std::copy(o.begin(), o.end(), out_strides);
        return OK;
    }
    int view_d = new_rank;
    i64 chunk_base = strides[rank - 1], tensor_n = 1, view_n = 1;
    for (int d = rank - 1; d >= 0; --d) {
        tensor_n *= shape[d];
        bool ends = d == 0 || (shape[d - 1] != 1 && strides[d - 1] != tensor_n * chunk_base);
        if (!ends) continue;
        while (view_d > 0 && (view_n < tensor_n || new_shape[view_d - 1] == 1)) {
            --view_d;
            out_strides[view_d] = view_n * chunk_base;
            view_n *= new_shape[view_d];
        }
        if (view_n != tensor_n) return 7;
        if (d > 0) { chunk_base = strides[d - 1]; tensor_n = 1; view_n = 1; }
    }
    return view_d == 0 ? OK : 7;
}

// Strides of clone() with the preserve format (tensor.rs:1535-1575): dense layouts keep their
// strides, others are packed in the same dimension order.
int ref_clone_strides(int rank, const i64* shape, const i64* strides, i64* out_strides) {
    View v = make_view(nullptr, 0, rank, shape, strides);
    std::vector<i64> o;
    if (v.elements() == 0 || is_non_overlapping_and_dense(v.shape, v.strides, v.elements())) o = v.strides;
    else if (int s = elementwise_output_strides(v.shape, {Layout{&v.shape, &v.strides}}, o)) return s;
    std::copy(o.begin(), o.end(), out_strides);
    return OK;
}

// MemoryFormat (memory_format.rs:5-15): 0 preserve, 1 contiguous, 2 channels_last, 3 channels_last_3d.
// is_contiguous_with_memory_format (tensor.rs:1004-1014, 3717-3724, 3765-3791).
int ref_is_contiguous_in_format(int format, int rank, const i64* shape, const i64* strides) {
    View v = make_view(nullptr, 0, rank, shape, strides);
    if (format <= 1) return layout_is_contiguous(v.shape, v.strides, v.elements()) ? 1 : 0;
    static const int order4[4] = {1, 3, 2, 0}, order5[5] = {1, 4, 3, 2, 0};
    const int want = format == 2 ? 4 : 5;
    const int* order = format == 2 ? order4 : order5;
    if (rank != want) return 0;
    bool empty = v.elements() == 0;
    u64 expected = 1;
    for (int p = 0; p < want; ++p) {
        int axis = order[p];
        if (v.shape[axis] == 1) continue;
        if ((u64)v.strides[axis] != expected) return 0;
        unsigned __int128 next = (unsigned __int128)expected * (u64)v.shape[axis];
        if (next > (unsigned __int128)UINT64_MAX && !empty) return 0;
        expected = (u64)next;
    }
    return 1;
}

// Strides of try_clone_with_memory_format (tensor.rs:1533-1575) when `for_clone`, else of
// try_contiguous (1606-1675) when it has to copy.  Returns a Status.
int ref_memory_format_strides(int format, int for_clone, int rank, const i64* shape, const i64* strides, i64* out_strides) {
    View v = make_view(nullptr, 0, rank, shape, strides);
    static const int order4[4] = {1, 3, 2, 0}, order5[5] = {1, 4, 3, 2, 0};
    const int want = format == 2 ? 4 : (format == 3 ? 5 : -1);
    std::vector<i64> o;
    if (want >= 0 && rank != want) {
        if (for_clone) { if (int s = contiguous_strides(v.shape, o)) return s; }   // preflight (1545-1549)
        return FORMAT_RANK;
    }
    int status = OK;
    if (format == 0) {
        if (!for_clone) return PRESERVE_UNSUPPORTED;
        if (v.elements() == 0 || is_non_overlapping_and_dense(v.shape, v.strides, v.elements())) o = v.strides;
        else status = elementwise_output_strides(v.shape, {Layout{&v.shape, &v.strides}}, o);
    } else if (format == 1) {
        status = contiguous_strides(v.shape, o);
    } else {
        status = strides_in_physical_order(v.shape, format == 2 ? order4 : order5, o);
    }
    if (status) return status;
    std::copy(o.begin(), o.end(), out_strides);
    return OK;
}

float ref_relu_value(float v) { return relu_value(v); }
float ref_relu_backward_value(float x, float g) { return relu_backward_value(x, g); }

}  // extern "C"
