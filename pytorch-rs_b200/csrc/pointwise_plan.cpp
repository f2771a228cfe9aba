// Planner and code generator for fused pointwise chains (host only).
//
// The reference runs one element loop per op and materialises every intermediate
// (src/tensor.rs:1805-1838, 2629-2716, 3546-3599).  Here a whole chain becomes one kernel that
// walks the OUTPUT's physical order: dims are sorted by the output's stride, adjacent dims that
// every operand strides through uniformly are merged, and each operand is classified by how it
// moves along the innermost output dim:
//   unit stride  -> 128-bit vector loads (scalar loads when the address is not 16-byte aligned)
//   stride 0     -> one scalar load broadcast over the vector (e.g. a per-row bias)
//   other stride -> if it is unit-stride along another dim, a 32x32 shared-memory staged
//                   transpose ("tiled" class); otherwise plain strided loads.
#include "pointwise_plan.h"

#include <algorithm>
#include <cstring>
#include <sstream>

#include "common.h"

namespace trs {

namespace {

struct Dim {
    long long size;
    long long in_s[TRS_MAX_INPUTS];
    long long out_s[TRS_MAX_OUTPUTS];
};

void magic_for(unsigned d, unsigned* magic, unsigned* shift) {
    // n / d == (umulhi(n, magic) + n) >> shift for 0 <= n < 2^31, 1 <= d < 2^31.
    unsigned s = 0;
    while ((1ull << s) < d) ++s;
    unsigned long long one = 1;
    *magic = (unsigned)(((one << 32) * ((one << s) - d)) / d + 1);
    *shift = s;
}

bool arity_ok(int op, int* n_args) {
    switch (op) {
        case TRS_OP_CONST: *n_args = 0; return true;
        case TRS_OP_ADD: case TRS_OP_SUB: case TRS_OP_MUL: case TRS_OP_DIV: case TRS_OP_RELU_VJP: case TRS_OP_NE:
            *n_args = 2; return true;
        case TRS_OP_NEG: case TRS_OP_RELU: case TRS_OP_EXP: case TRS_OP_RECIP: case TRS_OP_SQRT:
        case TRS_OP_SIN: case TRS_OP_COS: case TRS_OP_COPY:
            *n_args = 1; return true;
        default: return false;
    }
}

}  // namespace

int32_t pw_make_plan(const trs_program* prog, const trs_operand* inputs, const trs_operand* outputs, PwPlan* plan) {
    if (!prog || !outputs || !plan) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL program/outputs");
    const int n_in = prog->n_inputs, n_out = prog->n_outputs, n_ins = prog->n_instrs;
    if (n_in < 0 || n_in > TRS_MAX_INPUTS || n_out < 1 || n_out > TRS_MAX_OUTPUTS || n_ins < 0 || n_ins > TRS_MAX_INSTRS)
        return fail(TRS_ERR_INVALID_ARGUMENT, "program has %d inputs, %d instrs, %d outputs (limits %d/%d/%d)", n_in,
                    n_ins, n_out, TRS_MAX_INPUTS, TRS_MAX_INSTRS, TRS_MAX_OUTPUTS);
    if (n_in > 0 && !inputs) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL inputs");
    for (int j = 0; j < n_ins; ++j) {
        int args = 0;
        const trs_instr& in = prog->instrs[j];
        if (!arity_ok(in.op, &args)) return fail(TRS_ERR_INVALID_ARGUMENT, "instr %d: unknown op %d", j, in.op);
        if ((args >= 1 && (in.a < 0 || in.a >= n_in + j)) || (args >= 2 && (in.b < 0 || in.b >= n_in + j)))
            return fail(TRS_ERR_INVALID_ARGUMENT, "instr %d reads a value that is not defined before it", j);
    }
    for (int o = 0; o < n_out; ++o)
        if (prog->outputs[o] < 0 || prog->outputs[o] >= n_in + n_ins)
            return fail(TRS_ERR_INVALID_ARGUMENT, "output %d names value %d which does not exist", o, prog->outputs[o]);

    const int rank = outputs[0].rank;
    if (rank < 0 || rank > TRS_MAX_RANK) return fail(TRS_ERR_INVALID_ARGUMENT, "output rank %d out of range", rank);
    for (int o = 0; o < n_out; ++o) {
        if (outputs[o].rank != rank) return fail(TRS_ERR_INVALID_ARGUMENT, "outputs differ in rank");
        for (int a = 0; a < rank; ++a) {
            if (outputs[o].shape[a] != outputs[0].shape[a]) return fail(TRS_ERR_INVALID_ARGUMENT, "outputs differ in shape");
            if (outputs[o].shape[a] < 0 || outputs[o].stride[a] < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative size or stride");
        }
    }

    *plan = PwPlan();
    plan->n_in = n_in;
    plan->n_out = n_out;
    long long numel = 1;
    for (int a = 0; a < rank; ++a) {
        long long d = outputs[0].shape[a];
        if (d != 0 && numel > (long long)(INT64_MAX / d)) return fail(TRS_ERR_INVALID_ARGUMENT, "element count overflows");
        numel *= d;
    }
    plan->numel = numel;
    if (numel == 0) { plan->empty = true; return TRS_OK; }

    // Right-align inputs against the output shape; size-1 axes broadcast with stride 0.
    std::vector<Dim> dims;
    for (int a = 0; a < rank; ++a) {
        Dim d{};
        d.size = outputs[0].shape[a];
        for (int o = 0; o < n_out; ++o) d.out_s[o] = outputs[o].stride[a];
        for (int k = 0; k < n_in; ++k) {
            const trs_operand& in = inputs[k];
            if (in.rank < 0 || in.rank > rank) return fail(TRS_ERR_INVALID_ARGUMENT, "input %d has rank %d above the output rank %d", k, in.rank, rank);
            int lead = rank - in.rank;
            if (a < lead) { d.in_s[k] = 0; continue; }
            long long isz = in.shape[a - lead], ist = in.stride[a - lead];
            if (ist < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative stride");
            if (isz == d.size) d.in_s[k] = (isz == 1) ? 0 : ist;
            else if (isz == 1) d.in_s[k] = 0;
            else return fail(TRS_ERR_INVALID_ARGUMENT, "input %d axis %d has size %lld, not broadcastable to %lld", k, a - lead, isz, d.size);
        }
        if (d.size != 1) dims.push_back(d);
    }
    for (int k = 0; k < n_in; ++k) if (!inputs[k].base) return fail(TRS_ERR_INVALID_ARGUMENT, "input %d base is NULL", k);
    for (int o = 0; o < n_out; ++o) if (!outputs[o].base) return fail(TRS_ERR_INVALID_ARGUMENT, "output %d base is NULL", o);

    // A dimension of 2^31 or more elements is cut into (outer x inner) with a power-of-two inner
    // extent, so that every extent fits the 32-bit index arithmetic of the kernels.
    for (size_t j = 0; j < dims.size(); ++j) {
        if (dims[j].size < (1ll << 31)) continue;
        long long inner = 1ll << 30;
        while (inner > 1 && dims[j].size % inner != 0) inner >>= 1;
        if (dims[j].size / inner >= (1ll << 31))
            return fail(TRS_ERR_UNSUPPORTED, "a dimension of %lld elements cannot be split for 32-bit indexing", dims[j].size);
        Dim outer = dims[j];
        outer.size = dims[j].size / inner;
        for (int k = 0; k < n_in; ++k) outer.in_s[k] = dims[j].in_s[k] * inner;
        for (int o = 0; o < n_out; ++o) outer.out_s[o] = dims[j].out_s[o] * inner;
        dims[j].size = inner;
        dims.insert(dims.begin() + j, outer);      // the outer part precedes the inner part, like a leading axis
        ++j;
    }
    if (dims.empty()) { Dim d{}; d.size = 1; dims.push_back(d); }
    // Innermost first, by the first output's stride.
    std::stable_sort(dims.begin(), dims.end(), [](const Dim& x, const Dim& y) { return x.out_s[0] < y.out_s[0]; });
    // Merge dim j into its inner neighbour when every operand walks them as one run.
    std::vector<Dim> merged;
    merged.push_back(dims[0]);
    for (size_t j = 1; j < dims.size(); ++j) {
        Dim& prev = merged.back();
        bool ok = true;
        for (int k = 0; k < n_in && ok; ++k) ok = dims[j].in_s[k] == prev.in_s[k] * prev.size;
        for (int o = 0; o < n_out && ok; ++o) ok = dims[j].out_s[o] == prev.out_s[o] * prev.size;
        ok = ok && prev.size * dims[j].size < (1ll << 31);
        if (ok) prev.size *= dims[j].size;
        else merged.push_back(dims[j]);
    }
    const int nd = (int)merged.size();
    plan->ndim = nd;
    if (nd > TRS_MAX_RANK) return fail(TRS_ERR_UNSUPPORTED, "operand layout needs %d index dimensions (limit %d)", nd, TRS_MAX_RANK);

    PwParams& p = plan->params;
    std::memset(&p, 0, sizeof p);
    long long max_off = 0;
    for (int k = 0; k < n_in; ++k) {
        p.in[k] = (const float*)inputs[k].base + inputs[k].offset;
        long long ext = 0;
        for (int d = 0; d < nd; ++d) { p.in_stride[k][d] = merged[d].in_s[k]; ext += (merged[d].size - 1) * merged[d].in_s[k]; }
        max_off = std::max(max_off, ext);
    }
    for (int o = 0; o < n_out; ++o) {
        p.out[o] = (float*)outputs[o].base + outputs[o].offset;
        long long ext = 0;
        for (int d = 0; d < nd; ++d) { p.out_stride[o][d] = merged[d].out_s[o]; ext += (merged[d].size - 1) * merged[d].out_s[o]; }
        max_off = std::max(max_off, ext);
    }
    for (int d = 0; d < nd; ++d) p.size[d] = (unsigned)merged[d].size;
    plan->wide_offsets = max_off >= (1ll << 31) - 8;

    // ---- kernel class ---------------------------------------------------------------------
    bool outs_unit = true;
    for (int o = 0; o < n_out; ++o) outs_unit &= (p.out_stride[o][0] == 1) || merged[0].size == 1;
    int tdim = 0;
    if (outs_unit && nd >= 2) {
        for (int k = 0; k < n_in && !tdim; ++k) {
            if (p.in_stride[k][0] == 0 || p.in_stride[k][0] == 1) continue;
            for (int d = 1; d < nd; ++d)
                if (p.in_stride[k][d] == 1 && merged[d].size >= 8 && merged[0].size >= 8) { tdim = d; break; }
        }
    }
    if (tdim) {
        plan->tiled = true;
        plan->tdim = tdim;
        for (int k = 0; k < n_in; ++k)
            plan->in_kind[k] = (p.in_stride[k][tdim] == 1 && p.in_stride[k][0] != 1 && p.in_stride[k][0] != 0) ? IN_TRANSPOSED : IN_STRIDED;
        for (int o = 0; o < n_out; ++o) plan->out_kind[o] = OUT_STRIDED;
        // 128-bit variant: every operand's addresses stay 16-byte aligned when stepping 4 elements
        // along its own unit-stride axis, and both tiled extents are multiples of 4.
        bool vec = merged[0].size % 4 == 0 && merged[tdim].size % 4 == 0;
        auto strides_ok = [&](const void* base, const long long* st, int unit_dim) {
            if (((uintptr_t)base & 15u) != 0) return false;
            for (int d = 0; d < nd; ++d) if (d != unit_dim && st[d] % 4 != 0) return false;
            return true;
        };
        for (int k = 0; k < n_in && vec; ++k) {
            if (plan->in_kind[k] == IN_TRANSPOSED) vec = strides_ok(p.in[k], p.in_stride[k], tdim);
            else if (p.in_stride[k][0] == 1) vec = strides_ok(p.in[k], p.in_stride[k], 0);
            else vec = p.in_stride[k][0] == 0;              // broadcast along dim 0 is fine; other strides are not
        }
        for (int o = 0; o < n_out && vec; ++o) vec = p.out_stride[o][0] == 1 && strides_ok(p.out[o], p.out_stride[o], 0);
        int ntrans = 0;
        for (int k = 0; k < n_in; ++k) ntrans += plan->in_kind[k] == IN_TRANSPOSED;
        if (ntrans > 2) vec = false;                         // 64x65 floats of shared memory per staged input
        plan->tile_vec = vec;
        const long long tile = vec ? 64 : 32;
        unsigned long long tiles0 = (merged[0].size + tile - 1) / tile, tilest = (merged[tdim].size + tile - 1) / tile;
        unsigned long long total = tiles0 * tilest;
        for (int d = 1; d < nd; ++d) if (d != tdim) total *= (unsigned long long)merged[d].size;
        p.aux[0] = (unsigned)tiles0;
        p.aux[1] = (unsigned)tilest;
        p.total = total;
        plan->grid = total;
        plan->block = 256;
        plan->unroll = 1;
        if (total >= (1ull << 31)) return fail(TRS_ERR_UNSUPPORTED, "tiled pointwise launch of %llu tiles exceeds the grid limit", total);
        return TRS_OK;
    }

    // Vector class: 4 consecutive elements of the innermost dim per work item.
    const long long inner = merged[0].size;
    auto aligned = [&](const void* base, const long long* strides) {
        if (((uintptr_t)base & 15u) != 0) return false;
        for (int d = 1; d < nd; ++d) if (strides[d] % 4 != 0) return false;
        return true;
    };
    for (int k = 0; k < n_in; ++k) {
        long long s0 = p.in_stride[k][0];
        if (inner == 1 || s0 == 0) plan->in_kind[k] = IN_BCAST;
        else if (s0 == 1) plan->in_kind[k] = aligned(p.in[k], p.in_stride[k]) ? IN_VEC : IN_SCALAR4;
        else plan->in_kind[k] = IN_STRIDED;
    }
    for (int o = 0; o < n_out; ++o) {
        long long s0 = p.out_stride[o][0];
        if (s0 == 1 || inner == 1) plan->out_kind[o] = aligned(p.out[o], p.out_stride[o]) ? OUT_VEC : OUT_SCALAR4;
        else plan->out_kind[o] = OUT_STRIDED;
    }
    if (inner == 1) for (int o = 0; o < n_out; ++o) plan->out_kind[o] = OUT_STRIDED;
    plan->has_tail = (inner % 4) != 0;
    unsigned long long vecs0 = (unsigned long long)(inner + 3) / 4;
    unsigned long long total = vecs0;
    for (int d = 1; d < nd; ++d) total *= (unsigned long long)merged[d].size;
    p.aux[0] = (unsigned)vecs0;
    p.total = total;
    plan->wide_items = total >= (1ull << 31) - (1ull << 20);
    magic_for((unsigned)vecs0, &p.div_magic[0], &p.div_shift[0]);
    for (int d = 1; d < nd; ++d) magic_for(p.size[d], &p.div_magic[d], &p.div_shift[d]);
    int vec_inputs = 0;
    for (int k = 0; k < n_in; ++k) vec_inputs += plan->in_kind[k] != IN_BCAST;
    // Measured on B200: 2 vectors in flight per thread with 512-thread CTAs streams best for
    // chains with up to two streamed inputs (config 2: 6.66 TB/s against 6.54 with 4 x 256).
    plan->unroll = vec_inputs <= 4 ? 2 : 1;
    plan->block = vec_inputs <= 2 ? 512 : 256;
    unsigned long long per_cta = (unsigned long long)plan->block * plan->unroll;
    plan->grid = (total + per_cta - 1) / per_cta;
    if (plan->grid >= (1ull << 31)) return fail(TRS_ERR_UNSUPPORTED, "pointwise launch exceeds the grid limit");
    return TRS_OK;
}

// ---- code generation ---------------------------------------------------------------------------

namespace {

const char* kPreamble = R"SRC(
typedef unsigned int u32;
typedef unsigned long long u64;
struct Params {
    const float* in[8];
    float* out[4];
    long long in_stride[8][8];
    long long out_stride[4][8];
    u32 size[8];
    u32 div_magic[8];
    u32 div_shift[8];
    u64 total;
    u32 aux[4];
};
// Reference semantics (pytorch-rs src/tensor.rs:4388-4432): exact zeros keep their sign through
// relu, relu(NaN) is +0, the relu VJP passes the upstream for NaN or strictly positive inputs.
__device__ __forceinline__ float trs_relu(float v) {
    return (__float_as_uint(v) == 0x80000000u) ? v : fmaxf(v, 0.0f);      // fmaxf already keeps +0 and sends NaN to +0; only -0 needs the pass-through
}
__device__ __forceinline__ float trs_relu_vjp(float x, float g) {
    u32 b = __float_as_uint(x), mag = b & 0x7fffffffu;
    return (mag > 0x7f800000u || ((b >> 31) == 0u && mag != 0u)) ? g : 0.0f;
}
__device__ __forceinline__ float trs_neg(float v) { return __uint_as_float(__float_as_uint(v) ^ 0x80000000u); }
__device__ __forceinline__ float trs_sqrt(float v) {
    u32 b = __float_as_uint(v), mag = b & 0x7fffffffu;
    return ((b >> 31) != 0u && mag != 0u && mag <= 0x7f800000u) ? __uint_as_float(0x7fc00000u) : __fsqrt_rn(v);
}
// exp within 1 ulp of glibc's expf (the reference calls the platform's libm expf, src/tensor.rs:2398-2400; glibc's is
// within 0.502 ulp of the true value, CUDA's expf only within 2).  Cody-Waite reduction x = j ln2 + r with ln2 in two
// parts, |r| <= ln2/2, exp(r) as a degree-6 polynomial (minimax, error 3e-9) in Horner form, scaled by 2^j.  For
// |x| <= 87 the result is a normal number and the scaling is an add into the exponent field (j sits in the low
// mantissa bits of the rounding constant's sum); everything else -- overflow, subnormal results, inf, NaN -- takes
// the out-of-line path, which scales in two steps so that a subnormal result is rounded once.  Checked against glibc
// expf on every float32 in [-104.5, 89.5]: never more than 1 ulp apart.  exp(+-0) = exp(+-denormal) = 1,
// exp(x > 88.73) = +inf, exp(x < -103.98) = +0, NaN stays NaN.
__device__ __noinline__ float trs_exp_slow(float x) {
    const float t = x < -110.0f ? -110.0f : (x > 90.0f ? 90.0f : x);      // false for NaN: it passes through
    const float j = __fsub_rn(__fmaf_rn(t, 1.44269502f, 12582912.0f), 12582912.0f);
    float r = __fmaf_rn(j, -0.693145752f, t);
    r = __fmaf_rn(j, -1.42860677e-06f, r);
    float q = __uint_as_float(0x3ab6da3fu);
    q = __fmaf_rn(q, r, __uint_as_float(0x3c091dc9u));
    q = __fmaf_rn(q, r, __uint_as_float(0x3d2aaa2fu));
    q = __fmaf_rn(q, r, __uint_as_float(0x3e2aaa47u));
    q = __fmaf_rn(q, r, 0.5f);
    q = __fmaf_rn(q, r, 1.0f);
    const float p = __fmaf_rn(q, r, 1.0f);
    const int ji = __float2int_rn(j);                     // 0 for NaN
    const int h = ji >> 1;
    const float s1 = __uint_as_float((u32)(h + 127) << 23), s2 = __uint_as_float((u32)(ji - h + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}
__device__ __forceinline__ float trs_exp(float x) {
    if (!(fabsf(x) <= 87.0f)) return trs_exp_slow(x);
    const float m = __fmaf_rn(x, 1.44269502f, 12582912.0f);       // 1.5 * 2^23 + nearest integer to x / ln2
    const float j = __fsub_rn(m, 12582912.0f);
    float r = __fmaf_rn(j, -0.693145752f, x);
    r = __fmaf_rn(j, -1.42860677e-06f, r);
    float q = __uint_as_float(0x3ab6da3fu);               // 0x1.6db47ep-10
    q = __fmaf_rn(q, r, __uint_as_float(0x3c091dc9u));    // 0x1.123b92p-7
    q = __fmaf_rn(q, r, __uint_as_float(0x3d2aaa2fu));    // 0x1.55545ep-5
    q = __fmaf_rn(q, r, __uint_as_float(0x3e2aaa47u));    // 0x1.55548ep-3
    q = __fmaf_rn(q, r, 0.5f);
    q = __fmaf_rn(q, r, 1.0f);
    const float p = __fmaf_rn(q, r, 1.0f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(m) << 23));
}
__device__ __forceinline__ u32 trs_div(u32 n, u32 magic, u32 shift) { return (__umulhi(n, magic) + n) >> shift; }
)SRC";

std::string value_name(int v) { return "v" + std::to_string(v); }

void emit_chain(std::ostringstream& s, const trs_program* prog) {
    const int n_in = prog->n_inputs;
    s << "__device__ __forceinline__ void trs_chain(const float (&x)[NIN > 0 ? NIN : 1], float (&y)[NOUT]) {\n";
    for (int k = 0; k < n_in; ++k) s << "    const float v" << k << " = x[" << k << "];\n";
    for (int j = 0; j < prog->n_instrs; ++j) {
        const trs_instr& in = prog->instrs[j];
        std::string a = value_name(in.a), b = value_name(in.b), d = "    const float " + value_name(n_in + j) + " = ";
        switch (in.op) {
            case TRS_OP_CONST: {
                unsigned bits;
                std::memcpy(&bits, &in.imm, 4);
                char buf[64];
                snprintf(buf, sizeof buf, "__uint_as_float(0x%08xu)", bits);
                s << d << buf << ";\n";
                break;
            }
            case TRS_OP_ADD: s << d << "__fadd_rn(" << a << ", " << b << ");\n"; break;
            case TRS_OP_SUB: s << d << "__fsub_rn(" << a << ", " << b << ");\n"; break;
            case TRS_OP_MUL: s << d << "__fmul_rn(" << a << ", " << b << ");\n"; break;
            case TRS_OP_DIV: s << d << "__fdiv_rn(" << a << ", " << b << ");\n"; break;
            case TRS_OP_NEG: s << d << "trs_neg(" << a << ");\n"; break;
            case TRS_OP_RELU: s << d << "trs_relu(" << a << ");\n"; break;
            case TRS_OP_EXP: s << d << "trs_exp(" << a << ");\n"; break;
            case TRS_OP_RELU_VJP: s << d << "trs_relu_vjp(" << a << ", " << b << ");\n"; break;
            case TRS_OP_RECIP: s << d << "__fmul_rn(1.0f, __frcp_rn(" << a << "));\n"; break;
            case TRS_OP_SQRT: s << d << "trs_sqrt(" << a << ");\n"; break;
            case TRS_OP_SIN: s << d << "sinf(" << a << ");\n"; break;
            case TRS_OP_COS: s << d << "cosf(" << a << ");\n"; break;
            case TRS_OP_NE: s << d << "((" << a << " != " << b << ") ? 1.0f : 0.0f);\n"; break;
            default: s << d << a << ";\n"; break;
        }
    }
    for (int o = 0; o < prog->n_outputs; ++o) s << "    y[" << o << "] = " << value_name(prog->outputs[o]) << ";\n";
    s << "}\n";
}

const char* kVectorKernel = R"SRC(
// Vector class: one work item = 4 consecutive elements of the innermost output dim.
extern "C" __global__ void __launch_bounds__(BLOCK) trs_pw(const Params p) {
    // Launched with programmatic stream serialization: blocks of this grid become resident while the
    // previous kernel of the stream drains.  Nothing is read or written before that kernel has completed
    // and flushed; after that the next kernel's blocks may take the slots this grid frees.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    float xin[UNROLL][NIN > 0 ? NIN : 1][4];
    ofs_t ooff[UNROLL][NOUT];
    u32 nvalid[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const item_t item = (item_t)blockIdx.x * (BLOCK * UNROLL) + (item_t)u * BLOCK + threadIdx.x;
        nvalid[u] = 0;
        if (item < (item_t)p.total) {
            u32 c[NDIM];
#if NDIM == 1
            c[0] = (u32)item;
#elif WIDE_ITEMS
            item_t r = item;
            c[0] = (u32)(r % p.aux[0]); r /= p.aux[0];
#pragma unroll
            for (int d = 1; d < NDIM - 1; ++d) { c[d] = (u32)(r % p.size[d]); r /= p.size[d]; }
            c[NDIM - 1] = (u32)r;
#else
            u32 r = (u32)item;
            { u32 q = trs_div(r, p.div_magic[0], p.div_shift[0]); c[0] = r - q * p.aux[0]; r = q; }
#pragma unroll
            for (int d = 1; d < NDIM - 1; ++d) { u32 q = trs_div(r, p.div_magic[d], p.div_shift[d]); c[d] = r - q * p.size[d]; r = q; }
            c[NDIM - 1] = r;
#endif
            const u32 e0 = c[0] * 4u;
            const u32 left = p.size[0] - e0;
            nvalid[u] = HAS_TAIL ? (left < 4u ? left : 4u) : 4u;
#pragma unroll
            for (int k = 0; k < NIN; ++k) {
                ofs_t off = (ofs_t)e0 * (IN_KIND[k] == 2 ? (ofs_t)0 : (IN_KIND[k] == 3 ? (ofs_t)p.in_stride[k][0] : (ofs_t)1));
#pragma unroll
                for (int d = 1; d < NDIM; ++d) off += (ofs_t)c[d] * (ofs_t)p.in_stride[k][d];
                const float* src = p.in[k] + off;
                if (IN_KIND[k] == 0 && (!HAS_TAIL || nvalid[u] == 4u)) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(src));
                    xin[u][k][0] = t.x; xin[u][k][1] = t.y; xin[u][k][2] = t.z; xin[u][k][3] = t.w;
                } else if (IN_KIND[k] == 2) {
                    const float t = __ldg(src);
                    xin[u][k][0] = t; xin[u][k][1] = t; xin[u][k][2] = t; xin[u][k][3] = t;
                } else {
                    const ofs_t step = IN_KIND[k] == 3 ? (ofs_t)p.in_stride[k][0] : (ofs_t)1;
#pragma unroll
                    for (int e = 0; e < 4; ++e) xin[u][k][e] = (u32)e < nvalid[u] ? __ldg(src + (ofs_t)e * step) : 0.0f;
                }
            }
#pragma unroll
            for (int o = 0; o < NOUT; ++o) {
                ofs_t off = (ofs_t)e0 * (OUT_KIND[o] == 3 ? (ofs_t)p.out_stride[o][0] : (ofs_t)1);
#pragma unroll
                for (int d = 1; d < NDIM; ++d) off += (ofs_t)c[d] * (ofs_t)p.out_stride[o][d];
                ooff[u][o] = off;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        if (nvalid[u] == 0u) continue;
        float yout[4][NOUT];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float xs[NIN > 0 ? NIN : 1];
#pragma unroll
            for (int k = 0; k < NIN; ++k) xs[k] = xin[u][k][e];
            trs_chain(xs, yout[e]);
        }
#pragma unroll
        for (int o = 0; o < NOUT; ++o) {
            float* dst = p.out[o] + ooff[u][o];
            if (OUT_KIND[o] == 0 && (!HAS_TAIL || nvalid[u] == 4u)) {
                __stcs(reinterpret_cast<float4*>(dst), make_float4(yout[0][o], yout[1][o], yout[2][o], yout[3][o]));
            } else {
                const ofs_t step = OUT_KIND[o] == 3 ? (ofs_t)p.out_stride[o][0] : (ofs_t)1;
#pragma unroll
                for (int e = 0; e < 4; ++e) if ((u32)e < nvalid[u]) dst[(ofs_t)e * step] = yout[e][o];
            }
        }
    }
}
)SRC";

const char* kTiledKernel = R"SRC(
// Tiled class: 32x32 tiles over (dim 0 = the outputs' unit-stride dim, dim TDIM = the dim along
// which the "transposed" inputs are unit-stride).  Transposed inputs are read coalesced along
// TDIM into padded shared memory and consumed along dim 0; everything else is accessed along
// dim 0 directly, so every global access of the hot operands is coalesced.
extern "C" __global__ void __launch_bounds__(256) trs_pw(const Params p) {
    // Launched with programmatic stream serialization: blocks of this grid become resident while the
    // previous kernel of the stream drains.  Nothing is read or written before that kernel has completed
    // and flushed; after that the next kernel's blocks may take the slots this grid frees.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ float tile[NTRANS > 0 ? NTRANS : 1][32][33];
    u64 cta = blockIdx.x;
    const u32 t0 = (u32)(cta % p.aux[0]); cta /= p.aux[0];
    const u32 tt = (u32)(cta % p.aux[1]); cta /= p.aux[1];
    ofs_t in_off[NIN > 0 ? NIN : 1];
    ofs_t out_off[NOUT];
#pragma unroll
    for (int k = 0; k < NIN; ++k) in_off[k] = 0;
#pragma unroll
    for (int o = 0; o < NOUT; ++o) out_off[o] = 0;
#pragma unroll
    for (int d = 1; d < NDIM; ++d) {
        if (d == TDIM) continue;
        const u32 c = (u32)(cta % p.size[d]); cta /= p.size[d];
#pragma unroll
        for (int k = 0; k < NIN; ++k) in_off[k] += (ofs_t)c * (ofs_t)p.in_stride[k][d];
#pragma unroll
        for (int o = 0; o < NOUT; ++o) out_off[o] += (ofs_t)c * (ofs_t)p.out_stride[o][d];
    }
    const u32 tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
    const u32 size0 = p.size[0], sizet = p.size[TDIM];
    {
        int q = 0;
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
            if (IN_KIND[k] != 4) continue;
            const u32 it = tt * 32u + tx;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const u32 i0 = t0 * 32u + ty + 8u * j;
                if (i0 < size0 && it < sizet)
                    tile[q][ty + 8 * j][tx] = __ldcs(p.in[k] + in_off[k] + (ofs_t)i0 * (ofs_t)p.in_stride[k][0] + (ofs_t)it);
            }
            ++q;
        }
    }
    __syncthreads();
    const u32 i0 = t0 * 32u + tx;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const u32 it = tt * 32u + ty + 8u * j;
        if (i0 >= size0 || it >= sizet) continue;
        float xs[NIN > 0 ? NIN : 1];
        int q = 0;
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
            if (IN_KIND[k] == 4) { xs[k] = tile[q][tx][ty + 8 * j]; ++q; }
            else xs[k] = __ldg(p.in[k] + in_off[k] + (ofs_t)i0 * (ofs_t)p.in_stride[k][0] + (ofs_t)it * (ofs_t)p.in_stride[k][TDIM]);
        }
        float ys[NOUT];
        trs_chain(xs, ys);
#pragma unroll
        for (int o = 0; o < NOUT; ++o)
            p.out[o][out_off[o] + (ofs_t)i0 * (ofs_t)p.out_stride[o][0] + (ofs_t)it * (ofs_t)p.out_stride[o][TDIM]] = ys[o];
    }
}
)SRC";

const char* kTiledVecKernel = R"SRC(
// Tiled class, 128-bit variant: 64x64 tiles.  Staged inputs are read with float4 along TDIM
// (their unit-stride axis) into padded shared memory; everything else moves as float4 along dim 0.
extern "C" __global__ void __launch_bounds__(256) trs_pw(const Params p) {
    // Launched with programmatic stream serialization: blocks of this grid become resident while the
    // previous kernel of the stream drains.  Nothing is read or written before that kernel has completed
    // and flushed; after that the next kernel's blocks may take the slots this grid frees.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ float tile[NTRANS > 0 ? NTRANS : 1][64][65];
    u64 cta = blockIdx.x;
    const u32 t0 = (u32)(cta % p.aux[0]); cta /= p.aux[0];
    const u32 tt = (u32)(cta % p.aux[1]); cta /= p.aux[1];
    ofs_t in_off[NIN > 0 ? NIN : 1];
    ofs_t out_off[NOUT];
#pragma unroll
    for (int k = 0; k < NIN; ++k) in_off[k] = 0;
#pragma unroll
    for (int o = 0; o < NOUT; ++o) out_off[o] = 0;
#pragma unroll
    for (int d = 1; d < NDIM; ++d) {
        if (d == TDIM) continue;
        const u32 c = (u32)(cta % p.size[d]); cta /= p.size[d];
#pragma unroll
        for (int k = 0; k < NIN; ++k) in_off[k] += (ofs_t)c * (ofs_t)p.in_stride[k][d];
#pragma unroll
        for (int o = 0; o < NOUT; ++o) out_off[o] += (ofs_t)c * (ofs_t)p.out_stride[o][d];
    }
    const u32 q4 = (threadIdx.x & 15u) * 4u, r16 = threadIdx.x >> 4;
    const u32 size0 = p.size[0], sizet = p.size[TDIM];
    {
        int q = 0;
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
            if (IN_KIND[k] != 4) continue;
            const u32 it = tt * 64u + q4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const u32 i0l = r16 + 16u * j, i0 = t0 * 64u + i0l;
                if (i0 < size0 && it < sizet) {
                    const float4 v = __ldcs(reinterpret_cast<const float4*>(p.in[k] + in_off[k] + (ofs_t)i0 * (ofs_t)p.in_stride[k][0] + (ofs_t)it));
                    tile[q][i0l][q4] = v.x; tile[q][i0l][q4 + 1] = v.y; tile[q][i0l][q4 + 2] = v.z; tile[q][i0l][q4 + 3] = v.w;
                }
            }
            ++q;
        }
    }
    __syncthreads();
    const u32 i0 = t0 * 64u + q4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const u32 itl = r16 + 16u * j, it = tt * 64u + itl;
        if (i0 >= size0 || it >= sizet) continue;
        float xin[NIN > 0 ? NIN : 1][4];
        int q = 0;
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
            if (IN_KIND[k] == 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) xin[k][e] = tile[q][q4 + e][itl];
                ++q;
            } else {
                const float* src = p.in[k] + in_off[k] + (ofs_t)it * (ofs_t)p.in_stride[k][TDIM];
                if (p.in_stride[k][0] == 0) {
                    const float t = __ldg(src);
                    xin[k][0] = t; xin[k][1] = t; xin[k][2] = t; xin[k][3] = t;
                } else {
                    const float4 v = __ldcs(reinterpret_cast<const float4*>(src + i0));
                    xin[k][0] = v.x; xin[k][1] = v.y; xin[k][2] = v.z; xin[k][3] = v.w;
                }
            }
        }
        float yout[4][NOUT];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float xs[NIN > 0 ? NIN : 1];
#pragma unroll
            for (int k = 0; k < NIN; ++k) xs[k] = xin[k][e];
            trs_chain(xs, yout[e]);
        }
#pragma unroll
        for (int o = 0; o < NOUT; ++o)
            __stcs(reinterpret_cast<float4*>(p.out[o] + out_off[o] + (ofs_t)i0 + (ofs_t)it * (ofs_t)p.out_stride[o][TDIM]),
                   make_float4(yout[0][o], yout[1][o], yout[2][o], yout[3][o]));
    }
}
)SRC";

}  // namespace

// Everything the generated source depends on, as a short byte string: the kernel cache is keyed by it so
// that a cache hit does not have to build (and hash) kilobytes of source text per launch.
std::string pw_cache_key(const trs_program* prog, const PwPlan& plan) {
    std::string key;
    key.reserve(64 + (size_t)prog->n_instrs * sizeof(trs_instr));
    auto put = [&key](int v) { key.push_back((char)(v & 0xff)); key.push_back((char)((v >> 8) & 0xff)); };
    put(plan.n_in); put(plan.n_out); put(plan.ndim); put(plan.unroll); put(plan.block); put(plan.tdim);
    put((plan.has_tail ? 1 : 0) | (plan.wide_items ? 2 : 0) | (plan.wide_offsets ? 4 : 0) | (plan.tiled ? 8 : 0) | (plan.tile_vec ? 16 : 0));
    for (int k = 0; k < plan.n_in; ++k) put(plan.in_kind[k]);
    for (int o = 0; o < plan.n_out; ++o) put(plan.out_kind[o]);
    put(prog->n_inputs); put(prog->n_instrs); put(prog->n_outputs);
    for (int o = 0; o < prog->n_outputs; ++o) put(prog->outputs[o]);
    for (int j = 0; j < prog->n_instrs; ++j) {
        const trs_instr& in = prog->instrs[j];
        put(in.op); put(in.a);
        // only the fields the emitted text reads: `imm` of a constant, `b` of a binary op
        const bool binary = in.op == TRS_OP_ADD || in.op == TRS_OP_SUB || in.op == TRS_OP_MUL || in.op == TRS_OP_DIV ||
                            in.op == TRS_OP_RELU_VJP || in.op == TRS_OP_NE;
        if (in.op == TRS_OP_CONST) key.append(reinterpret_cast<const char*>(&in.imm), sizeof in.imm);
        else if (binary) put(in.b);
    }
    return key;
}

std::string pw_generate_source(const trs_program* prog, const PwPlan& plan) {
    std::ostringstream s;
    s << "#define NIN " << plan.n_in << "\n#define NOUT " << plan.n_out << "\n#define NDIM " << plan.ndim << "\n";
    s << "#define UNROLL " << plan.unroll << "\n#define BLOCK " << plan.block << "\n";
    s << "#define HAS_TAIL " << (plan.has_tail ? 1 : 0) << "\n#define WIDE_ITEMS " << (plan.wide_items ? 1 : 0) << "\n";
    s << "#define TDIM " << plan.tdim << "\n";
    int ntrans = 0;
    for (int k = 0; k < plan.n_in; ++k) ntrans += plan.in_kind[k] == IN_TRANSPOSED;
    s << "#define NTRANS " << ntrans << "\n";
    s << "typedef " << (plan.wide_offsets ? "long long" : "int") << " ofs_t;\n";
    s << "typedef " << (plan.wide_items ? "unsigned long long" : "unsigned int") << " item_t;\n";
    s << kPreamble;
    s << "__device__ constexpr int IN_KIND[" << std::max(plan.n_in, 1) << "] = {";
    for (int k = 0; k < std::max(plan.n_in, 1); ++k) s << (k ? ", " : "") << (k < plan.n_in ? plan.in_kind[k] : 0);
    s << "};\n__device__ constexpr int OUT_KIND[" << plan.n_out << "] = {";
    for (int o = 0; o < plan.n_out; ++o) s << (o ? ", " : "") << plan.out_kind[o];
    s << "};\n";
    emit_chain(s, prog);
    s << (plan.tiled ? (plan.tile_vec ? kTiledVecKernel : kTiledKernel) : kVectorKernel);
    return s.str();
}

}  // namespace trs
