// Lowering of a pending expression to the fusion IR and the matmul descriptor of the C ABI.
//
// materialize(S) turns the expression under storage S into ONE trs_pointwise launch: pending
// operands become SSA instructions, materialised views become inputs, and every pending
// intermediate that something else still holds (a user tensor, a saved tensor of the autograd
// tape, another pending expression) becomes an extra output, so nothing is computed twice.
// A pending matmul directly under add(bias) / relu / relu_vjp is run as a GEMM with that
// epilogue instead (bias+relu for the forward layer, relu-VJP for its backward).
#include <algorithm>
#include <unordered_map>

#include "engine.h"

namespace trsh {

namespace {

bool same_view(const View& a, const View& b) {
    return a.st.get() == b.st.get() && a.offset == b.offset && a.shape == b.shape && a.strides == b.strides;
}

trs_operand operand_of(float* base, i64 offset, const Shape& shape, const Shape& strides) {
    trs_operand op{};
    op.base = base;
    op.offset = offset;
    op.rank = (int32_t)shape.size();
    if (shape.size() > TRS_MAX_RANK) throw Error(ErrKind::InvalidArgument, "tensor rank above 8 is not supported on CUDA");
    for (size_t i = 0; i < shape.size(); ++i) { op.shape[i] = shape[i]; op.stride[i] = strides[i]; }
    return op;
}

float* alloc_values(Storage& st) { return alloc_floats(st.count, st.device); }

// ---- matmul ---------------------------------------------------------------------------------------

struct Epilogue {
    int kind = TRS_EPI_NONE;
    const float* bias = nullptr;
    const float* aux = nullptr;
    float* preact = nullptr;
};

// `out`: the storage that receives C; when `out_image` is set the matmul also writes C's lo image into it.
void run_matmul(Node& mm, float* c, const Epilogue& epi, int device, Storage* out = nullptr, bool out_image = false) {
    View& a = mm.args[0];
    View& b = mm.args[1];
    if (a.st->node) materialize(a.st, true);
    if (b.st->node) materialize(b.st, true);
    const bool batched = mm.shape.size() == 3;
    trs_gemm_desc d{};
    d.batch = batched ? mm.shape[0] : 1;
    d.m = mm.shape[mm.shape.size() - 2];
    d.n = mm.shape[mm.shape.size() - 1];
    d.k = a.shape.back();
    d.a = a.st->ptr + a.offset;
    d.b = b.st->ptr + b.offset;
    const size_t ar = a.shape.size(), br = b.shape.size();
    d.a_batch_stride = ar == 3 ? a.strides[0] : 0;
    d.a_row_stride = a.strides[ar - 2];
    d.a_col_stride = a.strides[ar - 1];
    d.b_batch_stride = br == 3 ? b.strides[0] : 0;
    d.b_row_stride = b.strides[br - 2];
    d.b_col_stride = b.strides[br - 1];
    d.c = c;
    d.c_batch_stride = d.m * d.n;
    d.c_row_stride = d.n;
    d.bias = epi.bias;
    d.aux = epi.aux;
    d.preact = epi.preact;
    d.epilogue = epi.kind;
    d.algo = TRS_GEMM_AUTO;
    // Operand images: a storage's lo values are computed once and kept beside it, so a weight, an activation that
    // feeds both a forward and a backward product, or any operand used twice is prepared once, not per call.
    trs_gemm_planes planes{};
    int32_t algo = 0, a_used = 0, b_used = 0;
    check_cuda(trs_matmul_plan(&d, &algo, &a_used, &b_used), "matmul");
    i64 a_numel = 1, b_numel = 1;
    for (i64 e : a.shape) a_numel *= e;
    for (i64 e : b.shape) b_numel *= e;
    if (a_used && ensure_lo_image(*a.st, a_numel)) { planes.a_lo = a.st->lo + a.offset; planes.a_flag = a.st->lo_flag; }
    if (b_used && ensure_lo_image(*b.st, b_numel)) { planes.b_lo = b.st->lo + b.offset; planes.b_flag = b.st->lo_flag; }
    const bool tensor_core = algo == TRS_GEMM_TCGEN05_3XTF32 || algo == TRS_GEMM_TCGEN05_3XTF32_2CTA;
    if (out && out_image && tensor_core && plane_cache_enabled() && !out->lo) {
        alloc_lo_image(*out);
        planes.c_lo = out->lo;
        planes.c_flag = out->lo_flag;
    }
    int32_t status = trs_matmul_f32_planes(&d, &planes, stream_for(device));
    if (status != TRS_OK && planes.c_lo) { free_floats(device, out->lo); out->lo = nullptr; out->lo_flag = nullptr; }
    check_cuda(status, "matmul");
}

bool is_pending_matmul(const View& v) { return v.st->node && v.st->node->op == OP_MATMUL; }

// A per-column bias: materialised, unit stride along the last axis, broadcast along all others.
bool is_column_bias(const View& v, const Shape& out_shape) {
    if (v.st->node || v.shape.empty()) return false;
    const i64 n = out_shape.back();
    if (v.shape.back() != n || (n > 1 && v.strides.back() != 1)) return false;
    for (size_t i = 0; i + 1 < v.shape.size(); ++i) if (v.shape[i] != 1) return false;
    return true;
}

// Holders of `st` other than the single expression edge that leads to it.
long external_holders(const std::shared_ptr<Storage>& st) { return st.use_count() - 1; }

// Tries the fused-epilogue forms with `root` as the outermost node.  Returns true when it ran.
bool try_fused_matmul(const std::shared_ptr<Storage>& root, bool for_matmul) {
    Node& r = *root->node;
    if (r.strides != contiguous_strides(r.shape) || r.shape.size() < 2) return false;
    const int device = root->device;
    auto bias_add = [&](Node& add, View** mm, View** bias) {
        if (add.op != TRS_OP_ADD) return false;
        for (int side = 0; side < 2; ++side) {
            View& m = add.args[side];
            View& b = add.args[1 - side];
            if (is_pending_matmul(m) && external_holders(m.st) == 0 && is_column_bias(b, add.shape)) { *mm = &m; *bias = &b; return true; }
        }
        return false;
    };
    View *mm = nullptr, *bias = nullptr;
    if (bias_add(r, &mm, &bias)) {                                         // X @ W + b
        float* c = alloc_values(*root);
        Epilogue e; e.kind = TRS_EPI_BIAS; e.bias = bias->st->ptr + bias->offset;
        run_matmul(*mm->st->node, c, e, device, root.get(), for_matmul);
        root->ptr = c; root->node.reset();
        return true;
    }
    if (r.op == TRS_OP_RELU) {
        View& inner = r.args[0];
        if (is_pending_matmul(inner) && external_holders(inner.st) == 0) {   // relu(X @ W)
            float* c = alloc_values(*root);
            Epilogue e; e.kind = TRS_EPI_RELU;
            run_matmul(*inner.st->node, c, e, device, root.get(), for_matmul);
            root->ptr = c; root->node.reset();
            return true;
        }
        if (inner.st->node && inner.st->node->op == TRS_OP_ADD && inner.st->node->strides == r.strides &&
            bias_add(*inner.st->node, &mm, &bias)) {                         // relu(X @ W + b)
            const bool keep_preact = external_holders(inner.st) > 0;        // e.g. saved for the relu VJP
            float* c = alloc_values(*root);
            Epilogue e; e.kind = TRS_EPI_BIAS_RELU; e.bias = bias->st->ptr + bias->offset;
            float* pre = nullptr;
            if (keep_preact) { pre = alloc_values(*inner.st); e.preact = pre; }
            std::shared_ptr<Storage> inner_st = inner.st;
            run_matmul(*mm->st->node, c, e, device, root.get(), for_matmul);
            if (keep_preact) { inner_st->ptr = pre; inner_st->node.reset(); }
            root->ptr = c; root->node.reset();
            return true;
        }
    }
    if (r.op == TRS_OP_RELU_VJP) {                                          // relu_vjp(Z, dY @ W^T)
        View& z = r.args[0];
        View& g = r.args[1];
        if (is_pending_matmul(g) && external_holders(g.st) == 0 && !z.st->node && z.shape == r.shape &&
            z.strides == r.strides) {
            float* c = alloc_values(*root);
            Epilogue e; e.kind = TRS_EPI_RELU_VJP; e.aux = z.st->ptr + z.offset;
            // dZ of a linear layer: its next reader is the weight-gradient product X^T @ dZ, so its image is written now
            run_matmul(*g.st->node, c, e, device, root.get(), true);
            root->ptr = c; root->node.reset();
            return true;
        }
    }
    return false;
}

// ---- pointwise ------------------------------------------------------------------------------------

struct Dag {
    std::vector<Storage*> order;                       // pending pointwise storages, operands first
    std::unordered_map<Storage*, int> refs;            // expression edges into each pending storage
    std::unordered_map<Storage*, int> value;           // SSA value index
    std::vector<const View*> leaves;
    std::vector<std::shared_ptr<Storage>> matmuls;     // pending matmuls found under the root
};

void collect(Storage* s, Dag& dag) {
    for (const View& a : s->node->args) {
        if (a.st->node) {
            if (a.st->node->op == OP_MATMUL) { dag.matmuls.push_back(a.st); continue; }
            const bool first = dag.refs.find(a.st.get()) == dag.refs.end();
            dag.refs[a.st.get()] += 1;
            if (first) collect(a.st.get(), dag);
        } else {
            bool seen = false;
            for (const View* l : dag.leaves) seen |= same_view(*l, a);
            if (!seen) dag.leaves.push_back(&a);
        }
    }
    dag.order.push_back(s);
}

}  // namespace

void materialize(const std::shared_ptr<Storage>& root, bool for_matmul) {
    std::lock_guard<std::recursive_mutex> lock(g_engine_mu);
    if (!root->node) return;
    const int device = root->device;
    if (root->node->op == OP_MATMUL) {
        float* c = alloc_values(*root);
        run_matmul(*root->node, c, Epilogue{}, device, root.get(), for_matmul);
        root->ptr = c;
        root->node.reset();
        return;
    }
    if (try_fused_matmul(root, for_matmul)) return;

    for (int attempt = 0; attempt < 64; ++attempt) {
        Dag dag;
        collect(root.get(), dag);
        if (!dag.matmuls.empty()) {
            for (auto& m : dag.matmuls) materialize(m);     // plain GEMMs, then they are ordinary inputs
            continue;
        }
        // Pending intermediates that something outside this expression still holds.
        std::vector<const View*> extra;
        for (Storage* s : dag.order) {
            if (s == root.get()) continue;
            for (Storage* user : dag.order)
                for (const View& a : user->node->args)
                    if (a.st.get() == s && a.st.use_count() > dag.refs[s]) {
                        bool seen = false;
                        for (const View* e : extra) seen |= e->st.get() == s;
                        if (!seen) extra.push_back(&a);
                    }
        }
        int instrs = (int)dag.order.size();
        if ((int)extra.size() > TRS_MAX_OUTPUTS - 1 || (int)dag.leaves.size() > TRS_MAX_INPUTS || instrs > TRS_MAX_INSTRS) {
            // Too large for one kernel: compute the held intermediates (or, failing that, the
            // root's own operands) first, which turns them into inputs, then try again.
            if (!extra.empty()) { std::shared_ptr<Storage> st = extra.front()->st; materialize(st); continue; }
            bool progressed = false;
            for (const View& a : root->node->args)
                if (a.st->node) { std::shared_ptr<Storage> st = a.st; materialize(st); progressed = true; break; }
            if (!progressed) throw Error(ErrKind::InvalidArgument, "pointwise expression exceeds the fusion limits");
            continue;
        }

        trs_program prog{};
        prog.n_inputs = (int32_t)dag.leaves.size();
        std::vector<trs_operand> ins(std::max<size_t>(dag.leaves.size(), 1));
        for (size_t i = 0; i < dag.leaves.size(); ++i) {
            const View& l = *dag.leaves[i];
            ins[i] = operand_of(l.st->ptr, l.offset, l.shape, l.strides);
        }
        auto value_of = [&](const View& a) -> int {
            if (a.st->node) return dag.value.at(a.st.get());
            for (size_t i = 0; i < dag.leaves.size(); ++i) if (same_view(*dag.leaves[i], a)) return (int)i;
            throw Error(ErrKind::InvalidArgument, "internal: operand not found while lowering");
        };
        int next = prog.n_inputs;
        for (Storage* s : dag.order) {
            const Node& n = *s->node;
            trs_instr& in = prog.instrs[prog.n_instrs++];
            in.op = n.op;
            in.imm = n.imm;
            in.a = n.args.size() > 0 ? value_of(n.args[0]) : 0;
            in.b = n.args.size() > 1 ? value_of(n.args[1]) : 0;
            dag.value[s] = next++;
        }
        std::vector<Storage*> out_st{root.get()};
        for (const View* e : extra) out_st.push_back(e->st.get());
        std::vector<trs_operand> outs(out_st.size());
        std::vector<float*> bufs(out_st.size());
        prog.n_outputs = (int32_t)out_st.size();
        for (size_t o = 0; o < out_st.size(); ++o) {
            bufs[o] = alloc_values(*out_st[o]);
            outs[o] = operand_of(bufs[o], 0, out_st[o]->node->shape, out_st[o]->node->strides);
            prog.outputs[o] = dag.value.at(out_st[o]);
        }
        int32_t status = trs_pointwise(&prog, ins.data(), outs.data(), stream_for(device));
        if (status != TRS_OK) {
            for (float* b : bufs) free_floats(device, b);
            check_cuda(status, "fused pointwise kernel");
        }
        // Commit: extras first (the root's expression still references them), the root last,
        // which releases the whole expression.
        for (size_t o = 1; o < out_st.size(); ++o) { out_st[o]->ptr = bufs[o]; }
        std::vector<std::shared_ptr<Node>> keep_alive;
        for (size_t o = 1; o < out_st.size(); ++o) keep_alive.push_back(std::move(out_st[o]->node));
        root->ptr = bufs[0];
        root->node.reset();
        return;
    }
    throw Error(ErrKind::InvalidArgument, "pointwise expression could not be lowered");
}

}  // namespace trsh
