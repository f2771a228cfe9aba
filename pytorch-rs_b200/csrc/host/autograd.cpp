// Backward engine for CUDA tensors (reference: run_backward / collect_topology / apply_grad_fn,
// src/tensor.rs:2881-3341).  Every VJP is expressed with the same recorded ops as the forward
// pass (grad mode off), so the pointwise VJPs fuse into single kernels and the matmul VJPs are
// GEMMs over transposed views; un-broadcast reductions use the deterministic device sums.
// Gradients are kept contiguous in logical order, like the reference's flat Vec<f32> buffers.
#include "autograd.h"

#include <algorithm>
#include <atomic>
#include <unordered_map>
#include <unordered_set>

namespace trsh {

namespace {
const char* kFreedMessage =
    "Trying to backward through the graph a second time (or directly access saved tensors after they have already been freed). "
    "Saved intermediate values of the graph are freed when you call .backward() or autograd.grad(). Specify retain_graph=True if "
    "you need to backward through the graph a second time or if you need to access saved tensors after calling backward.";

struct NoGrad {
    NoGrad() { set_grad_enabled(false); }
    ~NoGrad() { set_grad_enabled(true); }
};

TensorP contiguous_result(int op, std::vector<View> args, const Shape& shape, int device) {
    return pointwise_node(op, 0.f, std::move(args), shape, contiguous_strides(shape), device);
}

// Sum `g` (contiguous, logical shape `from`) over the axes that were broadcast from `to`
// (GradientAccumulator, src/tensor.rs:3204-3228).
TensorP unbroadcast(const TensorP& g, const Shape& from, const Shape& to) {
    if (from == to) return g;
    const int device = g->device();
    const size_t rank = from.size(), lead = rank - to.size();
    std::vector<bool> reduced(rank, false);
    for (size_t a = 0; a < rank; ++a) reduced[a] = a < lead || (to[a - lead] == 1 && from[a] != 1);
    i64 n_red = 1, n_keep = 1;
    for (size_t a = 0; a < rank; ++a) (reduced[a] ? n_red : n_keep) *= from[a];
    if (n_red == 1) return make_tensor(View{g->v.st, to, contiguous_strides(to), g->v.offset});
    // Bring the reduced axes to the front (a no-op when they already lead) so that the sum is a
    // [n_red, n_keep] column reduction, or keep them last for a row reduction.
    bool leading = true, trailing = true;
    {
        size_t first_keep = rank, last_keep = 0;
        bool any_keep = false;
        for (size_t a = 0; a < rank; ++a) if (!reduced[a] && from[a] != 1) { first_keep = std::min(first_keep, a); last_keep = a; any_keep = true; }
        for (size_t a = 0; a < rank; ++a) if (reduced[a] && from[a] != 1 && any_keep) { if (a > first_keep) leading = false; if (a < last_keep) trailing = false; }
    }
    TensorP src = g;
    if (!layout_is_contiguous(src->v.shape, src->v.strides)) src = contiguous(src);
    if (!leading && !trailing) {
        std::vector<i64> dims;
        for (size_t a = 0; a < rank; ++a) if (reduced[a]) dims.push_back((i64)a);
        for (size_t a = 0; a < rank; ++a) if (!reduced[a]) dims.push_back((i64)a);
        src = contiguous(permute(make_tensor(View{src->v.st, from, contiguous_strides(from), src->v.offset}), dims, 0));
        leading = true;
    }
    materialize(src->v.st);
    TensorP out = full(to, 0.0f, device);
    if (n_keep == 0 || n_red == 0) return out;
    const float* in = src->v.st->ptr + src->v.offset;
    if (leading) check_cuda(trs_unbroadcast_sum_f32(in, n_red, n_keep, 0, out->v.st->ptr, stream_for(device)), "un-broadcast sum");
    else check_cuda(trs_unbroadcast_sum_f32(in, n_keep, n_red, 1, out->v.st->ptr, stream_for(device)), "un-broadcast sum");
    return out;
}

TensorP transposed_last2(const View& v) {
    View t = v;
    const size_t r = t.shape.size();
    std::swap(t.shape[r - 1], t.shape[r - 2]);
    std::swap(t.strides[r - 1], t.strides[r - 2]);
    return make_tensor(std::move(t));
}

// Gradient contributions of one node, one per input edge (null when that input needs none).
std::vector<TensorP> apply(const GradFn& fn, const TensorP& g, int device) {
    std::vector<TensorP> out(fn.in.size());
    auto wants = [&](size_t i) { return fn.in[i].meta != nullptr; };
    switch (fn.kind) {
        case GK::Sum:        // fill the input shape with the upstream scalar (src/tensor.rs:3008-3013)
            if (wants(0)) out[0] = contiguous_result(TRS_OP_COPY, {g->v}, fn.in[0].shape, device);
            break;
        case GK::MulScalar:
            if (wants(0)) {
                TensorP c = pointwise_node(TRS_OP_CONST, fn.scalar, {}, fn.out_shape, contiguous_strides(fn.out_shape), device);
                out[0] = contiguous_result(TRS_OP_MUL, {g->v, c->v}, fn.out_shape, device);
            }
            break;
        case GK::Neg:
            if (wants(0)) out[0] = contiguous_result(TRS_OP_NEG, {g->v}, fn.out_shape, device);
            break;
        case GK::Identity:
        case GK::Copy:
            if (wants(0)) out[0] = g;
            break;
        case GK::Reshape:    // the gradient keeps its flat logical order and takes the input's shape
            if (wants(0)) {
                TensorP c = contiguous(g);
                out[0] = make_tensor(View{c->v.st, fn.in[0].shape, contiguous_strides(fn.in[0].shape), c->v.offset});
            }
            break;
        case GK::Relu:       // src/tensor.rs:3161-3176
            if (wants(0)) out[0] = contiguous_result(TRS_OP_RELU_VJP, {fn.saved[0], g->v}, fn.out_shape, device);
            break;
        case GK::Sin:        // upstream * cos(input) (src/tensor.rs:3178-3185)
            if (wants(0)) {
                TensorP c = contiguous_result(TRS_OP_COS, {fn.saved[0]}, fn.out_shape, device);
                out[0] = contiguous_result(TRS_OP_MUL, {g->v, c->v}, fn.out_shape, device);
            }
            break;
        case GK::Sqrt:       // upstream / (2.0 * sqrt(input)) (src/tensor.rs:4416-4419)
            if (wants(0)) {
                TensorP r = contiguous_result(TRS_OP_SQRT, {fn.saved[0]}, fn.out_shape, device);
                TensorP two = pointwise_node(TRS_OP_CONST, 2.0f, {}, fn.out_shape, contiguous_strides(fn.out_shape), device);
                TensorP d = contiguous_result(TRS_OP_MUL, {two->v, r->v}, fn.out_shape, device);
                out[0] = contiguous_result(TRS_OP_DIV, {g->v, d->v}, fn.out_shape, device);
            }
            break;
        case GK::Exp:        // d exp(x) = g * exp(x), with exp(x) the saved output
            if (wants(0)) out[0] = contiguous_result(TRS_OP_MUL, {g->v, fn.saved[0]}, fn.out_shape, device);
            break;
        case GK::Mul:        // src/tensor.rs:3031-3097
            if (wants(0)) out[0] = unbroadcast(contiguous_result(TRS_OP_MUL, {g->v, fn.saved[1]}, fn.out_shape, device), fn.out_shape, fn.in[0].shape);
            if (wants(1)) out[1] = unbroadcast(contiguous_result(TRS_OP_MUL, {g->v, fn.saved[0]}, fn.out_shape, device), fn.out_shape, fn.in[1].shape);
            break;
        case GK::Add:
            if (wants(0)) out[0] = unbroadcast(g, fn.out_shape, fn.in[0].shape);
            if (wants(1)) out[1] = unbroadcast(g, fn.out_shape, fn.in[1].shape);
            break;
        case GK::Sub:
            if (wants(0)) out[0] = unbroadcast(g, fn.out_shape, fn.in[0].shape);
            if (wants(1)) out[1] = unbroadcast(contiguous_result(TRS_OP_NEG, {g->v}, fn.out_shape, device), fn.out_shape, fn.in[1].shape);
            break;
        case GK::Permute:    // src/tensor.rs:3248-3298: scatter back through the inverse permutation
            if (wants(0)) {
                std::vector<i64> inverse(fn.dims.size());
                for (size_t o = 0; o < fn.dims.size(); ++o) inverse[fn.dims[o]] = (i64)o;
                TensorP gv = make_tensor(View{g->v.st, fn.out_shape, contiguous_strides(fn.out_shape), g->v.offset});
                out[0] = contiguous(permute(gv, inverse, 0));
            }
            break;
        case GK::Index:      // src/tensor.rs:3237-3247: zeros with the selected slab set to the upstream
            if (wants(0)) {
                TensorP z = full(fn.in[0].shape, 0.0f, device);
                const i64 slab = element_count(fn.out_shape);
                if (slab > 0) {
                    TensorP src = contiguous(g);
                    materialize(src->v.st);
                    check_cuda(trs_memcpy_d2d(z->v.st->ptr + fn.index * slab, src->v.st->ptr + src->v.offset, (size_t)slab * 4, stream_for(device)), "select backward");
                }
                out[0] = z;
            }
            break;
        case GK::Matmul: {   // dA = g @ B^T, dB = A^T @ g
            if (wants(0)) out[0] = matmul(g, transposed_last2(fn.saved[1]));
            if (wants(1)) out[1] = matmul(transposed_last2(fn.saved[0]), g);
            break;
        }
    }
    return out;
}

TensorP accumulate(const TensorP& have, const TensorP& more, int device) {
    // add_gradient (src/tensor.rs:3302-3317)
    if (!have) return more;
    return contiguous_result(TRS_OP_ADD, {have->v, more->v}, have->v.shape, device);
}

}  // namespace

void record(const TensorP& out, GK kind, const char* name, std::vector<const Tensor*> inputs, std::vector<View> saved,
            bool needs_values, float scalar, std::vector<i64> dims, i64 index) {
    auto fn = std::make_shared<GradFn>();
    fn->kind = kind;
    fn->name = name;
    for (const Tensor* t : inputs) fn->in.push_back(Edge{t->meta, t->v.shape});
    fn->saved = std::move(saved);
    fn->needs_values = needs_values;
    fn->scalar = scalar;
    fn->dims = std::move(dims);
    fn->index = index;
    fn->out_shape = out->v.shape;
    auto meta = std::make_shared<AutogradMeta>();
    meta->leaf = false;
    meta->grad_fn = fn;
    meta->device = out->device();
    out->meta = meta;
}

const char* grad_fn_name(const Tensor& t) {
    if (!t.meta || t.meta->leaf || !t.meta->grad_fn) return "";
    return t.meta->grad_fn->name;
}

// with_requires_grad (src/tensor.rs:780-798): a new leaf handle over the same storage.
TensorP set_requires_grad(const TensorP& t, bool on) {
    TensorP out = make_tensor(t->v);
    if (on) {
        auto meta = std::make_shared<AutogradMeta>();
        meta->leaf = true;
        meta->leaf_shape = t->v.shape;
        meta->device = t->device();
        out->meta = meta;
    }
    return out;
}

TensorP grad_of(const TensorP& t) {
    if (!t->meta || !t->meta->leaf) return nullptr;
    return t->meta->grad;
}

// Evaluates a leaf's finished gradient (contiguous, in a buffer of its own) and, for a first gradient, records the
// event a gradient exchange on another stream waits for.
static std::atomic<uint64_t> g_ready_counter{0};
static void finish_leaf_gradient(std::pair<AutogradMeta*, TensorP>& entry, int device) {
    AutogradMeta* m = entry.first;
    TensorP g = entry.second;
    if (!layout_is_contiguous(g->v.shape, g->v.strides)) g = contiguous(g);
    if (!m->grad && !g->v.st->node && g->v.st.use_count() > 1) g = contiguous_result(TRS_OP_COPY, {g->v}, g->v.shape, device);
    materialize(g->v.st);
    if (!m->grad) {
        if (!m->grad_ready) check_cuda(trs_event_create(&m->grad_ready), "creating the gradient event");
        check_cuda(trs_event_record(m->grad_ready, stream_for(device)), "recording the gradient event");
        m->ready_order = ++g_ready_counter;
    }
    entry.second = g;
}

// Moves the parents of a recorded op out of it, so that releasing the op does not release them.
static void take_parents(const std::shared_ptr<GradFn>& fn, std::vector<std::shared_ptr<AutogradMeta>>& pending) {
    if (!fn || fn.use_count() != 1) return;
    for (Edge& e : fn->in)
        if (e.meta) pending.push_back(std::move(e.meta));
}

AutogradMeta::~AutogradMeta() {
    if (grad_ready) trs_event_destroy(grad_ready);
    // src/tensor.rs:189-206: walk the chain of sole-owned ancestors with a work list instead of letting each
    // destructor call the next one.
    std::vector<std::shared_ptr<AutogradMeta>> pending;
    take_parents(grad_fn, pending);
    grad_fn.reset();
    while (!pending.empty()) {
        std::shared_ptr<AutogradMeta> parent = std::move(pending.back());
        pending.pop_back();
        if (parent.use_count() == 1) {
            take_parents(parent->grad_fn, pending);
            parent->grad_fn.reset();
        }
        // `parent` is released here; it has no parents left, so its own destructor does not descend
    }
}

void backward(const TensorP& root) {
    std::lock_guard<std::recursive_mutex> lock(g_engine_mu);
    // src/tensor.rs:884-898
    if (!root->requires_grad() || !root->meta)
        throw Error(ErrKind::DoesNotRequireGrad, "element 0 of tensors does not require grad and does not have a grad_fn");
    if (root->numel != 1)
        throw Error(ErrKind::BackwardRequiresScalar, "grad can be implicitly created only for scalar outputs");
    const int device = root->device();
    NoGrad guard;

    // Topology first (collect_topology, src/tensor.rs:2945-2994): depth-first from the root, the first input of a
    // node explored first, every node listed after all of its inputs; a freed value-dependent node aborts before
    // anything runs.  The nodes are then processed in the reverse of that list, as the reference does, so that
    // several contributions to one tensor are added in the reference's order.
    std::vector<std::shared_ptr<AutogradMeta>> topology;
    {
        struct Frame { std::shared_ptr<AutogradMeta> meta; bool exit; };
        std::vector<Frame> stack{{root->meta, false}};
        std::unordered_set<AutogradMeta*> seen;
        while (!stack.empty()) {
            Frame f = std::move(stack.back());
            stack.pop_back();
            if (f.exit) { topology.push_back(std::move(f.meta)); continue; }
            if (!seen.insert(f.meta.get()).second) continue;
            if (!f.meta->leaf && (f.meta->freed || !f.meta->grad_fn)) throw Error(ErrKind::BackwardGraphFreed, kFreedMessage);
            stack.push_back({f.meta, true});
            if (f.meta->leaf) continue;
            const std::vector<Edge>& in = f.meta->grad_fn->in;
            for (size_t i = in.size(); i-- > 0;)            // pushed last = explored first
                if (in[i].meta) stack.push_back({in[i].meta, false});
        }
    }

    std::unordered_map<AutogradMeta*, TensorP> grads;
    grads[root->meta.get()] = full(root->v.shape, 1.0f, device);
    std::vector<std::pair<AutogradMeta*, TensorP>> leaf_grads;
    std::vector<AutogradMeta*> visited_nodes;
    for (size_t pos = topology.size(); pos-- > 0;) {
        AutogradMeta* m = topology[pos].get();
        if (!m->leaf) visited_nodes.push_back(m);           // its saved values are consumed whether or not a gradient reaches it
        auto found = grads.find(m);
        if (found == grads.end()) continue;                 // nothing flowed here
        TensorP g = found->second;
        grads.erase(found);
        if (m->leaf) {
            // Every contribution to this leaf has been recorded.  A cheap gradient (a fused chain, a reduction) is
            // evaluated now; one that is still an unevaluated product waits for the end of the walk (see below).
            leaf_grads.emplace_back(m, g);
            if (!(g->v.st->node && g->v.st->node->op == OP_MATMUL)) finish_leaf_gradient(leaf_grads.back(), device);
            continue;
        }
        const GradFn& fn = *m->grad_fn;
        std::vector<TensorP> contributions = apply(fn, g, device);
        for (size_t i = 0; i < fn.in.size(); ++i) {
            AutogradMeta* target = fn.in[i].meta.get();
            if (!target || !contributions[i]) continue;
            auto have = grads.find(target);
            grads[target] = accumulate(have == grads.end() ? nullptr : have->second, contributions[i], device);
        }
    }

    // Weight gradients that are still unevaluated products run now, the largest first: a data-parallel host sums
    // each gradient over the ranks on a side stream as soon as its kernel has finished (all_reduce_grads), so the
    // exchange of a large gradient runs under the products that follow it and only the smallest one's is exposed.
    {
        std::vector<size_t> deferred;
        for (size_t i = 0; i < leaf_grads.size(); ++i)
            if (leaf_grads[i].second->v.st->node) deferred.push_back(i);
        std::stable_sort(deferred.begin(), deferred.end(), [&](size_t a, size_t b) { return leaf_grads[a].second->numel > leaf_grads[b].second->numel; });
        for (size_t i : deferred) finish_leaf_gradient(leaf_grads[i], device);
    }

    // Every VJP has been enqueued without error: commit (src/tensor.rs:2918-2938).  Leaf
    // gradients are contiguous; the first one is installed, later ones accumulate in place
    // (src/tensor.rs:3319-3341, src/storage.rs:85-100).
    for (auto& lg : leaf_grads) {
        AutogradMeta* leaf = lg.first;
        TensorP g = lg.second;
        if (!leaf->grad) {
            mark_written_in_place(*g->v.st);                  // later backward passes add into it
            leaf->grad = make_tensor(View{g->v.st, leaf->leaf_shape, contiguous_strides(leaf->leaf_shape), g->v.offset});
        } else {
            check_cuda(trs_accumulate_f32(leaf->grad->v.st->ptr + leaf->grad->v.offset, g->v.st->ptr + g->v.offset, leaf->grad->numel,
                                          stream_for(device)), "leaf gradient accumulation");
            if (!leaf->grad_ready) check_cuda(trs_event_create(&leaf->grad_ready), "creating the gradient event");
            check_cuda(trs_event_record(leaf->grad_ready, stream_for(device)), "recording the gradient event");
            leaf->ready_order = ++g_ready_counter;
        }
    }
    for (AutogradMeta* m : visited_nodes)
        if (m->grad_fn && m->grad_fn->needs_values) { m->grad_fn->saved.clear(); m->freed = true; }
}

}  // namespace trsh
