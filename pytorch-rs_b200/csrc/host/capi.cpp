// C API of the host engine: handle management and error translation (no exception crosses).
#include "../../../include/trs_host.h"

#include <algorithm>
#include <cstring>

#include "autograd.h"
#include "engine.h"

using namespace trsh;

struct trsh_tensor_s {
    TensorP t;
};

namespace {
thread_local std::string t_error;

template <class F>
int32_t guarded(F&& body) {
    std::lock_guard<std::recursive_mutex> lock(g_engine_mu);
    try {
        body();
        return TRSH_OK;
    } catch (const Error& e) {
        t_error = e.what();
        return (int32_t)e.kind;
    } catch (const std::bad_alloc&) {
        t_error = "host allocation failed";
        return TRSH_ALLOCATION_FAILED;
    } catch (const std::exception& e) {
        t_error = e.what();
        return TRSH_INVALID_ARGUMENT;
    }
}

trsh_tensor wrap(TensorP t) { return new trsh_tensor_s{std::move(t)}; }
const TensorP& get(trsh_tensor h) {
    if (!h || !h->t) throw Error(ErrKind::InvalidArgument, "NULL tensor handle");
    return h->t;
}
Shape shape_of(int32_t rank, const int64_t* dims) {
    if (rank < 0 || rank > TRS_MAX_RANK) throw Error(ErrKind::InvalidArgument, "rank must be between 0 and 8 on CUDA");
    return Shape(dims, dims + rank);
}
}  // namespace

extern "C" {

const char* trsh_last_error(void) { return t_error.c_str(); }

int32_t trsh_from_host(const float* data, int32_t rank, const int64_t* shape, int32_t device, trsh_tensor* out) {
    return guarded([&] { *out = wrap(from_host(data, shape_of(rank, shape), device)); });
}
int32_t trsh_from_pinned_host(const float* data, int32_t rank, const int64_t* shape, int32_t device, trsh_tensor* out) {
    return guarded([&] { *out = wrap(from_host(data, shape_of(rank, shape), device, true)); });
}
int32_t trsh_full(int32_t rank, const int64_t* shape, float value, int32_t device, trsh_tensor* out) {
    return guarded([&] { *out = wrap(full(shape_of(rank, shape), value, device)); });
}
int32_t trsh_to_host(trsh_tensor t, float* out) { return guarded([&] { to_host(*get(t), out); }); }
int32_t trsh_to_pinned_host_async(trsh_tensor t, float* out) { return guarded([&] { to_host_async(get(t), out); }); }
int32_t trsh_item(trsh_tensor t, float* out) { return guarded([&] { *out = item(*get(t)); }); }
int32_t trsh_release(trsh_tensor t) {
    return guarded([&] { delete t; });
}

int32_t trsh_rank(trsh_tensor t, int32_t* rank) { return guarded([&] { *rank = (int32_t)get(t)->v.shape.size(); }); }
int32_t trsh_layout(trsh_tensor t, int64_t* shape, int64_t* strides, int64_t* offset, int64_t* numel) {
    return guarded([&] {
        const Tensor& x = *get(t);
        for (size_t i = 0; i < x.v.shape.size(); ++i) {
            if (shape) shape[i] = x.v.shape[i];
            if (strides) strides[i] = x.v.strides[i];
        }
        if (offset) *offset = x.v.offset;
        if (numel) *numel = x.numel;
    });
}
int32_t trsh_device(trsh_tensor t, int32_t* device) { return guarded([&] { *device = get(t)->device(); }); }
int32_t trsh_flags(trsh_tensor t, int32_t* requires_grad, int32_t* is_leaf, int32_t* is_contiguous, int32_t* is_pending) {
    return guarded([&] {
        const Tensor& x = *get(t);
        if (requires_grad) *requires_grad = x.requires_grad();
        if (is_leaf) *is_leaf = x.is_leaf();
        if (is_contiguous) *is_contiguous = layout_is_contiguous(x.v.shape, x.v.strides);
        if (is_pending) *is_pending = x.v.st->node != nullptr;
    });
}
int32_t trsh_data_ptr(trsh_tensor t, void** ptr) {
    return guarded([&] {
        const Tensor& x = *get(t);
        materialize(x.v.st);
        mark_written_in_place(*x.v.st);      // whoever holds the address may write through it
        *ptr = x.v.st->ptr + x.v.offset;
    });
}
int32_t trsh_const_data_ptr(trsh_tensor t, const void** ptr) {
    return guarded([&] {
        const Tensor& x = *get(t);
        materialize(x.v.st);
        *ptr = x.v.st->ptr + x.v.offset;
    });
}
int32_t trsh_shares_storage(trsh_tensor a, trsh_tensor b, int32_t* shared) {
    return guarded([&] { *shared = get(a)->v.st.get() == get(b)->v.st.get(); });
}
const char* trsh_grad_fn_name(trsh_tensor t) { return (t && t->t) ? grad_fn_name(*t->t) : ""; }

int32_t trsh_permute(trsh_tensor t, int32_t n, const int64_t* dims, trsh_tensor* out) {
    return guarded([&] { *out = wrap(permute(get(t), std::vector<i64>(dims, dims + n), 0)); });
}
int32_t trsh_transpose(trsh_tensor t, int64_t d0, int64_t d1, trsh_tensor* out) {
    return guarded([&] { *out = wrap(transpose(get(t), d0, d1)); });
}
int32_t trsh_matrix_transpose(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(matrix_transpose(get(t))); }); }
int32_t trsh_reverse_dims(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(reverse_dims(get(t))); }); }
int32_t trsh_select0(trsh_tensor t, int64_t index, trsh_tensor* out) { return guarded([&] { *out = wrap(select0(get(t), index)); }); }
int32_t trsh_detach(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(detach(get(t))); }); }
int32_t trsh_contiguous(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(contiguous(get(t))); }); }

int32_t trsh_clone(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(clone(get(t))); }); }
static MemoryFormat format_arg(int32_t f) {
    if (f < 0 || f > 3) throw Error(ErrKind::InvalidArgument, "unknown memory format " + std::to_string(f));
    return (MemoryFormat)f;
}
int32_t trsh_clone_format(trsh_tensor t, int32_t memory_format, trsh_tensor* out) {
    return guarded([&] { *out = wrap(clone(get(t), format_arg(memory_format))); });
}
int32_t trsh_contiguous_format(trsh_tensor t, int32_t memory_format, trsh_tensor* out) {
    return guarded([&] { *out = wrap(contiguous(get(t), format_arg(memory_format))); });
}
int32_t trsh_is_contiguous_format(trsh_tensor t, int32_t memory_format, int32_t* result) {
    return guarded([&] {
        const Tensor& x = *get(t);
        *result = is_contiguous_in_format(x.v.shape, x.v.strides, format_arg(memory_format)) ? 1 : 0;
    });
}
int32_t trsh_reshape(trsh_tensor t, int32_t n, const int64_t* shape, int32_t view_only, trsh_tensor* out) {
    return guarded([&] { *out = wrap(reshape(get(t), std::vector<i64>(shape, shape + n), view_only != 0)); });
}
int32_t trsh_squeeze(trsh_tensor t, int32_t all, int64_t dimension, trsh_tensor* out) {
    return guarded([&] { *out = wrap(squeeze(get(t), all ? INT64_MIN : dimension)); });
}
int32_t trsh_equal(trsh_tensor a, trsh_tensor b, int32_t* result) { return guarded([&] { *result = equal(get(a), get(b)); }); }

int32_t trsh_unary(trsh_tensor t, int32_t op, trsh_tensor* out) { return guarded([&] { *out = wrap(unary(get(t), op)); }); }
int32_t trsh_scalar(trsh_tensor t, int32_t op, float scalar, int32_t reflected, trsh_tensor* out) {
    return guarded([&] { *out = wrap(scalar_op(get(t), op, scalar, reflected != 0)); });
}
int32_t trsh_binary(trsh_tensor l, trsh_tensor r, int32_t op, trsh_tensor* out) {
    return guarded([&] { *out = wrap(binary(get(l), get(r), op)); });
}
int32_t trsh_matmul(trsh_tensor l, trsh_tensor r, trsh_tensor* out) { return guarded([&] { *out = wrap(matmul(get(l), get(r))); }); }
int32_t trsh_sum(trsh_tensor t, trsh_tensor* out) { return guarded([&] { *out = wrap(sum(get(t))); }); }

int32_t trsh_set_requires_grad(trsh_tensor t, int32_t on, trsh_tensor* out) {
    return guarded([&] { *out = wrap(set_requires_grad(get(t), on != 0)); });
}
int32_t trsh_backward(trsh_tensor t) { return guarded([&] { backward(get(t)); }); }
int32_t trsh_grad(trsh_tensor t, trsh_tensor* out) {
    return guarded([&] {
        TensorP g = grad_of(get(t));
        *out = g ? wrap(g) : nullptr;
    });
}
int32_t trsh_set_grad_enabled(int32_t on) { return guarded([&] { set_grad_enabled(on != 0); }); }
int32_t trsh_is_grad_enabled(int32_t* on) { return guarded([&] { *on = grad_enabled(); }); }

int32_t trsh_plan_unary(int32_t rank, const int64_t* shape, const int64_t* strides, int64_t* out_strides) {
    return guarded([&] {
        Shape o = unary_output_strides(Shape(shape, shape + rank), Shape(strides, strides + rank));
        std::copy(o.begin(), o.end(), out_strides);
    });
}
int32_t trsh_plan_scalar(int32_t rank, const int64_t* shape, const int64_t* strides, int64_t* out_strides) {
    return guarded([&] {
        Shape o = scalar_output_strides(Shape(shape, shape + rank), Shape(strides, strides + rank));
        std::copy(o.begin(), o.end(), out_strides);
    });
}
int32_t trsh_plan_memory_format(int32_t memory_format, int32_t for_clone, int32_t rank, const int64_t* shape, const int64_t* strides,
                                int32_t* copies, int64_t* out_strides) {
    return guarded([&] {
        Shape o;
        const bool copy = memory_format_plan(Shape(shape, shape + rank), Shape(strides, strides + rank), format_arg(memory_format),
                                             for_clone != 0, &o);
        *copies = copy ? 1 : 0;
        if (copy) std::copy(o.begin(), o.end(), out_strides);
    });
}
int32_t trsh_plan_binary(int32_t lrank, const int64_t* lshape, const int64_t* lstrides, int32_t rrank,
                         const int64_t* rshape, const int64_t* rstrides, int32_t* out_rank, int64_t* out_shape,
                         int64_t* out_strides) {
    return guarded([&] {
        Shape shape, strides;
        binary_plan(Shape(lshape, lshape + lrank), Shape(lstrides, lstrides + lrank), Shape(rshape, rshape + rrank),
                    Shape(rstrides, rstrides + rrank), &shape, &strides);
        *out_rank = (int32_t)shape.size();
        std::copy(shape.begin(), shape.end(), out_shape);
        std::copy(strides.begin(), strides.end(), out_strides);
    });
}

int32_t trsh_set_plane_cache(int32_t on) { return guarded([&] { set_plane_cache(on != 0); }); }
int32_t trsh_has_operand_image(trsh_tensor t, int32_t* has) { return guarded([&] { *has = get(t)->v.st->lo != nullptr; }); }

int32_t trsh_comm_unique_id(char* id128) { return guarded([&] { comm_unique_id(id128); }); }
int32_t trsh_comm_init(int32_t device, int32_t nranks, int32_t rank, const char* id128) {
    return guarded([&] { comm_init(device, nranks, rank, id128); });
}
int32_t trsh_comm_destroy(void) { return guarded([&] { comm_destroy(); }); }
int32_t trsh_comm_size(int32_t* nranks) { return guarded([&] { *nranks = comm_size(); }); }
int32_t trsh_all_reduce_grads(const trsh_tensor* leaves, int32_t count) {
    return guarded([&] {
        std::vector<TensorP> v;
        for (int32_t i = 0; i < count; ++i) v.push_back(get(leaves[i]));
        all_reduce_grads(v);
    });
}
int32_t trsh_all_reduce(trsh_tensor t) { return guarded([&] { all_reduce_tensor(get(t)); }); }

int32_t trsh_materialize(trsh_tensor t) { return guarded([&] { materialize(get(t)->v.st); }); }
int32_t trsh_sync(int32_t device) { return guarded([&] { sync(device); }); }
int32_t trsh_stream(int32_t device, void** handle) { return guarded([&] { *handle = (void*)stream_for(device); }); }

}  // extern "C"
