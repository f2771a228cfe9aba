// Tensor creation, views, op recording and egress for CUDA tensors.
//
// Pointwise ops do not run when called: each returns a tensor whose storage is a pending
// expression node carrying the already planned shape and strides (which depend on metadata
// only, so .shape/.stride() answer at once).  fuse.cpp lowers a pending expression to the
// fusion IR of the C ABI and runs it as one kernel when a value is needed.
#include "engine.h"

#include "autograd.h"

#include <algorithm>
#include <cstring>
#include <map>

namespace trsh {

std::recursive_mutex g_engine_mu;

namespace {
thread_local int t_no_grad_depth = 0;
std::map<int, trs_stream>& g_streams = *new std::map<int, trs_stream>();   // never destroyed: storages may outlive static teardown
}  // namespace

bool grad_enabled() { return t_no_grad_depth == 0; }   // src/grad_mode.rs:5-56
void set_grad_enabled(bool on) {
    if (on) { if (t_no_grad_depth > 0) --t_no_grad_depth; }
    else ++t_no_grad_depth;
}

void check_cuda(int32_t status, const char* what) {
    if (status == TRS_OK) return;
    std::string msg = std::string(what) + ": " + trs_status_string(status) + ": " + trs_last_error_message();
    throw Error(status == TRS_ERR_ALLOCATION_FAILED ? ErrKind::AllocationFailed : ErrKind::Device, msg);
}

trs_stream stream_for(int device) {
    auto it = g_streams.find(device);
    if (it != g_streams.end()) return it->second;
    trs_stream s = nullptr;
    check_cuda(trs_stream_create(device, &s), "creating the device stream");
    g_streams[device] = s;
    return s;
}

namespace {
bool g_plane_cache = true;
}
void set_plane_cache(bool on) { g_plane_cache = on; }
bool plane_cache_enabled() { return g_plane_cache; }

// Blocks come from and go back to the device cache in the order of the engine's compute stream: a block freed
// here may still be read by kernels already queued on that stream, and the cache hands it to another stream
// only behind that work.
static float* alloc_floats_on(i64 count, int device, trs_stream stream) {
    void* p = nullptr;
    int32_t s = trs_malloc_async(device, (size_t)std::max<i64>(count, 1) * sizeof(float), stream, &p);
    if (s == TRS_ERR_ALLOCATION_FAILED)
        throw Error(ErrKind::AllocationFailed, "failed to allocate storage for " + std::to_string(count) + " elements");
    check_cuda(s, "device allocation");
    return (float*)p;
}

float* alloc_floats(i64 count, int device) { return alloc_floats_on(count, device, stream_for(device)); }

void free_floats(int device, void* ptr) {
    if (!ptr) return;
    auto it = g_streams.find(device);
    if (it != g_streams.end()) trs_free_async(device, ptr, it->second);
    else trs_free(device, ptr);
}

Storage::~Storage() {
    free_floats(device, ptr);
    free_floats(device, lo);         // the flag word lives in the same block
}

void mark_written_in_place(Storage& st) {
    st.written_in_place = true;
    if (st.lo) {                      // an image of values that may now change is worthless
        free_floats(st.device, st.lo);
        st.lo = nullptr;
        st.lo_flag = nullptr;
    }
}

// One block: `count` floats of lo values, then (512-byte aligned) the inf/NaN word.
void alloc_lo_image(Storage& st) {
    const i64 padded = (st.count + 127) / 128 * 128;
    float* block = alloc_floats(padded + 128, st.device);
    st.lo = block;
    st.lo_flag = reinterpret_cast<uint32_t*>(block + padded);
    check_cuda(trs_fill_f32(block + padded, 1, 0.0f, stream_for(st.device)), "clearing the operand flag");
}

bool ensure_lo_image(Storage& st, i64 view_numel) {
    if (st.lo) return true;
    // not for values that may change, nor for a small window of a large buffer
    if (!g_plane_cache || st.written_in_place || st.node || !st.ptr || st.count == 0 || view_numel * 64 < st.count) return false;
    const i64 padded = (st.count + 127) / 128 * 128;
    float* block = alloc_floats(padded + 128, st.device);
    int32_t s = trs_split_lo_f32(st.ptr, st.count, block, reinterpret_cast<uint32_t*>(block + padded), stream_for(st.device));
    if (s != TRS_OK) { free_floats(st.device, block); check_cuda(s, "operand image"); }
    st.lo = block;
    st.lo_flag = reinterpret_cast<uint32_t*>(block + padded);
    return true;
}

namespace {
// Read-backs in flight on the per-device egress stream: the tensor is kept alive (so its block is
// not handed out again) until the device has finished copying it.
struct Egress {
    trs_stream stream = nullptr;
    trs_event ready = nullptr;
    std::vector<TensorP> in_flight;
};
std::map<int, Egress> g_egress;
}  // namespace

void sync(int device) {
    check_cuda(trs_stream_sync(stream_for(device)), "stream sync");      // uploads are waited for by this stream already
    auto it = g_egress.find(device);
    if (it != g_egress.end() && it->second.stream) {
        check_cuda(trs_stream_sync(it->second.stream), "egress stream sync");
        it->second.in_flight.clear();
    }
}

// Device-to-host copy into page-locked memory that returns at once: it runs on a second stream
// (behind an event on the compute stream), so it overlaps later uploads and kernels.  The data
// is valid after sync(device).
void to_host_async(const TensorP& t, float* out) {
    if (t->numel == 0) return;
    const int device = t->device();
    TensorP src = t;
    if (!layout_is_contiguous(t->v.shape, t->v.strides))
        src = pointwise_node(TRS_OP_COPY, 0.f, {t->v}, t->v.shape, contiguous_strides(t->v.shape), device);
    materialize(src->v.st);
    Egress& e = g_egress[device];
    if (!e.stream) {
        check_cuda(trs_stream_create(device, &e.stream), "creating the egress stream");
        check_cuda(trs_event_create(&e.ready), "creating the egress event");
    }
    check_cuda(trs_event_record(e.ready, stream_for(device)), "egress event");
    check_cuda(trs_stream_wait_event(e.stream, e.ready), "egress wait");
    check_cuda(trs_memcpy_d2h(out, src->v.st->ptr + src->v.offset, (size_t)t->numel * 4, e.stream), "device to host copy");
    e.in_flight.push_back(src);
}

static std::shared_ptr<Storage> alloc_storage(i64 count, int device) {
    auto st = std::make_shared<Storage>();
    st->device = device;
    st->count = count;
    st->ptr = alloc_floats(count, device);
    return st;
}

TensorP make_tensor(View v) {
    auto t = std::make_shared<Tensor>();
    t->numel = element_count(v.shape);
    t->v = std::move(v);
    return t;
}

namespace {
// Uploads from page-locked memory run on a stream of their own, so that the upload of the next batch proceeds while
// the kernels of the current one are still running (a host that creates the next input tensor before it waits for
// the current result gets the overlap; the compute stream only waits for the copy it is about to read).
struct Ingress {
    trs_stream stream = nullptr;
    trs_event done = nullptr;
};
std::map<int, Ingress>& g_ingress = *new std::map<int, Ingress>();
}  // namespace

TensorP from_host(const float* data, const Shape& shape, int device, bool pinned) {
    for (i64 d : shape) if (d < 0) throw Error(ErrKind::InvalidArgument, "negative dimension");
    const i64 n = element_count(shape);
    if (n > 0 && pinned) {
        Ingress& in = g_ingress[device];
        if (!in.stream) {
            check_cuda(trs_stream_create(device, &in.stream), "creating the upload stream");
            check_cuda(trs_event_create(&in.done), "creating the upload event");
        }
        // The block is taken in the upload stream's order: if the compute stream freed it with work still queued, the
        // copy waits for exactly that work (not for what the compute stream was given afterwards).
        auto st = std::make_shared<Storage>();
        st->device = device;
        st->count = n;
        st->ptr = alloc_floats_on(n, device, in.stream);
        check_cuda(trs_memcpy_h2d(st->ptr, data, (size_t)n * sizeof(float), in.stream), "host to device copy");
        check_cuda(trs_event_record(in.done, in.stream), "upload event");
        check_cuda(trs_stream_wait_event(stream_for(device), in.done), "ordering kernels behind the upload");
        return make_tensor(View{st, shape, contiguous_strides(shape), 0});
    }
    auto st = alloc_storage(n, device);
    if (n > 0) {
        trs_stream s = stream_for(device);
        check_cuda(trs_memcpy_h2d(st->ptr, data, (size_t)n * sizeof(float), s), "host to device copy");
        check_cuda(trs_stream_sync(s), "host to device copy");      // a pageable source may be released by the caller at once
    }
    return make_tensor(View{st, shape, contiguous_strides(shape), 0});
}

TensorP full(const Shape& shape, float value, int device) {
    const i64 n = element_count(shape);
    auto st = alloc_storage(n, device);
    if (n > 0) check_cuda(trs_fill_f32(st->ptr, n, value, stream_for(device)), "fill");
    return make_tensor(View{st, shape, contiguous_strides(shape), 0});
}

TensorP zeros_like_shape(const Shape& shape, int device) { return full(shape, 0.0f, device); }

// ---- views (metadata only; src/tensor.rs:1082-1215, 1850-1973) -----------------------------------

TensorP detach(const TensorP& t) {
    auto out = make_tensor(t->v);
    return out;
}

static i64 wrap_dim(i64 dim, size_t rank) {
    // normalize_transpose_dimension (src/tensor.rs:3793-3813); message src/tensor_error.rs:252-263
    const i64 r = (i64)std::max<size_t>(rank, 1);
    if (dim < -r || dim >= r)
        throw Error(ErrKind::DimensionOutOfRange, "Dimension out of range (expected to be in range of [-" + std::to_string(r) + ", " +
                                                      std::to_string(r - 1) + "], but got " + std::to_string(dim) + ")");
    if (rank == 0) return 0;
    return dim < 0 ? dim + r : dim;
}

TensorP transpose(const TensorP& t, i64 d0, i64 d1) {
    const size_t rank = t->v.shape.size();
    const i64 a0 = wrap_dim(d0, rank), a1 = wrap_dim(d1, rank);
    std::vector<i64> dims(rank);
    for (size_t i = 0; i < rank; ++i) dims[i] = (i64)i;
    if (rank) std::swap(dims[a0], dims[a1]);
    return permute(t, dims, 1);
}

TensorP matrix_transpose(const TensorP& t) {
    const size_t rank = t->v.shape.size();
    if (rank == 1)
        throw Error(ErrKind::MatrixTransposeRequiresMatrix, "tensor.mT is only supported on matrices or batches of matrices. Got 1-D tensor.");
    if (rank == 0) return permute(t, {}, 1);
    return transpose(t, -2, -1);
}

TensorP reverse_dims(const TensorP& t) {
    std::vector<i64> dims(t->v.shape.size());
    for (size_t i = 0; i < dims.size(); ++i) dims[i] = (i64)(dims.size() - 1 - i);
    return permute(t, dims, 0);
}

// ---- op recording -------------------------------------------------------------------------------

static bool is_identity_view_of_pending(const View& v) {
    const Storage& st = *v.st;
    return st.node && v.offset == 0 && v.shape == st.node->shape && v.strides == st.node->strides;
}

TensorP pointwise_node(int op, float imm, std::vector<View> args, const Shape& shape, const Shape& strides, int device) {
    auto node = std::make_shared<Node>();
    node->op = op;
    node->imm = imm;
    node->shape = shape;
    node->strides = strides;
    int instrs = 1, leaves = 0;
    for (View& a : args) {
        if (a.st->device != device)
            throw Error(ErrKind::DeviceMismatch, "Expected all tensors to be on the same device, but found at least two devices, cuda:" +
                                                     std::to_string(device) + " and cuda:" + std::to_string(a.st->device) + "!");
        if (a.st->node) {
            // A pending operand fuses only when it is read element for element (identity view,
            // same logical shape); otherwise its values are needed in memory first.
            if (is_identity_view_of_pending(a) && a.shape == shape && a.st->node->n_instr + instrs <= 40 &&
                a.st->node->n_leaf + leaves <= TRS_MAX_INPUTS - 2) {
                instrs += a.st->node->n_instr;
                leaves += a.st->node->n_leaf;
                continue;
            }
            materialize(a.st);
        }
        leaves += 1;
    }
    node->n_instr = instrs;
    node->n_leaf = leaves;
    bool reads_mutable = false;
    for (const View& a : args) reads_mutable |= a.st->written_in_place;
    node->args = std::move(args);
    auto st = std::make_shared<Storage>();
    st->device = device;
    st->count = element_count(shape);
    st->node = node;
    // The reference computes every result at once.  Deferring is invisible only while the operands cannot change:
    // a value that may be written in place later (an accumulating leaf gradient, an exported buffer) is read now.
    if (reads_mutable) materialize(st);
    return make_tensor(View{st, shape, strides, 0});
}

void to_host(const Tensor& t, float* out) {
    if (t.numel == 0) return;
    const int device = t.device();
    materialize(t.v.st);
    trs_stream s = stream_for(device);
    if (layout_is_contiguous(t.v.shape, t.v.strides)) {
        check_cuda(trs_memcpy_d2h(out, t.v.st->ptr + t.v.offset, (size_t)t.numel * 4, s), "device to host copy");
        check_cuda(trs_stream_sync(s), "device to host copy");
        return;
    }
    // Gather into logical order on the device (one fused copy), then read back.
    TensorP packed = pointwise_node(TRS_OP_COPY, 0.f, {t.v}, t.v.shape, contiguous_strides(t.v.shape), device);
    materialize(packed->v.st);
    check_cuda(trs_memcpy_d2h(out, packed->v.st->ptr, (size_t)t.numel * 4, s), "device to host copy");
    check_cuda(trs_stream_sync(s), "device to host copy");
}

float item(const Tensor& t) {
    // src/tensor.rs:2438-2445
    if (t.numel != 1) throw Error(ErrKind::ItemRequiresOneElement, "item requires one element, got " + std::to_string(t.numel));
    materialize(t.v.st);
    float v = 0.f;
    trs_stream s = stream_for(t.device());
    check_cuda(trs_memcpy_d2h(&v, t.v.st->ptr + t.v.offset, 4, s), "device to host copy");
    check_cuda(trs_stream_sync(s), "device to host copy");
    return v;
}

// try_contiguous (src/tensor.rs:1606-1675): the tensor itself when it already has the requested layout,
// else a packed copy with that format's canonical strides.
TensorP contiguous(const TensorP& t, MemoryFormat format) {
    Shape strides;
    if (!memory_format_plan(t->v.shape, t->v.strides, format, false, &strides)) return t;
    TensorP out = pointwise_node(TRS_OP_COPY, 0.f, {t->v}, t->v.shape, strides, t->device());
    if (t->requires_grad() && grad_enabled()) record(out, GK::Copy, "CloneBackward0", {t.get()}, {}, false);
    return out;
}

}  // namespace trsh
