// Data-parallel gradient exchange for the host engine: the one collective of the hot path (the sum of the MLP
// weight gradients over the ranks), issued through the kernel library's NCCL entry points on a side stream.
//
// The reference has no distributed backend (python/torch_rs/distributed/distributed_c10d.py:39-74 reports every
// backend as unavailable); its only multi-process convention, LOCAL_RANK (same file, 71-72), picks the device.
// Each all-reduce waits only for the event recorded behind the kernel that produced that gradient, so the
// exchange of an early gradient (the last layer's) runs under the GEMMs of the earlier layers.
#include "autograd.h"
#include "engine.h"

#include <algorithm>
#include <map>

namespace trsh {

namespace {
struct Comm {
    trs_comm comm = nullptr;
    int device = 0;
    int size = 1;
    trs_stream stream = nullptr;     // the exchange runs here, beside the compute stream
    trs_event done = nullptr;
};
Comm g_comm;
}  // namespace

void comm_unique_id(char* id128) { check_cuda(trs_comm_unique_id(id128), "creating the communicator id"); }

void comm_init(int device, int nranks, int rank, const char* id128) {
    if (g_comm.comm) throw Error(ErrKind::InvalidArgument, "the communicator is already initialised");
    check_cuda(trs_comm_init_rank(device, nranks, rank, id128, &g_comm.comm), "joining the communicator");
    g_comm.device = device;
    g_comm.size = nranks;
    check_cuda(trs_stream_create(device, &g_comm.stream), "creating the exchange stream");
    check_cuda(trs_event_create(&g_comm.done), "creating the exchange event");
}

void comm_destroy() {
    if (!g_comm.comm) return;
    sync(g_comm.device);
    trs_stream_sync(g_comm.stream);
    trs_comm_destroy(g_comm.comm);
    trs_stream_destroy(g_comm.stream);
    trs_event_destroy(g_comm.done);
    g_comm = Comm{};
}

int comm_size() { return g_comm.comm ? g_comm.size : 1; }

static void exchange(Storage& st, float* data, i64 count, trs_event ready) {
    // the buffer is summed in place: nothing may still be waiting to read its old values lazily
    mark_written_in_place(st);
    trs_stream compute = stream_for(g_comm.device);
    if (ready) {
        check_cuda(trs_stream_wait_event(g_comm.stream, ready), "ordering the exchange behind the gradient");
    } else {
        check_cuda(trs_event_record(g_comm.done, compute), "ordering the exchange");
        check_cuda(trs_stream_wait_event(g_comm.stream, g_comm.done), "ordering the exchange");
    }
    check_cuda(trs_comm_allreduce_sum_f32(g_comm.comm, data, count, g_comm.stream), "gradient all-reduce");
}

static void join_compute_stream() {
    check_cuda(trs_event_record(g_comm.done, g_comm.stream), "exchange event");
    check_cuda(trs_stream_wait_event(stream_for(g_comm.device), g_comm.done), "waiting for the exchange");
}

void all_reduce_grads(const std::vector<TensorP>& leaves) {
    std::lock_guard<std::recursive_mutex> lock(g_engine_mu);
    if (!g_comm.comm || g_comm.size == 1) return;
    bool any = false;
    // in the order the gradients became ready on the compute stream, whatever order the caller names them in
    std::vector<TensorP> ordered;
    for (const TensorP& leaf : leaves)
        if (leaf && leaf->meta && leaf->meta->leaf && leaf->meta->grad) ordered.push_back(leaf);
    std::stable_sort(ordered.begin(), ordered.end(), [](const TensorP& a, const TensorP& b) { return a->meta->ready_order < b->meta->ready_order; });
    for (const TensorP& leaf : ordered) {
        Tensor& g = *leaf->meta->grad;
        if (g.device() != g_comm.device) throw Error(ErrKind::DeviceMismatch, "gradient lives on another device than the communicator");
        if (g.numel == 0) continue;
        exchange(*g.v.st, g.v.st->ptr + g.v.offset, g.numel, leaf->meta->grad_ready);
        any = true;
    }
    if (any) join_compute_stream();
}

void all_reduce_tensor(const TensorP& t) {
    std::lock_guard<std::recursive_mutex> lock(g_engine_mu);
    if (!g_comm.comm || g_comm.size == 1 || t->numel == 0) return;
    if (!layout_is_contiguous(t->v.shape, t->v.strides)) throw Error(ErrKind::InvalidArgument, "all_reduce needs a contiguous tensor");
    if (t->device() != g_comm.device) throw Error(ErrKind::DeviceMismatch, "tensor lives on another device than the communicator");
    materialize(t->v.st);
    exchange(*t->v.st, t->v.st->ptr + t->v.offset, t->numel, nullptr);
    join_compute_stream();
}

}  // namespace trsh
