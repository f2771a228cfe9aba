// The path's one collective behind the C ABI: sum of float32 buffers over the ranks of a job with NCCL
// (NVLink / NVSwitch inside a node).  New relative to the reference, which has no distributed backend
// (python/torch_rs/distributed/distributed_c10d.py:39-74); its LOCAL_RANK convention (same file, 71-72) is what a
// host uses to pick `device`.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) rather than at link time: a process that already carries an
// NCCL (for instance one that imported PyTorch) keeps using that one copy, and a host that never starts a
// communicator needs no NCCL at all.  Only the four stable entry points below are used; their types and enum
// values are restated here (ncclUniqueId is 128 opaque bytes, ncclFloat32 = 7, ncclSum = 0).
#include <dlfcn.h>

#include <mutex>

#include "common.h"

struct trs_comm_s {
    void* nccl;        // ncclComm_t
    int device;
    int nranks;
    int rank;
};

namespace trs {
namespace {

struct NcclId { char internal[128]; };
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(void**, int, NcclId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);

struct NcclApi {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn error_string = nullptr;
    std::string why;
};

NcclApi& api() {
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (a.handle) break;
        }
        if (!a.handle) { a.why = std::string("cannot load libnccl.so.2: ") + (dlerror() ? dlerror() : "not found"); return; }
        a.get_unique_id = (GetUniqueIdFn)dlsym(a.handle, "ncclGetUniqueId");
        a.comm_init_rank = (CommInitRankFn)dlsym(a.handle, "ncclCommInitRank");
        a.all_reduce = (AllReduceFn)dlsym(a.handle, "ncclAllReduce");
        a.comm_destroy = (CommDestroyFn)dlsym(a.handle, "ncclCommDestroy");
        a.error_string = (GetErrorStringFn)dlsym(a.handle, "ncclGetErrorString");
        if (!a.get_unique_id || !a.comm_init_rank || !a.all_reduce || !a.comm_destroy) {
            a.why = "libnccl.so.2 lacks an expected entry point";
            a.handle = nullptr;
        }
    });
    return a;
}

int32_t nccl_fail(int code, const char* what) {
    NcclApi& a = api();
    return fail(TRS_ERR_CUDA, "%s: NCCL error %d (%s)", what, code, a.error_string ? a.error_string(code) : "?");
}

}  // namespace
}  // namespace trs

using namespace trs;

extern "C" {

int32_t trs_comm_unique_id(char* id) {
    if (!id) return fail(TRS_ERR_INVALID_ARGUMENT, "id is NULL");
    NcclApi& a = api();
    if (!a.handle) return fail(TRS_ERR_UNSUPPORTED, "%s", a.why.c_str());
    NcclId nid;
    int r = a.get_unique_id(&nid);
    if (r != 0) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id, nid.internal, sizeof nid.internal);
    return TRS_OK;
}

int32_t trs_comm_init_rank(int32_t device, int32_t nranks, int32_t rank, const char* id, trs_comm* comm) {
    if (!comm || !id) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL argument");
    *comm = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail(TRS_ERR_INVALID_ARGUMENT, "rank %d outside a job of %d ranks", rank, nranks);
    if (device < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device %d", device);
    NcclApi& a = api();
    if (!a.handle) return fail(TRS_ERR_UNSUPPORTED, "%s", a.why.c_str());
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    NcclId nid;
    memcpy(nid.internal, id, sizeof nid.internal);
    void* c = nullptr;
    int r = a.comm_init_rank(&c, nranks, nid, rank);
    if (r != 0) return nccl_fail(r, "ncclCommInitRank");
    *comm = new trs_comm_s{c, device, nranks, rank};
    return TRS_OK;
}

int32_t trs_comm_allreduce_sum_f32(trs_comm comm, float* data, int64_t count, trs_stream stream) {
    if (!comm) return fail(TRS_ERR_INVALID_ARGUMENT, "comm is NULL (use trs_comm_init_rank)");
    TRS_TRY(check_stream(stream));
    if (count < 0 || (count > 0 && !data)) return fail(TRS_ERR_INVALID_ARGUMENT, "bad buffer");
    if (stream->device != comm->device)
        return fail(TRS_ERR_INVALID_ARGUMENT, "stream belongs to device %d, the communicator to device %d", stream->device, comm->device);
    if (count == 0) return TRS_OK;
    DeviceGuard guard(comm->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", comm->device);
    int r = api().all_reduce(data, data, (size_t)count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, comm->nccl, stream->stream);
    if (r != 0) return nccl_fail(r, "ncclAllReduce");
    count_launch();
    return TRS_OK;
}

int32_t trs_comm_info(trs_comm comm, int32_t* device, int32_t* nranks, int32_t* rank) {
    if (!comm) return fail(TRS_ERR_INVALID_ARGUMENT, "comm is NULL");
    if (device) *device = comm->device;
    if (nranks) *nranks = comm->nranks;
    if (rank) *rank = comm->rank;
    return TRS_OK;
}

int32_t trs_comm_destroy(trs_comm comm) {
    if (!comm) return TRS_OK;
    DeviceGuard guard(comm->device);
    if (comm->nccl) api().comm_destroy(comm->nccl);
    delete comm;
    return TRS_OK;
}

}  // extern "C"
