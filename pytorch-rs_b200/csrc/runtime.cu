// Devices, cached device memory, pinned host memory, streams, events and copies.
//
// The reference owns host Vec<f32> buffers (src/storage.rs:7-18); here a Storage is a block of
// HBM handed out by a per-device size-bucketed cache so that the per-op fresh output allocation
// the reference performs (from_owned_parts, src/tensor.rs:432-450) costs no cudaMalloc after
// warm-up.  A freed block remembers the stream whose queued work may still use it: the same stream
// gets it back at once (stream order protects it), another stream is first made to wait for that work,
// and a request that names no stream only gets it once that stream has drained.
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "gemm.h"

namespace trs {
thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};

namespace {
constexpr int kMaxDevices = 16;
struct FreeBlock {
    void* ptr;
    trs_stream last;       // stream whose queued work may still touch the block; NULL when nothing can
    cudaEvent_t freed;     // recorded on `last` when the block was handed back: everything that may touch it lies before
};
struct DeviceCache {
    std::mutex mu;
    std::multimap<size_t, FreeBlock> free_blocks;      // rounded size -> block
    std::unordered_map<void*, size_t> live;            // block -> rounded size
    std::vector<cudaEvent_t> spare_events;             // events of this device waiting for their next block
    int64_t in_use = 0, reserved = 0;
    int sms = 0;
};
DeviceCache g_cache[kMaxDevices];

size_t round_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);   // 2 MiB granularity above 1 MiB
}

void release_all(DeviceCache& c) {
    for (auto& kv : c.free_blocks) {
        cudaFree(kv.second.ptr);                          // cudaFree waits for the device to finish using the block
        if (kv.second.freed) c.spare_events.push_back(kv.second.freed);
        c.reserved -= (int64_t)kv.first;
    }
    c.free_blocks.clear();
}

// Events are pooled: one is needed per free, and creating one costs as much as the free itself.  Caller holds c.mu and
// has the device selected.
cudaEvent_t take_event(DeviceCache& c) {
    if (!c.spare_events.empty()) {
        cudaEvent_t e = c.spare_events.back();
        c.spare_events.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return e;
}
}  // namespace

int32_t check_stream(trs_stream s) {
    if (!s) return fail(TRS_ERR_INVALID_ARGUMENT, "stream must not be NULL (use trs_stream_create)");
    return TRS_OK;
}

int32_t malloc_on_stream(trs_stream stream, size_t bytes, void** ptr) { return trs_malloc_async(stream->device, bytes, stream, ptr); }
void free_on_stream(trs_stream stream, void* ptr) { trs_free_async(stream->device, ptr, stream); }

int sm_count(int device) {
    DeviceCache& c = g_cache[device];
    if (c.sms == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        c.sms = v;
    }
    return c.sms;
}
}  // namespace trs

using namespace trs;

extern "C" {

int32_t trs_device_count(int32_t* count) {
    if (!count) return fail(TRS_ERR_INVALID_ARGUMENT, "count is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return cuda_fail(e, "cudaGetDeviceCount");
    }
    *count = n;
    return TRS_OK;
}

int32_t trs_set_current_device(int32_t device) {
    if (device < 0 || device >= kMaxDevices) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device %d", device);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { cudaGetLastError(); return cuda_fail(e, "cudaSetDevice"); }
    return TRS_OK;
}

int32_t trs_device_pci_bus_id(int32_t device, char* buffer, int32_t length) {
    if (!buffer || length < 16) return fail(TRS_ERR_INVALID_ARGUMENT, "buffer of at least 16 bytes needed");
    TRS_CUDA(cudaDeviceGetPCIBusId(buffer, length, device));
    return TRS_OK;
}

static int32_t cache_malloc(int32_t device, size_t bytes, trs_stream stream, void** ptr) {
    if (!ptr || device < 0 || device >= kMaxDevices) return fail(TRS_ERR_INVALID_ARGUMENT, "bad trs_malloc arguments");
    if (stream && stream->device != device) return fail(TRS_ERR_INVALID_ARGUMENT, "stream belongs to device %d, not %d", stream->device, device);
    *ptr = nullptr;
    DeviceCache& c = g_cache[device];
    size_t rounded = round_size(bytes);
    std::lock_guard<std::mutex> lock(c.mu);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    // Reuse only a block that wastes at most 1/8 of itself, so large blocks stay available for large requests.
    // First choice: a block the requesting stream freed itself, or one nothing can touch any more.
    auto take = [&](std::multimap<size_t, FreeBlock>::iterator it) {
        FreeBlock& b = it->second;
        if (b.freed) c.spare_events.push_back(b.freed);       // a wait already enqueued keeps the state it saw
        *ptr = b.ptr;
        c.live[*ptr] = it->first;
        c.in_use += (int64_t)it->first;
        c.free_blocks.erase(it);
    };
    int busy_candidates = 0;
    for (auto it = c.free_blocks.lower_bound(rounded); it != c.free_blocks.end() && it->first <= rounded + rounded / 8; ++it) {
        FreeBlock& b = it->second;
        if (b.last != nullptr && b.last != stream) {
            const bool idle = b.freed ? cudaEventQuery(b.freed) == cudaSuccess : cudaStreamQuery(b.last->stream) == cudaSuccess;
            if (!idle) { cudaGetLastError(); ++busy_candidates; continue; }
        }
        take(it);
        return TRS_OK;
    }
    // Second choice: new memory.  Only blocks that another stream gave up with work still queued are left; taking one
    // would order the requester behind that work (an upload behind the kernels it is meant to overlap), whereas one
    // more block in the pool gives every later request of this kind an idle one.  The pool must not grow without
    // bound in a loop that never drains, though: once kMaxBusyCandidates such blocks are waiting, the oldest of them
    // (freed first, so its work finishes first) is taken instead, behind the work that was queued on the other stream
    // when it was freed (and no further: later work of that stream cannot touch a block it had given up).
    constexpr int kMaxBusyCandidates = 8;
    auto take_busy = [&]() {
        for (auto it = c.free_blocks.lower_bound(rounded); it != c.free_blocks.end() && it->first <= rounded + rounded / 8; ++it) {
            FreeBlock& b = it->second;
            if (!b.freed || b.last == nullptr || b.last == stream) continue;
            if (cudaStreamWaitEvent(stream->stream, b.freed, 0) != cudaSuccess) { cudaGetLastError(); continue; }
            take(it);
            return true;
        }
        return false;
    };
    if (stream && busy_candidates >= kMaxBusyCandidates && take_busy()) return TRS_OK;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, rounded);
    if (e == cudaErrorMemoryAllocation && stream && busy_candidates > 0) {
        cudaGetLastError();                  // memory is short: such a block after all
        if (take_busy()) return TRS_OK;
    }
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        release_all(c);                      // give cached blocks back and retry once
        e = cudaMalloc(&p, rounded);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(e, "cudaMalloc");
    }
    c.live[p] = rounded;
    c.in_use += (int64_t)rounded;
    c.reserved += (int64_t)rounded;
    *ptr = p;
    return TRS_OK;
}

static int32_t cache_free(int32_t device, void* ptr, trs_stream stream) {
    if (!ptr) return TRS_OK;
    if (device < 0 || device >= kMaxDevices) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device");
    DeviceCache& c = g_cache[device];
    std::lock_guard<std::mutex> lock(c.mu);
    auto it = c.live.find(ptr);
    if (it == c.live.end()) return fail(TRS_ERR_INVALID_ARGUMENT, "pointer was not allocated by trs_malloc on device %d", device);
    c.in_use -= (int64_t)it->second;
    cudaEvent_t freed = nullptr;
    if (stream) {
        DeviceGuard guard(device);
        if (guard.ok && (freed = take_event(c)) != nullptr && cudaEventRecord(freed, stream->stream) != cudaSuccess) {
            cudaGetLastError();
            c.spare_events.push_back(freed);
            freed = nullptr;                                // falls back to querying the stream itself
        }
    }
    c.free_blocks.emplace(it->second, FreeBlock{ptr, stream, freed});
    c.live.erase(it);
    return TRS_OK;
}

// A stream that is going away can no longer be waited for: it has been drained, so its blocks are free for all.
static void forget_stream(trs_stream stream) {
    DeviceCache& c = g_cache[stream->device];
    std::lock_guard<std::mutex> lock(c.mu);
    for (auto& kv : c.free_blocks)
        if (kv.second.last == stream) {
            kv.second.last = nullptr;
            if (kv.second.freed) { c.spare_events.push_back(kv.second.freed); kv.second.freed = nullptr; }
        }
}

int32_t trs_malloc(int32_t device, size_t bytes, void** ptr) { return cache_malloc(device, bytes, nullptr, ptr); }
int32_t trs_free(int32_t device, void* ptr) { return cache_free(device, ptr, nullptr); }
int32_t trs_malloc_async(int32_t device, size_t bytes, trs_stream stream, void** ptr) {
    TRS_TRY(check_stream(stream));
    return cache_malloc(device, bytes, stream, ptr);
}
int32_t trs_free_async(int32_t device, void* ptr, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (stream->device != device) return fail(TRS_ERR_INVALID_ARGUMENT, "stream belongs to device %d, not %d", stream->device, device);
    return cache_free(device, ptr, stream);
}

int32_t trs_empty_cache(int32_t device) {
    if (device < 0 || device >= kMaxDevices) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device");
    DeviceCache& c = g_cache[device];
    std::lock_guard<std::mutex> lock(c.mu);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    cudaDeviceSynchronize();
    release_all(c);
    return TRS_OK;
}

int32_t trs_memory_stats(int32_t device, int64_t* bytes_in_use, int64_t* bytes_reserved) {
    if (device < 0 || device >= kMaxDevices) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device");
    DeviceCache& c = g_cache[device];
    std::lock_guard<std::mutex> lock(c.mu);
    if (bytes_in_use) *bytes_in_use = c.in_use;
    if (bytes_reserved) *bytes_reserved = c.reserved;
    return TRS_OK;
}

int32_t trs_malloc_host(size_t bytes, void** ptr) {
    if (!ptr) return fail(TRS_ERR_INVALID_ARGUMENT, "ptr is NULL");
    TRS_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1));
    return TRS_OK;
}

int32_t trs_free_host(void* ptr) {
    if (ptr) TRS_CUDA(cudaFreeHost(ptr));
    return TRS_OK;
}

int32_t trs_stream_create(int32_t device, trs_stream* stream) {
    if (!stream) return fail(TRS_ERR_INVALID_ARGUMENT, "stream is NULL");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    cudaStream_t s;
    TRS_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = new trs_stream_s{device, s};
    return TRS_OK;
}

int32_t trs_stream_destroy(trs_stream stream) {
    if (!stream) return TRS_OK;
    DeviceGuard guard(stream->device);
    cudaStreamSynchronize(stream->stream);
    forget_stream(stream);
    cudaStreamDestroy(stream->stream);
    delete stream;
    return TRS_OK;
}

int32_t trs_stream_sync(trs_stream stream) {
    TRS_TRY(check_stream(stream));
    DeviceGuard guard(stream->device);
    TRS_CUDA(cudaStreamSynchronize(stream->stream));
    return gemm_check_status(stream->device);
}

int32_t trs_stream_device(trs_stream stream, int32_t* device) {
    TRS_TRY(check_stream(stream));
    if (device) *device = stream->device;
    return TRS_OK;
}

int32_t trs_stream_handle(trs_stream stream, void** cuda_stream) {
    TRS_TRY(check_stream(stream));
    if (cuda_stream) *cuda_stream = (void*)stream->stream;
    return TRS_OK;
}

int32_t trs_device_sync(int32_t device) {
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    TRS_CUDA(cudaDeviceSynchronize());
    return gemm_check_status(device);
}

int32_t trs_event_create(trs_event* event) {
    if (!event) return fail(TRS_ERR_INVALID_ARGUMENT, "event is NULL");
    *event = new trs_event_s{nullptr, -1};
    return TRS_OK;
}

int32_t trs_event_record(trs_event event, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (!event) return fail(TRS_ERR_INVALID_ARGUMENT, "event is NULL");
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    if (event->device != stream->device) {
        // a CUDA event belongs to the device that was current when it was created: (re)create it where it is used
        if (event->event) cudaEventDestroy(event->event);
        event->event = nullptr;
        event->device = -1;
        TRS_CUDA(cudaEventCreate(&event->event));
        event->device = stream->device;
    }
    TRS_CUDA(cudaEventRecord(event->event, stream->stream));
    return TRS_OK;
}

int32_t trs_event_sync(trs_event event) {
    if (!event) return fail(TRS_ERR_INVALID_ARGUMENT, "event is NULL");
    if (!event->event) return TRS_OK;                    // never recorded: nothing to wait for
    TRS_CUDA(cudaEventSynchronize(event->event));
    return TRS_OK;
}

int32_t trs_event_elapsed_ms(trs_event start, trs_event stop, float* ms) {
    if (!start || !stop || !ms) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL argument");
    if (!start->event || !stop->event) return fail(TRS_ERR_INVALID_ARGUMENT, "both events must have been recorded");
    TRS_CUDA(cudaEventElapsedTime(ms, start->event, stop->event));
    return TRS_OK;
}

int32_t trs_event_destroy(trs_event event) {
    if (!event) return TRS_OK;
    if (event->event) cudaEventDestroy(event->event);
    delete event;
    return TRS_OK;
}

int32_t trs_stream_wait_event(trs_stream stream, trs_event event) {
    TRS_TRY(check_stream(stream));
    if (!event) return fail(TRS_ERR_INVALID_ARGUMENT, "event is NULL");
    if (!event->event) return TRS_OK;                    // never recorded: nothing to wait for
    DeviceGuard guard(stream->device);
    TRS_CUDA(cudaStreamWaitEvent(stream->stream, event->event, 0));
    return TRS_OK;
}

static int32_t copy(void* dst, const void* src, size_t bytes, trs_stream stream, cudaMemcpyKind kind) {
    TRS_TRY(check_stream(stream));
    if (bytes == 0) return TRS_OK;
    if (!dst || !src) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL copy pointer");
    DeviceGuard guard(stream->device);
    TRS_CUDA(cudaMemcpyAsync(dst, src, bytes, kind, stream->stream));
    return TRS_OK;
}

int32_t trs_memcpy_h2d(void* dst, const void* src, size_t bytes, trs_stream stream) {
    return copy(dst, src, bytes, stream, cudaMemcpyHostToDevice);
}
int32_t trs_memcpy_d2h(void* dst, const void* src, size_t bytes, trs_stream stream) {
    return copy(dst, src, bytes, stream, cudaMemcpyDeviceToHost);
}
int32_t trs_memcpy_d2d(void* dst, const void* src, size_t bytes, trs_stream stream) {
    return copy(dst, src, bytes, stream, cudaMemcpyDeviceToDevice);
}

const char* trs_status_string(int32_t status) {
    switch (status) {
        case TRS_OK: return "ok";
        case TRS_ERR_INVALID_ARGUMENT: return "invalid argument";
        case TRS_ERR_ALLOCATION_FAILED: return "allocation failed";
        case TRS_ERR_CUDA: return "CUDA error";
        case TRS_ERR_JIT: return "kernel specialisation failed";
        case TRS_ERR_UNSUPPORTED: return "unsupported";
        case TRS_ERR_NO_DEVICE: return "no CUDA device";
        case TRS_ERR_DEVICE_STATUS: return "device-side status error";
        default: return "unknown status";
    }
}

const char* trs_last_error_message(void) { return g_last_error.c_str(); }
int64_t trs_kernel_launch_count(void) { return g_launches.load(); }

}  // extern "C"
