// Shared internals of libtrs_cuda.so: status plumbing, stream/event objects, launch accounting.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <utility>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/trs_cuda.h"

struct trs_stream_s {
    int device;
    cudaStream_t stream;
};
struct trs_event_s {
    cudaEvent_t event;     // created on the device of the first stream it is recorded on (an event belongs to one device)
    int device;            // -1 until then
};

namespace trs {

extern thread_local std::string g_last_error;
extern std::atomic<int64_t> g_launches;

inline int32_t fail(int32_t status, const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

inline int32_t cuda_fail(cudaError_t e, const char* what) {
    if (e == cudaErrorMemoryAllocation) return fail(TRS_ERR_ALLOCATION_FAILED, "%s: %s", what, cudaGetErrorString(e));
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInvalidDevice)
        return fail(TRS_ERR_NO_DEVICE, "%s: %s", what, cudaGetErrorString(e));
    return fail(TRS_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TRS_CUDA(call)                                             \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return ::trs::cuda_fail(e__, #call); \
    } while (0)

#define TRS_TRY(call)                   \
    do {                                \
        int32_t s__ = (call);           \
        if (s__ != TRS_OK) return s__;  \
    } while (0)

// Binds the calling thread to the stream's device for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (ok && cudaGetDevice(&cur) == cudaSuccess && cur != prev && prev >= 0) cudaSetDevice(prev);
    }
};

inline void count_launch(int64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#ifdef __CUDACC__
// Launch with programmatic stream serialization: the kernel's blocks may become resident while the
// stream's previous kernel drains.  Only for kernels that execute pdl_wait() before their first access
// to memory another kernel may have written.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// Waits until the kernels this one depends on have completed and their writes are visible, then lets the
// next kernel of the stream start taking the slots this grid frees.  A no-op in an ordinary launch.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}
#endif

int32_t check_stream(trs_stream s);
// Cached device blocks in stream order (see trs_malloc_async / trs_free_async).
int32_t malloc_on_stream(trs_stream stream, size_t bytes, void** ptr);
void free_on_stream(trs_stream stream, void* ptr);
int sm_count(int device);

}  // namespace trs
