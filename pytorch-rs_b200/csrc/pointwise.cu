// Fused pointwise chains: plan -> specialised kernel (NVRTC, cached) -> launch.
// Also the small fixed kernels for fill and in-place accumulation.
#include <nvrtc.h>
#include <unistd.h>

#include <cstdlib>

#include <mutex>
#include <unordered_map>

#include "common.h"
#include "pointwise_plan.h"
#include "reduce.h"

namespace trs {
namespace {

struct JitEntry {
    cudaLibrary_t library = nullptr;
    cudaKernel_t kernel = nullptr;
    std::string cubin;
};
std::mutex g_jit_mu;
std::unordered_map<std::string, JitEntry> g_jit_cache;   // key: pw_cache_key (what the generated source depends on)

int32_t compile_cubin(const std::string& source, std::string* cubin) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, source.c_str(), "trs_pw.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
        return fail(TRS_ERR_JIT, "nvrtcCreateProgram failed");
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "--ftz=false", "--prec-div=true",
                          "--prec-sqrt=true"};
    nvrtcResult r = nvrtcCompileProgram(prog, (int)(sizeof opts / sizeof opts[0]), opts);
    if (r != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        std::string log(n, '\0');
        if (n) nvrtcGetProgramLog(prog, &log[0]);
        nvrtcDestroyProgram(&prog);
        return fail(TRS_ERR_JIT, "NVRTC: %s\n%s", nvrtcGetErrorString(r), log.c_str());
    }
    size_t size = 0;
    if (nvrtcGetCUBINSize(prog, &size) != NVRTC_SUCCESS || size == 0) {
        nvrtcDestroyProgram(&prog);
        return fail(TRS_ERR_JIT, "NVRTC produced no cubin");
    }
    cubin->resize(size);
    nvrtcGetCUBIN(prog, &(*cubin)[0]);
    nvrtcDestroyProgram(&prog);
    return TRS_OK;
}

// ---- optional cache of compiled chains on disk -------------------------------------------------------
// Specialising a chain costs about 150 ms for the first one of a process (NVRTC start-up included) and 50-60 ms
// for each further one.  A process that names a directory in TRS_JIT_CACHE_DIR keeps the compiled code there and
// later processes read it back instead of compiling.  A file is named by a 64-bit hash of the generated source and
// holds a second hash and the source length, which must match too; it is written under a temporary name and
// renamed, so a reader never sees half a file.  Without the variable nothing touches the disk.
uint64_t fnv1a(const std::string& text, uint64_t seed) {
    uint64_t h = 1469598103934665603ull ^ seed;
    for (unsigned char c : text) { h ^= c; h *= 1099511628211ull; }
    return h;
}

struct DiskHeader {
    uint64_t magic, check, source_length, cubin_length;
};
constexpr uint64_t kDiskMagic = 0x31303062754a5254ull;      // "TRJub001"

std::string disk_path(const std::string& source) {
    const char* dir = getenv("TRS_JIT_CACHE_DIR");
    if (!dir || !*dir) return std::string();
    char name[64];
    snprintf(name, sizeof name, "/trs_pw_%016llx.cubin", (unsigned long long)fnv1a(source, 0));
    return std::string(dir) + name;
}

bool disk_load(const std::string& source, std::string* cubin) {
    const std::string path = disk_path(source);
    if (path.empty()) return false;
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    DiskHeader h{};
    bool ok = fread(&h, sizeof h, 1, f) == 1 && h.magic == kDiskMagic && h.check == fnv1a(source, 0x9e3779b97f4a7c15ull) &&
              h.source_length == source.size() && h.cubin_length > 0 && h.cubin_length < (64u << 20);
    if (ok) {
        cubin->resize(h.cubin_length);
        ok = fread(&(*cubin)[0], 1, h.cubin_length, f) == h.cubin_length;
    }
    fclose(f);
    if (!ok) cubin->clear();
    return ok;
}

void disk_store(const std::string& source, const std::string& cubin) {
    const std::string path = disk_path(source);
    if (path.empty()) return;
    char suffix[32];
    snprintf(suffix, sizeof suffix, ".tmp%ld", (long)getpid());
    const std::string tmp = path + suffix;
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return;                                   // an unwritable directory only means no cache
    DiskHeader h{kDiskMagic, fnv1a(source, 0x9e3779b97f4a7c15ull), source.size(), cubin.size()};
    const bool ok = fwrite(&h, sizeof h, 1, f) == 1 && fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
    if (fclose(f) != 0 || !ok || rename(tmp.c_str(), path.c_str()) != 0) remove(tmp.c_str());
}

// Returns the cache entry of this chain and plan, generating and compiling its source if needed; loads
// it onto the GPU when `load` is set (loading needs a device, compiling does not).
int32_t get_kernel(const trs_program* program, const PwPlan& plan, bool load, JitEntry** out) {
    const std::string key = pw_cache_key(program, plan);
    std::lock_guard<std::mutex> lock(g_jit_mu);
    JitEntry& e = g_jit_cache[key];
    if (e.cubin.empty()) {
        const std::string source = pw_generate_source(program, plan);
        if (!disk_load(source, &e.cubin)) {
            int32_t s = compile_cubin(source, &e.cubin);
            if (s != TRS_OK) { g_jit_cache.erase(key); return s; }
            disk_store(source, e.cubin);
        }
    }
    if (load && !e.kernel) {
        cudaError_t err = cudaLibraryLoadData(&e.library, e.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
        if (err != cudaSuccess) return cuda_fail(err, "cudaLibraryLoadData");
        err = cudaLibraryGetKernel(&e.kernel, e.library, "trs_pw");
        if (err != cudaSuccess) return cuda_fail(err, "cudaLibraryGetKernel");
    }
    *out = &e;
    return TRS_OK;
}

__global__ void __launch_bounds__(256) fill_kernel(float* __restrict__ dst, long long n, float value, int vec) {
    const long long n4 = vec ? (n >> 2) : 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    float4* d4 = reinterpret_cast<float4*>(dst);
    const float4 v = make_float4(value, value, value, value);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) __stcs(d4 + i, v);
    for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = value;
}

__global__ void __launch_bounds__(256) accumulate_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n,
                                                        int vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long done = 0;
    if (vec) {
        const long long n4 = n >> 2;
        float4* d4 = reinterpret_cast<float4*>(dst);
        const float4* s4 = reinterpret_cast<const float4*>(src);
        for (long long i = tid; i < n4; i += stride) {
            float4 a = d4[i];
            const float4 b = __ldcs(s4 + i);
            a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
            d4[i] = a;
        }
        done = n4 << 2;
    }
    for (long long i = done + tid; i < n; i += stride) dst[i] = __fadd_rn(dst[i], src[i]);
}

unsigned stream_grid(int device, long long work_items) {
    long long want = (work_items + 255) / 256;
    long long cap = (long long)sm_count(device) * 16;
    return (unsigned)std::max<long long>(1, std::min(want, cap));
}

}  // namespace

void fill_value_async(float* dst, long long count, float value, trs_stream stream) {
    if (count <= 0) return;
    const int vec = ((uintptr_t)dst & 15u) == 0;
    fill_kernel<<<stream_grid(stream->device, count / 4 + 1), 256, 0, stream->stream>>>(dst, count, value, vec);
    count_launch();
}
}  // namespace trs

using namespace trs;

extern "C" {

int32_t trs_pointwise_prepare(const trs_program* program, const trs_operand* inputs, const trs_operand* outputs,
                              char* klass) {
    PwPlan plan;
    TRS_TRY(pw_make_plan(program, inputs, outputs, &plan));
    if (klass) snprintf(klass, 16, "%s", plan.empty ? "empty" : (plan.tiled ? "tiled" : "vector"));
    if (plan.empty) return TRS_OK;
    JitEntry* entry = nullptr;
    return get_kernel(program, plan, false, &entry);
}

int32_t trs_pointwise(const trs_program* program, const trs_operand* inputs, const trs_operand* outputs,
                      trs_stream stream) {
    TRS_TRY(check_stream(stream));
    PwPlan plan;
    TRS_TRY(pw_make_plan(program, inputs, outputs, &plan));
    if (plan.empty) return TRS_OK;
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    JitEntry* entry = nullptr;
    TRS_TRY(get_kernel(program, plan, true, &entry));
    void* args[] = {&plan.params};
    // Programmatic dependent launch: the kernel starts with griddepcontrol.wait, so its blocks may be
    // scheduled while the stream's previous kernel drains (hides the launch gap between chained kernels).
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)plan.grid);
    cfg.blockDim = dim3(plan.block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream->stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    TRS_CUDA(cudaLaunchKernelExC(&cfg, (const void*)entry->kernel, args));
    count_launch();
    return TRS_OK;
}

int32_t trs_fill_f32(float* dst, int64_t count, float value, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (count < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative count");
    if (count == 0) return TRS_OK;
    if (!dst) return fail(TRS_ERR_INVALID_ARGUMENT, "fill destination is NULL");
    DeviceGuard guard(stream->device);
    fill_value_async(dst, count, value, stream);
    TRS_CUDA(cudaGetLastError());
    return TRS_OK;
}

int32_t trs_accumulate_f32(float* dst, const float* src, int64_t count, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (count < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative count");
    if (count == 0) return TRS_OK;
    if (!dst || !src) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL pointer");
    DeviceGuard guard(stream->device);
    int vec = (((uintptr_t)dst | (uintptr_t)src) & 15u) == 0;
    accumulate_kernel<<<stream_grid(stream->device, count / 4 + 1), 256, 0, stream->stream>>>(dst, src, count, vec);
    TRS_CUDA(cudaGetLastError());
    count_launch();
    return TRS_OK;
}

int32_t trs_jit_cache_size(int32_t* entries) {
    std::lock_guard<std::mutex> lock(g_jit_mu);
    if (entries) *entries = (int32_t)g_jit_cache.size();
    return TRS_OK;
}

}  // extern "C"
