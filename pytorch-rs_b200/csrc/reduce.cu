// Deterministic reductions: full sum of a strided view, and un-broadcast (row/column) sums.
//
// The reference sums sequentially in logical order (Tensor::sum, src/tensor.rs:2413-2431;
// GradientAccumulator, src/tensor.rs:3204-3228).  A GPU cannot keep that order at HBM speed, so
// these kernels use a fixed two-stage tree: the grouping depends only on the problem size, never
// on scheduling, so repeated runs give identical bits; the difference from the sequential order
// is rounding only and is covered by a stated tolerance in the tests.
//
// Both use scratch memory for the stage-1 partials.  The *_ws helpers take the scratch from the
// caller; the public entry points take it from the device cache.
#include <algorithm>
#include <vector>

#include <atomic>

#include "common.h"
#include "reduce.h"

namespace trs {
namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = 0.0f;
    if (warp == 0) {
        r = lane < (int)(blockDim.x >> 5) ? smem[lane] : 0.0f;
        r = warp_sum(r);
    }
    __syncthreads();
    return r;   // valid in thread 0
}

struct SumView {
    int ndim;
    long long size[TRS_MAX_RANK];     // dim 0 innermost (smallest stride)
    long long stride[TRS_MAX_RANK];
};

// Stage 1: each CTA sums a fixed, contiguous range of the (collapsed) logical index space.
__global__ void __launch_bounds__(kBlock) sum_stage1(const float* __restrict__ in, SumView v, long long n,
                                                    long long per_cta, float* __restrict__ partials) {
    __shared__ float smem[kBlock / 32];
    const long long begin = (long long)blockIdx.x * per_cta;
    const long long end = min(begin + per_cta, n);
    float acc = 0.0f;
    if (v.ndim == 1 && v.stride[0] == 1) {
        // 16-byte vector body when the CTA range is aligned, scalar otherwise.
        const float* p = in + begin;
        const long long len = end - begin;
        if ((((uintptr_t)p) & 15u) == 0) {
            const long long n4 = len >> 2;
            const float4* p4 = reinterpret_cast<const float4*>(p);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (long long i = threadIdx.x; i < n4; i += kBlock) {
                const float4 t = __ldcs(p4 + i);
                a0 = __fadd_rn(a0, t.x); a1 = __fadd_rn(a1, t.y); a2 = __fadd_rn(a2, t.z); a3 = __fadd_rn(a3, t.w);
            }
            acc = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
            for (long long i = (n4 << 2) + threadIdx.x; i < len; i += kBlock) acc = __fadd_rn(acc, p[i]);
        } else {
            for (long long i = threadIdx.x; i < len; i += kBlock) acc = __fadd_rn(acc, p[i]);
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kBlock) {
            long long rem = i, off = 0;
#pragma unroll 1
            for (int d = 0; d < v.ndim; ++d) {
                const long long c = rem % v.size[d];
                rem /= v.size[d];
                off += c * v.stride[d];
            }
            acc = __fadd_rn(acc, in[off]);
        }
    }
    const float total = block_sum(acc, smem);
    if (threadIdx.x == 0) partials[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kBlock) sum_stage2(const float* __restrict__ partials, int count, float* __restrict__ out) {
    __shared__ float smem[kBlock / 32];
    float acc = 0.0f;
    for (int i = threadIdx.x; i < count; i += kBlock) acc = __fadd_rn(acc, partials[i]);
    const float total = block_sum(acc, smem);
    if (threadIdx.x == 0) out[0] = total;
}

// Column sums, stage 1: CTA (x = 128-column tile, y = row chunk); 8 warps stride the rows.
__global__ void __launch_bounds__(kBlock) colsum_stage1(const float* __restrict__ in, long long rows, long long cols,
                                                       long long rows_per_chunk, float* __restrict__ partials, int vec) {
    __shared__ float smem[8][128];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long c0 = (long long)blockIdx.x * 128 + lane * 4;
    const long long r_begin = (long long)blockIdx.y * rows_per_chunk;
    const long long r_end = min(r_begin + rows_per_chunk, rows);
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec) {
        if (c0 < cols)
            for (long long r = r_begin + warp; r < r_end; r += 8) {
                const float4 t = __ldcs(reinterpret_cast<const float4*>(in + r * cols + c0));
                a[0] = __fadd_rn(a[0], t.x); a[1] = __fadd_rn(a[1], t.y); a[2] = __fadd_rn(a[2], t.z); a[3] = __fadd_rn(a[3], t.w);
            }
    } else {
        for (long long r = r_begin + warp; r < r_end; r += 8)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (c0 + e < cols) a[e] = __fadd_rn(a[e], in[r * cols + c0 + e]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) smem[warp][lane * 4 + e] = a[e];
    __syncthreads();
    if (threadIdx.x < 128) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s = __fadd_rn(s, smem[w][threadIdx.x]);
        const long long c = (long long)blockIdx.x * 128 + threadIdx.x;
        if (c < cols) partials[(long long)blockIdx.y * cols + c] = s;
    }
}

__global__ void __launch_bounds__(kBlock) colsum_stage2(const float* __restrict__ partials, int chunks, long long cols,
                                                       float* __restrict__ out) {
    const long long c = (long long)blockIdx.x * kBlock + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int k = 0; k < chunks; ++k) s = __fadd_rn(s, partials[(long long)k * cols + c]);
    out[c] = s;
}

// Row sums: one CTA per row, fixed tree.
__global__ void __launch_bounds__(kBlock) rowsum_kernel(const float* __restrict__ in, long long cols, float* __restrict__ out) {
    __shared__ float smem[kBlock / 32];
    const float* p = in + (long long)blockIdx.x * cols;
    float acc = 0.f;
    for (long long i = threadIdx.x; i < cols; i += kBlock) acc = __fadd_rn(acc, p[i]);
    const float total = block_sum(acc, smem);
    if (threadIdx.x == 0) out[blockIdx.x] = total;
}

}  // namespace

int sum_partials_needed(int device, long long n) {
    long long want = (n + (long long)kBlock * 16 - 1) / ((long long)kBlock * 16);
    long long cap = (long long)sm_count(device) * 8;
    return (int)std::max<long long>(1, std::min(want, cap));
}

int32_t reduce_sum_ws(const trs_operand* input, float* out, float* scratch, int scratch_floats, trs_stream stream) {
    const int rank = input->rank;
    if (rank < 0 || rank > TRS_MAX_RANK) return fail(TRS_ERR_INVALID_ARGUMENT, "rank %d out of range", rank);
    long long n = 1;
    for (int a = 0; a < rank; ++a) n *= input->shape[a];
    if (n == 0) {
        // Empty sum: Rust's f32 Iterator::sum folds from -0.0.
        fill_value_async(out, 1, -0.0f, stream);
        return TRS_OK;
    }
    // Sort by stride (innermost first) and merge uniform runs; summation order is free, so a
    // dense permuted view collapses to one contiguous range.
    struct D { long long size, stride; };
    std::vector<D> dims;
    for (int a = 0; a < rank; ++a) if (input->shape[a] != 1) dims.push_back({input->shape[a], input->stride[a]});
    std::stable_sort(dims.begin(), dims.end(), [](const D& x, const D& y) { return x.stride < y.stride; });
    SumView v{};
    v.ndim = 0;
    for (const D& d : dims) {
        if (v.ndim > 0 && d.stride == v.stride[v.ndim - 1] * v.size[v.ndim - 1]) v.size[v.ndim - 1] *= d.size;
        else { v.size[v.ndim] = d.size; v.stride[v.ndim] = d.stride; ++v.ndim; }
    }
    if (v.ndim == 0) { v.ndim = 1; v.size[0] = 1; v.stride[0] = 1; }
    const float* base = (const float*)input->base + input->offset;
    int ctas = std::min(sum_partials_needed(stream->device, n), scratch_floats);
    if (ctas < 1) return fail(TRS_ERR_INVALID_ARGUMENT, "reduction scratch is too small");
    long long per_cta = (n + ctas - 1) / ctas;
    per_cta = (per_cta + 3) & ~3ll;                       // keeps CTA ranges 16-byte aligned
    ctas = (int)((n + per_cta - 1) / per_cta);
    sum_stage1<<<ctas, kBlock, 0, stream->stream>>>(base, v, n, per_cta, scratch);
    sum_stage2<<<1, kBlock, 0, stream->stream>>>(scratch, ctas, out);
    TRS_CUDA(cudaGetLastError());
    count_launch(2);
    return TRS_OK;
}

void colsum_geometry_for(int sms, long long rows, long long cols, long long max_partials, int* chunks, long long* rows_per_chunk) {
    long long col_tiles = (cols + 127) / 128;
    long long want = std::max<long long>(1, ((long long)sms * 4) / col_tiles);
    long long c = std::min<long long>(want, std::max<long long>(1, rows / 64));
    c = std::min<long long>(c, 1024);
    // a bounded partials buffer (the allocation-free entry point) caps the number of row chunks
    if (max_partials > 0) c = std::min<long long>(c, std::max<long long>(1, max_partials / std::max<long long>(cols, 1)));
    *rows_per_chunk = (rows + c - 1) / c;
    *chunks = (int)((rows + *rows_per_chunk - 1) / *rows_per_chunk);
}

void colsum_geometry(int device, long long rows, long long cols, int* chunks, long long* rows_per_chunk) {
    colsum_geometry_for(sm_count(device), rows, cols, 0, chunks, rows_per_chunk);
}

int32_t unbroadcast_sum_ws(const float* input, long long rows, long long cols, int by_rows, float* out, float* scratch,
                           long long scratch_floats, trs_stream stream) {
    if (rows < 0 || cols < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative extent");
    if (by_rows) {
        if (rows == 0) return TRS_OK;
        if (cols == 0) { fill_value_async(out, rows, 0.0f, stream); return TRS_OK; }
        rowsum_kernel<<<(unsigned)rows, kBlock, 0, stream->stream>>>(input, cols, out);
        TRS_CUDA(cudaGetLastError());
        count_launch();
        return TRS_OK;
    }
    if (cols == 0) return TRS_OK;
    if (rows == 0) { fill_value_async(out, cols, 0.0f, stream); return TRS_OK; }
    int chunks = 0;
    long long rows_per_chunk = 0;
    colsum_geometry(stream->device, rows, cols, &chunks, &rows_per_chunk);
    if ((long long)chunks * cols > scratch_floats) return fail(TRS_ERR_INVALID_ARGUMENT, "un-broadcast scratch is too small");
    const int vec = (cols % 4 == 0) && (((uintptr_t)input & 15u) == 0);
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)chunks);
    colsum_stage1<<<grid, kBlock, 0, stream->stream>>>(input, rows, cols, rows_per_chunk, scratch, vec);
    colsum_stage2<<<(unsigned)((cols + kBlock - 1) / kBlock), kBlock, 0, stream->stream>>>(scratch, chunks, cols, out);
    TRS_CUDA(cudaGetLastError());
    count_launch(2);
    return TRS_OK;
}

}  // namespace trs

using namespace trs;

extern "C" {

int32_t trs_reduce_sum_f32(const trs_operand* input, float* out, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (!input || !out) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL argument");
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    long long n = 1;
    for (int a = 0; a < input->rank; ++a) n *= input->shape[a];
    const int need = sum_partials_needed(stream->device, std::max<long long>(n, 1));
    void* scratch = nullptr;
    TRS_TRY(malloc_on_stream(stream, (size_t)need * sizeof(float), &scratch));
    int32_t s = reduce_sum_ws(input, out, (float*)scratch, need, stream);
    free_on_stream(stream, scratch);     // reuse is ordered behind this stream's work
    return s;
}

int32_t trs_unbroadcast_sum_f32(const float* input, int64_t rows, int64_t cols, int32_t by_rows, float* out,
                                trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (!out || (!input && rows * cols != 0)) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL argument");
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    void* scratch = nullptr;
    long long floats = 0;
    if (!by_rows && rows > 0 && cols > 0) {
        int chunks = 0;
        long long rpc = 0;
        colsum_geometry(stream->device, rows, cols, &chunks, &rpc);
        floats = (long long)chunks * cols;
        TRS_TRY(malloc_on_stream(stream, (size_t)floats * sizeof(float), &scratch));
    }
    int32_t s = unbroadcast_sum_ws(input, rows, cols, by_rows, out, (float*)scratch, floats, stream);
    if (scratch) free_on_stream(stream, scratch);
    return s;
}


// ---- column sums for callers that must not allocate ---------------------------------------------
// Some hosts of this library run where a device allocation is not an option: inside a region that
// is being stream-captured, inside a callback that the driver runs, or in a service that sized its
// memory pool at start-up and forbids growth afterwards.  For them the stage-1 partials live in a
// fixed array that is part of the library image: 1 MiB per GPU that loads the library, held until
// the process exits.
constexpr long long kNoAllocScratchFloats = 262144;      // 1 MiB; also the largest `cols` accepted
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
static std::atomic<float*> g_noalloc_scratch_ptr[16];     // device address per device, resolved once

int32_t trs_colsum_f32_noalloc(const float* input, int64_t rows, int64_t cols, float* out, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (rows < 0 || cols < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative extent");
    if (!out || (!input && rows != 0 && cols != 0)) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL argument");
    if (cols > kNoAllocScratchFloats)
        return fail(TRS_ERR_UNSUPPORTED, "trs_colsum_f32_noalloc: %lld columns exceed the fixed scratch of %lld floats; "
                                         "use trs_unbroadcast_sum_f32", (long long)cols, kNoAllocScratchFloats);
    const int device = stream->device;
    if (device < 0 || device >= 16) return fail(TRS_ERR_INVALID_ARGUMENT, "bad device");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", device);
    if (cols == 0) return TRS_OK;
    // The array's name is only a host-side handle; the kernels need its address on THIS device.
    float* scratch = g_noalloc_scratch_ptr[device].load(std::memory_order_acquire);
    if (!scratch) {
        cudaError_t err = cudaGetSymbolAddress((void**)&scratch, g_noalloc_scratch);
        if (err != cudaSuccess) return cuda_fail(err, "cudaGetSymbolAddress(g_noalloc_scratch)");
        g_noalloc_scratch_ptr[device].store(scratch, std::memory_order_release);   // every thread resolves the same address
    }
    if (rows == 0) { fill_value_async(out, cols, 0.0f, stream); return TRS_OK; }
    int chunks = 0;
    long long rows_per_chunk = 0;
    // as many row chunks as the grid wants, but never more partials than the fixed array holds
    colsum_geometry_for(sm_count(device), rows, cols, kNoAllocScratchFloats, &chunks, &rows_per_chunk);
    const int vec = (cols % 4 == 0) && (((uintptr_t)input & 15u) == 0);
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)chunks);
    // Stage 1 writes every partial that stage 2 reads, so nothing left by an earlier call matters.
    colsum_stage1<<<grid, kBlock, 0, stream->stream>>>(input, rows, cols, rows_per_chunk, scratch, vec);
    colsum_stage2<<<(unsigned)((cols + kBlock - 1) / kBlock), kBlock, 0, stream->stream>>>(scratch, chunks, cols, out);
    TRS_CUDA(cudaGetLastError());
    count_launch(2);
    return TRS_OK;
}

int32_t trs_colsum_noalloc_geometry(int32_t sm_count, int64_t rows, int64_t cols, int32_t* chunks, int64_t* rows_per_chunk) {
    if (sm_count < 1 || rows < 1 || cols < 1 || cols > kNoAllocScratchFloats || !chunks || !rows_per_chunk)
        return fail(TRS_ERR_INVALID_ARGUMENT, "bad trs_colsum_noalloc_geometry arguments");
    int c = 0;
    long long rpc = 0;
    colsum_geometry_for(sm_count, rows, cols, kNoAllocScratchFloats, &c, &rpc);
    *chunks = c;
    *rows_per_chunk = rpc;
    return TRS_OK;
}

}  // extern "C"
