// FP32 SIMT matmul: register-tiled FFMA kernel for any operand strides.
//
// Replaces Tensor::matmul's loops (pytorch-rs src/tensor.rs:2453-2533, 3889-3966) for shapes
// the tensor-core path does not take (unaligned or tiny operands) and serves as the exact-FP32
// algorithm under float32 matmul precision "highest".  The reference accumulates k ascending
// with separate multiply and add roundings; this kernel accumulates k ascending per thread with
// fused multiply-add, which differs by rounding only (tolerance rel 1e-5*sqrt(K) in the tests).
#include <algorithm>
#include <mutex>

#include "common.h"
#include "gemm.h"

namespace trs {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, PAD = 4;

__device__ __forceinline__ float ref_relu(float v) {
    return ((__float_as_uint(v) & 0x7fffffffu) == 0u) ? v : fmaxf(v, 0.0f);
}
__device__ __forceinline__ float ref_relu_vjp(float x, float g) {
    const unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    return (mag > 0x7f800000u || ((b >> 31) == 0u && mag != 0u)) ? g : 0.0f;
}

__device__ __forceinline__ bool word_is(const unsigned int* p, unsigned int value) {
    return p != nullptr && *reinterpret_cast<const volatile unsigned int*>(p) == value;
}
__device__ __forceinline__ bool word_set(const unsigned int* p) {
    return p != nullptr && *reinterpret_cast<const volatile unsigned int*>(p) != 0u;
}

template <bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256, 2) gemm_simt_kernel(const trs_gemm_desc g, const SimtGate gate, float* c_lo, unsigned int* c_flag,
                                                       const long long tiles_x, const long long tiles_y, const long long total_tiles) {
    pdl_wait();
    // gated launch: runs only when the preparation of this very call (tagged `epoch`) or a prepared operand image met an inf / NaN
    if (gate.gated && !word_is(gate.word, gate.epoch) && !word_set(gate.flag_a) && !word_set(gate.flag_b)) return;
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // Output tiles are walked with a grid stride, so a gated launch can use a small grid.
  for (long long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const long long tile_x = tile % tiles_x, tile_y = (tile / tiles_x) % tiles_y, batch = tile / (tiles_x * tiles_y);
    const long long m0 = tile_y * BM, n0 = tile_x * BN;
    __syncthreads();        // the previous tile's shared-memory reads are done before this tile overwrites them
    const float* __restrict__ A = g.a + batch * g.a_batch_stride;
    const float* __restrict__ B = g.b + batch * g.b_batch_stride;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float ra[8], rb[8];
    auto load_tiles = [&](long long k0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = i * 256 + tid;
            const int kk = A_KFAST ? (e & 15) : (e >> 7);
            const int mm = A_KFAST ? (e >> 4) : (e & 127);
            const long long m = m0 + mm, k = k0 + kk;
            ra[i] = (m < g.m && k < g.k) ? __ldg(A + m * g.a_row_stride + k * g.a_col_stride) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = i * 256 + tid;
            const int kk = B_NFAST ? (e >> 7) : (e & 15);
            const int nn = B_NFAST ? (e & 127) : (e >> 4);
            const long long n = n0 + nn, k = k0 + kk;
            rb[i] = (n < g.n && k < g.k) ? __ldg(B + k * g.b_row_stride + n * g.b_col_stride) : 0.0f;
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = i * 256 + tid;
            const int kk = A_KFAST ? (e & 15) : (e >> 7);
            const int mm = A_KFAST ? (e >> 4) : (e & 127);
            As[buf][kk][mm] = ra[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = i * 256 + tid;
            const int kk = B_NFAST ? (e >> 7) : (e & 15);
            const int nn = B_NFAST ? (e & 127) : (e >> 4);
            Bs[buf][kk][nn] = rb[i];
        }
    };

    const long long k_tiles = (g.k + BK - 1) / BK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    for (long long t = 0; t < k_tiles; ++t) {
        const int buf = (int)(t & 1);
        if (t + 1 < k_tiles) load_tiles((t + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (t + 1 < k_tiles) store_tiles(buf ^ 1);
        __syncthreads();
    }

    float* __restrict__ C = g.c + batch * g.c_batch_stride;
    const float* __restrict__ aux = g.aux ? g.aux + batch * g.c_batch_stride : nullptr;
    float* __restrict__ pre = g.preact ? g.preact + batch * g.c_batch_stride : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= g.m) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= g.n) continue;
            float v = acc[i][j];
            const long long idx = m * g.c_row_stride + n;
            if (g.epilogue == TRS_EPI_BIAS || g.epilogue == TRS_EPI_BIAS_RELU) v = __fadd_rn(v, __ldg(g.bias + n));
            if (g.epilogue == TRS_EPI_BIAS_RELU && pre) pre[idx] = v;
            if (g.epilogue == TRS_EPI_BIAS_RELU || g.epilogue == TRS_EPI_RELU) v = ref_relu(v);
            if (g.epilogue == TRS_EPI_RELU_VJP) v = ref_relu_vjp(__ldg(aux + idx), v);
            C[idx] = v;
            if (c_lo) {
                // lo image of the result for the tensor-core matmul that reads it next: tf32(v - trunc_tf32(v))
                const unsigned bits = __float_as_uint(v);
                float lo = 0.0f;
                if ((bits & 0x7f800000u) == 0x7f800000u) {
                    *reinterpret_cast<volatile unsigned int*>(c_flag) = 1u;
                } else {
                    unsigned l;
                    const float rest = __fsub_rn(v, __uint_as_float(bits & 0xffffe000u));
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
                    lo = __uint_as_float(l);
                }
                c_lo[batch * g.c_batch_stride + idx] = lo;
            }
        }
    }
  }
}

}  // namespace

int32_t gemm_simt_launch(const trs_gemm_desc& g, const trs_gemm_planes* planes, trs_stream stream, const SimtGate& gate) {
    const long long tiles_x = (g.n + BN - 1) / BN, tiles_y = (g.m + BM - 1) / BM, total = tiles_x * tiles_y * g.batch;
    // A gated launch almost always returns at once: keep its grid small so that the no-op is cheap.
    const long long cap = gate.gated ? (long long)sm_count(stream->device) * 2 : (1ll << 31) - 1;
    const unsigned grid = (unsigned)std::max<long long>(1, std::min(total, cap));
    const bool a_kfast = g.a_col_stride == 1 || g.a_row_stride != 1;
    const bool b_nfast = g.b_col_stride == 1 || g.b_row_stride != 1;
    auto kernel = a_kfast ? (b_nfast ? gemm_simt_kernel<true, true> : gemm_simt_kernel<true, false>)
                          : (b_nfast ? gemm_simt_kernel<false, true> : gemm_simt_kernel<false, false>);
    if (gate.gated) {
        // A gated launch sits between tensor-core GEMMs and their preparation kernels: keep their shared-memory
        // configuration, so that no SM has to drain to switch it for a kernel that returns at once.  Function
        // attributes are per device.
        static std::once_flag once[16];
        std::call_once(once[stream->device & 15], [] {
            cudaFuncSetAttribute(gemm_simt_kernel<true, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaFuncSetAttribute(gemm_simt_kernel<true, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaFuncSetAttribute(gemm_simt_kernel<false, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaFuncSetAttribute(gemm_simt_kernel<false, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        });
    }
    TRS_CUDA(launch_dependent(kernel, dim3(grid), dim3(256), 0, stream->stream, g, gate, planes ? planes->c_lo : (float*)nullptr,
                               planes ? planes->c_flag : (unsigned int*)nullptr, tiles_x, tiles_y, total));
    count_launch();
    return TRS_OK;
}

}  // namespace trs
