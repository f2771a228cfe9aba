// Tensor-core float32 matmul for sm_100a: TMA-fed tcgen05.mma kind::tf32 with the 3-product
// error-compensated split ("3xTF32"), FP32 accumulation in tensor memory, fused epilogues.
//
// Replaces Tensor::matmul's loops (pytorch-rs src/tensor.rs:2453-2533, 3889-3966) for aligned
// shapes while honouring float32 matmul precision "highest": each operand a is split into
// hi = tf32(a) and lo = tf32(a - hi); the product uses hi*hi + hi*lo + lo*hi, dropping only the
// lo*lo term (relative 2^-22), so the result stays within the path's rel 1e-5*sqrt(K) tolerance.
//
// Kernels:
//   split_tf32_*            prepare operand planes in scratch memory.  An aligned operand is fed to the
//                           MMA as it lies (the MMA drops the low 13 mantissa bits, i.e. it sees
//                           hi = truncation) and only its lo plane is written, in the operand's own
//                           order: K-major ([rows, K_pad], K_pad a multiple of 32, zero padded) or, for
//                           row-contiguous operands on the pair kernel, MN-major ([K, rows]).  Other
//                           operands are re-laid into K-major hi and lo planes through shared memory.
//   gemm_tf32x3_kernel      persistent, one CTA per 128x256 output tile.  Warp 0 drives TMA (no
//                           multicast) into a 4-stage ring of {A_hi, A_lo, B_hi, B_lo} 64-byte-swizzled
//                           tiles, warp 1 issues 6 tcgen05.mma per stage into one of two 128x256 FP32
//                           accumulators in TMEM, warps 2-5 read the other back with tcgen05.ld and
//                           apply the epilogue.
//   gemm_tf32x3_pair_kernel the same pipeline on a cluster of two CTAs per 256x256 tile
//                           (tcgen05.mma.cta_group::2): each CTA stages half of B, which takes the
//                           shared-memory port off the critical path; reads K-major and MN-major
//                           operand tiles.  The default where M allows.
// Every wait on an mbarrier is bounded; on a timeout the kernel records an error word, releases
// its tensor memory and returns, and the host reports TRS_ERR_DEVICE_STATUS.
#include <cuda.h>

#include <mutex>

#include "common.h"
#include "gemm.h"

namespace trs {
namespace {

constexpr int BM = 128, BN = 256;
constexpr int BK = 16;                                // floats per pipeline stage along K: 8 / 16 / 32 -> 32- / 64- / 128-byte swizzled rows.
                                                      // Measured at 4096^3: 16 x 4 stages 256 TFLOP/s, 32 x 2 stages 223, 8 x 8 stages 155.
constexpr int STAGES = BK == 8 ? 8 : (BK == 16 ? 4 : 2);
constexpr int ROW_BYTES = BK * 4;
constexpr int A_TILE_BYTES = BM * ROW_BYTES;
constexpr int B_TILE_BYTES = BN * ROW_BYTES;
constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;   // 48 KiB (BK=16) or 96 KiB (BK=32)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;                        // two 128x256 FP32 accumulators
constexpr long long WAIT_CYCLES = 2000000000ll;        // bounded waits: about a second of SM clocks
constexpr int K_PAD = 32;                             // operand planes are padded along K to this many floats

// Written by the split kernels when an operand holds inf/NaN (the split cannot represent those): each
// tensor-core matmul call owns word (epoch % 8) and marks it with its epoch, so nothing has to be cleared.
__device__ unsigned int g_nonfinite_seen[8];

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Returns false when the wait ran out of iterations.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, long long limit_cycles) {
    const long long start = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - start > limit_cycles) return false;
    }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

// K-major operand tile whose rows are one swizzle span (128 or 64 bytes): 8-row groups are
// 8 * ROW_BYTES apart; layout type 2 = SWIZZLE_128B, 4 = SWIZZLE_64B.
template <int kRowBytes = ROW_BYTES>
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address
    d |= (uint64_t)((8 * kRowBytes) >> 4) << 32;       // stride between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version (sm_100)
    d |= (uint64_t)(kRowBytes == 128 ? 2 : (kRowBytes == 64 ? 4 : 6)) << 61;
    return d;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// kind::tf32, FP32 accumulate, A and B K-major, M=128, N=256.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p; }"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- two-CTA (cta_group::2) variants: the CTA pair of a cluster works on one 256x256 tile ----------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Cluster-window address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Load into this CTA's shared memory; the bytes are counted on `cluster_bar`, the leader CTA's barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// kind::tf32, FP32 accumulate, M=256 over the CTA pair (128 rows each), N=256; bit 15 / 16 set = A / B is MN-major.
constexpr uint32_t kInstrDescPair = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p; }"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// MN-major operand tile (the only form kind::tf32 takes for it: 128-byte rows swizzled in 32-byte chunks):
// 32 consecutive rows of the operand (128 bytes) per k, kRows k per group; groups of 32 rows lie kRows * 128
// bytes apart (leading byte offset), atoms of 4 k 512 bytes apart (stride byte offset).
template <int kRows>
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((kRows * 128) >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;                            // SWIZZLE_128B_BASE32B
    return d;
}
// Arrives on the barrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs issued so far retire.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}

__device__ __forceinline__ float ref_relu(float v) {
    return ((__float_as_uint(v) & 0x7fffffffu) == 0u) ? v : fmaxf(v, 0.0f);
}
__device__ __forceinline__ float ref_relu_vjp(float x, float g) {
    const unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    return (mag > 0x7f800000u || ((b >> 31) == 0u && mag != 0u)) ? g : 0.0f;
}

// lo part of the 3-product split for a value the MMA reads in place (hi = the value with its low 13 mantissa
// bits dropped): lo = tf32(v - hi).  Returns true for inf / NaN, which the split cannot represent (lo = 0).
__device__ __forceinline__ bool lo_of(float v, float& lo) {
    const uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7f800000u) == 0x7f800000u) { lo = 0.0f; return true; }
    const float rest = __fsub_rn(v, __uint_as_float(bits & 0xffffe000u));      // exact
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    lo = __uint_as_float(l);
    return false;
}

struct EpilogueArgs {
    float* c;
    const float* bias;
    const float* aux;
    float* preact;
    long long c_batch_stride, c_row_stride;
    int m, n, k_blocks, epilogue;
    int tiles_m, tiles_n, total_tiles;
    int whole_tiles;      // work items [0, whole_tiles) are complete tiles; each later tile is cut into `parts` items along K
    int total_items;
    int parts;            // K parts per tile of the last, partly filled round (1 = no cut)
    float* partials;      // [cut tile][part][tile rows][BN] partial sums of the cut tiles
    unsigned int* arrivals;  // [cut tile][row slab] zeroed counters: the last part to arrive adds the parts up and stores C
    int a_mn, b_mn;       // pair kernel: the operand's tiles are MN-major (unit stride along its rows) instead of K-major
    float* c_lo;          // optional: lo image of C (tf32(c - trunc_tf32(c))), laid out like C, for the matmul that reads C next
    unsigned int* c_flag; // with c_lo: set to 1 when an inf / NaN is stored
    unsigned int* error;  // word (mapped host memory) that receives the stage number when a bounded wait runs out
    long long wait_cycles;  // limit of every mbarrier wait, in SM clocks
};

// Tile order: bands of 16 tile rows, walked column by column, so that the ~148 tiles in flight at
// any time cover a roughly square 16 x 9 patch of C and share their A and B panels in L2.
template <int kGroup = 16>
__device__ __forceinline__ void decode_tile(int t, int tiles_m, int tiles_n, int& batch, int& tile_m, int& tile_n) {
    const int per_batch = tiles_m * tiles_n;
    batch = t / per_batch;
    const int rem = t - batch * per_batch;
    const int band = rem / (kGroup * tiles_n);
    const int first_m = band * kGroup;
    const int band_rows = min(kGroup, tiles_m - first_m);
    const int in_band = rem - band * kGroup * tiles_n;
    tile_n = in_band / band_rows;
    tile_m = first_m + (in_band - tile_n * band_rows);
}

// Work item -> tile and K-block range.  When the last round of tiles would leave SMs idle, its tiles are cut
// into `parts` items along K that run side by side.  Every item of a cut tile writes its partial sums to scratch;
// whichever arrives last adds the parts up in part order (so the result does not depend on who finishes when),
// applies the epilogue and stores C.  Nobody waits for anybody.
__device__ __forceinline__ void decode_item(int w, const EpilogueArgs& e, int& tile, int& kb_begin, int& kb_end, int& part) {
    if (w < e.whole_tiles) { tile = w; kb_begin = 0; kb_end = e.k_blocks; part = -1; return; }
    const int r = w - e.whole_tiles;
    const int cut = r / e.parts;
    part = r - cut * e.parts;
    tile = e.whole_tiles + cut;
    kb_begin = (int)(((long long)e.k_blocks * part) / e.parts);
    kb_end = (int)(((long long)e.k_blocks * (part + 1)) / e.parts);
}

// Fused epilogue and store of 32 consecutive columns of one output row.
__device__ __forceinline__ void finish_chunk(const EpilogueArgs& e, float (&v)[32], long long idx0, long long col0, bool vec_ok) {
    const bool full_cols = col0 + 32 <= e.n;
    if (e.epilogue == TRS_EPI_BIAS || e.epilogue == TRS_EPI_BIAS_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (full_cols || col0 + j < e.n) v[j] = __fadd_rn(v[j], __ldg(e.bias + col0 + j));
    }
    if (e.epilogue == TRS_EPI_BIAS_RELU && e.preact) {
        if (full_cols && vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(e.preact + idx0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
            for (int j = 0; j < 32; ++j) if (col0 + j < e.n) e.preact[idx0 + j] = v[j];
        }
    }
    if (e.epilogue == TRS_EPI_BIAS_RELU || e.epilogue == TRS_EPI_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = ref_relu(v[j]);
    }
    if (e.epilogue == TRS_EPI_RELU_VJP) {
        if (full_cols && vec_ok && ((reinterpret_cast<uintptr_t>(e.aux) & 15u) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 z = __ldcs(reinterpret_cast<const float4*>(e.aux + idx0 + j));
                v[j] = ref_relu_vjp(z.x, v[j]); v[j + 1] = ref_relu_vjp(z.y, v[j + 1]);
                v[j + 2] = ref_relu_vjp(z.z, v[j + 2]); v[j + 3] = ref_relu_vjp(z.w, v[j + 3]);
            }
        } else {
            for (int j = 0; j < 32; ++j) if (col0 + j < e.n) v[j] = ref_relu_vjp(e.aux[idx0 + j], v[j]);
        }
    }
    if (e.c_lo) {
        // lo image of the stored values, for the matmul that consumes C as an operand
        float l[32];
        bool nonfinite = false;
#pragma unroll
        for (int j = 0; j < 32; ++j) nonfinite |= lo_of(v[j], l[j]);
        if (full_cols && vec_ok && ((reinterpret_cast<uintptr_t>(e.c_lo) & 15u) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(e.c_lo + idx0 + j) = make_float4(l[j], l[j + 1], l[j + 2], l[j + 3]);
        } else {
            nonfinite = false;
            for (int j = 0; j < 32; ++j) if (col0 + j < e.n) { e.c_lo[idx0 + j] = l[j]; nonfinite |= (__float_as_uint(v[j]) & 0x7f800000u) == 0x7f800000u; }
        }
        if (nonfinite) *reinterpret_cast<volatile unsigned int*>(e.c_flag) = 1u;
    }
    if (full_cols && vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(e.c + idx0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
        for (int j = 0; j < 32; ++j) if (col0 + j < e.n) e.c[idx0 + j] = v[j];
    }
}

// Epilogue of one warp for one tile: reads its 32 accumulator rows (TMEM lanes) 32 columns at a time,
// hands the accumulator back as soon as the last columns are in registers, applies the fused
// epilogue and stores.  `tmem_acc` addresses the warp's lanes at the accumulator's first column;
// `empty_bar_addr` is the accumulator-empty barrier (a cluster address of the leader's barrier when kPair).
// For an item of a cut tile (`part` >= 0) the columns go to the partial-sum scratch instead; `slab` is this
// warp's 32-row slab of the tile (0 .. tile rows / 32 - 1) and `cut` the tile's index among the cut tiles.
template <bool kPair>
__device__ __forceinline__ void drain_accumulator(const EpilogueArgs& e, uint32_t tmem_acc, long long row, long long batch_off, int tile_n,
                                                  int part, int cut, int slab, bool vec_ok, int lane, uint32_t empty_bar_addr) {
    constexpr int kTileRows = kPair ? 2 * BM : BM;
    // partial sums of a slab: [32-column chunk][group of 4 columns][lane][4 floats], so that the 32 lanes of a warp
    // write (and the finishing warp reads) 512 consecutive bytes per instruction
    float* my_partial = nullptr;
    if (part >= 0) my_partial = e.partials + (((long long)cut * e.parts + part) * kTileRows + slab * 32) * BN + lane * 4;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_acc + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 == BN) {
            // every column of this accumulator has been read into registers: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) { if (kPair) mbar_arrive_cluster(empty_bar_addr); else mbar_arrive(empty_bar_addr); }
        }
        const long long col0 = (long long)tile_n * BN + c0;
        if (part >= 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) __stcg(reinterpret_cast<float4*>(my_partial + (c0 + j) * 32), make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])));
            continue;
        }
        if (row < e.m && col0 < e.n) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            finish_chunk(e, v, batch_off + row * e.c_row_stride + col0, col0, vec_ok);
        }
    }
    if (part < 0) return;
    // This slab's part is in scratch.  Count it; the last of the tile's parts to get here finishes the slab.
    __threadfence();
    __syncwarp();
    unsigned int earlier = 0;
    if (lane == 0) earlier = atomicAdd(e.arrivals + (long long)cut * (kTileRows / 32) + slab, 1u);
    earlier = __shfl_sync(0xffffffffu, earlier, 0);
    if (earlier != (unsigned int)(e.parts - 1)) return;
    __threadfence();
    const float* first = e.partials + (((long long)cut * e.parts) * kTileRows + slab * 32) * BN + lane * 4;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        const long long col0 = (long long)tile_n * BN + c0;
        if (!(row < e.m && col0 < e.n)) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(first + (c0 + j) * 32));
            v[j] = t.x; v[j + 1] = t.y; v[j + 2] = t.z; v[j + 3] = t.w;
        }
        for (int q = 1; q < e.parts; ++q) {                 // fixed order: part 0 + part 1 + ...
            const float* next = first + (long long)q * kTileRows * BN;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(next + (c0 + j) * 32));
                v[j] = __fadd_rn(v[j], t.x); v[j + 1] = __fadd_rn(v[j + 1], t.y); v[j + 2] = __fadd_rn(v[j + 2], t.z); v[j + 3] = __fadd_rn(v[j + 3], t.w);
            }
        }
        finish_chunk(e, v, batch_off + row * e.c_row_stride + col0, col0, vec_ok);
    }
}

// Persistent kernel: CTA i works on tiles i, i + gridDim.x, ...; the accumulator of tile j lives
// in TMEM columns (j & 1) * 256, so the epilogue of one tile overlaps the MMAs of the next.
__global__ void __launch_bounds__(192, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                   const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                   const EpilogueArgs e) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    // bars: [0,S) stage full, [S,2S) stage empty, [2S,2S+2) accumulator full, [2S+2,2S+4) accumulator empty
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                           // barriers and tensor memory are set up while the previous kernel drains

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            bool failed = false;
            uint32_t g = 0;                                           // stage uses so far, over all tiles
            for (int w = blockIdx.x; w < e.total_items && !failed; w += gridDim.x) {
                int t, kb_begin, kb_end, batch, tile_m, tile_n;
                int part;
                decode_item(w, e, t, kb_begin, kb_end, part);
                decode_tile(t, e.tiles_m, e.tiles_n, batch, tile_m, tile_n);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % STAGES, round = g / STAGES;
                    if (round > 0 && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, e.wait_cycles)) { failed = true; break; }
                    const uint32_t full = smem_u32(&full_bar[s]);
                    const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_3d(base, &map_a_hi, full, kb * BK, tile_m * BM, batch);
                    tma_load_3d(base + A_TILE_BYTES, &map_a_lo, full, kb * BK, tile_m * BM, batch);
                    tma_load_3d(base + 2 * A_TILE_BYTES, &map_b_hi, full, kb * BK, tile_n * BN, batch);
                    tma_load_3d(base + 2 * A_TILE_BYTES + B_TILE_BYTES, &map_b_lo, full, kb * BK, tile_n * BN, batch);
                }
            }
            if (failed) atomicExch_system(e.error, 1u);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            bool failed = false;
            uint32_t g = 0, it = 0;
            for (int w = blockIdx.x; w < e.total_items && !failed; w += gridDim.x, ++it) {
                int t, kb_begin, kb_end;
                int part;
                decode_item(w, e, t, kb_begin, kb_end, part);
                const uint32_t acc = it & 1, use = it >> 1;
                // the epilogue must have drained this accumulator's previous tile
                if (use > 0 && !mbar_wait(smem_u32(&acc_empty[acc]), (use - 1) & 1, e.wait_cycles)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + acc * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % STAGES;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (g / STAGES) & 1, e.wait_cycles)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t a_hi = smem_desc(base), a_lo = smem_desc(base + A_TILE_BYTES);
                    const uint64_t b_hi = smem_desc(base + 2 * A_TILE_BYTES), b_lo = smem_desc(base + 2 * A_TILE_BYTES + B_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 8; ++k) {
                        const uint64_t step = (uint64_t)((k * 8 * 4) >> 4);      // 32 bytes per UMMA K step
                        // small terms first, the dominant hi*hi product last
                        umma_tf32(d, a_lo + step, b_hi + step, (kb != kb_begin) || (k != 0));
                        umma_tf32(d, a_hi + step, b_lo + step, 1u);
                        umma_tf32(d, a_hi + step, b_hi + step, 1u);
                    }
                    umma_commit(smem_u32(&empty_bar[s]));                         // stage reusable once these MMAs retire
                }
                umma_commit(smem_u32(&acc_full[acc]));                            // accumulator complete (or abandoned)
            }
            if (failed) atomicExch_system(e.error, 2u);
        }
    } else {
        // ---- epilogue warps 2..5: TMEM lanes 32*(warp%4) .. +31 ----
        const int quarter = warp & 3;
        const bool vec_ok = (e.c_row_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(e.c) & 15u) == 0) && (e.c_batch_stride % 4 == 0) &&
                            (!e.preact || (reinterpret_cast<uintptr_t>(e.preact) & 15u) == 0);
        uint32_t it = 0;
        bool failed = false;
        for (int w = blockIdx.x; w < e.total_items && !failed; w += gridDim.x, ++it) {
            int t, kb_begin, kb_end, batch, tile_m, tile_n;
            int part;
            decode_item(w, e, t, kb_begin, kb_end, part);
            decode_tile(t, e.tiles_m, e.tiles_n, batch, tile_m, tile_n);
            const uint32_t acc = it & 1, use = it >> 1;
            if (!mbar_wait(smem_u32(&acc_full[acc]), use & 1, e.wait_cycles)) {
                if (lane == 0) atomicExch_system(e.error, 3u);
                failed = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const long long row = (long long)tile_m * BM + quarter * 32 + lane;
            const long long batch_off = (long long)batch * e.c_batch_stride;
            drain_accumulator<false>(e, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, row, batch_off, tile_n, part,
                                     (t - e.whole_tiles), quarter, vec_ok, lane, smem_u32(&acc_empty[acc]));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


// ---- two-CTA kernel --------------------------------------------------------------------------------
// A cluster of two CTAs (neighbouring SMs) owns one 256x256 tile: CTA r stages its own 128 rows of
// A and rows [128 r, 128 r + 128) of the B^T tile, so every byte of B is staged once per pair
// instead of once per CTA, and each SM's shared memory serves 8 KiB per MMA instead of 12 KiB (the
// one-CTA kernel is bound by exactly that port).  The leader (rank 0) issues every MMA
// (tcgen05.mma.cta_group::2, M=256); each CTA's tensor core accumulates its own 128 rows in its own
// TMEM, and each CTA's epilogue warps drain and store them.
//   stage full   (leader only)  one arrive.expect_tx by the leader's producer for the bytes of both CTAs
//   stage empty  (each CTA)     one multicast tcgen05.commit by the leader's MMA thread
//   acc full     (each CTA)     one multicast tcgen05.commit by the leader's MMA thread
//   acc empty    (leader only)  eight arrivals: the four epilogue warps of both CTAs
// Measured (TFLOP/s at 4096^3 / 8192^3 / 64 x 1024^3 with bias+relu): 32 floats x 3 stages 277 / 339 / 220,
// 16 x 6 stages 277 / 336 / 210, 16 x 4 stages 267 / 330 / 203; the one-CTA kernel reaches 259 / 320 / 191.
constexpr int PAIR_BK = 32;                                                       // 128-byte swizzled rows
constexpr int PAIR_STAGES = 3;
constexpr int PAIR_ROW_BYTES = PAIR_BK * 4;
constexpr int PAIR_A_TILE_BYTES = BM * PAIR_ROW_BYTES;
constexpr int PAIR_B_TILE_BYTES = (BN / 2) * PAIR_ROW_BYTES;
constexpr int PAIR_STAGE_BYTES = 2 * PAIR_A_TILE_BYTES + 2 * PAIR_B_TILE_BYTES;  // 64 KiB per CTA
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;
constexpr int PAIR_GROUP_M = 8;                                                   // bands of 8 x 256 rows
constexpr bool kMnMajorOperands = true;                                           // read row-contiguous operands MN-major ...
constexpr long long kMnMajorMaxReuse = 4096;                                      // ... when each element is used at most this often

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                        const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                        const EpilogueArgs e) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + PAIR_STAGES;
    uint64_t* acc_full = bars + 2 * PAIR_STAGES;
    uint64_t* acc_empty = bars + 2 * PAIR_STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PAIR_STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();             // 0: leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                   // the peer's barriers are initialised before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                           // barriers and tensor memory are set up while the previous kernel drains

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer (both CTAs) ----
            bool failed = false;
            uint32_t g = 0;
            for (int w = pair; w < e.total_items && !failed; w += pairs) {
                int t, kb_begin, kb_end, batch, tile_m, tile_n;
                int part;
                decode_item(w, e, t, kb_begin, kb_end, part);
                decode_tile<PAIR_GROUP_M>(t, e.tiles_m, e.tiles_n, batch, tile_m, tile_n);
                const int a_row = tile_m * (2 * BM) + (int)rank * BM;
                const int b_row = tile_n * BN + (int)rank * (BN / 2);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % PAIR_STAGES, round = g / PAIR_STAGES;
                    if (round > 0 && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, e.wait_cycles)) { failed = true; break; }
                    const uint32_t full = map_to_cta(smem_u32(&full_bar[s]), 0);
                    const uint32_t base = smem_u32(smem + s * PAIR_STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * PAIR_STAGE_BYTES);
                    if (e.a_mn) {
                        tma_load_4d_pair(base, &map_a_hi, full, 0, kb * PAIR_BK, a_row >> 5, batch);
                        tma_load_4d_pair(base + PAIR_A_TILE_BYTES, &map_a_lo, full, 0, kb * PAIR_BK, a_row >> 5, batch);
                    } else {
                        tma_load_3d_pair(base, &map_a_hi, full, kb * PAIR_BK, a_row, batch);
                        tma_load_3d_pair(base + PAIR_A_TILE_BYTES, &map_a_lo, full, kb * PAIR_BK, a_row, batch);
                    }
                    if (e.b_mn) {
                        tma_load_4d_pair(base + 2 * PAIR_A_TILE_BYTES, &map_b_hi, full, 0, kb * PAIR_BK, b_row >> 5, batch);
                        tma_load_4d_pair(base + 2 * PAIR_A_TILE_BYTES + PAIR_B_TILE_BYTES, &map_b_lo, full, 0, kb * PAIR_BK, b_row >> 5, batch);
                    } else {
                        tma_load_3d_pair(base + 2 * PAIR_A_TILE_BYTES, &map_b_hi, full, kb * PAIR_BK, b_row, batch);
                        tma_load_3d_pair(base + 2 * PAIR_A_TILE_BYTES + PAIR_B_TILE_BYTES, &map_b_lo, full, kb * PAIR_BK, b_row, batch);
                    }
                }
            }
            // stay until the leader's last commits have arrived on this CTA's barriers
            const uint32_t last = g < (uint32_t)PAIR_STAGES ? g : (uint32_t)PAIR_STAGES;
            for (uint32_t u = g - last; u < g && !failed; ++u)
                if (!mbar_wait(smem_u32(&empty_bar[u % PAIR_STAGES]), (u / PAIR_STAGES) & 1, e.wait_cycles)) failed = true;
            if (failed) atomicExch_system(e.error, 4u);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (leader CTA only) ----
            bool failed = false;
            uint32_t g = 0, it = 0;
            const uint32_t idesc = kInstrDescPair | (e.a_mn ? (1u << 15) : 0u) | (e.b_mn ? (1u << 16) : 0u);
            for (int w = pair; w < e.total_items && !failed; w += pairs, ++it) {
                int t, kb_begin, kb_end;
                int part;
                decode_item(w, e, t, kb_begin, kb_end, part);
                const uint32_t acc = it & 1, use = it >> 1;
                if (use > 0 && !mbar_wait(smem_u32(&acc_empty[acc]), (use - 1) & 1, e.wait_cycles)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + acc * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % PAIR_STAGES;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (g / PAIR_STAGES) & 1, e.wait_cycles)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t base = smem_u32(smem + s * PAIR_STAGE_BYTES);
                    const uint32_t a0 = base, a1 = base + PAIR_A_TILE_BYTES, b0 = base + 2 * PAIR_A_TILE_BYTES, b1 = b0 + PAIR_B_TILE_BYTES;
                    const uint64_t a_hi = e.a_mn ? smem_desc_mn<PAIR_BK>(a0) : smem_desc<PAIR_ROW_BYTES>(a0);
                    const uint64_t a_lo = e.a_mn ? smem_desc_mn<PAIR_BK>(a1) : smem_desc<PAIR_ROW_BYTES>(a1);
                    const uint64_t b_hi = e.b_mn ? smem_desc_mn<PAIR_BK>(b0) : smem_desc<PAIR_ROW_BYTES>(b0);
                    const uint64_t b_lo = e.b_mn ? smem_desc_mn<PAIR_BK>(b1) : smem_desc<PAIR_ROW_BYTES>(b1);
                    // 8 k per MMA: 32 bytes along a K-major row, or one 8-k-row atom (1024 bytes) of an MN-major tile
                    const uint64_t a_step = e.a_mn ? (1024 >> 4) : (32 >> 4), b_step = e.b_mn ? (1024 >> 4) : (32 >> 4);
#pragma unroll
                    for (int k = 0; k < PAIR_BK / 8; ++k) {
                        const uint64_t sa = a_step * k, sb = b_step * k;
                        umma_tf32_pair(d, a_lo + sa, b_hi + sb, idesc, (kb != kb_begin) || (k != 0));
                        umma_tf32_pair(d, a_hi + sa, b_lo + sb, idesc, 1u);
                        umma_tf32_pair(d, a_hi + sa, b_hi + sb, idesc, 1u);
                    }
                    umma_commit_pair(smem_u32(&empty_bar[s]), 3);
                }
                umma_commit_pair(smem_u32(&acc_full[acc]), 3);
            }
            // stay until the peer's epilogue has made its last arrivals on this CTA's barriers
            const uint32_t last = it < 2u ? it : 2u;
            for (uint32_t j = it - last; j < it && !failed; ++j)
                if (!mbar_wait(smem_u32(&acc_empty[j & 1]), (j >> 1) & 1, e.wait_cycles)) failed = true;
            if (failed) atomicExch_system(e.error, 5u);
        }
    } else {
        // ---- epilogue warps 2..5 of both CTAs: this CTA's 128 rows of the tile ----
        const int quarter = warp & 3;
        const bool vec_ok = (e.c_row_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(e.c) & 15u) == 0) && (e.c_batch_stride % 4 == 0) &&
                            (!e.preact || (reinterpret_cast<uintptr_t>(e.preact) & 15u) == 0);
        uint32_t it = 0;
        for (int w = pair; w < e.total_items; w += pairs, ++it) {
            int t, kb_begin, kb_end, batch, tile_m, tile_n;
            int part;
            decode_item(w, e, t, kb_begin, kb_end, part);
            decode_tile<PAIR_GROUP_M>(t, e.tiles_m, e.tiles_n, batch, tile_m, tile_n);
            const uint32_t acc = it & 1, use = it >> 1;
            if (!mbar_wait(smem_u32(&acc_full[acc]), use & 1, e.wait_cycles)) {
                if (lane == 0) atomicExch_system(e.error, 6u);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const long long row = (long long)tile_m * (2 * BM) + (long long)rank * BM + quarter * 32 + lane;
            const long long batch_off = (long long)batch * e.c_batch_stride;
            drain_accumulator<true>(e, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, row, batch_off, tile_n, part,
                                    (t - e.whole_tiles), (int)rank * 4 + quarter, vec_ok, lane, map_to_cta(smem_u32(&acc_empty[acc]), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                   // neither CTA frees tensor memory or exits while the other may still signal it
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


// ---- operand preparation: strided f32 -> K-major hi / lo planes -------------------------------------

struct SplitArgs {
    const float* src;
    float* hi;
    float* lo;
    long long batch_stride, row_stride, k_stride;     // source strides in elements
    long long rows, k, k_pad;
    unsigned int* nonfinite;
    int lo_only;          // the source itself serves as the hi operand (the MMA drops the low 13 bits): hi = truncation
    unsigned int epoch;   // value stored to *nonfinite when an inf / NaN is met
};

__device__ __forceinline__ void split_value(float a, float& hi, float& lo, unsigned int* nonfinite, unsigned int epoch, bool truncate_hi = false) {
    const uint32_t bits = __float_as_uint(a);
    if ((bits & 0x7f800000u) == 0x7f800000u) {         // inf / NaN: not representable by the split
        *reinterpret_cast<volatile unsigned int*>(nonfinite) = epoch;
        hi = a; lo = 0.0f;
        return;
    }
    uint32_t h;
    if (truncate_hi) {
        h = bits & 0xffffe000u;
    } else {
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(a));
        if ((h & 0x7f800000u) == 0x7f800000u) h = bits & 0xffffe000u;   // rounding overflowed: truncate instead
    }
    hi = __uint_as_float(h);
    const float rest = __fsub_rn(a, hi);                // exact
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    lo = __uint_as_float(l);
}

// Source unit-stride along k: each thread converts 4 consecutive k of one row.
__global__ void __launch_bounds__(256) split_tf32_kfast_kernel(const SplitArgs a, int vec) {
    pdl_wait();
    const long long quads = a.k_pad >> 2;
    const long long total = a.rows * quads;
    const long long batch = blockIdx.y;
    const float* src = a.src + batch * a.batch_stride;
    float* hi = a.hi + batch * a.rows * a.k_pad;
    float* lo = a.lo + batch * a.rows * a.k_pad;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / quads, k0 = (i - r * quads) << 2;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const float* p = src + r * a.row_stride + k0;
        if (vec && k0 + 4 <= a.k) {
            const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) if (k0 + e < a.k) v[e] = __ldg(p + e);
        }
        float h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_value(v[e], h[e], l[e], a.nonfinite, a.epoch, a.lo_only != 0);
        if (!a.lo_only) *reinterpret_cast<float4*>(hi + r * a.k_pad + k0) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(lo + r * a.k_pad + k0) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// Any other source layout (unit stride along rows, or fully strided): 32x32 tiles through shared
// memory, read along the rows axis, written along k.
__global__ void __launch_bounds__(256) split_tf32_tiled_kernel(const SplitArgs a) {
    pdl_wait();
    __shared__ float tile[32][33];
    const long long batch = blockIdx.z;
    const float* src = a.src + batch * a.batch_stride;
    float* hi = a.hi + batch * a.rows * a.k_pad;
    float* lo = a.lo + batch * a.rows * a.k_pad;
    const long long r0 = (long long)blockIdx.x * 32, k0 = (long long)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const long long k = k0 + ty + 8 * j, r = r0 + tx;
        tile[ty + 8 * j][tx] = (k < a.k && r < a.rows) ? __ldg(src + r * a.row_stride + k * a.k_stride) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const long long r = r0 + ty + 8 * j, k = k0 + tx;
        if (r < a.rows && k < a.k_pad) {
            float h, l;
            split_value(tile[tx][ty + 8 * j], h, l, a.nonfinite, a.epoch);
            hi[r * a.k_pad + k] = h;
            lo[r * a.k_pad + k] = l;
        }
    }
}

// Source unit-stride along rows (a transposed view) and 16-byte aligned: 64x64 tiles, float4 reads
// along rows, float4 hi/lo writes along k.
__global__ void __launch_bounds__(256) split_tf32_tiled64_kernel(const SplitArgs a) {
    pdl_wait();
    __shared__ float tile[64][65];                       // [k][row]
    const long long batch = blockIdx.z;
    const float* src = a.src + batch * a.batch_stride;
    float* hi = a.hi + batch * a.rows * a.k_pad;
    float* lo = a.lo + batch * a.rows * a.k_pad;
    const long long r0 = (long long)blockIdx.x * 64, k0 = (long long)blockIdx.y * 64;
    const int q4 = (threadIdx.x & 15) * 4, r16 = threadIdx.x >> 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int kl = r16 + 16 * j;
        const long long k = k0 + kl, r = r0 + q4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < a.k && r < a.rows) v = __ldcs(reinterpret_cast<const float4*>(src + k * a.k_stride + r));
        tile[kl][q4] = v.x; tile[kl][q4 + 1] = v.y; tile[kl][q4 + 2] = v.z; tile[kl][q4 + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int rl = r16 + 16 * j;
        const long long r = r0 + rl, k = k0 + q4;
        if (r < a.rows && k < a.k_pad) {
            float h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_value(tile[q4 + e][rl], h[e], l[e], a.nonfinite, a.epoch);
            *reinterpret_cast<float4*>(hi + r * a.k_pad + k) = make_float4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<float4*>(lo + r * a.k_pad + k) = make_float4(l[0], l[1], l[2], l[3]);
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int32_t make_operand_map(CUtensorMap* map, const float* base, long long rows, long long k_extent, long long batch,
                         long long row_stride, long long batch_stride, int box_rows, int bk) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return fail(TRS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)k_extent, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 4, (cuuint64_t)batch_stride * 4};
    void* plane = const_cast<float*>(base);
    cuuint32_t box[3] = {(cuuint32_t)bk, (cuuint32_t)box_rows, 1};             // rows of bk floats: one swizzle span
    const CUtensorMapSwizzle swizzle = bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, plane, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TRS_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return TRS_OK;
}

// Map over an operand whose rows are unit-stride in memory ([k, rows] with `pitch` elements between k):
// dims {32 rows, k, rows / 32, batch}, so that one box lands as groups of 32 rows x bk k x 128 bytes, swizzled in
// 32-byte chunks -- the MN-major tile form of smem_desc_mn.  `rows` must be a multiple of 32.
int32_t make_mn_operand_map(CUtensorMap* map, const float* base, long long rows, long long k_extent, long long batch,
                            long long pitch, long long batch_stride, int box_rows, int bk) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return fail(TRS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {32, (cuuint64_t)k_extent, (cuuint64_t)(rows / 32), (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)pitch * 4, 128, (cuuint64_t)batch_stride * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)bk, (cuuint32_t)(box_rows / 32), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TRS_ERR_CUDA, "cuTensorMapEncodeTiled (MN-major) failed with code %d", (int)r);
    return TRS_OK;
}

// Whether the pair kernel can read the operand MN-major as it lies: unit stride along its rows, rows a multiple
// of 32 (a box never straddles the end of a k line), 16-byte aligned lines.
bool mn_major_ok(const float* src, long long batch, long long rows, long long batch_stride, long long row_stride, long long k_stride, long long k) {
    if (row_stride != 1 || rows % 32 != 0 || (reinterpret_cast<uintptr_t>(src) & 15u) != 0 || k_stride % 4 != 0 || k_stride < rows) return false;
    if (batch > 1 && (batch_stride % 4 != 0 || batch_stride < k * k_stride)) return false;
    return k >= 1;
}

struct DeviceWords {
    unsigned int* error = nullptr;       // device-side address of host_error
    unsigned int* host_error = nullptr;  // page-locked, mapped: kernels write it, the host reads it without a copy
    unsigned int* nonfinite = nullptr;
    bool smem_set = false;
    unsigned int epoch = 0;     // tag of the latest tensor-core matmul call on this device
    int pair_clusters = 0;      // CTA pairs of the two-CTA kernel that can be resident at once
};
DeviceWords g_words[16];
std::mutex g_words_mu;

int32_t device_words(int device, DeviceWords** out, unsigned int* epoch) {
    std::lock_guard<std::mutex> lock(g_words_mu);
    DeviceWords& w = g_words[device];
    if (++w.epoch == 0) ++w.epoch;                       // 0 is the words' initial value: never a tag
    *epoch = w.epoch;
    if (!w.error) {
        unsigned int* host = nullptr;
        TRS_CUDA(cudaHostAlloc((void**)&host, sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable));
        *host = 0;
        unsigned int* dev = nullptr;
        if (cudaHostGetDevicePointer((void**)&dev, host, 0) != cudaSuccess) { cudaGetLastError(); cudaFreeHost(host); return fail(TRS_ERR_CUDA, "cannot map the status word"); }
        TRS_CUDA(cudaGetSymbolAddress((void**)&w.nonfinite, g_nonfinite_seen));
        w.host_error = host;
        w.error = dev;
    }
    if (!w.smem_set) {
        TRS_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        TRS_CUDA(cudaFuncSetAttribute(gemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
        // The preparation kernels use no shared memory, but their blocks share SMs with the blocks of the GEMM that
        // follows (programmatic dependent launch): ask for the same (largest) shared-memory configuration, or the SM
        // would have to drain to switch.  Measured: 2048^3 0.093 -> 0.082 ms.
        TRS_CUDA(cudaFuncSetAttribute(split_tf32_kfast_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        TRS_CUDA(cudaFuncSetAttribute(split_tf32_tiled64_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        TRS_CUDA(cudaFuncSetAttribute(split_tf32_tiled_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        const int sms = sm_count(device);
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sms / 2 * 2)); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tf32x3_pair_kernel, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            clusters = sms / 2;
        }
        w.pair_clusters = std::min(clusters, sms / 2);
        w.smem_set = true;
    }
    *out = &w;
    return TRS_OK;
}

int32_t make_plane_map(CUtensorMap* map, float* plane, long long rows, long long k_pad, long long batch, int box_rows, int bk) {
    return make_operand_map(map, plane, rows, k_pad, batch, k_pad, rows * k_pad, box_rows, bk);
}

// Whether the MMA can read the hi operand straight from the source (K-major, 16-byte aligned
// rows).  kind::tf32 ignores the low 13 mantissa bits of its FP32 operands, i.e. it sees
// hi = truncation(a); the lo plane is then tf32(a - truncation(a)) and no hi plane is written.
// (Checked on B200 with operands whose low 13 bits are all ones: results stay within 4e-6*sqrt(K)*rms
// of a float64 product, which a rounding MMA would miss by orders of magnitude.)
bool raw_hi_ok(const float* src, long long batch, long long rows, long long batch_stride, long long row_stride, long long k_stride, long long k) {
    if (k_stride != 1 || (reinterpret_cast<uintptr_t>(src) & 15u) != 0 || row_stride % 4 != 0 || row_stride < k) return false;
    if (batch > 1 && (batch_stride % 4 != 0 || batch_stride < rows * row_stride)) return false;
    return true;
}

int32_t launch_split(const float* src, long long batch, long long rows, long long k, long long k_pad, long long batch_stride,
                     long long row_stride, long long k_stride, float* hi, float* lo, unsigned int* nonfinite, unsigned int epoch,
                     trs_stream stream, int lo_only = 0) {
    SplitArgs a{src, hi, lo, batch_stride, row_stride, k_stride, rows, k, k_pad, nonfinite, lo_only, epoch};
    if (k_stride == 1 || k == 1) {
        const int vec = (row_stride % 4 == 0) && (batch_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0);
        const long long total = rows * (k_pad >> 2);
        unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, (long long)sm_count(stream->device) * 32);
        TRS_CUDA(launch_dependent(split_tf32_kfast_kernel, dim3(std::max(grid, 1u), (unsigned)batch), dim3(256), 0, stream->stream, a, vec));
    } else if (row_stride == 1 && rows % 4 == 0 && k_stride % 4 == 0 && batch_stride % 4 == 0 &&
               (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        dim3 grid((unsigned)((rows + 63) / 64), (unsigned)((k_pad + 63) / 64), (unsigned)batch);
        if (grid.y > 65535) return fail(TRS_ERR_UNSUPPORTED, "inner dimension too large for the operand split");
        TRS_CUDA(launch_dependent(split_tf32_tiled64_kernel, grid, dim3(256), 0, stream->stream, a));
    } else {
        dim3 grid((unsigned)((rows + 31) / 32), (unsigned)(k_pad / 32), (unsigned)batch);   // k_pad is a multiple of 32
        TRS_CUDA(launch_dependent(split_tf32_tiled_kernel, grid, dim3(256), 0, stream->stream, a));
    }
    TRS_CUDA(cudaGetLastError());
    count_launch();
    return TRS_OK;
}

// Whether AUTO takes the two-CTA kernel: it pays in 256-row tiles, so it wants at most one eighth
// of the rows it computes to be padding.
constexpr bool kPairDefault = true;

}  // namespace

bool gemm_tc_pair_preferred(const trs_gemm_desc& g) {
    if (!kPairDefault) return false;
    const long long padded = (g.m + 2 * BM - 1) / (2 * BM) * (2 * BM);
    const long long single = (g.m + BM - 1) / BM * BM;
    return padded * 8 <= single * 9;
}

bool gemm_tc_eligible(const trs_gemm_desc& g) {
    if (g.batch < 1 || g.batch > 65535 || g.k < 32 || g.m < 1 || g.n < 1) return false;
    if ((g.m + BM - 1) / BM > 65535) return false;
    // Small problems stay on the exact-FP32 SIMT kernel: the split's two extra passes do not pay off.
    return (double)g.m * (double)g.n * (double)g.k >= (double)(1 << 21);
}

namespace {

// How one operand reaches the MMA.
struct OperandRoute {
    bool raw = false;      // K-major, read in place as hi; only a lo image is needed
    bool mn = false;       // row-contiguous, read in place MN-major (pair kernel); only a lo image is needed
    bool given = false;    // the caller's lo image is used (raw or mn only)
    long long floats = 0;  // scratch this operand needs
};

// Whether a caller's lo image can stand beside the operand: same 16-byte phase as the operand itself.
bool lo_image_ok(const float* operand, const float* lo) {
    return lo != nullptr && ((reinterpret_cast<uintptr_t>(lo) & 15u) == (reinterpret_cast<uintptr_t>(operand) & 15u));
}

void route_operands(const trs_gemm_desc& g, const trs_gemm_planes* p, OperandRoute* ra, OperandRoute* rb) {
    const bool pair = g.algo == TRS_GEMM_TCGEN05_3XTF32_2CTA;
    const long long k_pad = (g.k + K_PAD - 1) / K_PAD * K_PAD;
    ra->raw = raw_hi_ok(g.a, g.batch, g.m, g.a_batch_stride, g.a_row_stride, g.a_col_stride, g.k);
    rb->raw = raw_hi_ok(g.b, g.batch, g.n, g.b_batch_stride, g.b_col_stride, g.b_row_stride, g.k);
    // An operand that is unit-stride along its rows (a transposed view, or the right operand of a plain A @ B) is
    // read MN-major as it lies by the pair kernel; only its lo image, in the same order, is needed.
    // Measured: the MMA reads an MN-major tile 1-3 % slower than a K-major one, while re-laying an operand costs
    // 4 more bytes of HBM traffic per element; the operand's reuse (the other output extent) decides which is cheaper.
    ra->mn = pair && kMnMajorOperands && !ra->raw && g.n <= kMnMajorMaxReuse &&
             mn_major_ok(g.a, g.batch, g.m, g.a_batch_stride, g.a_row_stride, g.a_col_stride, g.k);
    rb->mn = pair && kMnMajorOperands && !rb->raw && g.m <= kMnMajorMaxReuse &&
             mn_major_ok(g.b, g.batch, g.n, g.b_batch_stride, g.b_col_stride, g.b_row_stride, g.k);
    ra->given = (ra->raw || ra->mn) && p && lo_image_ok(g.a, p->a_lo);
    rb->given = (rb->raw || rb->mn) && p && lo_image_ok(g.b, p->b_lo);
    ra->floats = ra->given ? 0 : (ra->mn ? g.batch * g.k * g.m : (ra->raw ? 1 : 2) * g.batch * g.m * k_pad);
    rb->floats = rb->given ? 0 : (rb->mn ? g.batch * g.k * g.n : (rb->raw ? 1 : 2) * g.batch * g.n * k_pad);
}

// Elementwise lo image of a contiguous range (the form a host keeps beside a storage).
__global__ void __launch_bounds__(256) split_lo_kernel(const float* __restrict__ src, float* __restrict__ lo, long long count,
                                                       unsigned int* flag, int vec) {
    bool nonfinite = false;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (vec) {
        const long long quads = count >> 2;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += stride) {
            const float4 t = __ldcs(reinterpret_cast<const float4*>(src) + i);
            float4 l;
            nonfinite |= lo_of(t.x, l.x); nonfinite |= lo_of(t.y, l.y); nonfinite |= lo_of(t.z, l.z); nonfinite |= lo_of(t.w, l.w);
            reinterpret_cast<float4*>(lo)[i] = l;
        }
        for (long long i = (quads << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) nonfinite |= lo_of(src[i], lo[i]);
    } else {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) nonfinite |= lo_of(__ldg(src + i), lo[i]);
    }
    if (nonfinite) *reinterpret_cast<volatile unsigned int*>(flag) = 1u;
}

// Test aid for the bounded waits: waits, with the given limit, on a barrier that nothing ever arrives on, and
// reports the timeout through the same error word and host check as the GEMM kernels.  It returns by itself.
__global__ void wait_probe_kernel(unsigned int* error, long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(smem_u32(&bar), 0, limit_cycles)) atomicExch_system(error, 7u);
    }
}

}  // namespace

int32_t gemm_tc_plan(const trs_gemm_desc& g, bool* a_image, bool* b_image) {
    OperandRoute ra, rb;
    route_operands(g, nullptr, &ra, &rb);
    *a_image = ra.raw || ra.mn;
    *b_image = rb.raw || rb.mn;
    return TRS_OK;
}

int32_t gemm_split_lo(const float* src, long long count, float* lo, unsigned int* flag, trs_stream stream) {
    TRS_CUDA(cudaMemsetAsync(flag, 0, sizeof(unsigned int), stream->stream));
    if (count <= 0) return TRS_OK;
    const int vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(lo)) & 15u) == 0;
    const long long items = vec ? (count + 3) / 4 : count;
    const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((items + 255) / 256, (long long)sm_count(stream->device) * 16));
    split_lo_kernel<<<grid, 256, 0, stream->stream>>>(src, lo, count, flag, vec);
    TRS_CUDA(cudaGetLastError());
    count_launch();
    return TRS_OK;
}

namespace {
struct ScratchGuard {       // handed back when the call returns: reuse is ordered behind this stream's work
    trs_stream s;
    void* p;
    ~ScratchGuard() { if (p) free_on_stream(s, p); }
};
}  // namespace

// Split (where no image was given) + GEMM + the gated exact-FP32 recompute.
int32_t gemm_tc_launch(const trs_gemm_desc& g, const trs_gemm_planes* planes, trs_stream stream) {
    if (g.m > INT32_MAX || g.n > INT32_MAX) return fail(TRS_ERR_UNSUPPORTED, "matrix extent above 2^31");
    if (planes && planes->c_lo && !planes->c_flag) return fail(TRS_ERR_INVALID_ARGUMENT, "c_lo needs c_flag");
    DeviceWords* words = nullptr;
    unsigned int epoch = 0;
    TRS_TRY(device_words(stream->device, &words, &epoch));
    unsigned int* nonfinite = words->nonfinite + (epoch & 7u);
    const long long k_pad = (g.k + K_PAD - 1) / K_PAD * K_PAD;
    const bool pair = g.algo == TRS_GEMM_TCGEN05_3XTF32_2CTA;
    const int b_box = pair ? BN / 2 : BN;                // B^T rows one CTA stages
    const int bk = pair ? PAIR_BK : BK;                  // floats along K per pipeline stage
    OperandRoute ra, rb;
    route_operands(g, planes, &ra, &rb);
    // A[b, m, k]: rows = m.  B[b, k, n] is consumed as B^T[b, n, k]: rows = n, so its "row stride" is the column stride.
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    const long long a_bs = g.batch > 1 ? g.a_batch_stride : 0, b_bs = g.batch > 1 ? g.b_batch_stride : 0;
    if (ra.raw && make_operand_map(&ma_hi, g.a, g.m, g.k, g.batch, g.a_row_stride, a_bs ? a_bs : g.m * g.a_row_stride, BM, bk) != TRS_OK) ra.raw = ra.given = false;
    if (rb.raw && make_operand_map(&mb_hi, g.b, g.n, g.k, g.batch, g.b_col_stride, b_bs ? b_bs : g.n * g.b_col_stride, b_box, bk) != TRS_OK) rb.raw = rb.given = false;
    if (ra.mn && make_mn_operand_map(&ma_hi, g.a, g.m, g.k, g.batch, g.a_col_stride, a_bs ? a_bs : g.k * g.a_col_stride, BM, bk) != TRS_OK) ra.mn = ra.given = false;
    if (rb.mn && make_mn_operand_map(&mb_hi, g.b, g.n, g.k, g.batch, g.b_row_stride, b_bs ? b_bs : g.k * g.b_row_stride, b_box, bk) != TRS_OK) rb.mn = rb.given = false;
    // The caller's lo image has the operand's own strides: the same map geometry over the other base.
    if (ra.given && (ra.raw ? make_operand_map(&ma_lo, planes->a_lo, g.m, g.k, g.batch, g.a_row_stride, a_bs ? a_bs : g.m * g.a_row_stride, BM, bk)
                            : make_mn_operand_map(&ma_lo, planes->a_lo, g.m, g.k, g.batch, g.a_col_stride, a_bs ? a_bs : g.k * g.a_col_stride, BM, bk)) != TRS_OK) ra.given = false;
    if (rb.given && (rb.raw ? make_operand_map(&mb_lo, planes->b_lo, g.n, g.k, g.batch, g.b_col_stride, b_bs ? b_bs : g.n * g.b_col_stride, b_box, bk)
                            : make_mn_operand_map(&mb_lo, planes->b_lo, g.n, g.k, g.batch, g.b_row_stride, b_bs ? b_bs : g.k * g.b_row_stride, b_box, bk)) != TRS_OK) rb.given = false;
    const long long a_floats = ra.given ? 0 : (ra.mn ? g.batch * g.k * g.m : (ra.raw ? 1 : 2) * g.batch * g.m * k_pad);
    const long long b_floats = rb.given ? 0 : (rb.mn ? g.batch * g.k * g.n : (rb.raw ? 1 : 2) * g.batch * g.n * k_pad);
    float* scratch = nullptr;
    if (a_floats + b_floats > 0) TRS_TRY(malloc_on_stream(stream, (size_t)(a_floats + b_floats) * sizeof(float), (void**)&scratch));
    ScratchGuard scratch_guard{stream, scratch};
    // scratch layout: [A lo | A hi (re-laid only)] [B lo | B hi (re-laid only)]
    float* a_lo = scratch;
    float* a_hi = a_lo + g.batch * g.m * k_pad;
    float* b_lo = scratch + a_floats;
    float* b_hi = b_lo + g.batch * g.n * k_pad;
    if (!ra.given) {
        if (ra.mn) {
            // lo plane [batch, k, m]: the k-fast kernel with the roles of the axes exchanged (its "rows" are k, its "k" is m)
            TRS_TRY(launch_split(g.a, g.batch, g.k, g.m, g.m, g.a_batch_stride, g.a_col_stride, 1, a_lo, a_lo, nonfinite, epoch, stream, 1));
            TRS_TRY(make_mn_operand_map(&ma_lo, a_lo, g.m, g.k, g.batch, g.m, g.k * g.m, BM, bk));
        } else {
            TRS_TRY(launch_split(g.a, g.batch, g.m, g.k, k_pad, g.a_batch_stride, g.a_row_stride, g.a_col_stride, a_hi, a_lo, nonfinite, epoch, stream, ra.raw));
            if (!ra.raw) TRS_TRY(make_plane_map(&ma_hi, a_hi, g.m, k_pad, g.batch, BM, bk));
            TRS_TRY(make_plane_map(&ma_lo, a_lo, g.m, k_pad, g.batch, BM, bk));
        }
    }
    if (!rb.given) {
        if (rb.mn) {
            TRS_TRY(launch_split(g.b, g.batch, g.k, g.n, g.n, g.b_batch_stride, g.b_row_stride, 1, b_lo, b_lo, nonfinite, epoch, stream, 1));
            TRS_TRY(make_mn_operand_map(&mb_lo, b_lo, g.n, g.k, g.batch, g.n, g.k * g.n, b_box, bk));
        } else {
            TRS_TRY(launch_split(g.b, g.batch, g.n, g.k, k_pad, g.b_batch_stride, g.b_col_stride, g.b_row_stride, b_hi, b_lo, nonfinite, epoch, stream, rb.raw));
            if (!rb.raw) TRS_TRY(make_plane_map(&mb_hi, b_hi, g.n, k_pad, g.batch, b_box, bk));
            TRS_TRY(make_plane_map(&mb_lo, b_lo, g.n, k_pad, g.batch, b_box, bk));
        }
    }
    const long long tile_rows = pair ? 2 * BM : BM;
    const long long tiles_m = (g.m + tile_rows - 1) / tile_rows, tiles_n = (g.n + BN - 1) / BN;
    const long long total_tiles = tiles_m * tiles_n * g.batch;
    if (total_tiles > INT32_MAX) return fail(TRS_ERR_UNSUPPORTED, "too many output tiles");
    EpilogueArgs e{g.c, g.bias, g.aux, g.preact, g.c_batch_stride, g.c_row_stride, (int)g.m, (int)g.n, (int)(k_pad / bk), g.epilogue,
                   (int)tiles_m, (int)tiles_n, (int)total_tiles, (int)total_tiles, (int)total_tiles, 1, nullptr, nullptr, ra.mn ? 1 : 0, rb.mn ? 1 : 0,
                   planes ? planes->c_lo : nullptr, planes ? planes->c_flag : nullptr, words->error, WAIT_CYCLES};
    // units that work side by side: SMs, or resident CTA pairs
    const long long units = pair ? words->pair_clusters : sm_count(stream->device);
    // The last round of tiles rarely fills the GPU (256 tile pairs on 74 SM pairs: 3 rounds + 34).  Its tiles are cut
    // into `parts` items along K when that shortens the round: with p parts it takes ceil(tail * p / units) / p tile
    // times.  A cut item keeps a whole tile's epilogue (drain the accumulator, write 128 KiB per CTA, count itself) and
    // the finishing item reads every part back, so an item must carry enough MMA work to hide that: at least 2048 of
    // K per part.  Measured (us, cut / uncut): 4096^3 495 / 510, 512 x 4096 x 4096 97 / 121, 4096 x 4096 x 8192 960 / 1003;
    // with thinner parts the epilogues become the bottleneck (2048 x 4096 x 4096 cut in four: 317 against 256; 8 x 1024^3 cut
    // in four: 223 against 88).
    const long long tail = total_tiles % units;
    const int min_blocks_per_part = 2048 / bk;
    int parts = 1;
    if (tail > 0) {
        double best = 1.0;
        for (int p = 2; p <= 8 && e.k_blocks / p >= min_blocks_per_part; ++p) {
            const double t = (double)((tail * p + units - 1) / units) / p + 0.03 * (p - 1);
            if (t < best - 0.05) { best = t; parts = p; }
        }
    }
    ScratchGuard partial_guard{stream, nullptr};
    if (parts > 1) {
        const size_t slabs = (size_t)tail * (size_t)(tile_rows / 32);
        const size_t counter_bytes = (slabs * sizeof(unsigned int) + 511) & ~size_t(511);
        const size_t partial_bytes = (size_t)tail * parts * (size_t)tile_rows * BN * sizeof(float);
        void* block = nullptr;
        TRS_TRY(malloc_on_stream(stream, counter_bytes + partial_bytes, &block));
        partial_guard.p = block;
        e.arrivals = reinterpret_cast<unsigned int*>(block);
        e.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(block) + counter_bytes);
        e.parts = parts;
        e.whole_tiles = (int)(total_tiles - tail);
        e.total_items = (int)(e.whole_tiles + parts * tail);
        TRS_CUDA(cudaMemsetAsync(e.arrivals, 0, counter_bytes, stream->stream));
    }
    const unsigned grid = (unsigned)std::min<long long>(e.total_items, units);
    if (parts > 1) {
        // ordinary launch behind the memset of the counters: programmatic serialization is between kernels only
        if (pair) gemm_tf32x3_pair_kernel<<<2 * grid, 192, PAIR_SMEM_BYTES, stream->stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, e);
        else gemm_tf32x3_kernel<<<grid, 192, SMEM_BYTES, stream->stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, e);
        TRS_CUDA(cudaGetLastError());
    } else if (pair) {
        TRS_CUDA(launch_dependent(gemm_tf32x3_pair_kernel, dim3(2 * grid), dim3(192), PAIR_SMEM_BYTES, stream->stream, ma_hi, ma_lo, mb_hi, mb_lo, e));
    } else {
        TRS_CUDA(launch_dependent(gemm_tf32x3_kernel, dim3(grid), dim3(192), SMEM_BYTES, stream->stream, ma_hi, ma_lo, mb_hi, mb_lo, e));
    }
    count_launch();
    // inf / NaN operands: recompute with the exact-FP32 kernel (a no-op launch when none were seen),
    // which keeps the reference's inf/NaN classification of the result.
    SimtGate gate;
    gate.word = (ra.given && rb.given) ? nullptr : nonfinite;
    gate.epoch = epoch;
    gate.flag_a = ra.given ? planes->a_flag : nullptr;
    gate.flag_b = rb.given ? planes->b_flag : nullptr;
    gate.gated = true;
    TRS_TRY(gemm_simt_launch(g, planes, stream, gate));
    return TRS_OK;
}

// Reads (and clears) the error word of kernels with bounded waits; called after a stream or device sync.
// The word lives in page-locked host memory that the kernels write through a mapped pointer, so the check is a
// plain host read: any sync on the device sees (once) an error raised by a kernel that has completed.
int32_t gemm_check_status(int device) {
    if (device < 0 || device >= 16) return TRS_OK;
    unsigned int value = 0;
    {
        std::lock_guard<std::mutex> lock(g_words_mu);
        DeviceWords& w = g_words[device];
        if (!w.host_error) return TRS_OK;
        value = *reinterpret_cast<volatile unsigned int*>(w.host_error);
        if (value != 0) *reinterpret_cast<volatile unsigned int*>(w.host_error) = 0;
    }
    if (value != 0)
        return fail(TRS_ERR_DEVICE_STATUS, "tensor-core matmul: a bounded wait ran out (stage %u); the result is invalid", value);
    return TRS_OK;
}

int32_t gemm_wait_probe(trs_stream stream, long long limit_cycles) {
    DeviceWords* words = nullptr;
    unsigned int epoch = 0;
    TRS_TRY(device_words(stream->device, &words, &epoch));
    wait_probe_kernel<<<1, 32, 0, stream->stream>>>(words->error, limit_cycles);
    TRS_CUDA(cudaGetLastError());
    count_launch();
    return TRS_OK;
}

}  // namespace trs
