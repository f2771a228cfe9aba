// Internal matmul entry points.
#pragma once
#include "common.h"

namespace trs {
// When the exact-FP32 kernel runs as the recompute step behind a tensor-core product: it returns at once unless
// the preparation of this very call met an inf / NaN (*word == epoch) or a prepared operand image carries the
// mark (*flag_a / *flag_b non-zero).  `gated` false: an ordinary launch that always computes.
struct SimtGate {
    const unsigned int* word = nullptr;
    unsigned int epoch = 0;
    const unsigned int* flag_a = nullptr;
    const unsigned int* flag_b = nullptr;
    bool gated = false;
};
// `planes` (may be NULL): only c_lo / c_flag are honoured here, so that the result's lo image exists whichever kernel ran.
int32_t gemm_simt_launch(const trs_gemm_desc& g, const trs_gemm_planes* planes, trs_stream stream, const SimtGate& gate = SimtGate());
// Whether the tensor-core path can take this descriptor (alignment and size rules).
bool gemm_tc_eligible(const trs_gemm_desc& g);
// Whether the two-CTA (256x256 tiles) variant suits this descriptor better than the one-CTA kernel.
bool gemm_tc_pair_preferred(const trs_gemm_desc& g);
// `g.algo` picks the variant: TRS_GEMM_TCGEN05_3XTF32_2CTA the CTA-pair kernel, anything else the one-CTA kernel.
int32_t gemm_tc_launch(const trs_gemm_desc& g, const trs_gemm_planes* planes, trs_stream stream);
// Whether the tensor-core path would read a caller's lo image of A / B in place (g.algo resolved).
int32_t gemm_tc_plan(const trs_gemm_desc& g, bool* a_image, bool* b_image);
int32_t gemm_split_lo(const float* src, long long count, float* lo, unsigned int* flag, trs_stream stream);
int32_t gemm_check_status(int device);
// Launches one warp that waits `limit_cycles` SM clocks on a barrier nothing arrives on (test aid for the bounded waits).
int32_t gemm_wait_probe(trs_stream stream, long long limit_cycles);
}  // namespace trs
