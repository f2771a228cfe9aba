// Internal matmul entry points.
#pragma once
#include "common.h"

namespace trs {
// `gate`: optional device word; when non-NULL the kernel returns at once unless *gate == epoch.
int32_t gemm_simt_launch(const trs_gemm_desc& g, trs_stream stream, const unsigned int* gate = nullptr, unsigned int epoch = 0);
// Whether the tensor-core path can take this descriptor (alignment and size rules).
bool gemm_tc_eligible(const trs_gemm_desc& g);
// Whether the two-CTA (256x256 tiles) variant suits this descriptor better than the one-CTA kernel.
bool gemm_tc_pair_preferred(const trs_gemm_desc& g);
// `g.algo` picks the variant: TRS_GEMM_TCGEN05_3XTF32_2CTA the CTA-pair kernel, anything else the one-CTA kernel.
int32_t gemm_tc_launch(const trs_gemm_desc& g, trs_stream stream);
size_t gemm_tc_scratch_bytes(const trs_gemm_desc& g);
int32_t gemm_tc_launch_ws(const trs_gemm_desc& g, float* scratch, trs_stream stream);
int32_t gemm_check_status(int device);
}  // namespace trs
