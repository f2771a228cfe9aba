// Internal matmul entry points.
#pragma once
#include "common.h"

namespace trs {
int32_t gemm_simt_launch(const trs_gemm_desc& g, trs_stream stream);
// Whether the tensor-core path can take this descriptor (alignment and size rules).
bool gemm_tc_eligible(const trs_gemm_desc& g);
int32_t gemm_tc_launch(const trs_gemm_desc& g, trs_stream stream);
}  // namespace trs
