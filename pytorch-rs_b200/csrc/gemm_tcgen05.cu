// Placeholder translation unit for the tensor-core matmul (filled in by the tcgen05 kernel).
#include "gemm.h"

namespace trs {
bool gemm_tc_eligible(const trs_gemm_desc&) { return false; }
int32_t gemm_tc_launch(const trs_gemm_desc&, trs_stream) { return fail(TRS_ERR_UNSUPPORTED, "tensor-core matmul not built"); }
}  // namespace trs
