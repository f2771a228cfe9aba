// trs_matmul_f32: validation, algorithm choice, degenerate shapes.
#include "gemm.h"
#include "reduce.h"

using namespace trs;

namespace {
int32_t validate(const trs_gemm_desc* g) {
    if (!g) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL descriptor");
    if (g->batch < 0 || g->m < 0 || g->n < 0 || g->k < 0) return fail(TRS_ERR_INVALID_ARGUMENT, "negative extent");
    if (g->epilogue < TRS_EPI_NONE || g->epilogue > TRS_EPI_RELU_VJP) return fail(TRS_ERR_INVALID_ARGUMENT, "unknown epilogue %d", g->epilogue);
    if ((g->epilogue == TRS_EPI_BIAS || g->epilogue == TRS_EPI_BIAS_RELU) && !g->bias) return fail(TRS_ERR_INVALID_ARGUMENT, "bias epilogue without bias");
    if (g->epilogue == TRS_EPI_RELU_VJP && !g->aux) return fail(TRS_ERR_INVALID_ARGUMENT, "relu_vjp epilogue without aux");
    if (g->batch * g->m * g->n != 0 && (!g->c || (g->k != 0 && (!g->a || !g->b)))) return fail(TRS_ERR_INVALID_ARGUMENT, "NULL matrix pointer");
    if (g->algo < TRS_GEMM_AUTO || g->algo > TRS_GEMM_TCGEN05_3XTF32_2CTA) return fail(TRS_ERR_INVALID_ARGUMENT, "unknown algo %d", g->algo);
    return TRS_OK;
}
}  // namespace

extern "C" {

int32_t trs_matmul_select_algo(const trs_gemm_desc* desc, int32_t* algo) {
    TRS_TRY(validate(desc));
    if (!algo) return fail(TRS_ERR_INVALID_ARGUMENT, "algo is NULL");
    const bool tensor_core = desc->algo == TRS_GEMM_TCGEN05_3XTF32 || desc->algo == TRS_GEMM_TCGEN05_3XTF32_2CTA;
    if (tensor_core && !gemm_tc_eligible(*desc))
        return fail(TRS_ERR_UNSUPPORTED, "descriptor does not meet the tensor-core path's alignment rules");
    if (desc->algo != TRS_GEMM_AUTO) { *algo = desc->algo; return TRS_OK; }
    if (!gemm_tc_eligible(*desc)) *algo = TRS_GEMM_SIMT_FP32;
    else *algo = gemm_tc_pair_preferred(*desc) ? TRS_GEMM_TCGEN05_3XTF32_2CTA : TRS_GEMM_TCGEN05_3XTF32;
    return TRS_OK;
}

int32_t trs_matmul_f32_planes(const trs_gemm_desc* desc, const trs_gemm_planes* planes, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    int32_t algo = 0;
    TRS_TRY(trs_matmul_select_algo(desc, &algo));
    if (planes && planes->c_lo && !planes->c_flag) return fail(TRS_ERR_INVALID_ARGUMENT, "c_lo needs c_flag");
    if (desc->batch * desc->m * desc->n == 0) return TRS_OK;
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    // k == 0: the product is the zero matrix (reference: zero-filled output, src/tensor.rs:2473);
    // the SIMT kernel handles it (no k tiles) including the epilogue.
    if ((algo == TRS_GEMM_TCGEN05_3XTF32 || algo == TRS_GEMM_TCGEN05_3XTF32_2CTA) && desc->k > 0) {
        trs_gemm_desc chosen = *desc;
        chosen.algo = algo;
        return gemm_tc_launch(chosen, planes, stream);
    }
    return gemm_simt_launch(*desc, planes, stream);
}

int32_t trs_matmul_f32(const trs_gemm_desc* desc, trs_stream stream) { return trs_matmul_f32_planes(desc, nullptr, stream); }

int32_t trs_matmul_plan(const trs_gemm_desc* desc, int32_t* algo, int32_t* a_plane_used, int32_t* b_plane_used) {
    int32_t chosen_algo = 0;
    TRS_TRY(trs_matmul_select_algo(desc, &chosen_algo));
    bool a = false, b = false;
    if ((chosen_algo == TRS_GEMM_TCGEN05_3XTF32 || chosen_algo == TRS_GEMM_TCGEN05_3XTF32_2CTA) && desc->k > 0 &&
        desc->batch * desc->m * desc->n != 0) {
        trs_gemm_desc chosen = *desc;
        chosen.algo = chosen_algo;
        TRS_TRY(gemm_tc_plan(chosen, &a, &b));
    }
    if (algo) *algo = chosen_algo;
    if (a_plane_used) *a_plane_used = a ? 1 : 0;
    if (b_plane_used) *b_plane_used = b ? 1 : 0;
    return TRS_OK;
}

int32_t trs_split_lo_f32(const float* src, int64_t count, float* lo, uint32_t* flag, trs_stream stream) {
    TRS_TRY(check_stream(stream));
    if (count < 0 || !flag || (count > 0 && (!src || !lo))) return fail(TRS_ERR_INVALID_ARGUMENT, "bad trs_split_lo_f32 arguments");
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    return gemm_split_lo(src, count, lo, flag, stream);
}

int32_t trs_debug_wait_probe(trs_stream stream, int64_t limit_cycles) {
    TRS_TRY(check_stream(stream));
    if (limit_cycles < 0 || limit_cycles > 100000000) return fail(TRS_ERR_INVALID_ARGUMENT, "limit must be between 0 and 1e8 clocks");
    DeviceGuard guard(stream->device);
    if (!guard.ok) return fail(TRS_ERR_NO_DEVICE, "cannot select CUDA device %d", stream->device);
    return gemm_wait_probe(stream, limit_cycles);
}

}  // extern "C"
