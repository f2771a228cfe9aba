// Internal entry points of the reductions that take caller-provided scratch.
#pragma once
#include "common.h"

namespace trs {
int sum_partials_needed(int device, long long n);
int32_t reduce_sum_ws(const trs_operand* input, float* out, float* scratch, int scratch_floats, trs_stream stream);
// `max_partials` > 0 bounds chunks * cols (a fixed partials buffer); 0 = unbounded.
void colsum_geometry_for(int sms, long long rows, long long cols, long long max_partials, int* chunks, long long* rows_per_chunk);
void colsum_geometry(int device, long long rows, long long cols, int* chunks, long long* rows_per_chunk);
int32_t unbroadcast_sum_ws(const float* input, long long rows, long long cols, int by_rows, float* out, float* scratch,
                           long long scratch_floats, trs_stream stream);
// Enqueues dst[0..count) = value (any alignment).
void fill_value_async(float* dst, long long count, float value, trs_stream stream);
}  // namespace trs
