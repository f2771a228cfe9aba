// Host-side planning for fused pointwise chains: operand alignment, dimension sorting and
// collapsing, kernel-class choice and the generated kernel source.  Pure host code (no CUDA
// calls), so it is exercised by CPU-only tests.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/trs_cuda.h"

namespace trs {

// Must match `struct Params` in the generated kernel source byte for byte.
struct PwParams {
    const float* in[TRS_MAX_INPUTS];
    float* out[TRS_MAX_OUTPUTS];
    long long in_stride[TRS_MAX_INPUTS][TRS_MAX_RANK];    // [operand][collapsed dim], dim 0 innermost
    long long out_stride[TRS_MAX_OUTPUTS][TRS_MAX_RANK];
    unsigned size[TRS_MAX_RANK];
    unsigned div_magic[TRS_MAX_RANK];                     // fast division by vecs0 (slot 0) / size[d] (d >= 1)
    unsigned div_shift[TRS_MAX_RANK];
    unsigned long long total;                             // work items (vectors or tiles)
    unsigned aux[4];                                      // vector: {vecs0}; tiled: {tiles0, tiles_t}
};

enum InKind { IN_VEC = 0, IN_SCALAR4 = 1, IN_BCAST = 2, IN_STRIDED = 3, IN_TRANSPOSED = 4 };
enum OutKind { OUT_VEC = 0, OUT_SCALAR4 = 1, OUT_STRIDED = 3 };

struct PwPlan {
    bool empty = false;          // zero elements: nothing to launch
    bool tiled = false;          // shared-memory staged transpose class
    int ndim = 1;                // collapsed dims
    int tdim = 0;                // tiled class: the dim along which transposed inputs are unit-stride
    int n_in = 0, n_out = 0;
    int in_kind[TRS_MAX_INPUTS];
    int out_kind[TRS_MAX_OUTPUTS];
    bool wide_offsets = false;   // some element offset needs more than 31 bits
    bool wide_items = false;     // work-item count needs more than 31 bits
    bool has_tail = false;       // inner size not a multiple of the vector width
    bool tile_vec = false;       // tiled class: 64x64 tiles moved with 128-bit accesses (else 32x32 scalar)
    int unroll = 4;
    int block = 256;
    unsigned long long grid = 0;
    PwParams params;
    long long numel = 0;
};

// Validates the program and operands and fills `plan`.  Returns TRS_OK or an error status
// (message via trs_last_error_message).
int32_t pw_make_plan(const trs_program* program, const trs_operand* inputs, const trs_operand* outputs,
                     PwPlan* plan);

// CUDA source of the kernel specialised for (program, plan's baked choices).  The entry point is
// `trs_pw`.  Identical (program, class, kinds, ndim, flags) give identical text, which is the
// cache key.
std::string pw_generate_source(const trs_program* program, const PwPlan& plan);
std::string pw_cache_key(const trs_program* program, const PwPlan& plan);

}  // namespace trs
