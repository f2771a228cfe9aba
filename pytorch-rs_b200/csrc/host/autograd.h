// Define-by-run tape for CUDA tensors (reference: GradFn / SavedTensor / AutogradMeta,
// src/tensor.rs:23-106, and the Python-visible node names of src/autograd_node.rs:5-59).
#pragma once
#include "engine.h"

namespace trsh {

enum class GK {
    Sum,          // SumBackward0            src/tensor.rs:3008-3013
    MulScalar,    // MulBackward0 (scalar)   src/tensor.rs:3014-3021
    Neg,          // NegBackward0 / RsubBackward   src/tensor.rs:3022-3029
    Identity,     // AddBackward0 / SubBackward0 with a scalar   src/tensor.rs:3236
    Relu,         // ReluBackward0           src/tensor.rs:3161-3176
    Mul,          // MulBackward0            src/tensor.rs:3031-3097
    Permute,      // Permute/TransposeBackward0   src/tensor.rs:3248-3298
    Index,        // SelectBackward0         src/tensor.rs:3237-3247
    Copy,         // clone / contiguous      src/tensor.rs:3236
    Reshape,      // ViewBackward0: same flat logical order, other shape   src/tensor.rs:2127-2189, 3236
    Sin,          // SinBackward0            src/tensor.rs:3178-3185
    Sqrt,         // SqrtBackward0           src/tensor.rs:3187-3202, 4416-4419
    // Edges the reference does not record on CPU; CUDA tensors gain them:
    Add,          // AddBackward0 (tensor + tensor)
    Sub,          // SubBackward0 (tensor - tensor)
    Exp,          // ExpBackward0 (saves the output)
    Matmul,       // MmBackward0 / BmmBackward0
};

struct Edge {
    std::shared_ptr<AutogradMeta> meta;   // null: that input needs no gradient
    Shape shape;                           // the input's logical shape
};

struct GradFn {
    GK kind;
    std::vector<Edge> in;
    std::vector<View> saved;       // values needed by the VJP (released after a successful backward)
    bool needs_values = false;
    float scalar = 0.f;
    std::vector<i64> dims;         // Permute: output axis -> input axis
    i64 index = 0;                 // Index: selected position along dim 0
    Shape out_shape;
    const char* name = "";
};

void record(const TensorP& out, GK kind, const char* name, std::vector<const Tensor*> inputs, std::vector<View> saved,
            bool needs_values, float scalar = 0.f, std::vector<i64> dims = {}, i64 index = 0);
const char* grad_fn_name(const Tensor& t);

}  // namespace trsh
