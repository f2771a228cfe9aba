// Host engine: the C++ stand-in for the reference's Rust core (src/tensor.rs, src/storage.rs,
// src/autograd_node.rs) for tensors whose storage lives on a CUDA device.  It keeps the
// reference's metadata rules (shape / stride / broadcast planning, view construction, autograd
// tape) on the host and replaces its element loops by calls into the C ABI of libtrs_cuda.so.
// It links against nothing but that C ABI, exactly as the Rust crate would.
#pragma once
#include <cstdint>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/trs_cuda.h"

namespace trsh {

using i64 = int64_t;
using Shape = std::vector<i64>;

// Mirrors the TensorError variants the hot path can raise (src/tensor_error.rs:7-108); the
// messages are the reference's Display strings (src/tensor_error.rs:110-393).
enum class ErrKind : int {
    None = 0,
    ShapeMismatch = 1,
    MatmulRequiresMatrices = 2,
    MatmulInnerDimensionMismatch = 3,
    ItemRequiresOneElement = 4,
    IndexOutOfBounds = 5,
    DimensionOutOfRange = 6,
    PermutationRankMismatch = 7,
    PermutationDimensionOutOfRange = 8,
    DuplicatePermutationDimension = 9,
    MatrixTransposeRequiresMatrix = 10,
    StrideCalculationOverflow = 11,
    ElementCountOverflow = 12,
    AllocationFailed = 13,
    BackwardRequiresScalar = 14,
    DoesNotRequireGrad = 15,
    BackwardGraphFreed = 16,
    InvalidScalarIndex = 17,
    DeviceMismatch = 18,
    Device = 19,            // a libtrs_cuda call failed (no device, CUDA error, ...)
    InvalidArgument = 20,
    ShapeDataMismatch = 21,
    ReshapeInvalid = 22,
    ViewIncompatibleLayout = 23,
    ContiguousPreserveFormatUnsupported = 24,
    ContiguousMemoryFormatRankMismatch = 25,
};

// MemoryFormat (src/memory_format.rs:5-15)
enum class MemoryFormat : int { Preserve = 0, Contiguous = 1, ChannelsLast = 2, ChannelsLast3d = 3 };

struct Error : std::runtime_error {
    ErrKind kind;
    Error(ErrKind k, const std::string& m) : std::runtime_error(m), kind(k) {}
};

struct Node;

// Device buffer or a pending (not yet computed) pointwise result.  Immutable once filled, except
// a leaf gradient, which is accumulated in place (src/storage.rs:85-100).
struct Storage {
    int device = 0;
    float* ptr = nullptr;
    i64 count = 0;
    std::shared_ptr<Node> node;   // non-null while the values are still an unevaluated expression
    // Set once something may write the values in place after construction (a leaf gradient that is accumulated
    // into, a buffer handed out through data_ptr / DLPack, the target of an all-reduce).  Such a storage is never
    // a leaf of a pending expression (readers run at record time) and never gets a cached lo image.
    bool written_in_place = false;
    // Cached operand image for the tensor-core matmul: lo[i] = tf32(ptr[i] - trunc_tf32(ptr[i])) for the whole
    // storage, and a device word that is non-zero when the storage holds an inf / NaN.  The values of a storage
    // never change (src/storage.rs:7-18), so the image is computed at most once and dies with the storage.
    float* lo = nullptr;
    uint32_t* lo_flag = nullptr;
    ~Storage();
};

struct View {
    std::shared_ptr<Storage> st;
    Shape shape, strides;
    i64 offset = 0;
};

constexpr int OP_MATMUL = 100;   // lazy matmul node (so bias / relu / relu-VJP can fuse as epilogue)

struct Node {
    int op = 0;                  // trs_op or OP_MATMUL
    float imm = 0.f;
    std::vector<View> args;
    Shape shape, strides;        // layout of the value this node produces (offset 0)
    int n_instr = 1, n_leaf = 0; // conservative size of the pending expression under this node
};

struct GradFn;
struct Tensor;

struct AutogradMeta {
    bool leaf = false;
    std::shared_ptr<GradFn> grad_fn;          // non-leaf; reset when the graph is freed
    bool freed = false;
    std::shared_ptr<Tensor> grad;             // leaf: accumulated gradient (contiguous)
    Shape leaf_shape;
    int device = 0;
    // leaf: recorded on the compute stream right behind the kernel that produced the latest gradient, so that a
    // gradient all-reduce on another stream can start while the rest of the backward pass still runs
    trs_event grad_ready = nullptr;
    uint64_t ready_order = 0;                 // position of that event among all gradient events of the process
    // Releases a chain of recorded ops with a loop, not by recursion (the reference's iterative Drop,
    // src/tensor.rs:189-206): a 100,000-op chain must not overflow the stack when its last handle goes.
    ~AutogradMeta();
};

struct Tensor {
    View v;
    i64 numel = 0;
    std::shared_ptr<AutogradMeta> meta;
    bool view_requires_grad = false;
    bool requires_grad() const { return meta != nullptr || view_requires_grad; }
    bool is_leaf() const { return !meta || meta->leaf; }
    int device() const { return v.st->device; }
};
using TensorP = std::shared_ptr<Tensor>;

// ---- layout rules (layout.cpp) -----------------------------------------------------------------
i64 element_count(const Shape& shape);
Shape contiguous_strides(const Shape& shape);
bool layout_is_contiguous(const Shape& shape, const Shape& strides);
bool is_non_overlapping_and_dense(const Shape& shape, const Shape& strides);
Shape unary_output_strides(const Shape& shape, const Shape& strides);
Shape scalar_output_strides(const Shape& shape, const Shape& strides);
bool reshape_view_strides(const Shape& shape, const Shape& strides, const Shape& new_shape, Shape* out);
Shape clone_strides(const Shape& shape, const Shape& strides);
const char* memory_format_name(MemoryFormat f);
bool is_contiguous_in_format(const Shape& shape, const Shape& strides, MemoryFormat f);
Shape memory_format_strides(const Shape& shape, MemoryFormat f);
int memory_format_rank(MemoryFormat f);
bool memory_format_plan(const Shape& shape, const Shape& strides, MemoryFormat f, bool for_clone, Shape* out);
void binary_plan(const Shape& lshape, const Shape& lstrides, const Shape& rshape, const Shape& rstrides,
                 Shape* shape, Shape* strides);

// ---- engine (engine.cpp) -------------------------------------------------------------------------
bool grad_enabled();
void set_grad_enabled(bool on);
trs_stream stream_for(int device);
void check_cuda(int32_t status, const char* what);

TensorP from_host(const float* data, const Shape& shape, int device, bool pinned = false);
TensorP full(const Shape& shape, float value, int device);
void to_host(const Tensor& t, float* out);                 // logical row-major order
void to_host_async(const std::shared_ptr<Tensor>& t, float* out);   // pinned destination; valid after sync(device)
float item(const Tensor& t);
// `for_matmul`: the value is about to be read as a matmul operand; a matmul that produces it also writes its lo image.
void materialize(const std::shared_ptr<Storage>& st, bool for_matmul = false);
// Device blocks in the order of the engine's stream.
float* alloc_floats(i64 count, int device);
void free_floats(int device, void* ptr);
// The cached lo image of a storage (computed on first use); false when the storage does not qualify.
bool ensure_lo_image(Storage& st, i64 view_numel);
void alloc_lo_image(Storage& st);                  // empty image + cleared flag, to be filled by a matmul epilogue
void set_plane_cache(bool on);
bool plane_cache_enabled();
void mark_written_in_place(Storage& st);
void sync(int device);

TensorP permute(const TensorP& t, const std::vector<i64>& dims, int node_kind);
TensorP transpose(const TensorP& t, i64 d0, i64 d1);
TensorP matrix_transpose(const TensorP& t);
TensorP reverse_dims(const TensorP& t);
TensorP select0(const TensorP& t, i64 index);
TensorP detach(const TensorP& t);
TensorP contiguous(const TensorP& t, MemoryFormat format = MemoryFormat::Contiguous);
TensorP clone(const TensorP& t, MemoryFormat format = MemoryFormat::Preserve);
TensorP squeeze(const TensorP& t, i64 dimension);    // INT64_MIN: every singleton dimension
TensorP reshape(const TensorP& t, const std::vector<i64>& requested, bool view_only);
bool equal(const TensorP& a, const TensorP& b);

TensorP unary(const TensorP& t, int op);                   // relu, exp, neg, sin, sqrt, reciprocal
TensorP scalar_op(const TensorP& t, int op, float s, bool reflected);
TensorP binary(const TensorP& l, const TensorP& r, int op);
TensorP matmul(const TensorP& l, const TensorP& r);
TensorP sum(const TensorP& t);

TensorP set_requires_grad(const TensorP& t, bool on);
void backward(const TensorP& root);
TensorP grad_of(const TensorP& t);

// Data-parallel gradient exchange (comm.cpp): one NCCL communicator per process.
void comm_unique_id(char* id128);
void comm_init(int device, int nranks, int rank, const char* id128);
void comm_destroy();
int comm_size();
// Sums the gradients of the given leaves over all ranks, in place, on a side stream: each all-reduce starts as
// soon as that gradient's kernel has finished, under the rest of the backward pass; the compute stream waits
// for the last one.
void all_reduce_grads(const std::vector<TensorP>& leaves);
void all_reduce_tensor(const TensorP& t);

// Internal helpers shared with autograd.cpp
TensorP make_tensor(View v);
TensorP pointwise_node(int op, float imm, std::vector<View> args, const Shape& shape, const Shape& strides, int device);
TensorP zeros_like_shape(const Shape& shape, int device);
extern std::recursive_mutex g_engine_mu;

}  // namespace trsh
