/*
 * trs_host.h — C API of libtrs_host.so, the host engine that stands in for the reference's
 * Rust core (`Tensor`, `Storage`, autograd tape; src/tensor.rs, src/storage.rs) for tensors on
 * a CUDA device.  The reference's PyO3 layer calls `crate::Tensor` methods
 * (src/python.rs:3848-3952, 4067-4133); a binding layer calls these functions the same way.
 * The engine itself only calls the kernel ABI in trs_cuda.h.
 *
 * Handles are opaque and owned by the caller (trsh_release).  Every function returns 0 or a
 * trsh_error_kind; trsh_last_error() holds the reference's message for that error
 * (src/tensor_error.rs:110-393).  Shapes and strides are in elements.
 */
#ifndef TRS_HOST_H
#define TRS_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct trsh_tensor_s* trsh_tensor;

/* Values of trsh error codes (TensorError variants reachable on this path). */
enum {
    TRSH_OK = 0, TRSH_SHAPE_MISMATCH = 1, TRSH_MATMUL_REQUIRES_MATRICES = 2, TRSH_MATMUL_INNER_MISMATCH = 3,
    TRSH_ITEM_REQUIRES_ONE_ELEMENT = 4, TRSH_INDEX_OUT_OF_BOUNDS = 5, TRSH_DIMENSION_OUT_OF_RANGE = 6,
    TRSH_PERMUTATION_RANK_MISMATCH = 7, TRSH_PERMUTATION_DIM_OUT_OF_RANGE = 8, TRSH_DUPLICATE_PERMUTATION_DIM = 9,
    TRSH_MATRIX_TRANSPOSE_REQUIRES_MATRIX = 10, TRSH_STRIDE_OVERFLOW = 11, TRSH_ELEMENT_COUNT_OVERFLOW = 12,
    TRSH_ALLOCATION_FAILED = 13, TRSH_BACKWARD_REQUIRES_SCALAR = 14, TRSH_DOES_NOT_REQUIRE_GRAD = 15,
    TRSH_BACKWARD_GRAPH_FREED = 16, TRSH_INVALID_SCALAR_INDEX = 17, TRSH_DEVICE_MISMATCH = 18, TRSH_DEVICE = 19,
    TRSH_INVALID_ARGUMENT = 20, TRSH_SHAPE_DATA_MISMATCH = 21, TRSH_RESHAPE_INVALID = 22,
    TRSH_VIEW_INCOMPATIBLE_LAYOUT = 23
};

const char* trsh_last_error(void);

/* creation / egress: Tensor::from_vec, zeros/ones/full (src/tensor.rs:302-423), try_to_vec, item (2438) */
int32_t trsh_from_host(const float* data, int32_t rank, const int64_t* shape, int32_t device, trsh_tensor* out);
/* Same, for page-locked host memory (trs_malloc_host): returns once the copy is enqueued; the caller
 * keeps the source unchanged until the device stream has passed it (trsh_sync or a later read-back).
 * The copy runs on an upload stream of its own: it proceeds while kernels queued earlier are still
 * running, and only kernels that come after this call wait for it -- a host that creates the next
 * batch's tensor before it waits for the current result overlaps the upload with the computation. */
int32_t trsh_from_pinned_host(const float* data, int32_t rank, const int64_t* shape, int32_t device, trsh_tensor* out);
int32_t trsh_full(int32_t rank, const int64_t* shape, float value, int32_t device, trsh_tensor* out);
int32_t trsh_to_host(trsh_tensor t, float* out);          /* logical row-major order, numel floats */
/* Read-back into page-locked memory that does not wait: the copy runs on a second stream behind the
 * kernels that produce `t`, overlapping later uploads and kernels; `out` is valid after trsh_sync. */
int32_t trsh_to_pinned_host_async(trsh_tensor t, float* out);
int32_t trsh_item(trsh_tensor t, float* out);
int32_t trsh_release(trsh_tensor t);

/* metadata accessors (src/tensor.rs:453-771) */
int32_t trsh_rank(trsh_tensor t, int32_t* rank);
int32_t trsh_layout(trsh_tensor t, int64_t* shape, int64_t* strides, int64_t* offset, int64_t* numel);
int32_t trsh_device(trsh_tensor t, int32_t* device);
int32_t trsh_flags(trsh_tensor t, int32_t* requires_grad, int32_t* is_leaf, int32_t* is_contiguous, int32_t* is_pending);
/* Storage::data_ptr (src/storage.rs:154): forces the value; device address of element 0.  The holder of the
 * address may write through it, so from here on the engine reads this storage eagerly and keeps no derived
 * copies of it; trsh_const_data_ptr is the read-only form without that effect. */
int32_t trsh_data_ptr(trsh_tensor t, void** ptr);
int32_t trsh_const_data_ptr(trsh_tensor t, const void** ptr);
int32_t trsh_shares_storage(trsh_tensor a, trsh_tensor b, int32_t* shared);
const char* trsh_grad_fn_name(trsh_tensor t);

/* views (src/tensor.rs:1082-1215, 1850-1973) */
int32_t trsh_permute(trsh_tensor t, int32_t n, const int64_t* dims, trsh_tensor* out);
int32_t trsh_transpose(trsh_tensor t, int64_t dim0, int64_t dim1, trsh_tensor* out);
int32_t trsh_matrix_transpose(trsh_tensor t, trsh_tensor* out);    /* .mT */
int32_t trsh_reverse_dims(trsh_tensor t, trsh_tensor* out);        /* .T  */
int32_t trsh_select0(trsh_tensor t, int64_t index, trsh_tensor* out);
int32_t trsh_detach(trsh_tensor t, trsh_tensor* out);
int32_t trsh_contiguous(trsh_tensor t, trsh_tensor* out);
/* materialising layout ops: try_clone (src/tensor.rs:1517-1575), reshape / view (2032-2189; `view_only`
 * fails instead of copying), PartialEq (286-293) */
int32_t trsh_clone(trsh_tensor t, trsh_tensor* out);
/* Memory formats (MemoryFormat, src/memory_format.rs:5-15): 0 preserve_format, 1 contiguous_format,
 * 2 channels_last (rank 4), 3 channels_last_3d (rank 5).  try_clone_with_memory_format
 * (src/tensor.rs:1533-1575), try_contiguous (1606-1675; returns the same tensor when the layout already
 * matches, rejects preserve_format otherwise), is_contiguous_with_memory_format (1004-1014). */
int32_t trsh_clone_format(trsh_tensor t, int32_t memory_format, trsh_tensor* out);
int32_t trsh_contiguous_format(trsh_tensor t, int32_t memory_format, trsh_tensor* out);
int32_t trsh_is_contiguous_format(trsh_tensor t, int32_t memory_format, int32_t* result);
int32_t trsh_reshape(trsh_tensor t, int32_t n, const int64_t* shape, int32_t view_only, trsh_tensor* out);
int32_t trsh_equal(trsh_tensor a, trsh_tensor b, int32_t* result);
/* squeeze() (all != 0) / squeeze(dim): metadata-only (src/tensor.rs:1305-1336) */
int32_t trsh_squeeze(trsh_tensor t, int32_t all, int64_t dimension, trsh_tensor* out);

/* pointwise (src/tensor.rs:2197-2410); `op` is a trs_op from trs_cuda.h */
int32_t trsh_unary(trsh_tensor t, int32_t op, trsh_tensor* out);
int32_t trsh_scalar(trsh_tensor t, int32_t op, float scalar, int32_t reflected, trsh_tensor* out);
int32_t trsh_binary(trsh_tensor l, trsh_tensor r, int32_t op, trsh_tensor* out);
/* contraction and reduction (src/tensor.rs:2453-2533, 2413-2431) */
int32_t trsh_matmul(trsh_tensor l, trsh_tensor r, trsh_tensor* out);
int32_t trsh_sum(trsh_tensor t, trsh_tensor* out);

/* autograd (src/tensor.rs:780-898, src/grad_mode.rs) */
int32_t trsh_set_requires_grad(trsh_tensor t, int32_t on, trsh_tensor* out);
int32_t trsh_backward(trsh_tensor t);
int32_t trsh_grad(trsh_tensor t, trsh_tensor* out);       /* *out = NULL when no gradient has been accumulated */
int32_t trsh_set_grad_enabled(int32_t on);                /* nests: off increments a depth counter */
int32_t trsh_is_grad_enabled(int32_t* on);

/* layout planning only (no device needed): the output strides the ops above give their results
 * (unary_output_strides 2751-2766, map_scalar 2718-2727, zip_map 2535-2557 / BroadcastPlan 3601-3693) */
int32_t trsh_plan_unary(int32_t rank, const int64_t* shape, const int64_t* strides, int64_t* out_strides);
int32_t trsh_plan_scalar(int32_t rank, const int64_t* shape, const int64_t* strides, int64_t* out_strides);
/* clone(memory_format) when `for_clone`, else contiguous(memory_format): `copies` = 0 when contiguous() keeps
 * the tensor's storage, else `out_strides` holds the strides of the packed copy. */
int32_t trsh_plan_memory_format(int32_t memory_format, int32_t for_clone, int32_t rank, const int64_t* shape, const int64_t* strides,
                                int32_t* copies, int64_t* out_strides);
int32_t trsh_plan_binary(int32_t lrank, const int64_t* lshape, const int64_t* lstrides, int32_t rrank,
                         const int64_t* rshape, const int64_t* rstrides, int32_t* out_rank, int64_t* out_shape,
                         int64_t* out_strides);

/* Operand images for the tensor-core matmul (trs_gemm_planes in trs_cuda.h): kept beside each storage that a
 * matmul reads, on by default; off = every matmul prepares its operands per call.  trsh_has_operand_image
 * tells whether `t`'s storage currently carries one. */
int32_t trsh_set_plane_cache(int32_t on);
int32_t trsh_has_operand_image(trsh_tensor t, int32_t* has);

/* Data-parallel gradient exchange: the reference has no distributed backend
 * (python/torch_rs/distributed/distributed_c10d.py:39-74); LOCAL_RANK (71-72) picks the device.  One
 * communicator per process (trs_comm_* in trs_cuda.h underneath).  trsh_all_reduce_grads sums the .grad of the
 * given leaves over the ranks in place on a side stream, each one as soon as its own kernel has finished, and
 * makes the compute stream wait for the last; trsh_all_reduce does the same for one contiguous tensor. */
int32_t trsh_comm_unique_id(char* id128);
int32_t trsh_comm_init(int32_t device, int32_t nranks, int32_t rank, const char* id128);
int32_t trsh_comm_destroy(void);
int32_t trsh_comm_size(int32_t* nranks);
int32_t trsh_all_reduce_grads(const trsh_tensor* leaves, int32_t count);
int32_t trsh_all_reduce(trsh_tensor t);

/* execution control: force pending work of `t` onto the device / wait for the device stream */
int32_t trsh_materialize(trsh_tensor t);
int32_t trsh_sync(int32_t device);
int32_t trsh_stream(int32_t device, void** trs_stream_handle);   /* the engine's trs_stream for that device */

#ifdef __cplusplus
}
#endif
#endif /* TRS_HOST_H */
