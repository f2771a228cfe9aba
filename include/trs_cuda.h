/*
 * trs_cuda.h — C ABI of libtrs_cuda.so, the sm_100a (B200) execution path for
 * pytorch-rs's data-parallel hot path: fused pointwise chains over strided and
 * broadcast float32 views, float32 matmul/bmm with fused bias/relu epilogues,
 * and the reductions and accumulations their autograd backward needs.
 *
 * The boundary sits under the reference `Tensor` op methods: the host keeps
 * shape / stride / broadcast planning and the autograd tape, and calls these
 * entry points instead of running its element loops when a tensor's storage
 * lives on a CUDA device.  Each declaration names the reference loop it
 * replaces (path:line inside the pytorch-rs project).
 *
 * Conventions
 *   - plain C types only; every function returns a trs_status (0 == success);
 *     nothing throws, aborts or traps.  trs_last_error_message() gives detail.
 *   - strides and offsets are in ELEMENTS (float32), never negative; a stride
 *     of 0 marks a broadcast axis.  Shapes follow the reference Tensor
 *     (src/tensor.rs:212-221).
 *   - outputs are caller-allocated device buffers; the library never keeps a
 *     caller pointer past the call except through stream ordering.
 *   - work is enqueued on the given trs_stream and returns immediately; only
 *     trs_stream_sync, trs_device_sync and trs_memcpy_d2h (pageable) block.
 *   - thread-safe per device; callable with the host interpreter lock held.
 *   - scratch memory the library needs inside a call is taken from and returned to the device cache in the
 *     order of the call's stream (see trs_malloc_async), so calls on different streams of one device never
 *     share scratch that is still in use.
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point returns TRS_ERR_NO_DEVICE.
 */
#ifndef TRS_CUDA_H
#define TRS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRS_MAX_RANK 8
#define TRS_MAX_INPUTS 8
#define TRS_MAX_OUTPUTS 4
#define TRS_MAX_INSTRS 64

typedef enum trs_status {
    TRS_OK = 0,
    TRS_ERR_INVALID_ARGUMENT = 1,
    TRS_ERR_ALLOCATION_FAILED = 2,   /* maps to TensorError::AllocationFailed (src/tensor_error.rs) */
    TRS_ERR_CUDA = 3,                /* a CUDA runtime call failed; see trs_last_error_message */
    TRS_ERR_JIT = 4,                 /* specialising a fused chain failed (compile log in the message) */
    TRS_ERR_UNSUPPORTED = 5,
    TRS_ERR_NO_DEVICE = 6,
    TRS_ERR_DEVICE_STATUS = 7        /* a kernel reported a bounded wait running out or a failed self-check */
} trs_status;

typedef struct trs_stream_s* trs_stream;   /* a CUDA stream bound to one device */
typedef struct trs_event_s* trs_event;
typedef struct trs_comm_s* trs_comm;       /* one rank's end of a multi-process communicator */

/* A strided view of a float32 device buffer (reference: storage + shape + strides + offset,
 * src/tensor.rs:212-221).  Element (i0..i{rank-1}) lives at base[offset + sum(i_k * stride[k])]. */
typedef struct trs_operand {
    void* base;
    int64_t offset;
    int32_t rank;
    int64_t shape[TRS_MAX_RANK];
    int64_t stride[TRS_MAX_RANK];
} trs_operand;

/* Fusion IR: a straight-line SSA program over float32 values.  Value k < n_inputs is the
 * element of input k at the current logical index; value n_inputs + j is the result of
 * instrs[j].  Unary ops read `a`; binary ops read `a` then `b` (operand order is the
 * reference closure's order); TRS_OP_CONST yields `imm`. */
typedef enum trs_op {
    TRS_OP_CONST = 0,
    TRS_OP_ADD = 1,        /* a + b      src/tensor.rs:2197  (one IEEE add, never contracted) */
    TRS_OP_SUB = 2,        /* a - b      src/tensor.rs:2207 */
    TRS_OP_MUL = 3,        /* a * b      src/tensor.rs:2217 */
    TRS_OP_DIV = 4,        /* a / b      src/tensor.rs:2245 */
    TRS_OP_NEG = 5,        /* sign flip  src/tensor.rs:4388 */
    TRS_OP_RELU = 6,       /* src/tensor.rs:4392-4400: +-0 pass through, NaN -> +0 */
    TRS_OP_EXP = 7,        /* src/tensor.rs:2398 (libm expf; here within 1 ulp of glibc's) */
    TRS_OP_RELU_VJP = 8,   /* a = saved input, b = upstream   src/tensor.rs:4422-4432 */
    TRS_OP_RECIP = 9,      /* 1.0 * (1.0 / a)   src/tensor.rs:2348-2355 */
    TRS_OP_SQRT = 10,      /* src/tensor.rs:4402-4414 */
    TRS_OP_SIN = 11,       /* src/tensor.rs:2388 */
    TRS_OP_COS = 12,       /* used by the sin VJP, src/tensor.rs:3178-3185 */
    TRS_OP_COPY = 13,      /* identity; materialises a view (src/tensor.rs:1805-1838) */
    TRS_OP_NE = 14         /* a != b ? 1.0 : 0.0 (IEEE: NaN differs from everything, -0 equals +0); Tensor::eq src/tensor.rs:286-293 */
} trs_op;

typedef struct trs_instr {
    int32_t op;
    int32_t a;
    int32_t b;
    float imm;
} trs_instr;

typedef struct trs_program {
    int32_t n_inputs;
    int32_t n_instrs;
    int32_t n_outputs;
    int32_t outputs[TRS_MAX_OUTPUTS];   /* value index written to output k */
    trs_instr instrs[TRS_MAX_INSTRS];
} trs_program;

/* GEMM epilogues fused into the store of C. */
typedef enum trs_epilogue {
    TRS_EPI_NONE = 0,
    TRS_EPI_BIAS = 1,        /* C = A@B + bias[n]                                     */
    TRS_EPI_BIAS_RELU = 2,   /* C = relu(A@B + bias[n]) ; optional pre-activation copy */
    TRS_EPI_RELU = 3,
    TRS_EPI_RELU_VJP = 4     /* C = relu_vjp(aux[m,n], A@B): dZ = relu'(Z) * (dY @ W2^T) */
} trs_epilogue;

typedef enum trs_gemm_algo {
    TRS_GEMM_AUTO = 0,
    TRS_GEMM_SIMT_FP32 = 1,      /* register-tiled FFMA kernel, any strides          */
    TRS_GEMM_TCGEN05_3XTF32 = 2,      /* TMA + tcgen05.mma kind::tf32, 3-product split, one CTA per 128x256 tile */
    TRS_GEMM_TCGEN05_3XTF32_2CTA = 3  /* same product, cta_group::2: a CTA pair per 256x256 tile                 */
} trs_gemm_algo;

/* Batched float32 matmul C[b] = A[b] @ B[b].  All strides in elements.  Replaces
 * Tensor::matmul (src/tensor.rs:2453-2533, 3889-3966) and extends it to a batch. */
typedef struct trs_gemm_desc {
    int64_t batch, m, n, k;
    const float* a; int64_t a_batch_stride, a_row_stride, a_col_stride;   /* A[b,m,k] */
    const float* b; int64_t b_batch_stride, b_row_stride, b_col_stride;   /* B[b,k,n] */
    float* c;       int64_t c_batch_stride, c_row_stride;                 /* C[b,m,n], unit column stride */
    const float* bias;        /* [n] or NULL */
    const float* aux;         /* RELU_VJP: saved pre-activation, laid out like C */
    float* preact;            /* BIAS_RELU: optional copy of A@B+bias, laid out like C, or NULL */
    int32_t epilogue;         /* trs_epilogue */
    int32_t algo;             /* trs_gemm_algo */
} trs_gemm_desc;

/* ---- devices, memory, streams --------------------------------------------------------
 * New relative to the reference, whose Device has the single variant Cpu (src/device.rs:5-9)
 * and whose Storage owns a Vec<f32> (src/storage.rs:7-18, 116-134). */
int32_t trs_device_count(int32_t* count);
/* Makes `device` the calling thread's current CUDA device.  Every entry point that takes a stream or a device
 * selects that device itself for the duration of the call; this only decides where resources that name no
 * device land (page-locked host memory from trs_malloc_host).  A process that follows the reference's LOCAL_RANK
 * convention (python/torch_rs/distributed/distributed_c10d.py:71-72) calls it once with that rank, so that it
 * never creates a context on another rank's GPU. */
int32_t trs_set_current_device(int32_t device);
/* PCI bus id ("0000:1b:00.0") of a device, for placing host staging memory on the device's NUMA node. */
int32_t trs_device_pci_bus_id(int32_t device, char* buffer, int32_t length);
int32_t trs_malloc(int32_t device, size_t bytes, void** ptr);       /* cached blocks; Storage::from_owned */
int32_t trs_free(int32_t device, void* ptr);                        /* Storage drop */
/* Stream-ordered forms.  trs_free_async hands the block back while work that uses it may still be queued on
 * `stream`; the cache remembers that stream and an event recorded on it at that moment.  trs_malloc_async returns
 * such a block at once to the same stream (stream order protects it).  Another stream gets a block nothing can touch
 * any more, else new memory (so that, say, an upload stream is never queued behind the kernels it should overlap),
 * and a block that is still in use -- the one freed longest ago, behind the work its stream had queued when it
 * was freed -- only once eight such blocks are waiting (a loop that never drains must not grow the pool without
 * bound) or when memory is short.  Plain trs_malloc only returns a remembered block once that work has finished, and plain trs_free states
 * that nothing queued anywhere still uses the block. */
int32_t trs_malloc_async(int32_t device, size_t bytes, trs_stream stream, void** ptr);
int32_t trs_free_async(int32_t device, void* ptr, trs_stream stream);
int32_t trs_empty_cache(int32_t device);
int32_t trs_memory_stats(int32_t device, int64_t* bytes_in_use, int64_t* bytes_reserved);
int32_t trs_malloc_host(size_t bytes, void** ptr);                  /* pinned staging memory */
int32_t trs_free_host(void* ptr);
int32_t trs_stream_create(int32_t device, trs_stream* stream);
int32_t trs_stream_destroy(trs_stream stream);
int32_t trs_stream_sync(trs_stream stream);
int32_t trs_stream_device(trs_stream stream, int32_t* device);
int32_t trs_stream_handle(trs_stream stream, void** cuda_stream);   /* the underlying cudaStream_t */
int32_t trs_device_sync(int32_t device);
int32_t trs_event_create(trs_event* event);
int32_t trs_event_record(trs_event event, trs_stream stream);
int32_t trs_event_sync(trs_event event);
int32_t trs_event_elapsed_ms(trs_event start, trs_event stop, float* ms);
int32_t trs_event_destroy(trs_event event);
int32_t trs_stream_wait_event(trs_stream stream, trs_event event);
/* Tensor ingestion/egress (src/python.rs:10329-10403 flatten_buffer; 4031-4052 numpy_array_copy). */
int32_t trs_memcpy_h2d(void* dst, const void* src, size_t bytes, trs_stream stream);
int32_t trs_memcpy_d2h(void* dst, const void* src, size_t bytes, trs_stream stream);
int32_t trs_memcpy_d2d(void* dst, const void* src, size_t bytes, trs_stream stream);

/* ---- pointwise -------------------------------------------------------------------------
 * One kernel for a whole recorded chain.  Replaces zip_map / map_scalar / unary_map and their
 * materialize_* loops (src/tensor.rs:2535-2789, 1805-1838, 3376-3599) and the pointwise VJP
 * arms of apply_grad_fn (src/tensor.rs:3014-3029, 3161-3176).  Inputs are broadcast to the
 * outputs' shape by stride-0 axes; all outputs share one shape; outputs must not overlap
 * inputs.  The chain is specialised (compiled once per program + layout class, then cached). */
int32_t trs_pointwise(const trs_program* program, const trs_operand* inputs, const trs_operand* outputs,
                      trs_stream stream);
/* Compile (without launching) the kernel trs_pointwise would use; needs no GPU. Writes the
 * chosen kernel class ("vector", "tiled") to `klass` when non-NULL (at least 16 bytes). */
int32_t trs_pointwise_prepare(const trs_program* program, const trs_operand* inputs, const trs_operand* outputs,
                              char* klass);
/* filled_storage (src/tensor.rs:4434-4442): Sum VJP fill, zeros/ones/full. */
int32_t trs_fill_f32(float* dst, int64_t count, float value, trs_stream stream);
/* accumulate_shared_gradient (src/storage.rs:85-100) and add_gradient (src/tensor.rs:3302-3317):
 * dst[i] += src[i]. */
int32_t trs_accumulate_f32(float* dst, const float* src, int64_t count, trs_stream stream);

/* ---- reductions ----------------------------------------------------------------------------
 * Tensor::sum (src/tensor.rs:2413-2431): all elements of a view -> one float at *out (device).
 * Deterministic two-stage tree; differs from the reference's sequential order by rounding only. */
int32_t trs_reduce_sum_f32(const trs_operand* input, float* out, trs_stream stream);
/* GradientAccumulator (src/tensor.rs:3204-3228): out[j] = sum over rows r of in[r*cols + j]
 * (un-broadcast of a leading axis, e.g. db1 = sum_rows dZ), or with by_rows != 0
 * out[r] = sum over j of in[r*cols + j] (un-broadcast of a trailing axis). Deterministic. */
int32_t trs_unbroadcast_sum_f32(const float* input, int64_t rows, int64_t cols, int32_t by_rows, float* out,
                                trs_stream stream);

/* Column sums without any allocation: out[j] = sum over r of input[r*cols + j], the same result as
 * trs_unbroadcast_sum_f32(..., by_rows = 0, ...).  No counterpart in the reference; it exists for
 * callers that cannot allocate device memory at the point of the call (a stream being captured, a
 * driver callback, a service whose memory pool is fixed after start-up).  The partial sums live in a
 * fixed 1 MiB array inside the library (held on every GPU that loads it, until exit), so `cols` may be
 * at most 262144; larger requests fail with TRS_ERR_UNSUPPORTED.  It calls no cudaMalloc / cudaFree
 * and no allocating library routine.  The first call on each device resolves the array's device
 * address (once); make that call before starting any stream capture.  All calls share the one
 * array: two calls whose kernels can overlap on the GPU (different streams) race and must be ordered
 * by the caller.  Nothing has to be cleared between calls. */
int32_t trs_colsum_f32_noalloc(const float* input, int64_t rows, int64_t cols, float* out, trs_stream stream);
/* The row chunking trs_colsum_f32_noalloc uses on a GPU with `sm_count` SMs (no launch, no device needed):
 * chunks * cols never exceeds the fixed array.  No counterpart in the reference. */
int32_t trs_colsum_noalloc_geometry(int32_t sm_count, int64_t rows, int64_t cols, int32_t* chunks, int64_t* rows_per_chunk);

/* ---- matmul ----------------------------------------------------------------------------------
 * Honours float32 matmul precision "highest" (python/torch_rs/__init__.py:81-85): either exact
 * FP32 FMA accumulation or the 3xTF32 error-compensated split with FP32 accumulation. */
int32_t trs_matmul_f32(const trs_gemm_desc* desc, trs_stream stream);
/* Which algorithm TRS_GEMM_AUTO resolves to for this descriptor (no launch). */
int32_t trs_matmul_select_algo(const trs_gemm_desc* desc, int32_t* algo);

/* Prepared operand planes for the tensor-core matmul.  New: the reference multiplies FP32 values
 * directly (src/tensor.rs:3919-3966) and needs no operand preparation.  The 3xTF32 split feeds the
 * tensor core each operand element a as hi = a with its low 13 mantissa bits dropped (read in place)
 * and lo = tf32(a - hi), which otherwise costs a pass over the operand in every call.  A reference
 * Storage is immutable after construction (src/storage.rs:7-18), so the lo values are a pure function
 * of a storage: a host may compute them once (trs_split_lo_f32), keep them beside the storage, and hand
 * them to every matmul that reads it; a matmul can also write the lo values of its own result while it
 * stores it, for the matmul that consumes the result next.
 *   a_lo / b_lo  lo image of A / B: the lo value of the element at a[i] is at a_lo[i], for every i the
 *                descriptor's strides reach (the same base offset and strides as the operand); NULL =
 *                prepare per call.  Ignored where the kernel has to re-lay the operand anyway
 *                (trs_matmul_plan tells).
 *   a_flag/b_flag device word that is non-zero when the operand holds an inf or NaN (as written by
 *                trs_split_lo_f32 or through c_flag); NULL = the caller vouches that all values are finite.
 *   c_lo         when non-NULL, the lo image of C is written alongside C (same layout as C).
 *   c_flag       device word, zeroed by the caller beforehand, set to 1 when C receives an inf or NaN;
 *                required with c_lo. */
typedef struct trs_gemm_planes {
    const float* a_lo;
    const float* b_lo;
    float* c_lo;
    const uint32_t* a_flag;
    const uint32_t* b_flag;
    uint32_t* c_flag;
} trs_gemm_planes;

/* lo[i] = tf32(src[i] - trunc_tf32(src[i])) for i in [0, count); *flag = 1 when any src[i] is inf / NaN,
 * else 0.  `src` and `lo` 16-byte aligned for full speed (any alignment works). */
int32_t trs_split_lo_f32(const float* src, int64_t count, float* lo, uint32_t* flag, trs_stream stream);
/* trs_matmul_f32 with prepared planes (`planes` may be NULL: identical to trs_matmul_f32).  The result
 * is bit-identical to the call without planes. */
int32_t trs_matmul_f32_planes(const trs_gemm_desc* desc, const trs_gemm_planes* planes, trs_stream stream);
/* What trs_matmul_f32_planes would do with this descriptor (no launch): the algorithm, and whether it
 * would read a prepared lo image of A / of B (0 when the operand is re-laid or the FP32 kernel runs). */
int32_t trs_matmul_plan(const trs_gemm_desc* desc, int32_t* algo, int32_t* a_plane_used, int32_t* b_plane_used);

/* ---- the one collective -------------------------------------------------------------------------
 * New: the reference has no distributed backend (python/torch_rs/distributed/distributed_c10d.py:39-74); a host
 * keeps its LOCAL_RANK convention (same file, 71-72) to choose `device`.  The data-parallel MLP step sums the
 * weight gradients of all ranks; everything else on the path shards with no exchange.  NCCL (NVLink / NVSwitch)
 * is loaded on first use; without it these return TRS_ERR_UNSUPPORTED.
 *   trs_comm_unique_id   rank 0 fills 128 bytes and hands them to every rank by any means the host has
 *   trs_comm_init_rank   collective over all ranks; one communicator per rank, bound to `device`
 *   trs_comm_allreduce_sum_f32  in place, enqueued on `stream` (same device); ordered like any other work on it
 *   trs_comm_destroy     after the stream has drained */
int32_t trs_comm_unique_id(char* id128);
int32_t trs_comm_init_rank(int32_t device, int32_t nranks, int32_t rank, const char* id128, trs_comm* comm);
int32_t trs_comm_allreduce_sum_f32(trs_comm comm, float* data, int64_t count, trs_stream stream);
int32_t trs_comm_info(trs_comm comm, int32_t* device, int32_t* nranks, int32_t* rank);
int32_t trs_comm_destroy(trs_comm comm);

/* ---- diagnostics -------------------------------------------------------------------------------- */
/* Test aid for the bounded waits of the matmul kernels (no reference counterpart): one warp waits at most
 * `limit_cycles` SM clocks (<= 1e8) on a barrier that nothing arrives on, through the kernels' own wait loop,
 * and reports the timeout the way they do -- the next trs_stream_sync / trs_device_sync on the device returns
 * TRS_ERR_DEVICE_STATUS once.  The kernel returns by itself; nothing traps or spins unbounded. */
int32_t trs_debug_wait_probe(trs_stream stream, int64_t limit_cycles);
const char* trs_status_string(int32_t status);
const char* trs_last_error_message(void);          /* thread-local, valid until the next failing call */
int64_t trs_kernel_launch_count(void);             /* kernels launched by this library since load */
int32_t trs_jit_cache_size(int32_t* entries);

#ifdef __cplusplus
}
#endif
#endif /* TRS_CUDA_H */
