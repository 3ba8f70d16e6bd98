/*
 * vkml_b200.h -- C ABI of the B200 (sm_100a) execution backend for vkML.
 *
 * This is the whole boundary between vkML's host framework and the CUDA
 * backend: plain pointers, sizes and POD structs, status codes instead of
 * exceptions, no C++ or torch types.  One `b200_ctx` is one CUDA device with
 * one compute stream; everything submitted through a context is ordered on
 * that stream.
 *
 * The only intended caller inside vkML is an adapter class deriving from
 * `vkml::Backend` (include/vkml/backend/api/backend.h:49-125); each entry
 * point below names the virtual it replaces.  Numeric values of `b200_op` and
 * `b200_dtype` equal vkML's `OpKind` (include/vkml/graph/op.h:30-139) and
 * `DType` (include/vkml/core/dtype.h:17-23) so a node is flattened by copying
 * fields, and `params` carries the raw 64 `OpParams` bytes
 * (include/vkml/graph/op.h:199-221).
 */
#ifndef VKML_B200_H
#define VKML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1
#define B200_MAX_DIMS 4   /* vkml::kMaxDims, include/vkml/core/shape.h:25 */
#define B200_MAX_SRC 4    /* vkml::kMaxSrc,  include/vkml/graph/op.h:148 */
#define B200_PARAM_BYTES 64

/* Status codes. Each maps to one vkML exception type
 * (include/vkml/util/error.h:7-38); the adapter rethrows. */
typedef enum b200_status {
    B200_OK = 0,
    B200_SHAPE_ERROR = 1,
    B200_DTYPE_ERROR = 2,
    B200_DEVICE_ERROR = 3,
    B200_INDEX_ERROR = 4,
    B200_NOT_IMPLEMENTED = 5,
    B200_INTERNAL_ERROR = 6,
    B200_OUT_OF_MEMORY = 7,
    B200_INVALID_ARGUMENT = 8,
    B200_TIMEOUT = 9
} b200_status;

/* vkml::DType */
typedef enum b200_dtype {
    B200_F32 = 0,
    B200_F16 = 1,
    B200_I32 = 2,
    B200_I64 = 3,
    B200_BOOL = 4
} b200_dtype;

/* vkml::OpKind, same order and values. */
typedef enum b200_op {
    B200_OP_INPUT = 0, B200_OP_CONST, B200_OP_FULL, B200_OP_ARANGE, B200_OP_RAND,
    B200_OP_RESHAPE, B200_OP_PERMUTE, B200_OP_SLICE, B200_OP_BROADCAST, B200_OP_SQUEEZE,
    B200_OP_UNSQUEEZE, B200_OP_CONTIGUOUS, B200_OP_CAST, B200_OP_CAT, B200_OP_ADD,
    B200_OP_SUB, B200_OP_MUL, B200_OP_SCALED_ADD, B200_OP_DIV, B200_OP_POW,
    B200_OP_MAXIMUM, B200_OP_MINIMUM, B200_OP_EQUAL, B200_OP_LESS, B200_OP_GREATER,
    B200_OP_LESS_EQUAL, B200_OP_GREATER_EQUAL, B200_OP_NOT_EQUAL, B200_OP_NEG, B200_OP_ABS,
    B200_OP_SIGN, B200_OP_SQUARE, B200_OP_SQRT, B200_OP_RSQRT, B200_OP_RECIPROCAL,
    B200_OP_EXP, B200_OP_LOG, B200_OP_ERF, B200_OP_ERFC, B200_OP_SIN,
    B200_OP_COS, B200_OP_TANH, B200_OP_SIGMOID, B200_OP_RELU, B200_OP_GELU,
    B200_OP_SILU, B200_OP_CLAMP, B200_OP_SUM, B200_OP_MEAN, B200_OP_MAX,
    B200_OP_MIN, B200_OP_PROD, B200_OP_ARGMAX, B200_OP_ARGMIN, B200_OP_MATMUL,
    B200_OP_SOFTMAX, B200_OP_LOG_SOFTMAX, B200_OP_IM2COL, B200_OP_COL2IM, B200_OP_MAX_POOL2D,
    B200_OP_MAX_POOL2D_BACKWARD, B200_OP_INDEX_SELECT, B200_OP_SCATTER_ADD,
    B200_OP_SLICE_BACKWARD, B200_OP_WHERE, B200_OP_TRIU, B200_OP_TRIL,
    B200_OP_COUNT
} b200_op;

/* A strided view of device memory: vkml::Shape (byte strides, rank <= 4,
 * stride 0 with extent > 1 marks a broadcast; include/vkml/core/shape.h:60-153)
 * plus the node's address `storage->data() + storage_offset`
 * (include/vkml/graph/node.h:144-149). */
typedef struct b200_tensor {
    void* data;
    int64_t dims[B200_MAX_DIMS];
    int64_t strides[B200_MAX_DIMS]; /* bytes */
    int32_t ndim;
    int32_t dtype; /* b200_dtype */
} b200_tensor;

/* One graph node as the backend sees it (vkml::Node, node.h:69-157). */
typedef struct b200_node {
    uint32_t op;    /* b200_op */
    uint32_t n_src; /* 0..4 */
    b200_tensor out;
    b200_tensor src[B200_MAX_SRC];
    uint8_t params[B200_PARAM_BYTES];
} b200_node;

/* vkml::BufferCopy (backend.h:18-24) with the storage base already added. */
typedef struct b200_copy {
    void* dst;
    const void* src;
    size_t nbytes;
} b200_copy;

/* Subset of vkml::DeviceCapabilities (capabilities.h:23-119) the adapter fills
 * from the device. */
typedef struct b200_caps {
    char name[128];
    int32_t cc_major, cc_minor;
    uint32_t sm_count;
    uint32_t warp_size;
    uint32_t max_threads_per_block;
    size_t max_shared_memory_bytes;
    size_t total_memory_bytes;
    size_t min_buffer_alignment;
} b200_caps;

/* Allocator and launch counters: the figures vkML's VulkanStats exposes
 * (include/vkml/backend/vulkan/vulkan_backend.h:41-58). */
typedef struct b200_stats {
    uint64_t reserved_bytes;     /* held from the driver */
    uint64_t in_use_bytes;       /* handed out and not yet freed */
    uint64_t peak_in_use_bytes;
    uint64_t live_allocations;
    uint64_t total_allocations;
    uint64_t driver_allocations; /* cudaMalloc calls: growth of the cache */
    uint64_t compute_calls;      /* b200_compute calls (= submissions) */
    uint64_t kernel_launches;    /* kernels launched by this library */
    uint64_t nodes_computed;
    uint64_t comm_bytes;         /* bytes all-reduced */
} b200_stats;

typedef struct b200_ctx b200_ctx;

/* b200_compute flags */
#define B200_COMPUTE_DEFAULT 0u
#define B200_COMPUTE_SYNC 1u        /* synchronise before returning (eager mode, executor.cpp:134-144) */
#define B200_COMPUTE_GRAD_SYNC 2u   /* all-reduce (average) the span's gradients across ranks: the buffers
                                       registered with b200_dist_mark_grad, or, when none are registered,
                                       every f32 output of the span that no later node of the span reads */

/* GEMM arithmetic: 3xTF32 split on the tensor cores (default), single-pass
 * TF32 (explicit opt-in), or plain fp32 FMA on the CUDA cores. */
typedef enum b200_gemm_precision {
    B200_GEMM_3XTF32 = 0,
    B200_GEMM_TF32 = 1,
    B200_GEMM_FP32 = 2
} b200_gemm_precision;

/* -- lifetime: replaces vkml::vulkan_backend(index) (vulkan_backend.cpp:2991) -- */
int b200_abi_version(void);
int b200_device_count(int* count);
int b200_create(int cuda_ordinal, b200_ctx** out);
void b200_destroy(b200_ctx* ctx);

/* Backend::capabilities() (backend.h:62). */
int b200_get_caps(b200_ctx* ctx, b200_caps* out);

/* Allocator::allocate / Storage deleter (allocator.h:44, storage.h:33).
 * Thread-safe; memory is recycled in stream order, so a buffer may be freed
 * while kernels that use it are still queued. nbytes == 0 yields *out = NULL. */
int b200_alloc(b200_ctx* ctx, size_t nbytes, void** out);
int b200_free(b200_ctx* ctx, void* ptr);
/* Return every cached, unused block to the driver. */
int b200_trim(b200_ctx* ctx);

/* Backend::supports(const Node&) (backend.h:67). 1 = can evaluate, 0 = cannot. */
int b200_supports(const b200_node* node);

/* Backend::compute(span<Node* const>) (backend.h:79): evaluates the non-view,
 * non-leaf nodes in order on the context's stream. Returns once the work is
 * ordered, not finished, unless B200_COMPUTE_SYNC is set. */
int b200_compute(b200_ctx* ctx, const b200_node* nodes, size_t n_nodes, uint32_t flags);

/* Backend::copy_from_host / copy_to_host (backend.h:82-86). copy_to_host
 * returns after the bytes are in `dst`. */
int b200_copy_from_host(b200_ctx* ctx, void* dst_device, const void* src_host, size_t nbytes);
int b200_copy_to_host(b200_ctx* ctx, void* dst_host, const void* src_device, size_t nbytes);

/* Backend::copy_device_to_device(span<const BufferCopy>) (backend.h:108):
 * disjoint ranges, one unit of work. */
int b200_copy_device_to_device(b200_ctx* ctx, const b200_copy* copies, size_t n);

/* Backend::synchronize() (backend.h:124). Also reports errors the device
 * recorded since the last call (an out-of-range index in index_select /
 * scatter_add -> B200_INDEX_ERROR; a bounded wait that ran out -> B200_TIMEOUT). */
int b200_synchronize(b200_ctx* ctx);

/* Text of the last error on this context (empty string if none). */
const char* b200_last_error(b200_ctx* ctx);
const char* b200_status_name(int status);

int b200_get_stats(b200_ctx* ctx, b200_stats* out);

/* Per-dispatch device timing, the counterpart of the Vulkan backend's timestamp
 * queries and last_profile() (include/vkml/backend/vulkan/vulkan_backend.h:163-203):
 * while enabled, every kernel launch is bracketed by CUDA events on the
 * context's stream. b200_profile_read synchronises, resolves the events into
 * (label, milliseconds) records in launch order and clears the list. */
typedef struct b200_profile_record {
    char label[48];
    float ms;
    uint32_t op;         /* b200_op of the node the launch belongs to */
    uint32_t submission; /* the b200_compute call it was launched by, counted from 1 per context */
} b200_profile_record;
int b200_profile_enable(b200_ctx* ctx, int on);
int b200_profile_read(b200_ctx* ctx, b200_profile_record* out, size_t capacity, size_t* count);

/* A stopwatch on the context's stream: begin records a CUDA event, end records
 * a second one, waits for it and returns the device time between them. */
int b200_timer_begin(b200_ctx* ctx);
int b200_timer_end(b200_ctx* ctx, float* milliseconds);

/* Page-locked host memory for uploads and downloads that should run at full
 * PCIe rate (the role of the Vulkan backend's staging buffers,
 * src/backend/vulkan/vulkan_backend.cpp:2720-2793). */
int b200_alloc_host(b200_ctx* ctx, size_t nbytes, void** out);
int b200_free_host(b200_ctx* ctx, void* ptr);

/* Matmul kernel policy: replaces the VKML_GEMM_* switches
 * (vulkan_backend.cpp:2160-2178). */
int b200_set_gemm_precision(b200_ctx* ctx, int precision);
int b200_get_gemm_precision(b200_ctx* ctx);
/* Which kernel family b200_compute would launch for this matmul node, and why: the fact the
 * Vulkan backend publishes under the site "matmul.kernel"
 * (vulkan_backend.cpp:2363-2375) so that a run can be tied to the arithmetic that produced it.
 * Names: fp32_simt (CUDA cores), tcgen05_3xtf32 (operand planes), tcgen05_3xtf32_stream (the large
 * operand streamed once through tensor memory), tcgen05_3xtf32_direct (fp32 tiles split inside
 * the kernel), and the tcgen05_tf32* forms under the plain-TF32 precision.  The node is judged by
 * itself: inside a span, planes shared with another matmul keep a product on the plane scheme. */
int b200_matmul_kernel(b200_ctx* ctx, const b200_node* node, char* name, size_t name_len, char* reason,
                       size_t reason_len);

/* The CUDA stream (cudaStream_t) every call on this context is ordered on, so
 * a caller that owns other device work can order against it with events. */
void* b200_stream(b200_ctx* ctx);

/* Diagnostic (no counterpart in vkML): queues one block that waits `limit_ns` (at most one second)
 * on a barrier nobody arrives on, through the bounded wait the GEMM kernels use.  The wait gives
 * up, the kernel returns by itself, and the next b200_synchronize / b200_copy_to_host reports
 * B200_TIMEOUT; the context stays usable.  Nothing faults and nothing hangs: it lets a caller's
 * handling of an expired device wait be tested. */
int b200_debug_expire_wait(b200_ctx* ctx, uint64_t limit_ns);

/* b200_compute replays a span that comes back unchanged (same nodes, same addresses, same library
 * state) as one CUDA graph: captured at its second sighting, launched from then on -- vkML's
 * planned "re-submit the cached command buffer" (docs/ARCHITECTURE.md:565-569) without any change
 * above the backend interface.  How many spans were served by a launch of a kept graph, and how
 * many graphs were captured.  VKML_B200_SPAN_GRAPHS=0 turns the cache off. */
int b200_span_graph_stats(b200_ctx* ctx, uint64_t* hits, uint64_t* captures);

/* -- data-parallel training (no counterpart in vkML, which is single-device:
 *    src/dispatch/executor.cpp:96-103). One process per GPU. -- */
#define B200_UNIQUE_ID_BYTES 128
int b200_dist_unique_id(void* out_id /* B200_UNIQUE_ID_BYTES */);
int b200_dist_init(b200_ctx* ctx, int rank, int world_size, const void* id);
/* The same with an explicit deadline: the communicator is created in NCCL's non-blocking mode and
 * polled; if the ranks have not all joined after `timeout_ms` it is aborted and the call returns
 * B200_TIMEOUT (0 = wait for ever, as ncclCommInitRank does).  b200_dist_init uses
 * VKML_B200_DIST_INIT_TIMEOUT_MS, default two minutes.  Once initialised, b200_synchronize also
 * polls NCCL's asynchronous error state and, with VKML_B200_COMM_TIMEOUT_MS set, gives outstanding
 * collectives that long before it aborts the communicator and reports B200_TIMEOUT. */
int b200_dist_init_deadline(b200_ctx* ctx, int rank, int world_size, const void* id, int timeout_ms);
int b200_dist_destroy(b200_ctx* ctx);
/* Average `count` f32 values in place across ranks on the communication
 * stream; ordered after everything submitted so far and before everything
 * submitted after b200_dist_wait. */
int b200_dist_all_reduce_mean(b200_ctx* ctx, void* data, size_t count);
int b200_dist_wait(b200_ctx* ctx);
/* Register gradient buffers: a b200_compute call with B200_COMPUTE_GRAD_SYNC
 * all-reduces each registered buffer as soon as the node that writes it has
 * been launched, overlapping communication with the rest of the span. */
int b200_dist_mark_grad(b200_ctx* ctx, void* data, size_t count);
int b200_dist_clear_grads(b200_ctx* ctx);

/* -- step tape (no counterpart in vkML today; its plan is to "re-submit the cached command
 *    buffer" of an unchanged step, docs/ARCHITECTURE.md:565-569) --
 *
 * A tape replays the backend calls of whole training steps -- the allocations, frees,
 * uploads, compute spans, batched device copies and downloads the framework's executor,
 * Tensor::from_host/to_host and assign() make (src/dispatch/executor.cpp:105-144,
 * src/core/tensor.cpp:101-111,178-201,397-425) -- from flat arrays of 64-bit words in which
 * buffers are named by position (prologue allocation j, or allocation j of the step d steps
 * back) instead of by address.  Each event becomes exactly one call of this ABI, in the
 * recorded order, so a replayed step does the same device work as the framework's step at
 * the host cost of native code.  The word format is documented in vkml_b200/csrc/tape.cu and
 * produced by vkml_b200/tape.py from a recorded program.
 *
 * `lookback` is how many steps back a template may refer.  A prologue template allocates the
 * buffers that live for the whole run (parameters, optimiser state); every other template is
 * one step.  `uploads[i]` / `downloads[i]` are the host buffers of the template's i-th upload /
 * download (a NULL upload leaves the device buffer as it is).  Spans recorded as gradient
 * spans are computed with `grad_sync_flags` (0 or B200_COMPUTE_GRAD_SYNC). */
typedef struct b200_tape b200_tape;
int b200_tape_create(b200_ctx* ctx, int lookback, b200_tape** out);
int b200_tape_add_template(b200_tape* tape, const int64_t* words, size_t n_words, int is_prologue, int* index);
int b200_tape_run(b200_tape* tape, int index, const void* const* uploads, size_t n_uploads,
                  void* const* downloads, size_t n_downloads, uint32_t grad_sync_flags);
/* Graph mode: once the allocator hands a step the same device addresses as an earlier step
 * (the steady state of training), the step's device work is captured from the stream into a
 * CUDA graph and later steps with those addresses are one cudaGraphLaunch.  Same kernels, same
 * order, same arguments as the eager replay.  Needs page-locked upload buffers at unchanged
 * addresses (b200_alloc_host); anything else, profiling, and gradient-synchronising steps fall
 * back to the eager replay by themselves.  A step then returns after its one synchronisation. */
int b200_tape_enable_graphs(b200_tape* tape, int on);
int b200_tape_stats(b200_tape* tape, uint64_t* steps, uint64_t* graph_launches, uint64_t* graph_captures);
void b200_tape_destroy(b200_tape* tape);

/* -- an entry point that allocates nothing (no counterpart in vkML: its backends
 *    always own an allocator) --
 *
 * out[c] = sum over r of in[r * row_pitch + c], f32, for callers that are not allowed
 * to allocate device memory: code inside a latency-critical loop or a host callback, a
 * process whose device memory was budgeted once at start-up, a plug-in that was given a
 * stream and buffers and nothing else.  It needs no b200_ctx.  The split reduction's
 * partial sums live in a fixed array inside the library image (4 MiB + 16 KiB, held on
 * every GPU the library is loaded on until the process exits), so:
 *   - cols may not exceed B200_NOALLOC_MAX_COLUMNS; larger inputs are refused with
 *     B200_INVALID_ARGUMENT and a message in `error` (use a sum node through b200_compute);
 *   - the first call on each device looks the array's device address up; make that call
 *     before any stream capture begins on that device;
 *   - every call shares the one array: calls that overlap on the GPU (different streams)
 *     race with each other and must be serialised by the caller.
 * `in`, `out` are device pointers, `row_pitch` is in elements (>= cols), `stream` is a
 * cudaStream_t (NULL = the default stream); the work is ordered on it, not finished, when
 * the call returns.  `error` (may be NULL) receives a message when the status is not B200_OK.
 * The summation order is fixed, so repeated calls give identical bytes. */
#define B200_NOALLOC_MAX_COLUMNS 1048576
int b200_sum_columns_f32_noalloc(const float* in, int64_t rows, int64_t cols, int64_t row_pitch,
                                 float* out, void* stream, char* error, size_t error_len);

#ifdef __cplusplus
}
#endif

#endif /* VKML_B200_H */
