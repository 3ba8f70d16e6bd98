// The backend context: one CUDA device, one compute stream, a caching
// allocator, a device status word and counters.
#pragma once

#include "common.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <utility>
#include <vector>

namespace b200 {

// Caching device allocator.
//
// vkML allocates a fresh buffer for every computed node
// (src/dispatch/executor.cpp:40-45) and drops it whenever the last handle goes
// away, possibly while kernels that use it are still queued.  All work of a
// context runs on ONE in-order stream, so a block that is freed and handed out
// again is only ever touched by later work on the same stream: recycling needs
// no events.  Blocks come from cudaMalloc in size classes and return to
// per-size free lists (lowest address first); nothing goes back to the driver until trim().
class CachingAllocator {
public:
    void* allocate(size_t nbytes);
    void release(void* ptr);
    size_t size_of(void* ptr);  // bytes of a block that is currently handed out (0 if unknown)
    void trim();
    ~CachingAllocator();

    uint64_t reserved = 0, in_use = 0, peak = 0, live = 0, total = 0, driver_allocs = 0;
    uint64_t driver_frees = 0;  // blocks handed back to the driver (trim, or making room after a failed allocation)

private:
    static size_t round_size(size_t n);
    std::mutex mu_;
    std::map<size_t, std::set<void*>> free_;      // size -> free blocks, lowest address handed out first
    std::unordered_map<void*, size_t> sizes_;     // every block ever handed out
    std::unordered_map<void*, size_t> live_;      // blocks currently out (ptr -> size)
};

// Words behind b200_ctx::d_counters: 4096 arrival counters of split reductions, 64 words for the
// persistent GEMM's tile counter, 1024 arrival counters of the streamed-operand GEMM's split-K fold.
constexpr size_t kArrivalCounters = 4096 + 64 + 1024;

struct DistState;  // dist.cu

struct ProfEntry {
    char label[48];
    uint32_t op;
    uint32_t submission;  // which b200_compute call the launch belongs to (counted from 1)
    cudaEvent_t begin, end;
};

struct GradBuffer {
    void* data;
    size_t count;
};

// A matmul operand as it lies in memory: `rows` lines of `cols` elements, batched.  Two uses of
// the same memory (a weight in forward and in the input-gradient product; an activation in
// forward and, transposed, in the weight-gradient product) give the same key.
struct PlaneKey {
    const void* src;
    int64_t v[8];  // rows, cols, row stride, column stride, inner batch extent, batch strides, batches
    bool operator<(const PlaneKey& o) const {
        if (src != o.src) return src < o.src;
        for (int i = 0; i < 8; ++i) {
            if (v[i] != o.v[i]) return v[i] < o.v[i];
        }
        return false;
    }
};

// The TF32 hi / lo planes of one operand, kept for the rest of the compute span.
struct PlaneEntry {
    float* hi;
    float* lo;
    size_t bytes;
    int uses_left;
    const char* src_begin;
    const char* src_end;
};

}  // namespace b200

namespace b200 {
class Uploader;
}

struct b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    b200::CachingAllocator alloc;    // the caller's buffers (b200_alloc / b200_free)
    // The library's own scratch (workspace, shared operand planes) comes from a second pool, so it
    // can never land on a block the caller has already freed on the host but whose last reader
    // is not queued yet (a replay that books a step's frees before issuing its work does that).
    b200::CachingAllocator scratch;

    uint32_t* d_status = nullptr;  // device status word (DeviceStatusBits)
    uint32_t* h_status = nullptr;  // pinned mirror
    unsigned* d_counters = nullptr;  // arrival counters of split reductions (self-resetting)

    // Scratch the library owns (GEMM operand splits, reduction partials). Grown
    // on demand, never shrunk; reused by every launch on the stream.
    void* workspace = nullptr;
    size_t workspace_bytes = 0;

    // Uploads from pageable host memory, staged through pinned slots by a few threads (upload.cu).
    // VKML_B200_UPLOAD_THREADS: 0 or 1 leave such copies to the runtime's own single-threaded staging.
    b200::Uploader* uploader = nullptr;
    int upload_threads = 4;  // set from the host's core count at creation (2..8)

    int gemm_precision = B200_GEMM_3XTF32;
    // VKML_B200_GEMM_SCHEDULE: how the persistent GEMM's CTAs get their tiles. -1 (auto): a fixed
    // round-robin walk, except in a gradient-synchronising span, where tiles are drawn from a
    // counter so that CTAs sharing their SM with an all-reduce do not stretch the kernel; 0 / 1
    // force the fixed / drawn order.
    int gemm_schedule = -1;
    // VKML_B200_GEMM_OPERANDS: planes (0) = split each operand into TF32 planes in HBM first; direct (1)
    // = the GEMM kernel reads fp32 operands and splits them on the way into shared memory; auto (-1).
    int gemm_operands = -1;
    // VKML_B200_GEMM_STREAM: the streamed-operand kernel for products bound by HBM (a small left
    // operand or a short K, the large right operand read exactly once).  auto (-1): such products,
    // where the layout allows it and no other operand scheme was asked for by name; 0: never; 1:
    // every product whose layout allows it, whatever its size (A/B runs).
    int gemm_stream = -1;
    int gemm_group_m = 0;      // VKML_B200_GEMM_GROUP_M: M-tiles per L2 group of the tile walk (0: the built-in 16)
    int gemm_bn_override = 0;  // VKML_B200_GEMM_BN: force the N extent of the tensor-core tile (tuning aid)
    // SMs the persistent GEMM kernel leaves free while a span's gradients are being all-reduced,
    // so the communication kernels always find room (VKML_B200_COMM_SMS, default 0: measured no gain at 2 GPUs).
    int comm_sms = 0;
    // Hoist each gradient-producing node of a grad-sync span to just after its last input
    // is produced, so its all-reduce overlaps the rest of backward (VKML_B200_HOIST_GRADIENTS).
    bool hoist_gradients = false;  // measured at 2 GPUs: 13.5 ms/step hoisted, 13.1 ms in the recorded order
    // Lazy joining (VKML_B200_LAZY_JOIN, default on): a gradient span returns without waiting for its
    // all-reduces; the compute stream waits for each one where its buffer is next touched, and the
    // nodes of a later span are taken in the order their gradients arrive, so the optimiser's
    // updates of the early-reduced parameters run under the tail of the communication.
    bool lazy_join = true;
    bool bucket_grads = true;  // small gradients of a span leave as one grouped NCCL launch (VKML_B200_BUCKET)
    size_t bucket_flush_bytes = size_t(1) << 20;  // ... which leaves when it holds this much (VKML_B200_BUCKET_FLUSH_BYTES), or at the end of the span
    bool fuse = true;  // in-span fusion of the node sequences autograd always emits (VKML_B200_FUSE, fuse.cu)
    bool pdl = true;  // programmatic dependent launch between consecutive kernels (VKML_B200_PDL)
    bool in_grad_sync_span = false;
    bool comm_pending = false;  // an all-reduce was issued in this span and has not been joined yet

    std::atomic<uint64_t> compute_calls{0}, kernel_launches{0}, nodes_computed{0}, comm_bytes{0};

    std::mutex err_mu;
    std::string last_error;

    cudaEvent_t timer_begin = nullptr, timer_end = nullptr;
    bool profiling = false;
    bool capturing = false;  // the stream is being captured into a CUDA graph (tape.cu): no events, no waits
    uint32_t current_op = 0;
    std::vector<b200::ProfEntry> prof;
    std::vector<cudaEvent_t> event_pool;

    // Spans that come back unchanged -- same nodes, same addresses, same library state -- are replayed
    // as one CUDA graph each (context.cu, span_graph_*): a training loop driven through
    // Backend::compute is handed the same addresses again every few steps, so after a short
    // warm-up its large spans cost one launch.  VKML_B200_SPAN_GRAPHS=0 turns it off.
    struct SpanGraph {
        cudaGraphExec_t exec = nullptr;
        std::vector<unsigned char> nodes;  // the span it was captured from, byte for byte
        uint64_t launches = 0, node_count = 0;
        uint64_t state = 0;                // library state it depends on (see span_graph_state)
    };
    std::unordered_map<uint64_t, SpanGraph> span_graphs;
    std::unordered_map<uint64_t, uint32_t> span_seen;
    bool span_graph_cache = true;
    uint64_t span_graph_hits = 0, span_graph_captures = 0;

    b200::DistState* dist = nullptr;
    std::vector<b200::GradBuffer> grads;

    // Operand planes shared between the matmuls of ONE compute span (gemm_tc.cu).  A span's
    // outputs are distinct live buffers, each written once by its producer before any reader
    // (include/vkml/backend/api/backend.h:34-45), so a plane stays valid until the span ends.
    std::map<b200::PlaneKey, int> plane_uses;               // counted before the span runs
    std::map<b200::PlaneKey, b200::PlaneEntry> plane_cache;
    size_t plane_cache_bytes = 0;
    bool share_planes = true;  // VKML_B200_SHARE_PLANES=0 splits every operand afresh (A/B aid)
    uint64_t plane_hits = 0;

    void* ensure_workspace(size_t nbytes);
    void count_launch(uint64_t n = 1) { kernel_launches.fetch_add(n, std::memory_order_relaxed); }
};

namespace b200 {

// The one place kernels are launched from.  With programmatic dependent launch enabled
// (VKML_B200_PDL, default on) the launch carries the stream-serialization attribute that
// pdl_prologue() in the kernels relies on.
template <typename... Params, typename... Args>
inline void launch_kernel(b200_ctx* ctx, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    // a failed launch is picked up by check_last_launch() at the call site
    (void)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Per-family launchers (one translation unit each). Each reads the node, picks a
// kernel from the operand layouts, and launches on ctx->stream.
void launch_elementwise(b200_ctx* ctx, const b200_node& node);  // unary, binary, compare, where, scaled_add, cast, contiguous, full, arange, rand, tri, cat, slice_backward
void launch_reduce(b200_ctx* ctx, const b200_node& node);       // sum, mean, max, min, argmax, argmin
void launch_softmax(b200_ctx* ctx, const b200_node& node);      // softmax, log_softmax
void launch_movement(b200_ctx* ctx, const b200_node& node);     // im2col, col2im, max_pool2d(+backward), index_select, scatter_add
void launch_matmul(b200_ctx* ctx, const b200_node& node);       // matmul (all kernels)

bool supports_node(const b200_node& node);

// fuse.cu: serves the head of `seq` (the span's remaining computed nodes, in execution order)
// with one fused launch if it matches a known pattern; returns how many nodes it covered, or 0.
size_t launch_fused(b200_ctx* ctx, const b200_node* const* seq, size_t avail);
// movement.cu: max_pool2d_backward + the where() of ReLU's backward rule behind it, one launch; false: not that case
bool launch_pool_backward_where(b200_ctx* ctx, const b200_node& pool, const b200_node& where, int result_is_x,
                                const void* constant);
// elementwise.cu: the leading run of tiny elementwise nodes (a loss prologue) as one single-block launch
size_t launch_tiny_chain(b200_ctx* ctx, const b200_node* const* seq, size_t avail);
size_t launch_scaled_add_group(b200_ctx* ctx, const b200_node* const* seq, size_t avail, bool* picked);

// dist.cu
void dist_destroy(b200_ctx* ctx);
void dist_after_node(b200_ctx* ctx, const b200_node& node);  // all-reduce a registered gradient once its producer is queued
void dist_all_reduce_now(b200_ctx* ctx, void* data, size_t count);  // average across ranks on the comm stream
void dist_join(b200_ctx* ctx);                                // make the compute stream wait for outstanding all-reduces
// upload.cu: true when the copy was served by the threaded staging (src is reusable on return)
bool staged_upload(b200_ctx* ctx, void* dst, const void* src, size_t nbytes);
void destroy_uploader(b200_ctx* ctx);
void dist_wait_range(b200_ctx* ctx, const void* lo, const void* hi);  // ... for those touching [lo, hi) (nullptr: all)
int dist_pending_index(const b200_ctx* ctx, const void* lo, const void* hi);
bool dist_has_pending(const b200_ctx* ctx);
void dist_check_health(b200_ctx* ctx);  // asynchronous NCCL errors and the host deadline for collectives

void check_last_launch(const char* what);

// Brackets the launches made inside its lifetime with CUDA events when profiling is on.
class ProfScope {
public:
    ProfScope(b200_ctx* ctx, const char* label);
    ~ProfScope();
    ProfScope(const ProfScope&) = delete;
    ProfScope& operator=(const ProfScope&) = delete;

private:
    b200_ctx* ctx_;
    int index_ = -1;
};

const char* op_label(uint32_t op);

}  // namespace b200
