// C-ABI entry points, the caching allocator and the per-node dispatch.
#include "context.h"
#include "gemm.h"

#include <algorithm>
#include <cstdlib>
#include <new>
#include <thread>

namespace b200 {

void check_last_launch(const char* what) {
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        cudaGetLastError();  // clear the sticky launch error so the context stays usable
        fail(B200_DEVICE_ERROR, std::string(what) + ": launch failed: " + cudaGetErrorString(err));
    }
}

ProfScope::ProfScope(b200_ctx* ctx, const char* label) : ctx_(ctx) {
    if (!ctx->profiling || ctx->capturing) {
        return;
    }
    ProfEntry e{};
    std::snprintf(e.label, sizeof(e.label), "%s", label);
    e.op = ctx->current_op;
    e.submission = static_cast<uint32_t>(ctx->compute_calls.load(std::memory_order_relaxed));
    // events are recycled: creating a pair per launch would cost more than a small kernel
    for (cudaEvent_t* ev : {&e.begin, &e.end}) {
        if (!ctx->event_pool.empty()) {
            *ev = ctx->event_pool.back();
            ctx->event_pool.pop_back();
        } else if (cudaEventCreate(ev) != cudaSuccess) {
            cudaGetLastError();
            if (ev == &e.end) ctx->event_pool.push_back(e.begin);
            return;
        }
    }
    cudaEventRecord(e.begin, ctx->stream);
    ctx->prof.push_back(e);
    index_ = static_cast<int>(ctx->prof.size()) - 1;
}

ProfScope::~ProfScope() {
    if (index_ >= 0) {
        cudaEventRecord(ctx_->prof[static_cast<size_t>(index_)].end, ctx_->stream);
    }
}

const char* op_label(uint32_t op) {
    static const char* const names[B200_OP_COUNT] = {
        "input", "const", "full", "arange", "rand", "reshape", "permute", "slice", "broadcast", "squeeze",
        "unsqueeze", "contiguous", "cast", "cat", "add", "sub", "mul", "scaled_add", "div", "pow", "maximum",
        "minimum", "equal", "less", "greater", "less_equal", "greater_equal", "not_equal", "neg", "abs", "sign",
        "square", "sqrt", "rsqrt", "reciprocal", "exp", "log", "erf", "erfc", "sin", "cos", "tanh", "sigmoid",
        "relu", "gelu", "silu", "clamp", "sum", "mean", "max", "min", "prod", "argmax", "argmin", "matmul",
        "softmax", "log_softmax", "im2col", "col2im", "max_pool2d", "max_pool2d_backward", "index_select",
        "scatter_add", "slice_backward", "where", "triu", "tril"};
    return op < B200_OP_COUNT ? names[op] : "?";
}

// ---------------------------------------------------------------------------
// CachingAllocator
// ---------------------------------------------------------------------------

size_t CachingAllocator::round_size(size_t n) {
    // 512-byte classes up to 1 MiB, 2 MiB classes above: a freed activation
    // buffer is then reusable by the next step's buffer of the same shape, and
    // near-equal shapes share a class.
    if (n <= (size_t(1) << 20)) {
        return (n + 511) & ~size_t(511);
    }
    const size_t mb2 = size_t(2) << 20;
    return (n + mb2 - 1) / mb2 * mb2;
}

void* CachingAllocator::allocate(size_t nbytes) {
    if (nbytes == 0) {
        return nullptr;
    }
    const size_t size = round_size(nbytes);
    std::lock_guard<std::mutex> lock(mu_);
    void* ptr = nullptr;
    auto it = free_.lower_bound(size);
    // accept a cached block up to 25 % larger than needed; within a class the lowest address goes
    // out first.  The allocator's state is then the SET of free blocks, with no memory of the
    // order they were freed in, so a loop that allocates and frees the same shapes every
    // iteration is handed the same addresses again after a few iterations (2 to 6 for the
    // recorded training steps) -- which is what lets a step be replayed as a CUDA graph.
    if (it != free_.end() && it->first <= size + size / 4) {
        ptr = *it->second.begin();
        it->second.erase(it->second.begin());
        if (it->second.empty()) free_.erase(it);
    } else {
        cudaError_t err = cudaMalloc(&ptr, size);
        if (err != cudaSuccess) {
            // give the cache back to the driver and try once more
            cudaGetLastError();
            for (auto& kv : free_) {
                for (void* block : kv.second) {
                    cudaFree(block);
                    reserved -= kv.first;
                    sizes_.erase(block);
                    ++driver_frees;
                }
            }
            free_.clear();
            err = cudaMalloc(&ptr, size);
            if (err != cudaSuccess) {
                cudaGetLastError();
                fail(B200_OUT_OF_MEMORY, "device allocation of " + std::to_string(size) +
                                             " bytes failed: " + cudaGetErrorString(err));
            }
        }
        sizes_[ptr] = size;
        reserved += size;
        ++driver_allocs;
    }
    const size_t got = sizes_[ptr];
    live_[ptr] = got;
    in_use += got;
    peak = std::max(peak, in_use);
    ++live;
    ++total;
    return ptr;
}

void CachingAllocator::release(void* ptr) {
    if (ptr == nullptr) {
        return;
    }
    std::lock_guard<std::mutex> lock(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) {
        fail(B200_INVALID_ARGUMENT, "b200_free: pointer was not allocated by this context");
    }
    in_use -= it->second;
    --live;
    free_[it->second].insert(ptr);
    live_.erase(it);
}

size_t CachingAllocator::size_of(void* ptr) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = live_.find(ptr);
    return it == live_.end() ? 0 : it->second;
}

void CachingAllocator::trim() {
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& kv : free_) {
        for (void* block : kv.second) {
            cudaFree(block);
            reserved -= kv.first;
            sizes_.erase(block);
            ++driver_frees;
        }
    }
    free_.clear();
}

CachingAllocator::~CachingAllocator() {
    for (auto& kv : sizes_) {
        cudaFree(kv.first);
    }
}

// ---------------------------------------------------------------------------
// supports / dispatch
// ---------------------------------------------------------------------------

namespace {

bool is_view_or_leaf(uint32_t op) {
    return op == B200_OP_INPUT || op == B200_OP_CONST ||
           (op >= B200_OP_RESHAPE && op <= B200_OP_UNSQUEEZE);
}

bool dense(const b200_tensor& t) {
    int64_t numel = 1;
    for (int i = 0; i < t.ndim; ++i) numel *= t.dims[i];
    if (numel == 0) return true;
    int64_t expected = static_cast<int64_t>(dtype_size(t.dtype));
    for (int i = t.ndim - 1; i >= 0; --i) {
        if (t.dims[i] == 1) continue;
        if (t.strides[i] != expected) return false;
        expected *= t.dims[i];
    }
    return true;
}

bool srcs_f32(const b200_node& n, int count) {
    if (static_cast<int>(n.n_src) < count) return false;
    for (int i = 0; i < count; ++i) {
        if (n.src[i].dtype != B200_F32) return false;
    }
    return true;
}

bool cast_pair_ok(int from, int to) {
    if (from == to) return true;
    switch (from) {
        case B200_F32: return to == B200_I32 || to == B200_I64 || to == B200_BOOL || to == B200_F16;
        case B200_F16: return to == B200_F32;
        case B200_I32: return to == B200_F32 || to == B200_I64;
        case B200_I64: return to == B200_F32 || to == B200_I32;
        case B200_BOOL: return to == B200_F32 || to == B200_I64;
        default: return false;
    }
}

GemmProblem matmul_problem(const b200_node& node) {
    const View out = make_view(node.out);
    const View a = make_view(node.src[0]);
    const View b = make_view(node.src[1]);
    if (node.out.ndim != 4 || node.src[0].ndim != 4 || node.src[1].ndim != 4) {
        fail(B200_SHAPE_ERROR, "matmul expects rank-4 operands");
    }
    if (out.dtype != B200_F32 || a.dtype != B200_F32 || b.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, "matmul: only f32 is implemented");
    }
    if (!out.contiguous) {
        fail(B200_NOT_IMPLEMENTED, "matmul output must be contiguous");
    }
    GemmProblem p{};
    p.a = reinterpret_cast<const float*>(a.data);
    p.b = reinterpret_cast<const float*>(b.data);
    p.out = reinterpret_cast<float*>(out.data);
    p.b0 = out.dim[0];
    p.b1 = out.dim[1];
    p.m = out.dim[2];
    p.n = out.dim[3];
    p.k = a.dim[3];
    if (b.dim[2] != p.k || a.dim[2] != p.m || b.dim[3] != p.n || a.dim[0] != p.b0 ||
        a.dim[1] != p.b1 || b.dim[0] != p.b0 || b.dim[1] != p.b1) {
        fail(B200_SHAPE_ERROR, "matmul: operand extents disagree");
    }
    for (int i = 0; i < 4; ++i) {
        p.a_s[i] = a.stride[i];
        p.b_s[i] = b.stride[i];
    }
    return p;
}

void dispatch_matmul(b200_ctx* ctx, const b200_node& node) {
    const GemmProblem p = matmul_problem(node);
    if (ctx->gemm_precision != B200_GEMM_FP32 && gemm_tc_eligible(ctx, p)) {
        gemm_tc(ctx, p, ctx->gemm_precision == B200_GEMM_3XTF32);
    } else {
        gemm_simt(ctx, p);
    }
}

// Counts, before a span runs, how often each operand matrix feeds a tensor-core matmul, so
// that a matrix used twice (a weight in forward and backward, an activation in forward and in
// the weight gradient) is split into its TF32 planes only once.
void count_matmul_operands(b200_ctx* ctx, const b200_node* nodes, size_t n_nodes) {
    if (ctx->gemm_precision == B200_GEMM_FP32 || !ctx->share_planes) return;
    size_t matmuls = 0;
    for (size_t i = 0; i < n_nodes; ++i) matmuls += nodes[i].op == B200_OP_MATMUL ? 1 : 0;
    if (matmuls < 2) return;
    for (size_t i = 0; i < n_nodes; ++i) {
        const b200_node& node = nodes[i];
        if (node.op != B200_OP_MATMUL || node.out.data == nullptr || node.n_src < 2 ||
            node.src[0].data == nullptr || node.src[1].data == nullptr) {
            continue;
        }
        try {
            const GemmProblem p = matmul_problem(node);
            if (p.b0 * p.b1 * p.m * p.n * p.k != 0 && gemm_tc_eligible(ctx, p)) {
                gemm_tc_note_uses(ctx, p);
            }
        } catch (const Error&) {
            // reported when the node is dispatched
        }
    }
}

bool touches_f16(const b200_node& n) {
    if (n.op == B200_OP_CAST || n.op == B200_OP_FULL) return false;  // these handle F16 themselves
    if (n.out.dtype == B200_F16) return true;
    for (uint32_t s = 0; s < n.n_src && s < B200_MAX_SRC; ++s) {
        if (n.src[s].dtype == B200_F16) return true;
    }
    return false;
}

b200_tensor dense_f32_like(const b200_tensor& like, void* data) {
    b200_tensor t = like;
    t.dtype = B200_F32;
    t.data = data;
    int64_t stride = 4;
    for (int d = like.ndim - 1; d >= 0; --d) {
        t.strides[d] = stride;
        stride *= like.dims[d];
    }
    return t;
}

void dispatch_node(b200_ctx* ctx, const b200_node& node);

// F16 is storage, never arithmetic, in vkML (src/backend/cpu/kernels_elementwise.cpp:89-99; fp32
// accumulation everywhere, docs/ARCHITECTURE.md 7.3): every kernel widens Half on load, computes in
// float and narrows once, round-to-nearest-even, on store.  A node that touches F16 therefore runs
// here as the same node on widened copies with the result narrowed -- bit-identical to the CPU
// backend's Half kernels for every family (pinned on the CPU by the oracle tests) -- at the price
// of the temporaries' traffic.  It is the coverage path; the fp32 kernels are the tuned ones.
void dispatch_f16(b200_ctx* ctx, const b200_node& node) {
    b200_node w = node;
    void* temps[B200_MAX_SRC + 1] = {};
    struct Release {
        b200_ctx* c;
        void** t;
        ~Release() {
            for (int i = 0; i <= B200_MAX_SRC; ++i) {
                if (t[i] != nullptr) c->scratch.release(t[i]);  // stream-ordered: safe with work queued
            }
        }
    } release{ctx, temps};
    auto numel_of = [](const b200_tensor& t) {
        int64_t n = 1;
        for (int d = 0; d < t.ndim; ++d) n *= t.dims[d];
        return n;
    };
    for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
        if (node.src[s].dtype != B200_F16) continue;
        const int64_t n = numel_of(node.src[s]);
        temps[s] = ctx->scratch.allocate(static_cast<size_t>(std::max<int64_t>(n, 1)) * 4);
        b200_node c{};
        c.op = B200_OP_CAST;
        c.n_src = 1;
        c.src[0] = node.src[s];
        c.out = dense_f32_like(node.src[s], temps[s]);
        if (n > 0) {
            ProfScope scope(ctx, "f16.widen");
            launch_elementwise(ctx, c);
        }
        w.src[s] = c.out;
    }
    if (node.out.dtype == B200_F16) {
        const int64_t n = numel_of(node.out);
        temps[B200_MAX_SRC] = ctx->scratch.allocate(static_cast<size_t>(std::max<int64_t>(n, 1)) * 4);
        w.out = dense_f32_like(node.out, temps[B200_MAX_SRC]);
    }
    dispatch_node(ctx, w);
    if (node.out.dtype == B200_F16) {
        b200_node c{};
        c.op = B200_OP_CAST;
        c.n_src = 1;
        c.src[0] = w.out;
        c.out = node.out;
        ctx->current_op = B200_OP_CAST;
        ProfScope scope(ctx, "f16.narrow");
        launch_elementwise(ctx, c);
    }
}

void dispatch_node(b200_ctx* ctx, const b200_node& node) {
    const uint32_t op = node.op;
    ctx->current_op = op;
    if (touches_f16(node)) {
        // the elementwise families read and write half storage themselves (elementwise.cu, HalfIO);
        // everything else runs on widened copies
        const bool elementwise = op == B200_OP_WHERE || op == B200_OP_SCALED_ADD || op == B200_OP_CLAMP ||
                                 (op >= B200_OP_ADD && op <= B200_OP_NOT_EQUAL) || (op >= B200_OP_NEG && op <= B200_OP_SILU);
        bool all_half = true;
        for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
            all_half = all_half && node.src[s].dtype != B200_F32;
        }
        if (elementwise && all_half && node.out.dtype != B200_F32) {
            ProfScope scope(ctx, op_label(op));
            launch_elementwise(ctx, node);
        } else {
            dispatch_f16(ctx, node);
        }
        return;
    }
    if (op == B200_OP_MATMUL) {
        dispatch_matmul(ctx, node);  // times its kernels one by one
        return;
    }
    ProfScope scope(ctx, op_label(op));
    if (op == B200_OP_SOFTMAX || op == B200_OP_LOG_SOFTMAX) {
        launch_softmax(ctx, node);
    } else if (op >= B200_OP_SUM && op <= B200_OP_ARGMIN) {
        launch_reduce(ctx, node);
    } else if (op == B200_OP_IM2COL || op == B200_OP_COL2IM || op == B200_OP_MAX_POOL2D ||
               op == B200_OP_MAX_POOL2D_BACKWARD || op == B200_OP_INDEX_SELECT ||
               op == B200_OP_SCATTER_ADD) {
        launch_movement(ctx, node);
    } else {
        launch_elementwise(ctx, node);
    }
}

void set_error(b200_ctx* ctx, const std::string& msg) {
    if (ctx == nullptr) return;
    std::lock_guard<std::mutex> lock(ctx->err_mu);
    ctx->last_error = msg;
}

// Runs `fn`, converting Error / bad_alloc into a status code and message.
template <typename Fn>
int guarded(b200_ctx* ctx, Fn&& fn) {
    try {
        if (ctx != nullptr) {
            cudaError_t err = cudaSetDevice(ctx->device);
            if (err != cudaSuccess) {
                set_error(ctx, std::string("cudaSetDevice: ") + cudaGetErrorString(err));
                return B200_DEVICE_ERROR;
            }
        }
        fn();
        return B200_OK;
    } catch (const Error& e) {
        set_error(ctx, e.message);
        return e.status;
    } catch (const std::bad_alloc&) {
        set_error(ctx, "host allocation failed");
        return B200_OUT_OF_MEMORY;
    } catch (const std::exception& e) {
        set_error(ctx, e.what());
        return B200_INTERNAL_ERROR;
    }
}

}  // namespace

// Mirrors VulkanBackend::supports (src/backend/vulkan/vulkan_backend.cpp:1012-1187):
// f32 natively, f16 storage through widened copies (dispatch_f16).  Honest rather than optimistic:
// a false here becomes NotImplementedError at realize, there is no fallback.
bool supports_node(const b200_node& n) {
    const uint32_t op = n.op;
    if (is_view_or_leaf(op)) return true;
    if (op >= B200_OP_COUNT) return false;
    if (n.n_src > B200_MAX_SRC) return false;
    if (!dense(n.out)) return false;
    if (touches_f16(n)) {
        // vkML's rule for its GPU backend: the floating operands and the result share one dtype
        // (vulkan_backend.cpp:1055-1184); the node then runs as its f32 self on widened copies
        b200_node w = n;
        auto widen = [](b200_tensor& t) {
            t.dtype = B200_F32;
            for (int d = 0; d < t.ndim; ++d) t.strides[d] *= 2;
        };
        bool f32_seen = n.out.dtype == B200_F32;
        if (n.out.dtype == B200_F16) widen(w.out);
        for (uint32_t s = 0; s < n.n_src; ++s) {
            f32_seen = f32_seen || n.src[s].dtype == B200_F32;
            if (n.src[s].dtype == B200_F16) widen(w.src[s]);
        }
        if (op == B200_OP_RAND) return false;  // F32 only in vkML as well (vulkan_backend.cpp:1037)
        return !f32_seen && supports_node(w);
    }
    const int dt = n.out.dtype;
    switch (op) {
        case B200_OP_FULL: return dt == B200_F32 || dt == B200_F16 || dt == B200_I64 || dt == B200_I32 || dt == B200_BOOL;
        case B200_OP_ARANGE: return dt == B200_F32 || dt == B200_I64;
        case B200_OP_RAND: return dt == B200_F32;
        case B200_OP_CONTIGUOUS: return n.n_src >= 1 && n.src[0].dtype == dt;
        case B200_OP_CAST: return n.n_src >= 1 && cast_pair_ok(n.src[0].dtype, dt);
        case B200_OP_CAT: return dt == B200_F32 && srcs_f32(n, 2);
        case B200_OP_SCALED_ADD:
        case B200_OP_ADD: case B200_OP_SUB: case B200_OP_MUL: case B200_OP_DIV: case B200_OP_POW:
        case B200_OP_MAXIMUM: case B200_OP_MINIMUM:
            return dt == B200_F32 && srcs_f32(n, 2);
        case B200_OP_EQUAL: case B200_OP_LESS: case B200_OP_GREATER: case B200_OP_LESS_EQUAL:
        case B200_OP_GREATER_EQUAL: case B200_OP_NOT_EQUAL:
            return dt == B200_BOOL && srcs_f32(n, 2);
        case B200_OP_WHERE:
            return dt == B200_F32 && n.n_src >= 3 && n.src[0].dtype == B200_BOOL &&
                   n.src[1].dtype == B200_F32 && n.src[2].dtype == B200_F32;
        case B200_OP_TRIU: case B200_OP_TRIL: return dt == B200_F32 && srcs_f32(n, 1) && n.out.ndim >= 2;
        case B200_OP_SUM: case B200_OP_MEAN: case B200_OP_MAX: case B200_OP_MIN:
        case B200_OP_PROD:  // in index order, as on the CPU (vkML's own GPU backend declines it)
            return dt == B200_F32 && srcs_f32(n, 1);
        case B200_OP_ARGMAX: case B200_OP_ARGMIN: return dt == B200_I64 && srcs_f32(n, 1);
        case B200_OP_MATMUL: return dt == B200_F32 && srcs_f32(n, 2) && n.out.ndim == 4;
        case B200_OP_SOFTMAX: case B200_OP_LOG_SOFTMAX: return dt == B200_F32 && srcs_f32(n, 1);
        case B200_OP_IM2COL: case B200_OP_COL2IM: case B200_OP_MAX_POOL2D:
            return dt == B200_F32 && srcs_f32(n, 1);
        case B200_OP_MAX_POOL2D_BACKWARD: return dt == B200_F32 && srcs_f32(n, 2);
        case B200_OP_INDEX_SELECT:
            return (dtype_size(dt) == 4 || dtype_size(dt) == 8) && n.n_src >= 2 &&
                   n.src[0].dtype == dt && n.src[1].dtype == B200_I64;
        case B200_OP_SCATTER_ADD:
            return dt == B200_F32 && n.n_src >= 2 && n.src[0].dtype == B200_F32 &&
                   n.src[1].dtype == B200_I64;
        case B200_OP_SLICE_BACKWARD: return dt == B200_F32 && srcs_f32(n, 1);
        default:
            if (op >= B200_OP_NEG && op <= B200_OP_CLAMP) return dt == B200_F32 && srcs_f32(n, 1);
            return false;
    }
}

}  // namespace b200

void* b200_ctx::ensure_workspace(size_t nbytes) {
    if (nbytes <= workspace_bytes) {
        return workspace;
    }
    // Work already queued may still be using the old buffer; the stream is
    // in-order, so freeing it through the stream-ordered cache is safe.
    if (workspace != nullptr) {
        scratch.release(workspace);
        workspace = nullptr;
        workspace_bytes = 0;
    }
    const size_t want = std::max(nbytes, size_t(8) << 20);
    workspace = scratch.allocate(want);
    workspace_bytes = want;
    return workspace;
}

using namespace b200;

extern "C" {

int b200_abi_version(void) { return B200_ABI_VERSION; }

const char* b200_status_name(int status) {
    switch (status) {
        case B200_OK: return "ok";
        case B200_SHAPE_ERROR: return "shape error";
        case B200_DTYPE_ERROR: return "dtype error";
        case B200_DEVICE_ERROR: return "device error";
        case B200_INDEX_ERROR: return "index error";
        case B200_NOT_IMPLEMENTED: return "not implemented";
        case B200_INTERNAL_ERROR: return "internal error";
        case B200_OUT_OF_MEMORY: return "out of memory";
        case B200_INVALID_ARGUMENT: return "invalid argument";
        case B200_TIMEOUT: return "timeout";
        default: return "unknown status";
    }
}

int b200_device_count(int* count) {
    if (count == nullptr) return B200_INVALID_ARGUMENT;
    int n = 0;
    const cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess) {
        cudaGetLastError();
        *count = 0;
        return B200_DEVICE_ERROR;
    }
    *count = n;
    return B200_OK;
}

int b200_create(int cuda_ordinal, b200_ctx** out) {
    if (out == nullptr) return B200_INVALID_ARGUMENT;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || cuda_ordinal < 0 || cuda_ordinal >= n) {
        cudaGetLastError();
        return B200_DEVICE_ERROR;  // no CUDA device: there is no CPU fallback in this library
    }
    b200_ctx* ctx = new (std::nothrow) b200_ctx();
    if (ctx == nullptr) return B200_OUT_OF_MEMORY;
    ctx->device = cuda_ordinal;
    const int rc = guarded(ctx, [&] {
        B200_CUDA_CHECK(cudaGetDeviceProperties(&ctx->prop, cuda_ordinal));
        if (ctx->prop.major != 10) {
            fail(B200_DEVICE_ERROR, std::string("device '") + ctx->prop.name +
                                        "' is not compute capability 10.x; this library is built for sm_100a only");
        }
        B200_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        B200_CUDA_CHECK(cudaMalloc(&ctx->d_status, sizeof(uint32_t)));
        B200_CUDA_CHECK(cudaMemset(ctx->d_status, 0, sizeof(uint32_t)));
        B200_CUDA_CHECK(cudaMalloc(&ctx->d_counters, sizeof(unsigned) * kArrivalCounters));
        B200_CUDA_CHECK(cudaMemset(ctx->d_counters, 0, sizeof(unsigned) * kArrivalCounters));
        B200_CUDA_CHECK(cudaMallocHost(&ctx->h_status, sizeof(uint32_t)));
        *ctx->h_status = 0;
        // VKML_B200_GEMM_PRECISION = 3xtf32 (default) | tf32 | fp32, read once per context:
        // the counterpart of the VKML_GEMM_* switches (vulkan_backend.cpp:2160-2178)
        if (const char* e = std::getenv("VKML_B200_GEMM_GROUP_M")) {
            ctx->gemm_group_m = std::max(0, std::min(1024, std::atoi(e)));
        }
        if (const char* e = std::getenv("VKML_B200_GEMM_BN")) {
            ctx->gemm_bn_override = std::atoi(e);
        }
        if (const char* e = std::getenv("VKML_B200_GEMM_OPERANDS")) {
            const std::string v(e);
            if (v == "planes") ctx->gemm_operands = 0;
            else if (v == "direct") ctx->gemm_operands = 1;
            else if (v == "auto") ctx->gemm_operands = -1;
            else fail(B200_INVALID_ARGUMENT, "VKML_B200_GEMM_OPERANDS must be auto, planes or direct");
        }
        if (const char* e = std::getenv("VKML_B200_GEMM_STREAM")) {
            const std::string v(e);
            if (v == "auto") ctx->gemm_stream = -1;
            else if (v == "0" || v == "1") ctx->gemm_stream = v == "1" ? 1 : 0;
            else fail(B200_INVALID_ARGUMENT, "VKML_B200_GEMM_STREAM must be auto, 0 or 1");
        }
        if (const char* e = std::getenv("VKML_B200_GEMM_SCHEDULE")) {
            const std::string v(e);
            if (v == "static") ctx->gemm_schedule = 0;
            else if (v == "dynamic") ctx->gemm_schedule = 1;
            else if (v == "auto") ctx->gemm_schedule = -1;
            else fail(B200_INVALID_ARGUMENT, "VKML_B200_GEMM_SCHEDULE must be auto, static or dynamic");
        }
        if (const char* e = std::getenv("VKML_B200_SHARE_PLANES")) {
            ctx->share_planes = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_FUSE")) {
            ctx->fuse = std::atoi(e) != 0;
        }
        ctx->upload_threads = std::max(2, std::min(8, static_cast<int>(std::thread::hardware_concurrency()) / 2));
        if (const char* e = std::getenv("VKML_B200_UPLOAD_THREADS")) {
            ctx->upload_threads = std::max(0, std::min(16, std::atoi(e)));
        }
        if (const char* e = std::getenv("VKML_B200_SPAN_GRAPHS")) {
            ctx->span_graph_cache = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_PDL")) {
            ctx->pdl = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_BUCKET")) {
            ctx->bucket_grads = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_BUCKET_FLUSH_BYTES")) {
            ctx->bucket_flush_bytes = static_cast<size_t>(std::max<long long>(1, std::atoll(e)));
        }
        if (const char* e = std::getenv("VKML_B200_LAZY_JOIN")) {
            ctx->lazy_join = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_HOIST_GRADIENTS")) {
            ctx->hoist_gradients = std::atoi(e) != 0;
        }
        if (const char* e = std::getenv("VKML_B200_COMM_SMS")) {
            const int v = std::atoi(e);
            if (v < 0 || v > 64) fail(B200_INVALID_ARGUMENT, "VKML_B200_COMM_SMS must be 0..64");
            ctx->comm_sms = v;
        }
        if (const char* e = std::getenv("VKML_B200_GEMM_PRECISION")) {
            const std::string v(e);
            if (v == "tf32") ctx->gemm_precision = B200_GEMM_TF32;
            else if (v == "fp32") ctx->gemm_precision = B200_GEMM_FP32;
            else if (v == "3xtf32" || v.empty()) ctx->gemm_precision = B200_GEMM_3XTF32;
            else fail(B200_INVALID_ARGUMENT, "VKML_B200_GEMM_PRECISION must be 3xtf32, tf32 or fp32");
        }
    });
    if (rc != B200_OK) {
        b200_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return B200_OK;
}

void b200_destroy(b200_ctx* ctx) {
    if (ctx == nullptr) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream != nullptr) cudaStreamSynchronize(ctx->stream);
    destroy_uploader(ctx);
    for (auto& kv : ctx->span_graphs) {
        if (kv.second.exec != nullptr) cudaGraphExecDestroy(kv.second.exec);
    }
    dist_destroy(ctx);
    if (ctx->stream != nullptr) cudaStreamDestroy(ctx->stream);
    if (ctx->d_status != nullptr) cudaFree(ctx->d_status);
    if (ctx->d_counters != nullptr) cudaFree(ctx->d_counters);
    if (ctx->h_status != nullptr) cudaFreeHost(ctx->h_status);
    for (cudaEvent_t ev : ctx->event_pool) cudaEventDestroy(ev);
    if (ctx->timer_begin != nullptr) cudaEventDestroy(ctx->timer_begin);
    if (ctx->timer_end != nullptr) cudaEventDestroy(ctx->timer_end);
    cudaGetLastError();
    delete ctx;
}

int b200_get_caps(b200_ctx* ctx, b200_caps* out) {
    if (ctx == nullptr || out == nullptr) return B200_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof(*out));
    std::snprintf(out->name, sizeof(out->name), "%s", ctx->prop.name);
    out->cc_major = ctx->prop.major;
    out->cc_minor = ctx->prop.minor;
    out->sm_count = static_cast<uint32_t>(ctx->prop.multiProcessorCount);
    out->warp_size = static_cast<uint32_t>(ctx->prop.warpSize);
    out->max_threads_per_block = static_cast<uint32_t>(ctx->prop.maxThreadsPerBlock);
    out->max_shared_memory_bytes = ctx->prop.sharedMemPerBlockOptin;
    out->total_memory_bytes = ctx->prop.totalGlobalMem;
    out->min_buffer_alignment = 512;
    return B200_OK;
}

int b200_alloc(b200_ctx* ctx, size_t nbytes, void** out) {
    if (ctx == nullptr || out == nullptr) return B200_INVALID_ARGUMENT;
    *out = nullptr;
    return guarded(ctx, [&] { *out = ctx->alloc.allocate(nbytes); });
}

int b200_free(b200_ctx* ctx, void* ptr) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        if (ptr != nullptr && dist_has_pending(ctx)) {
            // a buffer still being all-reduced: later work that reuses the block must come after it
            dist_wait_range(ctx, ptr, static_cast<const char*>(ptr) + std::max<size_t>(ctx->alloc.size_of(ptr), 1));
        }
        ctx->alloc.release(ptr);
    });
}

static void drop_span_graphs(b200_ctx* ctx);

int b200_trim(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        drop_span_graphs(ctx);
        ctx->alloc.trim();
        ctx->scratch.trim();
    });
}

int b200_supports(const b200_node* node) {
    if (node == nullptr) return 0;
    return supports_node(*node) ? 1 : 0;
}

// Queues one span, node by node (fused groups aside).
static void compute_span(b200_ctx* ctx, const b200_node* nodes, size_t n_nodes, uint32_t flags) {
    const bool grad_sync = (flags & B200_COMPUTE_GRAD_SYNC) != 0 && ctx->dist != nullptr;
    // With no buffers registered, the gradients are the span's SINKS: f32 outputs that
    // no later node of the span reads.  backward() realises exactly the leaf gradients
    // (src/autograd/autograd.cpp:627-666), so every other output is consumed in-span.
    ctx->in_grad_sync_span = grad_sync && ctx->dist != nullptr;
    struct SpanGuard {
        b200_ctx* c;
        ~SpanGuard() {
            c->in_grad_sync_span = false;
            gemm_tc_end_span(c);
        }
    } span_guard{ctx};
    count_matmul_operands(ctx, nodes, n_nodes);
    std::vector<char> is_sink;
    if (grad_sync && ctx->grads.empty()) {
        is_sink.assign(n_nodes, 0);
        auto bytes_of = [](const b200_tensor& t) {
            size_t n = dtype_size(t.dtype);
            for (int d = 0; d < t.ndim; ++d) n *= static_cast<size_t>(t.dims[d]);
            return n;
        };
        for (size_t i = 0; i < n_nodes; ++i) {
            const b200_node& node = nodes[i];
            if (is_view_or_leaf(node.op) || node.out.dtype != B200_F32 || node.out.data == nullptr) continue;
            const char* lo = static_cast<const char*>(node.out.data);
            const char* hi = lo + bytes_of(node.out);
            bool consumed = false;
            for (size_t j = i + 1; j < n_nodes && !consumed; ++j) {
                for (uint32_t k = 0; k < nodes[j].n_src && k < B200_MAX_SRC; ++k) {
                    const char* p = static_cast<const char*>(nodes[j].src[k].data);
                    if (p >= lo && p < hi) {
                        consumed = true;
                        break;
                    }
                }
            }
            is_sink[i] = consumed ? 0 : 1;
        }
    }
    // Execution order.  Only dependency order is contractual (backend.h:34-45), and the
    // executor's depth-first order puts every parameter gradient at the tail of the span.
    // When gradients are exchanged, each sink is hoisted to just after the last node it
    // reads from, so its all-reduce runs under the remaining backward work instead of
    // after it.  Every node still computes the same values from the same inputs.
    std::vector<size_t> order;
    order.reserve(n_nodes);
    if (!is_sink.empty() && ctx->hoist_gradients) {
        std::vector<std::vector<size_t>> deps(n_nodes);
        std::vector<size_t> pending;
        auto bytes_of = [](const b200_tensor& t) {
            size_t n = dtype_size(t.dtype);
            for (int d = 0; d < t.ndim; ++d) n *= static_cast<size_t>(t.dims[d]);
            return n;
        };
        for (size_t j = 0; j < n_nodes; ++j) {
            if (!is_sink[j]) continue;
            pending.push_back(j);
            for (uint32_t k = 0; k < nodes[j].n_src && k < B200_MAX_SRC; ++k) {
                const char* p = static_cast<const char*>(nodes[j].src[k].data);
                for (size_t i = j; i-- > 0;) {  // latest earlier writer of that address
                    if (is_view_or_leaf(nodes[i].op) || nodes[i].out.data == nullptr) continue;
                    const char* lo = static_cast<const char*>(nodes[i].out.data);
                    if (p >= lo && p < lo + bytes_of(nodes[i].out)) {
                        deps[j].push_back(i);
                        break;
                    }
                }
            }
        }
        std::vector<char> emitted(n_nodes, 0);
        auto flush = [&] {
            for (size_t q = 0; q < pending.size();) {
                const size_t j = pending[q];
                bool ready = true;
                for (size_t d : deps[j]) ready = ready && emitted[d];
                if (ready) {
                    order.push_back(j);
                    emitted[j] = 1;
                    pending.erase(pending.begin() + static_cast<std::ptrdiff_t>(q));
                } else {
                    ++q;
                }
            }
        };
        flush();
        for (size_t i = 0; i < n_nodes; ++i) {
            if (is_sink[i]) continue;
            order.push_back(i);
            emitted[i] = 1;
            flush();
        }
    } else {
        for (size_t i = 0; i < n_nodes; ++i) order.push_back(i);
    }
    auto tensor_bytes = [](const b200_tensor& t) {
        size_t n = dtype_size(t.dtype);
        for (int d = 0; d < t.ndim; ++d) n *= static_cast<size_t>(t.dims[d]);
        return n;
    };
    // All-reduces of an earlier gradient span may still be running.  Nodes are taken in the
    // order their inputs become available: key = the latest pending all-reduce a node depends
    // on, directly or through producers inside this span; a stable sort by that key keeps
    // every producer before its consumers and leaves a span that touches no gradient as it is.
    if (dist_has_pending(ctx) && n_nodes > 1) {
        std::vector<int> key(n_nodes, -1);
        for (size_t j = 0; j < n_nodes; ++j) {
            const b200_node& node = nodes[j];
            if (is_view_or_leaf(node.op)) continue;
            int k = -1;
            if (node.out.data != nullptr) {
                k = std::max(k, dist_pending_index(ctx, node.out.data,
                                                   static_cast<const char*>(node.out.data) + tensor_bytes(node.out)));
            }
            for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
                const char* p = static_cast<const char*>(node.src[s].data);
                if (p == nullptr) continue;
                k = std::max(k, dist_pending_index(ctx, p, p + 1));
                for (size_t i = j; i-- > 0;) {  // latest earlier writer of that address
                    if (is_view_or_leaf(nodes[i].op) || nodes[i].out.data == nullptr) continue;
                    const char* lo = static_cast<const char*>(nodes[i].out.data);
                    if (p >= lo && p < lo + tensor_bytes(nodes[i].out)) {
                        k = std::max(k, key[i]);
                        break;
                    }
                }
            }
            key[j] = k;
        }
        std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return key[a] < key[b]; });
    }
    // What a node needs before its kernel may be queued, and what follows it.
    auto prepare = [&](size_t i) {
        const b200_node& node = nodes[i];
        if (node.out.data == nullptr) {
            fail(B200_INVALID_ARGUMENT, "node has no storage");
        }
        for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
            int64_t sn = 1;
            for (int d = 0; d < node.src[s].ndim; ++d) sn *= node.src[s].dims[d];
            if (sn != 0 && node.src[s].data == nullptr) {
                fail(B200_INVALID_ARGUMENT, "source " + std::to_string(s) + " has no storage");
            }
        }
        if (dist_has_pending(ctx)) {
            dist_wait_range(ctx, node.out.data, static_cast<const char*>(node.out.data) + tensor_bytes(node.out));
            for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
                const char* p = static_cast<const char*>(node.src[s].data);
                if (p != nullptr) dist_wait_range(ctx, p, p + 1);
            }
        }
        if (!ctx->plane_cache.empty()) {
            // cannot happen under the caller's contract (outputs are fresh buffers), but a
            // plane must never outlive the data it was split from
            gemm_tc_invalidate(ctx, node.out.data, static_cast<const char*>(node.out.data) + tensor_bytes(node.out));
        }
    };
    auto finish = [&](size_t i) {
        const b200_node& node = nodes[i];
        ctx->nodes_computed.fetch_add(1, std::memory_order_relaxed);
        if (grad_sync) {
            if (!is_sink.empty()) {
                if (is_sink[i]) {
                    int64_t numel = 1;
                    for (int d = 0; d < node.out.ndim; ++d) numel *= node.out.dims[d];
                    dist_all_reduce_now(ctx, node.out.data, static_cast<size_t>(numel));
                }
            } else {
                dist_after_node(ctx, node);
            }
        }
    };
    // the nodes that need a kernel, in execution order
    std::vector<size_t> exec;
    exec.reserve(order.size());
    for (const size_t i : order) {
        const b200_node& node = nodes[i];
        if (is_view_or_leaf(node.op)) {
            continue;  // resolved by the executor through aliasing (backend.h:34-45)
        }
        if (node.op >= B200_OP_COUNT) {
            fail(B200_NOT_IMPLEMENTED, "unknown op " + std::to_string(node.op));
        }
        // zero-element tensors are legal and need no work (vulkan_backend.cpp:1233-1236)
        int64_t numel = 1;
        for (int d = 0; d < node.out.ndim; ++d) numel *= node.out.dims[d];
        if (numel != 0) exec.push_back(i);
    }
    // Buffers a `full` node of this span filled with one value: a later elementwise node that
    // reads such a buffer whole is handed a stride-0 view of its first element instead, and
    // reads 4 bytes where it would have read the tensor (ReLU's backward mask compares against,
    // and its `where` selects from, activation-sized tensors of zeros).
    std::map<const void*, size_t> constants;
    std::vector<char> done(exec.size(), 0);  // served ahead of its turn by a grouped launch
    for (size_t p = 0; p < exec.size();) {
        if (done[p]) {
            ++p;
            continue;
        }
        const size_t i = exec[p];
        const b200_node& node = nodes[i];
        if (ctx->fuse && exec.size() - p >= 2 &&
            (node.op == B200_OP_ADD || node.op == B200_OP_FULL || node.op == B200_OP_EQUAL ||
             node.op == B200_OP_EXP)) {
            const size_t avail = std::min<size_t>(exec.size() - p, 5);
            const b200_node* seq[5];
            bool eligible = true;
            for (size_t k = 0; k < avail; ++k) {
                seq[k] = &nodes[exec[p + k]];
                // a gradient that this span all-reduces is exchanged as soon as its own kernel is queued
                eligible = eligible && (is_sink.empty() || !is_sink[exec[p + k]]) && seq[k]->out.data != nullptr;
                eligible = eligible && (!grad_sync || !is_sink.empty() || ctx->grads.empty());
            }
            if (eligible) {
                for (size_t k = 0; k < avail; ++k) prepare(exec[p + k]);
                ctx->current_op = node.op;
                const size_t taken = launch_fused(ctx, seq, avail);
                if (taken > 0) {
                    for (size_t k = 0; k < taken; ++k) {
                        if (seq[k]->op == B200_OP_FULL && seq[k]->out.dtype == B200_F32) {
                            constants[seq[k]->out.data] = tensor_bytes(seq[k]->out);
                        }
                        finish(exec[p + k]);
                    }
                    p += taken;
                    continue;
                }
            }
        }
        if (ctx->fuse && exec.size() - p >= 3 &&
            (node.op == B200_OP_FULL || node.op == B200_OP_ARANGE || node.op == B200_OP_CONTIGUOUS || node.op == B200_OP_CAST ||
             node.op == B200_OP_NEG || node.op == B200_OP_DIV || node.op == B200_OP_MUL || node.op == B200_OP_EQUAL)) {
            // a run of tiny elementwise nodes (the prologue of a loss): one block walks it
            constexpr size_t kLook = 12;
            const size_t avail = std::min<size_t>(exec.size() - p, kLook);
            const b200_node* seq[kLook];
            size_t run = 0;
            while (run < avail && !done[p + run]) {
                const size_t idx = exec[p + run];
                const bool sink = !is_sink.empty() && is_sink[idx];
                if (sink || (grad_sync && is_sink.empty() && !ctx->grads.empty())) break;
                int64_t numel = 1;
                for (int d = 0; d < nodes[idx].out.ndim; ++d) numel *= nodes[idx].out.dims[d];
                if (numel > 4096) break;
                seq[run] = &nodes[idx];
                ++run;
            }
            if (run >= 3) {
                for (size_t k = 0; k < run; ++k) prepare(exec[p + k]);
                ctx->current_op = node.op;
                const size_t taken = launch_tiny_chain(ctx, seq, run);
                if (taken > 0) {
                    for (size_t k = 0; k < taken; ++k) {
                        if (seq[k]->op == B200_OP_FULL && seq[k]->out.dtype == B200_F32) {
                            constants[seq[k]->out.data] = tensor_bytes(seq[k]->out);
                        } else {
                            constants.erase(seq[k]->out.data);
                        }
                        finish(exec[p + k]);
                    }
                    p += taken;
                    continue;
                }
            }
        }
        if (ctx->fuse && node.op == B200_OP_MAX_POOL2D_BACKWARD && p + 1 < exec.size() && !done[p + 1]) {
            // ReLU's backward rule behind a pooling layer: where(mask, zeros, pooling gradient)
            const b200_node& wn = nodes[exec[p + 1]];
            auto same_tensor = [](const b200_tensor& a, const b200_tensor& b) {
                if (a.data != b.data || a.dtype != b.dtype || a.ndim != b.ndim) return false;
                for (int d = 0; d < a.ndim; ++d) {
                    if (a.dims[d] != b.dims[d] || (a.dims[d] > 1 && a.strides[d] != b.strides[d])) return false;
                }
                return true;
            };
            auto filled = [&](const b200_tensor& t) {
                if (t.dtype != B200_F32 || t.data == nullptr) return false;
                const auto it = constants.find(t.data);
                if (it != constants.end() && it->second == tensor_bytes(t)) return true;
                for (int d = 0; d < t.ndim; ++d) {
                    if (t.dims[d] > 1 && t.strides[d] != 0) return false;
                }
                return true;
            };
            bool eligible = wn.op == B200_OP_WHERE && wn.n_src == 3 && node.out.data != nullptr && wn.out.data != nullptr;
            for (const size_t k : {p, p + 1}) {
                eligible = eligible && (is_sink.empty() || !is_sink[exec[k]]);
            }
            eligible = eligible && (!grad_sync || !is_sink.empty() || ctx->grads.empty());
            int side = -1;
            if (eligible && same_tensor(wn.src[1], node.out) && filled(wn.src[2])) side = 1;
            if (eligible && same_tensor(wn.src[2], node.out) && filled(wn.src[1])) side = 0;
            if (side >= 0) {
                prepare(exec[p]);
                prepare(exec[p + 1]);
                ctx->current_op = node.op;
                if (launch_pool_backward_where(ctx, node, wn, side, wn.src[side == 1 ? 2 : 1].data)) {
                    constants.erase(node.out.data);
                    constants.erase(wn.out.data);
                    finish(exec[p]);
                    finish(exec[p + 1]);
                    p += 2;
                    continue;
                }
            }
        }
        if (ctx->fuse && node.op == B200_OP_SCALED_ADD && exec.size() - p >= 2 && !grad_sync) {
            // the optimiser's spans: independent scaled_add nodes, one launch for the dense ones among
            // the next 24 nodes (a transposed gradient in between keeps its own kernel)
            constexpr size_t kLook = 24;
            const size_t avail = std::min<size_t>(exec.size() - p, kLook);
            const b200_node* seq[kLook];
            bool picked[kLook];
            size_t run = 0;
            while (run < avail && !done[p + run]) {
                seq[run] = &nodes[exec[p + run]];
                ++run;
            }
            if (run >= 2) {
                for (size_t k = 0; k < run; ++k) prepare(exec[p + k]);
                ctx->current_op = node.op;
                if (launch_scaled_add_group(ctx, seq, run, picked) > 0) {
                    for (size_t k = 0; k < run; ++k) {
                        if (picked[k]) {
                            constants.erase(seq[k]->out.data);
                            finish(exec[p + k]);
                            done[p + k] = 1;
                        }
                    }
                    if (done[p]) {
                        ++p;
                        continue;
                    }
                }
            }
        }
        prepare(i);
        const bool elementwise = node.op == B200_OP_WHERE || (node.op >= B200_OP_ADD && node.op <= B200_OP_NOT_EQUAL);
        if (ctx->fuse && elementwise && !constants.empty()) {
            b200_node lean = node;
            bool changed = false;
            for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
                const auto it = constants.find(node.src[s].data);
                if (it != constants.end() && node.src[s].dtype == B200_F32 && it->second == tensor_bytes(node.src[s])) {
                    for (int d = 0; d < lean.src[s].ndim; ++d) lean.src[s].strides[d] = 0;
                    changed = true;
                }
            }
            dispatch_node(ctx, changed ? lean : node);
        } else {
            dispatch_node(ctx, node);
        }
        if (node.op == B200_OP_FULL && node.out.dtype == B200_F32) {
            constants[node.out.data] = tensor_bytes(node.out);
        } else {
            constants.erase(node.out.data);  // (outputs are fresh buffers; kept exact regardless)
        }
        finish(i);
        ++p;
    }
    if (grad_sync) {
        dist_join(ctx);
    }
    if ((flags & B200_COMPUTE_SYNC) && !ctx->capturing) {
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    }
}

// ---- spans replayed as CUDA graphs ----
//
// What a span queues is a function of its nodes (ops, shapes, strides, ADDRESSES, parameters) and
// of a little library state: the GEMM precision, the workspace and the scratch pool the planes
// come from.  When all of that comes back unchanged, so do the launches -- and vkML's training
// loops do come back: the caching allocator hands a loop the same addresses again every few steps.
// The second time a span of at least kSpanGraphMinNodes nodes is seen in the same state, its
// launches are captured from the stream (relaxed mode, the same code path as the eager run) and
// kept; from then on the span is one cudaGraphLaunch.  A graph is only ever launched for a span
// that matches the captured one byte for byte, and everything is dropped when device memory goes
// back to the driver.  Spans that exchange gradients, spans queued while an all-reduce is still
// pending, and profiled spans always run eagerly.
constexpr size_t kSpanGraphMinNodes = 6;
constexpr size_t kSpanGraphMax = 256;
static_assert(sizeof(b200_node) % 8 == 0 && alignof(b200_node) >= 8, "spans are hashed in 8-byte words");

static uint64_t span_graph_state(const b200_ctx* ctx) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
    mix(static_cast<uint64_t>(ctx->gemm_precision));
    mix(reinterpret_cast<uintptr_t>(ctx->workspace));
    mix(ctx->workspace_bytes);
    mix(ctx->scratch.driver_allocs);
    mix(ctx->alloc.driver_frees + ctx->scratch.driver_frees);
    return h;
}

static void drop_span_graphs(b200_ctx* ctx) {
    for (auto& kv : ctx->span_graphs) {
        if (kv.second.exec != nullptr) cudaGraphExecDestroy(kv.second.exec);
    }
    ctx->span_graphs.clear();
    ctx->span_seen.clear();
}

// True when the span was served by a graph (launched, or captured and launched).
static bool span_graph_run(b200_ctx* ctx, const b200_node* nodes, size_t n_nodes, uint32_t flags) {
    if (!ctx->span_graph_cache || ctx->capturing || ctx->profiling || n_nodes < kSpanGraphMinNodes ||
        (flags & ~static_cast<uint32_t>(B200_COMPUTE_SYNC)) != 0 || dist_has_pending(ctx)) {
        return false;
    }
    const size_t bytes = n_nodes * sizeof(b200_node);
    const unsigned char* raw = reinterpret_cast<const unsigned char*>(nodes);
    uint64_t key = 1469598103934665603ull;
    {
        const uint64_t* w = reinterpret_cast<const uint64_t*>(raw);  // b200_node is a multiple of 8 bytes, 8-aligned
        for (size_t i = 0; i < bytes / 8; ++i) key = (key ^ w[i]) * 1099511628211ull;
    }
    const uint64_t state = span_graph_state(ctx);
    key = (key ^ state) * 1099511628211ull;
    auto finish = [&](b200_ctx::SpanGraph& g) {
        B200_CUDA_CHECK(cudaGraphLaunch(g.exec, ctx->stream));
        ctx->kernel_launches.fetch_add(g.launches, std::memory_order_relaxed);
        ctx->nodes_computed.fetch_add(g.node_count, std::memory_order_relaxed);
        if (flags & B200_COMPUTE_SYNC) B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    };
    if (auto it = ctx->span_graphs.find(key); it != ctx->span_graphs.end()) {
        b200_ctx::SpanGraph& g = it->second;
        if (g.state == state && g.nodes.size() == bytes && std::memcmp(g.nodes.data(), raw, bytes) == 0) {
            finish(g);
            ++ctx->span_graph_hits;
            return true;
        }
        return false;  // a different span under the same key: leave it to the eager path
    }
    if (ctx->span_seen.size() > 65536) ctx->span_seen.clear();  // a caller whose addresses never come back
    if (++ctx->span_seen[key] < 2 || ctx->span_graphs.size() >= kSpanGraphMax) {
        return false;
    }
    // second sighting: capture what the eager path queues for this span
    const uint64_t launches0 = ctx->kernel_launches.load(), nodes0 = ctx->nodes_computed.load();
    cudaGraph_t graph = nullptr;
    B200_CUDA_CHECK(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    bool ok = true;
    try {
        compute_span(ctx, nodes, n_nodes, flags);
    } catch (const Error&) {
        ok = false;
    }
    ctx->capturing = false;
    if (cudaStreamEndCapture(ctx->stream, &graph) != cudaSuccess || graph == nullptr) {
        cudaGetLastError();
        ok = false;
    }
    b200_ctx::SpanGraph g;
    ok = ok && span_graph_state(ctx) == state;  // nothing grew while capturing
    if (ok && cudaGraphInstantiate(&g.exec, graph, 0) != cudaSuccess) {
        cudaGetLastError();
        ok = false;
    }
    if (graph != nullptr) cudaGraphDestroy(graph);
    // the capture pass counted the span once; a launch counts it again below
    const uint64_t launches = ctx->kernel_launches.load() - launches0, node_count = ctx->nodes_computed.load() - nodes0;
    ctx->kernel_launches.fetch_sub(launches, std::memory_order_relaxed);
    ctx->nodes_computed.fetch_sub(node_count, std::memory_order_relaxed);
    if (!ok) {
        ctx->span_seen[key] = 0x40000000u;  // never try this one again; the eager path reports whatever is wrong
        if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
        return false;
    }
    g.nodes.assign(raw, raw + bytes);
    g.launches = launches;
    g.node_count = node_count;
    g.state = state;
    auto placed = ctx->span_graphs.emplace(key, std::move(g));
    ++ctx->span_graph_captures;
    finish(placed.first->second);
    return true;
}

int b200_compute(b200_ctx* ctx, const b200_node* nodes, size_t n_nodes, uint32_t flags) {
    if (ctx == nullptr || (nodes == nullptr && n_nodes != 0)) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        ctx->compute_calls.fetch_add(1, std::memory_order_relaxed);
        if (!span_graph_run(ctx, nodes, n_nodes, flags)) {
            compute_span(ctx, nodes, n_nodes, flags);
        }
    });
}

int b200_copy_from_host(b200_ctx* ctx, void* dst_device, const void* src_host, size_t nbytes) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    if (nbytes == 0) return B200_OK;
    if (dst_device == nullptr || src_host == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        // For pageable memory the runtime stages the bytes before returning, so
        // the caller may reuse `src_host` immediately; pinned memory is read
        // asynchronously, in stream order.
        dist_wait_range(ctx, dst_device, static_cast<const char*>(dst_device) + nbytes);
        cudaPointerAttributes attr{};
        const cudaError_t e = cudaPointerGetAttributes(&attr, src_host);
        if (e != cudaSuccess) cudaGetLastError();
        const bool pageable = e != cudaSuccess || attr.type == cudaMemoryTypeUnregistered;
        if (pageable && staged_upload(ctx, dst_device, src_host, nbytes)) {
            return;  // large and pageable: staged by several threads, `src_host` has been read
        }
        B200_CUDA_CHECK(cudaMemcpyAsync(dst_device, src_host, nbytes, cudaMemcpyHostToDevice, ctx->stream));
        if (e == cudaSuccess && attr.type == cudaMemoryTypeHost) {
            // pinned source: the copy is truly asynchronous; wait so the
            // "caller may reuse the buffer" contract of copy_from_host holds
            B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        }
    });
}

static int report_device_status(b200_ctx* ctx) {
    const uint32_t bits = *ctx->h_status;
    if (bits == 0) return B200_OK;
    *ctx->h_status = 0;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(uint32_t), ctx->stream);
    // a kernel that gave up may have left arrival counters of a split reduction half-counted
    cudaMemsetAsync(ctx->d_counters, 0, sizeof(unsigned) * kArrivalCounters, ctx->stream);
    if (bits & kStatusIndexOutOfRange) {
        set_error(ctx, "an index passed to index_select / scatter_add was out of range");
        return B200_INDEX_ERROR;
    }
    if (bits & kStatusWaitTimedOut) {
        set_error(ctx, "a bounded device-side wait ran out");
        return B200_TIMEOUT;
    }
    set_error(ctx, "a kernel reported an internal error (status bits " + std::to_string(bits) + ")");
    return B200_INTERNAL_ERROR;
}

int b200_copy_to_host(b200_ctx* ctx, void* dst_host, const void* src_device, size_t nbytes) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    if (nbytes == 0) return B200_OK;
    if (dst_host == nullptr || src_device == nullptr) return B200_INVALID_ARGUMENT;
    // Reading a tensor back is the framework's normal way of observing a result, so an error the
    // device recorded while producing it (an out-of-range index that was clamped) is reported
    // here, with the bytes, and not only at a later explicit synchronize: the CPU backend rejects
    // such an index before any value is visible (src/backend/cpu/kernels_movement.cpp:362,419).
    int device_rc = B200_OK;
    const int rc = guarded(ctx, [&] {
        dist_wait_range(ctx, src_device, static_cast<const char*>(src_device) + nbytes);
        B200_CUDA_CHECK(cudaMemcpyAsync(dst_host, src_device, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
        if (!ctx->capturing) {
            B200_CUDA_CHECK(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(uint32_t),
                                            cudaMemcpyDeviceToHost, ctx->stream));
        }
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        if (!ctx->capturing) device_rc = report_device_status(ctx);
    });
    return rc != B200_OK ? rc : device_rc;
}

int b200_copy_device_to_device(b200_ctx* ctx, const b200_copy* copies, size_t n) {
    if (ctx == nullptr || (copies == nullptr && n != 0)) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        for (size_t i = 0; i < n; ++i) {
            if (copies[i].nbytes == 0) continue;
            if (copies[i].dst == nullptr || copies[i].src == nullptr) {
                fail(B200_INVALID_ARGUMENT, "null pointer in copy_device_to_device");
            }
            dist_wait_range(ctx, copies[i].dst, static_cast<const char*>(copies[i].dst) + copies[i].nbytes);
            dist_wait_range(ctx, copies[i].src, static_cast<const char*>(copies[i].src) + copies[i].nbytes);
            B200_CUDA_CHECK(cudaMemcpyAsync(copies[i].dst, copies[i].src, copies[i].nbytes,
                                            cudaMemcpyDeviceToDevice, ctx->stream));
        }
    });
}

int b200_synchronize(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    int device_rc = B200_OK;
    const int rc = guarded(ctx, [&] {
        dist_check_health(ctx);
        dist_wait_range(ctx, nullptr, nullptr);  // "everything submitted" includes the all-reduces
        B200_CUDA_CHECK(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(uint32_t),
                                        cudaMemcpyDeviceToHost, ctx->stream));
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        device_rc = report_device_status(ctx);
    });
    return rc != B200_OK ? rc : device_rc;
}

const char* b200_last_error(b200_ctx* ctx) {
    if (ctx == nullptr) return "";
    std::lock_guard<std::mutex> lock(ctx->err_mu);
    // the string lives in the context until the next error replaces it
    return ctx->last_error.c_str();
}

int b200_get_stats(b200_ctx* ctx, b200_stats* out) {
    if (ctx == nullptr || out == nullptr) return B200_INVALID_ARGUMENT;
    out->reserved_bytes = ctx->alloc.reserved + ctx->scratch.reserved;  // both pools
    out->in_use_bytes = ctx->alloc.in_use;
    out->peak_in_use_bytes = ctx->alloc.peak;
    out->live_allocations = ctx->alloc.live;
    out->total_allocations = ctx->alloc.total;
    out->driver_allocations = ctx->alloc.driver_allocs + ctx->scratch.driver_allocs;
    out->compute_calls = ctx->compute_calls.load();
    out->kernel_launches = ctx->kernel_launches.load();
    out->nodes_computed = ctx->nodes_computed.load();
    out->comm_bytes = ctx->comm_bytes.load();
    return B200_OK;
}

int b200_profile_enable(b200_ctx* ctx, int on) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        for (ProfEntry& e : ctx->prof) {
            ctx->event_pool.push_back(e.begin);
            ctx->event_pool.push_back(e.end);
        }
        ctx->prof.clear();
        ctx->profiling = on != 0;
    });
}

int b200_profile_read(b200_ctx* ctx, b200_profile_record* out, size_t capacity, size_t* count) {
    if (ctx == nullptr || count == nullptr || (out == nullptr && capacity != 0)) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        size_t n = 0;
        for (ProfEntry& e : ctx->prof) {
            if (n < capacity) {
                float ms = 0.0F;
                if (cudaEventElapsedTime(&ms, e.begin, e.end) != cudaSuccess) {
                    cudaGetLastError();
                    ms = -1.0F;
                }
                std::memcpy(out[n].label, e.label, sizeof(out[n].label));
                out[n].ms = ms;
                out[n].op = e.op;
                out[n].submission = e.submission;
                ++n;
            }
            ctx->event_pool.push_back(e.begin);
            ctx->event_pool.push_back(e.end);
        }
        ctx->prof.clear();
        *count = n;
    });
}

int b200_timer_begin(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        if (ctx->timer_begin == nullptr) {
            B200_CUDA_CHECK(cudaEventCreate(&ctx->timer_begin));
            B200_CUDA_CHECK(cudaEventCreate(&ctx->timer_end));
        }
        B200_CUDA_CHECK(cudaEventRecord(ctx->timer_begin, ctx->stream));
    });
}

int b200_timer_end(b200_ctx* ctx, float* milliseconds) {
    if (ctx == nullptr || milliseconds == nullptr) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        if (ctx->timer_begin == nullptr) fail(B200_INVALID_ARGUMENT, "b200_timer_end without b200_timer_begin");
        dist_wait_range(ctx, nullptr, nullptr);
        B200_CUDA_CHECK(cudaEventRecord(ctx->timer_end, ctx->stream));
        B200_CUDA_CHECK(cudaEventSynchronize(ctx->timer_end));
        B200_CUDA_CHECK(cudaEventElapsedTime(milliseconds, ctx->timer_begin, ctx->timer_end));
    });
}

int b200_alloc_host(b200_ctx* ctx, size_t nbytes, void** out) {
    if (ctx == nullptr || out == nullptr) return B200_INVALID_ARGUMENT;
    *out = nullptr;
    if (nbytes == 0) return B200_OK;
    return guarded(ctx, [&] { B200_CUDA_CHECK(cudaMallocHost(out, nbytes)); });
}

int b200_free_host(b200_ctx* ctx, void* ptr) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    if (ptr == nullptr) return B200_OK;
    return guarded(ctx, [&] { B200_CUDA_CHECK(cudaFreeHost(ptr)); });
}

int b200_set_gemm_precision(b200_ctx* ctx, int precision) {
    if (ctx == nullptr || precision < B200_GEMM_3XTF32 || precision > B200_GEMM_FP32) {
        return B200_INVALID_ARGUMENT;
    }
    ctx->gemm_precision = precision;
    return B200_OK;
}

int b200_get_gemm_precision(b200_ctx* ctx) { return ctx == nullptr ? -1 : ctx->gemm_precision; }

int b200_matmul_kernel(b200_ctx* ctx, const b200_node* node, char* name, size_t name_len, char* reason,
                       size_t reason_len) {
    if (ctx == nullptr || node == nullptr || name == nullptr || name_len == 0) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] {
        if (node->op != B200_OP_MATMUL) fail(B200_INVALID_ARGUMENT, "b200_matmul_kernel: not a matmul node");
        const GemmProblem p = matmul_problem(*node);
        const char* kernel = "fp32_simt";
        const char* why = "the shape is too small or too ragged for a tensor-core tile";
        if (ctx->gemm_precision == B200_GEMM_FP32) {
            why = "plain fp32 arithmetic was asked for";
        } else if (gemm_tc_eligible(ctx, p)) {
            const bool three = ctx->gemm_precision == B200_GEMM_3XTF32;
            if (gemm_tc_streams(ctx, p)) {
                kernel = three ? "tcgen05_3xtf32_stream" : "tcgen05_tf32_stream";
                why = "bound by memory (a small left operand or a short K): the right operand is read as fp32 and split on the way";
            } else if (gemm_tc_reads_directly(ctx, p)) {
                kernel = three ? "tcgen05_3xtf32_direct" : "tcgen05_tf32_direct";
                why = "the plane passes would cost more than the product: fp32 tiles by TMA, split inside the kernel";
            } else {
                kernel = three ? "tcgen05_3xtf32" : "tcgen05_tf32";
                why = "operands split into TF32 planes, tensor-core tiles fed by TMA";
            }
        }
        std::snprintf(name, name_len, "%s", kernel);
        if (reason != nullptr && reason_len != 0) std::snprintf(reason, reason_len, "%s", why);
    });
}

void* b200_stream(b200_ctx* ctx) { return ctx == nullptr ? nullptr : ctx->stream; }

int b200_span_graph_stats(b200_ctx* ctx, uint64_t* hits, uint64_t* captures) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    if (hits != nullptr) *hits = ctx->span_graph_hits;
    if (captures != nullptr) *captures = ctx->span_graph_captures;
    return B200_OK;
}

int b200_debug_expire_wait(b200_ctx* ctx, uint64_t limit_ns) {
    if (ctx == nullptr || limit_ns == 0 || limit_ns > 1000000000ULL) return B200_INVALID_ARGUMENT;
    return guarded(ctx, [&] { gemm_tc_wait_probe(ctx, limit_ns); });
}

}  // extern "C"
