// Data-parallel gradient exchange: one process per GPU, NCCL all-reduce over
// NVLink/NVSwitch on a communication stream that runs beside the compute stream.
//
// vkML itself is single-device (src/dispatch/executor.cpp:96-103), so this has
// no counterpart there.  backward() realises every leaf gradient in ONE compute
// span (src/autograd/autograd.cpp:627-666); with B200_COMPUTE_GRAD_SYNC the
// dispatcher calls dist_after_node() after queueing each node, and a gradient
// buffer registered with b200_dist_mark_grad is all-reduced as soon as its
// producer is queued, while the rest of the span keeps the SMs busy.
//
// NCCL is opened with dlopen at b200_dist_init so the library has no link-time
// dependency on it; a process that already loaded a libnccl.so.2 (for instance
// through PyTorch) shares that copy.
#include "context.h"

#include <dlfcn.h>
#include <nccl.h>  // types and initialisers only (ncclConfig_t): the library itself is opened with dlopen

#include <chrono>
#include <thread>

namespace b200 {

namespace {

// The handful of NCCL declarations used here (public API, nccl.h).
struct NcclUniqueId {
    char internal[128];
};
using NcclComm = void*;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclAvg = 4;

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommInitRankConfig)(NcclComm*, int, NcclUniqueId, int, ncclConfig_t*) = nullptr;
    int (*CommGetAsyncError)(NcclComm, int*) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (a.handle == nullptr) {
            a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        }
        if (a.handle != nullptr) {
            a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
            a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
            a.CommInitRankConfig =
                reinterpret_cast<decltype(a.CommInitRankConfig)>(dlsym(a.handle, "ncclCommInitRankConfig"));
            a.CommGetAsyncError =
                reinterpret_cast<decltype(a.CommGetAsyncError)>(dlsym(a.handle, "ncclCommGetAsyncError"));
            a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(dlsym(a.handle, "ncclCommAbort"));
            a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
            a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
            a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(dlsym(a.handle, "ncclGroupStart"));
            a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(dlsym(a.handle, "ncclGroupEnd"));
            a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
        }
        return a;
    }();
    return api;
}

void require_nccl() {
    const NcclApi& a = nccl();
    if (a.handle == nullptr || a.GetUniqueId == nullptr || a.CommInitRank == nullptr ||
        a.AllReduce == nullptr || a.CommDestroy == nullptr) {
        fail(B200_DEVICE_ERROR, "NCCL (libnccl.so.2) could not be loaded");
    }
}

void nccl_check(int rc, const char* what) {
    if (rc != 0) {
        const char* s = nccl().GetErrorString != nullptr ? nccl().GetErrorString(rc) : "?";
        fail(B200_DEVICE_ERROR, std::string(what) + ": NCCL error " + std::to_string(rc) + " (" + s + ")");
    }
}

// A communicator created in non-blocking mode (b200_dist_init_deadline) stays non-blocking: any
// call on it may return ncclInProgress, and the work is only known to be ENQUEUED on its stream
// once ncclCommGetAsyncError stops saying so.  Events recorded behind a collective must come
// after that point, so every call is settled before the host goes on.
void nccl_settle(NcclComm comm, int rc, const char* what) {
    if (rc == static_cast<int>(ncclInProgress) && nccl().CommGetAsyncError != nullptr) {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(60);
        int state = rc;
        do {
            if (nccl().CommGetAsyncError(comm, &state) != 0) {
                state = 1;
                break;
            }
            if (state != static_cast<int>(ncclInProgress)) break;
            std::this_thread::yield();
        } while (std::chrono::steady_clock::now() < deadline);
        rc = state;
    }
    nccl_check(rc, what);
}

}  // namespace

struct DistState {
    NcclComm comm = nullptr;
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t produced = nullptr;  // compute -> comm
    cudaEvent_t reduced = nullptr;   // comm -> compute
    bool pending = false;
    std::vector<char> done;          // per registered gradient, within one span
    // all-reduces that the compute stream has not been made to wait for yet, in issue order
    struct Lazy {
        const char* lo;
        const char* hi;
        cudaEvent_t done;
    };
    std::vector<Lazy> lazy;
    std::vector<cudaEvent_t> event_pool;
    std::mutex lazy_mu;  // b200_free may arrive from any thread (a Storage deleter) and looks at `lazy`
    // Small gradients of the running span, held back so that they leave as ONE grouped NCCL
    // launch: eight biases and 3x3 kernels of a few KB each would otherwise be eight launches of
    // a latency-bound collective on a step that takes a millisecond.
    struct Deferred {
        void* data;
        size_t count;
    };
    std::vector<Deferred> bucket;
    size_t bucket_bytes = 0;
    bool aborted = false;
    int comm_timeout_ms = 0;  // host deadline for outstanding collectives at a synchronisation (0: none)
};

constexpr size_t kBucketEachBytes = size_t(4) << 20;    // gradients below this are grouped

// Issues the all-reduces of `items` on the communication stream, ordered after everything queued
// on the compute stream so far; more than one item goes out as one NCCL group (one launch).
static void issue_all_reduces(b200_ctx* ctx, const DistState::Deferred* items, size_t n) {
    DistState* d = ctx->dist;
    if (n == 0) return;
    if (d->aborted) fail(B200_DEVICE_ERROR, "the communicator was aborted after an error or a timeout");
    B200_CUDA_CHECK(cudaEventRecord(d->produced, ctx->stream));
    B200_CUDA_CHECK(cudaStreamWaitEvent(d->comm_stream, d->produced, 0));
    const bool group = n > 1 && nccl().GroupStart != nullptr && nccl().GroupEnd != nullptr;
    if (group) nccl_check(nccl().GroupStart(), "ncclGroupStart");
    for (size_t i = 0; i < n; ++i) {
        const int rc = nccl().AllReduce(items[i].data, items[i].data, items[i].count, kNcclFloat32, kNcclAvg, d->comm,
                                        d->comm_stream);
        if (group) {
            // inside a group nothing is launched yet: in-progress is the expected answer
            if (rc != static_cast<int>(ncclInProgress)) nccl_check(rc, "ncclAllReduce");
        } else {
            nccl_settle(d->comm, rc, "ncclAllReduce");
        }
        ctx->comm_bytes.fetch_add(items[i].count * sizeof(float), std::memory_order_relaxed);
    }
    if (group) nccl_settle(d->comm, nccl().GroupEnd(), "ncclGroupEnd");
    d->pending = true;
    ctx->comm_pending = true;
    if (ctx->lazy_join) {
        std::lock_guard<std::mutex> lock(d->lazy_mu);
        for (size_t i = 0; i < n; ++i) {
            cudaEvent_t ev = nullptr;
            if (!d->event_pool.empty()) {
                ev = d->event_pool.back();
                d->event_pool.pop_back();
            } else {
                B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            }
            B200_CUDA_CHECK(cudaEventRecord(ev, d->comm_stream));
            d->lazy.push_back(DistState::Lazy{static_cast<const char*>(items[i].data),
                                              static_cast<const char*>(items[i].data) + items[i].count * sizeof(float), ev});
        }
    }
}

static void flush_bucket(b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr || d->bucket.empty()) return;
    std::vector<DistState::Deferred> items;
    items.swap(d->bucket);
    d->bucket_bytes = 0;
    issue_all_reduces(ctx, items.data(), items.size());
}

// `may_defer`: inside a gradient span a small buffer waits for its neighbours (flushed when the
// group is large enough, when anything touches one of its buffers, and at the end of the span).
static void all_reduce_mean(b200_ctx* ctx, void* data, size_t count, bool may_defer = false) {
    DistState* d = ctx->dist;
    const size_t bytes = count * sizeof(float);
    if (may_defer && ctx->bucket_grads && bytes < kBucketEachBytes) {
        d->bucket.push_back(DistState::Deferred{data, count});
        d->bucket_bytes += bytes;
        if (d->bucket_bytes >= ctx->bucket_flush_bytes) flush_bucket(ctx);
        return;
    }
    const DistState::Deferred one{data, count};
    issue_all_reduces(ctx, &one, 1);
}

// Makes the compute stream wait for the pending all-reduces that overlap [lo, hi) and for every
// one issued before them (the communication stream is in order); nullptr: for all of them.
void dist_wait_range(b200_ctx* ctx, const void* lo, const void* hi) {
    DistState* d = ctx->dist;
    if (d == nullptr) return;
    if (!d->bucket.empty()) {
        // a held-back gradient that something is about to touch must be on its way first
        bool touches = lo == nullptr;
        for (const DistState::Deferred& e : d->bucket) {
            const char* b0 = static_cast<const char*>(e.data);
            touches = touches || (static_cast<const char*>(lo) < b0 + e.count * sizeof(float) && b0 < static_cast<const char*>(hi));
        }
        if (touches) flush_bucket(ctx);
    }
    std::lock_guard<std::mutex> lock(d->lazy_mu);
    if (d->lazy.empty()) return;
    const char* a = static_cast<const char*>(lo);
    const char* b = static_cast<const char*>(hi);
    int last = -1;
    for (size_t i = 0; i < d->lazy.size(); ++i) {
        if (lo == nullptr || (a < d->lazy[i].hi && d->lazy[i].lo < b)) last = static_cast<int>(i);
    }
    if (last < 0) return;
    B200_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, d->lazy[static_cast<size_t>(last)].done, 0));
    for (int i = 0; i <= last; ++i) d->event_pool.push_back(d->lazy[static_cast<size_t>(i)].done);
    d->lazy.erase(d->lazy.begin(), d->lazy.begin() + last + 1);
    if (d->lazy.empty()) d->pending = false;
}

// Position (in issue order) of the last pending all-reduce overlapping [lo, hi), or -1.
int dist_pending_index(const b200_ctx* ctx, const void* lo, const void* hi) {
    DistState* d = ctx->dist;
    if (d == nullptr) return -1;
    std::lock_guard<std::mutex> lock(d->lazy_mu);
    const char* a = static_cast<const char*>(lo);
    const char* b = static_cast<const char*>(hi);
    int last = -1;
    for (size_t i = 0; i < d->lazy.size(); ++i) {
        if (a < d->lazy[i].hi && d->lazy[i].lo < b) last = static_cast<int>(i);
    }
    return last;
}

bool dist_has_pending(const b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr) return false;
    if (!d->bucket.empty()) return true;
    std::lock_guard<std::mutex> lock(d->lazy_mu);
    return !d->lazy.empty();
}

void dist_all_reduce_now(b200_ctx* ctx, void* data, size_t count) {
    if (ctx->dist != nullptr && count != 0) {
        all_reduce_mean(ctx, data, count, /*may_defer=*/true);
    }
}

void dist_after_node(b200_ctx* ctx, const b200_node& node) {
    DistState* d = ctx->dist;
    if (d == nullptr || ctx->grads.empty()) {
        return;
    }
    if (d->done.size() != ctx->grads.size()) {
        d->done.assign(ctx->grads.size(), 0);
    }
    size_t nbytes = dtype_size(node.out.dtype);
    for (int i = 0; i < node.out.ndim; ++i) {
        nbytes *= static_cast<size_t>(node.out.dims[i]);
    }
    const char* lo = static_cast<const char*>(node.out.data);
    const char* hi = lo + nbytes;
    for (size_t i = 0; i < ctx->grads.size(); ++i) {
        const char* g = static_cast<const char*>(ctx->grads[i].data);
        if (!d->done[i] && g >= lo && g < hi) {
            all_reduce_mean(ctx, ctx->grads[i].data, ctx->grads[i].count, /*may_defer=*/true);
            d->done[i] = 1;
        }
    }
}

void dist_join(b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr) {
        return;
    }
    // gradients whose producer was not in this span (already computed earlier)
    for (size_t i = 0; i < ctx->grads.size(); ++i) {
        if (d->done.size() == ctx->grads.size() && !d->done[i]) {
            all_reduce_mean(ctx, ctx->grads[i].data, ctx->grads[i].count);
        }
    }
    d->done.clear();
    flush_bucket(ctx);
    if (d->pending && !ctx->lazy_join) {
        B200_CUDA_CHECK(cudaEventRecord(d->reduced, d->comm_stream));
        B200_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, d->reduced, 0));
        d->pending = false;
    }
    // with lazy joining the compute stream waits where a reduced buffer is next touched
    ctx->comm_pending = false;
}

void dist_destroy(b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr) {
        return;
    }
    if (d->comm_stream != nullptr && !d->aborted) cudaStreamSynchronize(d->comm_stream);
    if (d->comm != nullptr && !d->aborted && nccl().CommDestroy != nullptr) nccl().CommDestroy(d->comm);
    for (auto& l : d->lazy) cudaEventDestroy(l.done);
    for (cudaEvent_t e : d->event_pool) cudaEventDestroy(e);
    if (d->produced != nullptr) cudaEventDestroy(d->produced);
    if (d->reduced != nullptr) cudaEventDestroy(d->reduced);
    if (d->comm_stream != nullptr) cudaStreamDestroy(d->comm_stream);
    delete d;
    ctx->dist = nullptr;
}

// Gives up on the communicator: NCCL's kernels are told to stop, nothing further is issued on it.
static void abort_comm(b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr || d->aborted) return;
    d->aborted = true;
    if (d->comm != nullptr && nccl().CommAbort != nullptr) nccl().CommAbort(d->comm);
    d->comm = nullptr;
    std::lock_guard<std::mutex> lock(d->lazy_mu);
    for (auto& l : d->lazy) d->event_pool.push_back(l.done);
    d->lazy.clear();
    d->bucket.clear();
    d->pending = false;
}

// Called where the host is about to block on device work that may include collectives: an error
// NCCL noticed by itself (a peer that went away) or a collective that outlives the host deadline
// ends with the communicator aborted and an error code, not with a process that waits for ever.
void dist_check_health(b200_ctx* ctx) {
    DistState* d = ctx->dist;
    if (d == nullptr || d->aborted || d->comm == nullptr) return;
    flush_bucket(ctx);
    auto async_error = [&]() -> int {
        int state = 0;
        if (nccl().CommGetAsyncError == nullptr) return 0;
        if (nccl().CommGetAsyncError(d->comm, &state) != 0) return -1;
        return state == static_cast<int>(ncclInProgress) ? 0 : state;
    };
    if (const int e = async_error()) {
        abort_comm(ctx);
        fail(B200_DEVICE_ERROR, "NCCL reported an asynchronous error (" + std::to_string(e) + "); the communicator was aborted");
    }
    if (d->comm_timeout_ms <= 0) return;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(d->comm_timeout_ms);
    while (cudaStreamQuery(d->comm_stream) == cudaErrorNotReady) {
        if (const int e = async_error()) {
            abort_comm(ctx);
            fail(B200_DEVICE_ERROR, "NCCL reported an asynchronous error (" + std::to_string(e) + "); the communicator was aborted");
        }
        if (std::chrono::steady_clock::now() > deadline) {
            abort_comm(ctx);
            fail(B200_TIMEOUT, "a collective did not finish within " + std::to_string(d->comm_timeout_ms) +
                                   " ms (VKML_B200_COMM_TIMEOUT_MS); the communicator was aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    cudaGetLastError();
}

namespace {
template <typename Fn>
int guarded_dist(b200_ctx* ctx, Fn&& fn) {
    try {
        if (ctx != nullptr) {
            cudaSetDevice(ctx->device);
        }
        fn();
        return B200_OK;
    } catch (const Error& e) {
        if (ctx != nullptr) {
            std::lock_guard<std::mutex> lock(ctx->err_mu);
            ctx->last_error = e.message;
        }
        return e.status;
    } catch (const std::exception& e) {
        if (ctx != nullptr) {
            std::lock_guard<std::mutex> lock(ctx->err_mu);
            ctx->last_error = e.what();
        }
        return B200_INTERNAL_ERROR;
    }
}
}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_dist_unique_id(void* out_id) {
    if (out_id == nullptr) return B200_INVALID_ARGUMENT;
    static_assert(sizeof(NcclUniqueId) == B200_UNIQUE_ID_BYTES);
    return guarded_dist(nullptr, [&] {
        require_nccl();
        NcclUniqueId id;
        nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
        std::memcpy(out_id, &id, sizeof(id));
    });
}

int b200_dist_init_deadline(b200_ctx* ctx, int rank, int world_size, const void* id, int timeout_ms) {
    if (ctx == nullptr || id == nullptr || world_size < 1 || rank < 0 || rank >= world_size || timeout_ms < 0) {
        return B200_INVALID_ARGUMENT;
    }
    return guarded_dist(ctx, [&] {
        require_nccl();
        if (ctx->dist != nullptr) {
            fail(B200_INVALID_ARGUMENT, "b200_dist_init: already initialised");
        }
        DistState* d = new DistState();
        ctx->dist = d;
        d->rank = rank;
        d->world = world_size;
        if (const char* e = std::getenv("VKML_B200_COMM_TIMEOUT_MS")) d->comm_timeout_ms = std::max(0, std::atoi(e));
        // highest priority: when SMs free up, the all-reduce's blocks are placed before the next
        // compute blocks, so communication is never starved by a queue of GEMM tiles
        int least = 0, greatest = 0;
        B200_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        B200_CUDA_CHECK(cudaStreamCreateWithPriority(&d->comm_stream, cudaStreamNonBlocking, greatest));
        B200_CUDA_CHECK(cudaEventCreateWithFlags(&d->produced, cudaEventDisableTiming));
        B200_CUDA_CHECK(cudaEventCreateWithFlags(&d->reduced, cudaEventDisableTiming));
        NcclUniqueId uid;
        std::memcpy(&uid, id, sizeof(uid));
        const bool can_poll = nccl().CommInitRankConfig != nullptr && nccl().CommGetAsyncError != nullptr &&
                              nccl().CommAbort != nullptr;
        if (timeout_ms == 0 || !can_poll) {
            nccl_check(nccl().CommInitRank(&d->comm, world_size, uid, rank), "ncclCommInitRank");
            return;
        }
        // Non-blocking initialisation: the call returns while the ranks are still finding each
        // other, and the host polls with a deadline -- a rank that never joins ends this one with
        // B200_TIMEOUT and an aborted communicator instead of a process stuck inside NCCL.
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.blocking = 0;
        int rc = nccl().CommInitRankConfig(&d->comm, world_size, uid, rank, &config);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        int state = rc;
        while (rc == 0 || rc == static_cast<int>(ncclInProgress)) {
            if (d->comm == nullptr || nccl().CommGetAsyncError(d->comm, &state) != 0) {
                state = -1;
                break;
            }
            if (state != static_cast<int>(ncclInProgress)) break;
            if (std::chrono::steady_clock::now() > deadline) {
                nccl().CommAbort(d->comm);
                d->comm = nullptr;
                dist_destroy(ctx);
                fail(B200_TIMEOUT, "the ranks did not all join within " + std::to_string(timeout_ms) +
                                       " ms; the communicator was aborted");
            }
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
        if (state != 0) {
            if (d->comm != nullptr) nccl().CommAbort(d->comm);
            d->comm = nullptr;
            dist_destroy(ctx);
            nccl_check(state > 0 ? state : 1, "ncclCommInitRankConfig");
        }
    });
}

int b200_dist_init(b200_ctx* ctx, int rank, int world_size, const void* id) {
    int timeout_ms = 120000;
    if (const char* e = std::getenv("VKML_B200_DIST_INIT_TIMEOUT_MS")) timeout_ms = std::max(0, std::atoi(e));
    return b200_dist_init_deadline(ctx, rank, world_size, id, timeout_ms);
}

int b200_dist_destroy(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded_dist(ctx, [&] { dist_destroy(ctx); });
}

int b200_dist_all_reduce_mean(b200_ctx* ctx, void* data, size_t count) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    if (count == 0) return B200_OK;
    return guarded_dist(ctx, [&] {
        if (ctx->dist == nullptr) fail(B200_INVALID_ARGUMENT, "b200_dist_init has not been called");
        all_reduce_mean(ctx, data, count);
    });
}

int b200_dist_wait(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    return guarded_dist(ctx, [&] {
        if (ctx->dist == nullptr) return;
        DistState* d = ctx->dist;
        dist_wait_range(ctx, nullptr, nullptr);
        if (d->pending) {
            B200_CUDA_CHECK(cudaEventRecord(d->reduced, d->comm_stream));
            B200_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, d->reduced, 0));
            d->pending = false;
        }
    });
}

int b200_dist_mark_grad(b200_ctx* ctx, void* data, size_t count) {
    if (ctx == nullptr || data == nullptr) return B200_INVALID_ARGUMENT;
    return guarded_dist(ctx, [&] { ctx->grads.push_back(GradBuffer{data, count}); });
}

int b200_dist_clear_grads(b200_ctx* ctx) {
    if (ctx == nullptr) return B200_INVALID_ARGUMENT;
    ctx->grads.clear();
    if (ctx->dist != nullptr) ctx->dist->done.clear();
    return B200_OK;
}

}  // extern "C"
