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
};

static void all_reduce_mean(b200_ctx* ctx, void* data, size_t count) {
    DistState* d = ctx->dist;
    B200_CUDA_CHECK(cudaEventRecord(d->produced, ctx->stream));
    B200_CUDA_CHECK(cudaStreamWaitEvent(d->comm_stream, d->produced, 0));
    nccl_check(nccl().AllReduce(data, data, count, kNcclFloat32, kNcclAvg, d->comm, d->comm_stream),
               "ncclAllReduce");
    d->pending = true;
    ctx->comm_pending = true;
    ctx->comm_bytes.fetch_add(count * sizeof(float), std::memory_order_relaxed);
    if (ctx->lazy_join) {
        std::lock_guard<std::mutex> lock(d->lazy_mu);
        cudaEvent_t ev = nullptr;
        if (!d->event_pool.empty()) {
            ev = d->event_pool.back();
            d->event_pool.pop_back();
        } else {
            B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        }
        B200_CUDA_CHECK(cudaEventRecord(ev, d->comm_stream));
        d->lazy.push_back(DistState::Lazy{static_cast<const char*>(data),
                                          static_cast<const char*>(data) + count * sizeof(float), ev});
    }
}

// Makes the compute stream wait for the pending all-reduces that overlap [lo, hi) and for every
// one issued before them (the communication stream is in order); nullptr: for all of them.
void dist_wait_range(b200_ctx* ctx, const void* lo, const void* hi) {
    DistState* d = ctx->dist;
    if (d == nullptr) return;
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
    std::lock_guard<std::mutex> lock(d->lazy_mu);
    return !d->lazy.empty();
}

void dist_all_reduce_now(b200_ctx* ctx, void* data, size_t count) {
    if (ctx->dist != nullptr && count != 0) {
        all_reduce_mean(ctx, data, count);
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
            all_reduce_mean(ctx, ctx->grads[i].data, ctx->grads[i].count);
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
    if (d->comm_stream != nullptr) cudaStreamSynchronize(d->comm_stream);
    if (d->comm != nullptr && nccl().CommDestroy != nullptr) nccl().CommDestroy(d->comm);
    for (auto& l : d->lazy) cudaEventDestroy(l.done);
    for (cudaEvent_t e : d->event_pool) cudaEventDestroy(e);
    if (d->produced != nullptr) cudaEventDestroy(d->produced);
    if (d->reduced != nullptr) cudaEventDestroy(d->reduced);
    if (d->comm_stream != nullptr) cudaStreamDestroy(d->comm_stream);
    delete d;
    ctx->dist = nullptr;
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

int b200_dist_init(b200_ctx* ctx, int rank, int world_size, const void* id) {
    if (ctx == nullptr || id == nullptr || world_size < 1 || rank < 0 || rank >= world_size) {
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
        // highest priority: when SMs free up, the all-reduce's blocks are placed before the next
        // compute blocks, so communication is never starved by a queue of GEMM tiles
        int least = 0, greatest = 0;
        B200_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        B200_CUDA_CHECK(cudaStreamCreateWithPriority(&d->comm_stream, cudaStreamNonBlocking, greatest));
        B200_CUDA_CHECK(cudaEventCreateWithFlags(&d->produced, cudaEventDisableTiming));
        B200_CUDA_CHECK(cudaEventCreateWithFlags(&d->reduced, cudaEventDisableTiming));
        NcclUniqueId uid;
        std::memcpy(&uid, id, sizeof(uid));
        nccl_check(nccl().CommInitRank(&d->comm, world_size, uid, rank), "ncclCommInitRank");
    });
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
