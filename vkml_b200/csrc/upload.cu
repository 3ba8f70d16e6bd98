// Uploads from pageable host memory.
//
// vkML hands copy_from_host whatever the caller's tensor lives in -- normally pageable memory
// (include/vkml/backend/api/allocator.h: copy_from_host(dst, src, nbytes) must leave `src` reusable
// on return).  The CUDA runtime serves such a copy by staging it through its own pinned buffer on
// the calling thread, which runs at the speed of ONE host memcpy (measured: 18 GB/s, 1.86 ms for
// the 33.5 MB batch of the wide MLP -- more than the rest of the host side of that step together).
// Here the staging is spread over a few threads: each owns a ring of pinned slots, copies its
// chunks of the source into them and queues the slot's DMA on the context's stream itself, so the
// host copies run side by side and overlap the transfers.  The call returns when every chunk has
// been read from the source; the DMAs complete in stream order, ahead of anything queued later.
#include "context.h"

#include <condition_variable>
#include <cstring>
#include <thread>

namespace b200 {

class Uploader {
public:
    static constexpr size_t kChunk = size_t(1) << 20;
    static constexpr int kSlotsPerThread = 4;

    Uploader(int device, cudaStream_t stream, int threads)
        : device_(device), stream_(stream), threads_(threads), slots_(static_cast<size_t>(threads) * kSlotsPerThread) {
        B200_CUDA_CHECK(cudaHostAlloc(&pinned_, slots_.size() * kChunk, cudaHostAllocDefault));
        for (size_t i = 0; i < slots_.size(); ++i) {
            slots_[i].buffer = static_cast<char*>(pinned_) + i * kChunk;
            B200_CUDA_CHECK(cudaEventCreateWithFlags(&slots_[i].done, cudaEventDisableTiming));
        }
        for (int t = 1; t < threads_; ++t) {
            workers_.emplace_back([this, t] { worker_loop(t); });
        }
    }

    ~Uploader() {
        {
            std::lock_guard<std::mutex> lock(mu_);
            quit_ = true;
        }
        wake_.notify_all();
        for (std::thread& w : workers_) w.join();
        for (Slot& s : slots_) cudaEventDestroy(s.done);
        cudaFreeHost(pinned_);
    }

    // Returns when `src` may be reused; the transfers themselves are ordered on the stream.
    void copy(void* dst, const void* src, size_t nbytes) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            dst_ = static_cast<char*>(dst);
            src_ = static_cast<const char*>(src);
            nbytes_ = nbytes;
            chunks_ = (nbytes + kChunk - 1) / kChunk;
            pending_ = threads_ - 1;
            error_ = cudaSuccess;
            ++job_;
        }
        wake_.notify_all();
        const cudaError_t mine = run(0);
        std::unique_lock<std::mutex> lock(mu_);
        done_.wait(lock, [this] { return pending_ == 0; });
        const cudaError_t e = mine != cudaSuccess ? mine : error_;
        if (e != cudaSuccess) {
            fail(B200_INTERNAL_ERROR, std::string("copy_from_host (staged upload): ") + cudaGetErrorString(e));
        }
    }

private:
    struct Slot {
        char* buffer = nullptr;
        cudaEvent_t done = nullptr;
        bool used = false;
    };

    // Thread t takes chunks t, t + T, t + 2T ... and walks its own slots round-robin, so a slot's
    // previous transfer was queued by the same thread and its event is already recorded.
    cudaError_t run(int t) {
        size_t turn = 0;
        for (size_t c = static_cast<size_t>(t); c < chunks_; c += static_cast<size_t>(threads_), ++turn) {
            Slot& s = slots_[static_cast<size_t>(t) * kSlotsPerThread + turn % kSlotsPerThread];
            if (s.used) {
                if (const cudaError_t e = cudaEventSynchronize(s.done); e != cudaSuccess) return e;
            }
            const size_t off = c * kChunk;
            const size_t n = std::min(kChunk, nbytes_ - off);
            std::memcpy(s.buffer, src_ + off, n);
            if (const cudaError_t e = cudaMemcpyAsync(dst_ + off, s.buffer, n, cudaMemcpyHostToDevice, stream_);
                e != cudaSuccess) {
                return e;
            }
            if (const cudaError_t e = cudaEventRecord(s.done, stream_); e != cudaSuccess) return e;
            s.used = true;
        }
        return cudaSuccess;
    }

    void worker_loop(int t) {
        cudaSetDevice(device_);
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(mu_);
                wake_.wait(lock, [&] { return quit_ || job_ != seen; });
                if (quit_) return;
                seen = job_;
            }
            const cudaError_t e = run(t);
            std::lock_guard<std::mutex> lock(mu_);
            if (e != cudaSuccess && error_ == cudaSuccess) error_ = e;
            if (--pending_ == 0) done_.notify_one();
        }
    }

    int device_;
    cudaStream_t stream_;
    int threads_;
    void* pinned_ = nullptr;
    std::vector<Slot> slots_;
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable wake_, done_;
    bool quit_ = false;
    uint64_t job_ = 0;
    int pending_ = 0;
    cudaError_t error_ = cudaSuccess;
    char* dst_ = nullptr;
    const char* src_ = nullptr;
    size_t nbytes_ = 0, chunks_ = 0;
};

bool staged_upload(b200_ctx* ctx, void* dst, const void* src, size_t nbytes) {
    if (ctx->upload_threads < 2 || nbytes < 2 * Uploader::kChunk || ctx->capturing) {
        return false;
    }
    if (ctx->uploader == nullptr) {
        ctx->uploader = new Uploader(ctx->device, ctx->stream, ctx->upload_threads);
    }
    ctx->uploader->copy(dst, src, nbytes);
    return true;
}

void destroy_uploader(b200_ctx* ctx) {
    delete ctx->uploader;
    ctx->uploader = nullptr;
}

}  // namespace b200
