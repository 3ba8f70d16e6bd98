// Step tape: replays the exact sequence of backend calls a framework makes for one
// training step -- allocations, frees, uploads, compute spans, batched device copies,
// downloads -- from a flat array of 64-bit words, with buffers named by position instead
// of by address.  It is the host half of vkML's executor reduced to what reaches the
// backend (src/dispatch/executor.cpp:105-144, src/core/tensor.cpp:101-111,178-201,397-425):
// every event becomes exactly one call of the public C ABI, in the recorded order, so a
// step costs what the same calls cost from the framework's C++ and not what a scripting
// language adds on top.  vkML plans the same thing one level up ("re-submit the cached
// command buffer" for an unchanged step, docs/ARCHITECTURE.md:565-569).
//
// Word format, one template = a sequence of events:
//   1 ALLOC   bytes
//   2 FREE    where j
//   3 H2D     where j offset bytes upload#
//   4 COMPUTE n_nodes grad_sync  then per node: op n_src params[8 words] out src[n_src]
//             tensor = where j offset dtype ndim dims[4] strides[4]
//   5 D2D     n  then n x (dst where, j, offset, src where, j, offset, bytes)
//   6 D2H     where j offset bytes download#
//   7 SYNC
// A buffer reference is (where, j): where = -1 the j-th allocation of the prologue,
// -2 no buffer, d >= 0 the j-th allocation of the step d steps back (0 = the running one).
//
// Graph mode (b200_tape_enable_graphs).  The caching allocator is deterministic, so once
// training is in its steady state every step is handed the same device addresses as an
// earlier one.  A step is then run in two passes: first its allocations and frees alone
// (they only move blocks between the allocator's lists), then -- if the addresses, the
// upload pointers, the library scratch and the allocator's block set all match a step seen
// before -- one cudaGraphLaunch of that step's device work, which was captured from the
// stream the second time the addresses came up.  Kernels, their order and their arguments
// are exactly those of the eager replay; only the host cost per launch goes away.
#include "context.h"

#include <cstring>
#include <deque>
#include <unordered_map>

namespace {

struct Slot {
    void* p = nullptr;
    bool live = false;
};

struct GraphEntry {
    cudaGraphExec_t exec = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
};

struct Template {
    std::vector<int64_t> words;
    bool is_prologue = false;
    bool capturable = true;
    size_t download_bytes = 0;
    std::unordered_map<uint64_t, int> seen;          // address signature -> times seen
    std::unordered_map<uint64_t, GraphEntry> graphs;
};

}  // namespace

struct b200_tape {
    b200_ctx* ctx = nullptr;
    int lookback = 1;
    bool use_graphs = false;
    std::vector<Template> templates;
    std::vector<Slot> pro;
    std::deque<std::vector<Slot>> history;  // newest last
    std::vector<b200_node> nodes;
    std::vector<b200_copy> copies;
    // pinned landing area of a graph step's downloads, copied to the caller's buffers after the
    // step's single synchronisation
    char* stage = nullptr;
    size_t stage_bytes = 0;
    uint64_t steps_run = 0, graph_launches = 0, graph_captures = 0;
};

namespace {

using namespace b200;

enum : int64_t { kAlloc = 1, kFree = 2, kH2D = 3, kCompute = 4, kD2D = 5, kD2H = 6, kSync = 7 };
constexpr int kTensorWords = 13;

enum class Pass { Eager, MemoryOnly, DeviceEager, DeviceCapture };

struct Reader {
    const int64_t* w;
    size_t n, pos = 0;
    int64_t next() {
        if (pos >= n) fail(B200_INVALID_ARGUMENT, "tape: template ends inside an event");
        return w[pos++];
    }
    void skip(size_t k) {
        if (pos + k > n) fail(B200_INVALID_ARGUMENT, "tape: template ends inside an event");
        pos += k;
    }
    bool done() const { return pos >= n; }
};

Slot* slot(b200_tape* t, std::vector<Slot>& current, int64_t where, int64_t j) {
    std::vector<Slot>* list = nullptr;
    if (where == -1) {
        list = &t->pro;
    } else if (where == 0) {
        list = &current;
    } else if (where > 0 && static_cast<size_t>(where) < t->history.size()) {
        list = &t->history[t->history.size() - 1 - static_cast<size_t>(where)];
    }
    if (list == nullptr || j < 0 || static_cast<size_t>(j) >= list->size()) {
        fail(B200_INVALID_ARGUMENT, "tape: buffer reference out of range");
    }
    return &(*list)[static_cast<size_t>(j)];
}

// The address stays readable after the slot was freed: in the two-pass order the frees of a
// step are booked before its device work is issued (the work itself keeps the recorded order).
char* address(b200_tape* t, std::vector<Slot>& current, int64_t where, int64_t j, int64_t offset) {
    if (where == -2) return nullptr;
    void* base = slot(t, current, where, j)->p;
    return base == nullptr ? nullptr : static_cast<char*>(base) + offset;
}

void read_tensor(b200_tape* t, std::vector<Slot>& current, Reader& r, b200_tensor& out) {
    const int64_t where = r.next(), j = r.next(), offset = r.next();
    out.data = address(t, current, where, j, offset);
    out.dtype = static_cast<int32_t>(r.next());
    out.ndim = static_cast<int32_t>(r.next());
    for (int d = 0; d < B200_MAX_DIMS; ++d) out.dims[d] = r.next();
    for (int d = 0; d < B200_MAX_DIMS; ++d) out.strides[d] = r.next();
}

void check(b200_tape* t, int status, const char* what) {
    if (status != B200_OK) {
        const char* msg = b200_last_error(t->ctx);
        fail(static_cast<b200_status>(status), std::string("tape: ") + what + ": " + (msg != nullptr ? msg : ""));
    }
}

struct HostBuffers {
    const void* const* uploads;
    size_t n_uploads;
    void* const* downloads;
    size_t n_downloads;
    const void* upload(int64_t i) const {
        return (uploads != nullptr && i >= 0 && static_cast<size_t>(i) < n_uploads) ? uploads[i] : nullptr;
    }
    void* download(int64_t i) const {
        return (downloads != nullptr && i >= 0 && static_cast<size_t>(i) < n_downloads) ? downloads[i] : nullptr;
    }
};

// Walks one template.  Eager: every event in order.  MemoryOnly: allocations and frees.
// DeviceEager / DeviceCapture: everything else, against the slots MemoryOnly filled; in capture
// the copies are recorded without their synchronisation and downloads land in the pinned stage.
void run_template(b200_tape* t, const std::vector<int64_t>& words, std::vector<Slot>& current, Pass pass,
                  const HostBuffers& host, uint32_t grad_flags) {
    const bool memory = pass == Pass::Eager || pass == Pass::MemoryOnly;
    const bool device = pass != Pass::MemoryOnly;
    const bool capture = pass == Pass::DeviceCapture;
    cudaStream_t stream = t->ctx->stream;
    size_t stage_offset = 0;
    Reader r{words.data(), words.size()};
    while (!r.done()) {
        const int64_t ev = r.next();
        if (ev == kAlloc) {
            const int64_t bytes = r.next();
            if (memory) {
                void* p = nullptr;
                check(t, b200_alloc(t->ctx, static_cast<size_t>(bytes), &p), "allocate");
                current.push_back(Slot{p, true});
            }
        } else if (ev == kFree) {
            const int64_t where = r.next(), j = r.next();
            if (memory) {
                Slot* s = slot(t, current, where, j);
                if (s->live) {
                    check(t, b200_free(t->ctx, s->p), "free");
                    s->live = false;
                }
            }
        } else if (ev == kH2D) {
            const int64_t where = r.next(), j = r.next(), offset = r.next(), bytes = r.next(), index = r.next();
            const void* src = host.upload(index);
            if (device && src != nullptr && bytes > 0) {
                char* dst = address(t, current, where, j, offset);
                if (capture) {
                    B200_CUDA_CHECK(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyHostToDevice, stream));
                } else {
                    check(t, b200_copy_from_host(t->ctx, dst, src, static_cast<size_t>(bytes)), "upload");
                }
            }
        } else if (ev == kCompute) {
            const int64_t n_nodes = r.next(), grad_sync = r.next();
            if (!device) {
                for (int64_t i = 0; i < n_nodes; ++i) {
                    r.next();
                    const int64_t n_src = r.next();
                    r.skip(static_cast<size_t>(B200_PARAM_BYTES / 8 + kTensorWords * (1 + n_src)));
                }
                continue;
            }
            t->nodes.resize(static_cast<size_t>(n_nodes));
            for (int64_t i = 0; i < n_nodes; ++i) {
                b200_node& node = t->nodes[static_cast<size_t>(i)];
                std::memset(&node, 0, sizeof node);
                node.op = static_cast<uint32_t>(r.next());
                node.n_src = static_cast<uint32_t>(r.next());
                if (node.n_src > B200_MAX_SRC) fail(B200_INVALID_ARGUMENT, "tape: too many sources");
                for (int k = 0; k < B200_PARAM_BYTES / 8; ++k) {
                    const int64_t v = r.next();
                    std::memcpy(node.params + 8 * k, &v, 8);
                }
                read_tensor(t, current, r, node.out);
                for (uint32_t s = 0; s < node.n_src; ++s) read_tensor(t, current, r, node.src[s]);
            }
            check(t, b200_compute(t->ctx, t->nodes.data(), t->nodes.size(), grad_sync != 0 ? grad_flags : 0u),
                  "compute");
        } else if (ev == kD2D) {
            const int64_t n = r.next();
            if (!device) {
                r.skip(static_cast<size_t>(7 * n));
                continue;
            }
            t->copies.resize(static_cast<size_t>(n));
            for (int64_t i = 0; i < n; ++i) {
                const int64_t dw = r.next(), dj = r.next(), doff = r.next();
                const int64_t sw = r.next(), sj = r.next(), soff = r.next();
                b200_copy& c = t->copies[static_cast<size_t>(i)];
                c.dst = address(t, current, dw, dj, doff);
                c.src = address(t, current, sw, sj, soff);
                c.nbytes = static_cast<size_t>(r.next());
            }
            check(t, b200_copy_device_to_device(t->ctx, t->copies.data(), t->copies.size()), "device copy");
        } else if (ev == kD2H) {
            const int64_t where = r.next(), j = r.next(), offset = r.next(), bytes = r.next(), index = r.next();
            if (!device) continue;
            if (capture) {
                B200_CUDA_CHECK(cudaMemcpyAsync(t->stage + stage_offset, address(t, current, where, j, offset),
                                                static_cast<size_t>(bytes), cudaMemcpyDeviceToHost, stream));
                stage_offset += static_cast<size_t>((bytes + 15) / 16 * 16);
            } else {
                void* dst = host.download(index);
                if (dst == nullptr) fail(B200_INVALID_ARGUMENT, "tape: a download has no host buffer");
                check(t, b200_copy_to_host(t->ctx, dst, address(t, current, where, j, offset),
                                           static_cast<size_t>(bytes)), "download");
            }
        } else if (ev == kSync) {
            if (device && !capture) check(t, b200_synchronize(t->ctx), "synchronize");
        } else {
            fail(B200_INVALID_ARGUMENT, "tape: unknown event " + std::to_string(ev));
        }
    }
}

// Consumes the words of one event whose kind has just been read (everything but a download).
void skip_event(Reader& r, int64_t ev) {
    if (ev == kAlloc) {
        r.skip(1);
    } else if (ev == kFree) {
        r.skip(2);
    } else if (ev == kH2D) {
        r.skip(5);
    } else if (ev == kCompute) {
        const int64_t n_nodes = r.next();
        r.skip(1);
        for (int64_t i = 0; i < n_nodes; ++i) {
            r.next();
            const int64_t n_src = r.next();
            r.skip(static_cast<size_t>(B200_PARAM_BYTES / 8 + kTensorWords * (1 + n_src)));
        }
    } else if (ev == kD2D) {
        const int64_t n = r.next();
        r.skip(static_cast<size_t>(7 * n));
    } else if (ev != kSync) {
        fail(B200_INVALID_ARGUMENT, "tape: unknown event " + std::to_string(ev));
    }
}

// Visits the downloads of a template in order: fn(bytes, download index, offset in the stage).
template <typename Fn>
void for_each_download(const std::vector<int64_t>& words, Fn&& fn) {
    size_t stage_offset = 0;
    Reader r{words.data(), words.size()};
    while (!r.done()) {
        const int64_t ev = r.next();
        if (ev != kD2H) {
            skip_event(r, ev);
            continue;
        }
        r.skip(3);
        const int64_t bytes = r.next(), index = r.next();
        fn(bytes, index, stage_offset);
        stage_offset += static_cast<size_t>((bytes + 15) / 16 * 16);
    }
}

// After a graph step's one synchronisation: hand the staged downloads to the caller.
void deliver_downloads(b200_tape* t, const std::vector<int64_t>& words, const HostBuffers& host) {
    for_each_download(words, [&](int64_t bytes, int64_t index, size_t stage_offset) {
        void* dst = host.download(index);
        if (dst == nullptr) fail(B200_INVALID_ARGUMENT, "tape: a download has no host buffer");
        std::memcpy(dst, t->stage + stage_offset, static_cast<size_t>(bytes));
    });
}

// Size of the pinned stage a template's downloads need; walking it also validates the event stream.
size_t staged_download_bytes(const std::vector<int64_t>& words) {
    size_t total = 0;
    for_each_download(words, [&](int64_t bytes, int64_t, size_t) { total += static_cast<size_t>((bytes + 15) / 16 * 16); });
    return total;
}

void release_list(b200_tape* t, std::vector<Slot>& list) {
    for (Slot& s : list) {
        if (s.live) {
            b200_free(t->ctx, s.p);
            s.live = false;
        }
    }
}

void mix(uint64_t& h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
}

// Everything a captured step's device work depends on besides the template itself.
uint64_t signature(b200_tape* t, const HostBuffers& host) {
    uint64_t h = 1469598103934665603ull;
    for (const Slot& s : t->pro) mix(h, reinterpret_cast<uintptr_t>(s.p));
    for (const auto& list : t->history) {
        mix(h, list.size());
        for (const Slot& s : list) mix(h, reinterpret_cast<uintptr_t>(s.p));
    }
    for (size_t i = 0; i < host.n_uploads; ++i) mix(h, reinterpret_cast<uintptr_t>(host.uploads[i]));
    mix(h, t->ctx->alloc.driver_allocs);
    mix(h, t->ctx->scratch.driver_allocs);  // same scratch blocks => the same ones are free for the planes
    mix(h, static_cast<uint64_t>(t->ctx->gemm_precision));
    return h;
}

bool uploads_are_pinned(const HostBuffers& host) {
    for (size_t i = 0; i < host.n_uploads; ++i) {
        if (host.uploads[i] == nullptr) continue;
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, host.uploads[i]) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (attr.type != cudaMemoryTypeHost) return false;
    }
    return true;
}

void finish_graph_step(b200_tape* t, const Template& tpl, const HostBuffers& host) {
    check(t, b200_synchronize(t->ctx), "synchronize");
    if (tpl.download_bytes != 0) deliver_downloads(t, tpl.words, host);
}

// One step with graphs enabled.  Returns false when the step has to be issued eagerly
// (its allocations and frees have been made either way).
bool run_graph_step(b200_tape* t, Template& tpl, std::vector<Slot>& current, const HostBuffers& host) {
    b200_ctx* ctx = t->ctx;
    run_template(t, tpl.words, current, Pass::MemoryOnly, host, 0);
    if (!tpl.capturable || ctx->profiling || !uploads_are_pinned(host)) return false;
    const uint64_t sig = signature(t, host);
    auto hit = tpl.graphs.find(sig);
    if (hit != tpl.graphs.end() && hit->second.workspace == ctx->workspace &&
        hit->second.workspace_bytes == ctx->workspace_bytes) {
        B200_CUDA_CHECK(cudaGraphLaunch(hit->second.exec, ctx->stream));
        ++t->graph_launches;
        finish_graph_step(t, tpl, host);
        return true;
    }
    if (++tpl.seen[sig] < 2 || tpl.graphs.size() >= 16) return false;

    // second sighting of these addresses: capture the step's device work, then launch it
    if (t->stage_bytes < tpl.download_bytes) {
        if (t->stage != nullptr) cudaFreeHost(t->stage);
        t->stage = nullptr;
        t->stage_bytes = 0;
        B200_CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&t->stage), tpl.download_bytes));
        t->stage_bytes = tpl.download_bytes;
        for (Template& other : t->templates) {  // older graphs point at the old stage
            for (auto& kv : other.graphs) cudaGraphExecDestroy(kv.second.exec);
            other.graphs.clear();
        }
    }
    cudaGraph_t graph = nullptr;
    B200_CUDA_CHECK(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    bool ok = true;
    std::string why;
    try {
        run_template(t, tpl.words, current, Pass::DeviceCapture, host, 0);
    } catch (const Error& e) {
        ok = false;
        why = e.message;
    }
    ctx->capturing = false;
    const cudaError_t end = cudaStreamEndCapture(ctx->stream, &graph);
    if (end != cudaSuccess || graph == nullptr) {
        cudaGetLastError();
        ok = false;
    }
    GraphEntry entry;
    if (ok && cudaGraphInstantiate(&entry.exec, graph, 0) != cudaSuccess) {
        cudaGetLastError();
        ok = false;
    }
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (!ok) {
        tpl.capturable = false;  // this template stays on the eager path
        return false;
    }
    entry.workspace = ctx->workspace;
    entry.workspace_bytes = ctx->workspace_bytes;
    tpl.graphs[sig] = entry;
    ++t->graph_captures;
    B200_CUDA_CHECK(cudaGraphLaunch(entry.exec, ctx->stream));
    ++t->graph_launches;
    finish_graph_step(t, tpl, host);
    return true;
}

template <typename Fn>
int tape_guarded(b200_tape* t, Fn&& fn) {
    try {
        if (t != nullptr && t->ctx != nullptr) {
            const cudaError_t err = cudaSetDevice(t->ctx->device);
            if (err != cudaSuccess) return B200_DEVICE_ERROR;
        }
        fn();
        return B200_OK;
    } catch (const Error& e) {
        if (t != nullptr && t->ctx != nullptr) {
            std::lock_guard<std::mutex> lock(t->ctx->err_mu);
            t->ctx->last_error = e.message;
        }
        return e.status;
    } catch (const std::bad_alloc&) {
        return B200_OUT_OF_MEMORY;
    } catch (const std::exception&) {
        return B200_INTERNAL_ERROR;
    }
}

}  // namespace

extern "C" {

int b200_tape_create(b200_ctx* ctx, int lookback, b200_tape** out) {
    if (ctx == nullptr || out == nullptr || lookback < 0) return B200_INVALID_ARGUMENT;
    b200_tape* t = new (std::nothrow) b200_tape();
    if (t == nullptr) return B200_OUT_OF_MEMORY;
    t->ctx = ctx;
    t->lookback = lookback;
    *out = t;
    return B200_OK;
}

int b200_tape_add_template(b200_tape* tape, const int64_t* words, size_t n_words, int is_prologue, int* index) {
    if (tape == nullptr || (words == nullptr && n_words != 0)) return B200_INVALID_ARGUMENT;
    return tape_guarded(tape, [&] {
        Template tpl;
        tpl.words.assign(words, words + n_words);
        tpl.is_prologue = is_prologue != 0;
        tpl.download_bytes = staged_download_bytes(tpl.words);  // also validates the event stream
        tape->templates.push_back(std::move(tpl));
        if (index != nullptr) *index = static_cast<int>(tape->templates.size()) - 1;
    });
}

int b200_tape_enable_graphs(b200_tape* tape, int on) {
    if (tape == nullptr) return B200_INVALID_ARGUMENT;
    tape->use_graphs = on != 0;
    return B200_OK;
}

int b200_tape_run(b200_tape* tape, int index, const void* const* uploads, size_t n_uploads, void* const* downloads,
                  size_t n_downloads, uint32_t grad_sync_flags) {
    if (tape == nullptr || index < 0 || static_cast<size_t>(index) >= tape->templates.size()) {
        return B200_INVALID_ARGUMENT;
    }
    return tape_guarded(tape, [&] {
        Template& tpl = tape->templates[static_cast<size_t>(index)];
        const HostBuffers host{uploads, uploads != nullptr ? n_uploads : 0, downloads,
                               downloads != nullptr ? n_downloads : 0};
        if (tpl.is_prologue) {
            run_template(tape, tpl.words, tape->pro, Pass::Eager, host, grad_sync_flags);
            return;
        }
        tape->history.emplace_back();
        std::vector<Slot>& current = tape->history.back();
        if (tape->use_graphs && grad_sync_flags == 0) {
            if (!run_graph_step(tape, tpl, current, host)) {
                run_template(tape, tpl.words, current, Pass::DeviceEager, host, 0);
            }
        } else {
            run_template(tape, tpl.words, current, Pass::Eager, host, grad_sync_flags);
        }
        // allocations older than any template reaches back are dropped, as the framework's
        // last handle to them is
        while (tape->history.size() > static_cast<size_t>(tape->lookback) + 1) {
            release_list(tape, tape->history.front());
            tape->history.pop_front();
        }
        ++tape->steps_run;
    });
}

int b200_tape_stats(b200_tape* tape, uint64_t* steps, uint64_t* graph_launches, uint64_t* graph_captures) {
    if (tape == nullptr) return B200_INVALID_ARGUMENT;
    if (steps != nullptr) *steps = tape->steps_run;
    if (graph_launches != nullptr) *graph_launches = tape->graph_launches;
    if (graph_captures != nullptr) *graph_captures = tape->graph_captures;
    return B200_OK;
}

void b200_tape_destroy(b200_tape* tape) {
    if (tape == nullptr) return;
    if (tape->ctx != nullptr) cudaSetDevice(tape->ctx->device);
    for (Template& tpl : tape->templates) {
        for (auto& kv : tpl.graphs) cudaGraphExecDestroy(kv.second.exec);
    }
    for (auto& list : tape->history) release_list(tape, list);
    release_list(tape, tape->pro);
    if (tape->stage != nullptr) cudaFreeHost(tape->stage);
    delete tape;
}

}  // extern "C"
