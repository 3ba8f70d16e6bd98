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
#include "context.h"

#include <cstring>
#include <deque>

struct b200_tape {
    b200_ctx* ctx = nullptr;
    int lookback = 1;
    bool prologue_done = false;
    std::vector<std::vector<int64_t>> templates;
    std::vector<char> is_prologue;
    std::vector<void*> pro;
    std::deque<std::vector<void*>> history;  // newest last
    std::vector<b200_node> nodes;
    std::vector<b200_copy> copies;
    uint64_t steps_run = 0;
};

namespace {

using namespace b200;

enum : int64_t { kAlloc = 1, kFree = 2, kH2D = 3, kCompute = 4, kD2D = 5, kD2H = 6, kSync = 7 };

struct Reader {
    const int64_t* w;
    size_t n, pos = 0;
    int64_t next() {
        if (pos >= n) fail(B200_INVALID_ARGUMENT, "tape: template ends inside an event");
        return w[pos++];
    }
    bool done() const { return pos >= n; }
};

void** slot(b200_tape* t, std::vector<void*>& current, int64_t where, int64_t j) {
    std::vector<void*>* list = nullptr;
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

char* address(b200_tape* t, std::vector<void*>& current, int64_t where, int64_t j, int64_t offset) {
    if (where == -2) return nullptr;
    void* base = *slot(t, current, where, j);
    return base == nullptr ? nullptr : static_cast<char*>(base) + offset;
}

void read_tensor(b200_tape* t, std::vector<void*>& current, Reader& r, b200_tensor& out) {
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

void run_template(b200_tape* t, const std::vector<int64_t>& words, std::vector<void*>& current,
                  const void* const* uploads, size_t n_uploads, void* const* downloads, size_t n_downloads,
                  uint32_t grad_flags) {
    Reader r{words.data(), words.size()};
    while (!r.done()) {
        const int64_t ev = r.next();
        if (ev == kAlloc) {
            void* p = nullptr;
            check(t, b200_alloc(t->ctx, static_cast<size_t>(r.next()), &p), "allocate");
            current.push_back(p);
        } else if (ev == kFree) {
            const int64_t where = r.next(), j = r.next();
            void** s = slot(t, current, where, j);
            if (*s != nullptr) {
                check(t, b200_free(t->ctx, *s), "free");
                *s = nullptr;
            }
        } else if (ev == kH2D) {
            const int64_t where = r.next(), j = r.next(), offset = r.next(), bytes = r.next(), index = r.next();
            const void* src = (uploads != nullptr && index >= 0 && static_cast<size_t>(index) < n_uploads)
                                  ? uploads[index] : nullptr;
            if (src != nullptr && bytes > 0) {
                check(t, b200_copy_from_host(t->ctx, address(t, current, where, j, offset), src,
                                             static_cast<size_t>(bytes)), "upload");
            }
        } else if (ev == kCompute) {
            const int64_t n_nodes = r.next(), grad_sync = r.next();
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
            void* dst = (downloads != nullptr && index >= 0 && static_cast<size_t>(index) < n_downloads)
                            ? downloads[index] : nullptr;
            if (dst == nullptr) fail(B200_INVALID_ARGUMENT, "tape: a download has no host buffer");
            check(t, b200_copy_to_host(t->ctx, dst, address(t, current, where, j, offset),
                                       static_cast<size_t>(bytes)), "download");
        } else if (ev == kSync) {
            check(t, b200_synchronize(t->ctx), "synchronize");
        } else {
            fail(B200_INVALID_ARGUMENT, "tape: unknown event " + std::to_string(ev));
        }
    }
}

void release_list(b200_tape* t, std::vector<void*>& list) {
    for (void*& p : list) {
        if (p != nullptr) {
            b200_free(t->ctx, p);
            p = nullptr;
        }
    }
}

template <typename Fn>
int tape_guarded(b200_tape* t, Fn&& fn) {
    try {
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
        tape->templates.emplace_back(words, words + n_words);
        tape->is_prologue.push_back(is_prologue != 0 ? 1 : 0);
        if (index != nullptr) *index = static_cast<int>(tape->templates.size()) - 1;
    });
}

int b200_tape_run(b200_tape* tape, int index, const void* const* uploads, size_t n_uploads, void* const* downloads,
                  size_t n_downloads, uint32_t grad_sync_flags) {
    if (tape == nullptr || index < 0 || static_cast<size_t>(index) >= tape->templates.size()) {
        return B200_INVALID_ARGUMENT;
    }
    return tape_guarded(tape, [&] {
        const std::vector<int64_t>& words = tape->templates[static_cast<size_t>(index)];
        if (tape->is_prologue[static_cast<size_t>(index)]) {
            run_template(tape, words, tape->pro, uploads, n_uploads, downloads, n_downloads, grad_sync_flags);
            tape->prologue_done = true;
            return;
        }
        tape->history.emplace_back();
        run_template(tape, words, tape->history.back(), uploads, n_uploads, downloads, n_downloads,
                     grad_sync_flags);
        // allocations older than any template reaches back are dropped, as the framework's
        // last handle to them is
        while (tape->history.size() > static_cast<size_t>(tape->lookback) + 1) {
            release_list(tape, tape->history.front());
            tape->history.pop_front();
        }
        ++tape->steps_run;
    });
}

void b200_tape_destroy(b200_tape* tape) {
    if (tape == nullptr) return;
    for (auto& list : tape->history) release_list(tape, list);
    release_list(tape, tape->pro);
    delete tape;
}

}  // extern "C"
