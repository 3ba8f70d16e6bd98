// ref_harness.cpp -- drives the UNMODIFIED vkML reference (compiled from its own
// sources by oracle/Makefile into oracle/_ref/) for the tests and for the timed
// CPU baseline.  TEST INFRASTRUCTURE ONLY: nothing in the product path links,
// loads or calls it.
//
// Three services, all `extern "C"`:
//   vkml_ref_compute      evaluate b200_node descriptors (host pointers) with the
//                         reference's own CPU backend kernels
//                         (src/backend/cpu/cpu_backend.cpp:60-91) -- used to pin
//                         the C restatement in vkml_oracle.c bit for bit;
//   vkml_ref_matmul_mt    the same matmul kernel over row slabs of A on several
//                         host threads (each output element's dot product is
//                         independent, so per-element arithmetic is unchanged) --
//                         the timed multi-core CPU baseline;
//   vkml_ref_train_*      whole training runs (forward, backward(), SGD with
//                         momentum, assign) through the reference's public C++
//                         API on a chosen device: the CPU backend, or -- when
//                         built with WITH_B200 -- the B200 adapter registered as
//                         Device::vulkan(0).  Same graphs, same bytes, two
//                         devices: the loss curves are the training parity test.
//                         With device 2 nothing is computed: a recording backend
//                         writes every call the framework makes on its device
//                         (allocations, uploads, compute spans with their node
//                         descriptors, device copies, downloads) to a JSON-lines
//                         file, which vkml_b200/replay.py plays back through the C
//                         ABI -- the exact submissions of the real framework, at
//                         any size, without the CPU having to execute them.
#include "vkml_b200.h"

#include "vkml/api/ops.h"
#include "vkml/api/tensor.h"
#include "vkml/autograd/autograd.h"
#include "vkml/backend/api/backend.h"
#include "vkml/dispatch/executor.h"
#include "vkml/graph/node.h"
#include "vkml/util/error.h"

#ifdef WITH_B200
#include "b200_backend.h"
#endif

#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;

int status_of(const std::exception& e) {
    g_error = e.what();
    if (dynamic_cast<const vkml::ShapeError*>(&e)) return B200_SHAPE_ERROR;
    if (dynamic_cast<const vkml::DTypeError*>(&e)) return B200_DTYPE_ERROR;
    if (dynamic_cast<const vkml::DeviceError*>(&e)) return B200_DEVICE_ERROR;
    if (dynamic_cast<const vkml::IndexError*>(&e)) return B200_INDEX_ERROR;
    if (dynamic_cast<const vkml::NotImplementedError*>(&e)) return B200_NOT_IMPLEMENTED;
    if (dynamic_cast<const vkml::OutOfMemoryError*>(&e)) return B200_OUT_OF_MEMORY;
    return B200_INTERNAL_ERROR;
}

// Bytes spanned by a strided view, so the borrowed Storage can state a size.
size_t span_bytes(const b200_tensor& t) {
    const size_t esz = vkml::dtype_size(static_cast<vkml::DType>(t.dtype));
    size_t last = 0;
    for (int i = 0; i < t.ndim; ++i) {
        if (t.dims[i] == 0) return 0;
        last += static_cast<size_t>(t.dims[i] - 1) * static_cast<size_t>(t.strides[i] < 0 ? 0 : t.strides[i]);
    }
    return last + esz;
}

vkml::NodePtr borrow(const b200_tensor& t, vkml::OpKind op) {
    const auto dt = static_cast<vkml::DType>(t.dtype);
    const std::span<const int64_t> dims{t.dims, static_cast<size_t>(t.ndim)};
    const std::span<const int64_t> strides{t.strides, static_cast<size_t>(t.ndim)};
    auto n = vkml::make_node(op, vkml::Shape::strided(dims, strides, vkml::dtype_size(dt)), dt,
                             vkml::Device::cpu());
    const size_t nbytes = t.data == nullptr ? 0 : span_bytes(t);
    n->storage = std::make_shared<vkml::Storage>(t.data, nbytes, vkml::Device::cpu(), vkml::Storage::Deleter{});
    n->storage_offset = 0;
    return n;
}

vkml::NodePtr rebuild(const b200_node& d) {
    auto out = borrow(d.out, static_cast<vkml::OpKind>(d.op));
    std::memcpy(out->params.raw.data(), d.params, B200_PARAM_BYTES);
    out->n_src = static_cast<int>(d.n_src);
    for (uint32_t i = 0; i < d.n_src && i < B200_MAX_SRC; ++i) {
        out->src[i] = borrow(d.src[i], vkml::OpKind::Input);
        out->src[i]->flags |= vkml::kFlagComputed;
    }
    return out;
}

// ---------------------------------------------------------------------------
// Recording backend: vkml::Backend registered as Device::vulkan(9).  Memory is
// virtual (addresses are never dereferenced), compute() only logs.
// ---------------------------------------------------------------------------
constexpr uint64_t kArenaBase = uint64_t(1) << 44;
constexpr int kArenaShift = 38;  // 256 GiB of address space per allocation

class RecordingBackend final : public vkml::Backend {
public:
    RecordingBackend() : alloc_(this) {
        caps_.asynchronous = true;
        caps_.host_accessible_buffers = false;
        caps_.total_memory_bytes = size_t(180) << 30;
    }
    void open(const char* path) {
        if (file_ != nullptr) std::fclose(file_);
        file_ = std::fopen(path, "w");
        if (file_ == nullptr) throw vkml::DeviceError(std::string("cannot open ") + path);
    }
    void close() {
        if (file_ != nullptr) std::fclose(file_);
        file_ = nullptr;
    }
    void mark(const char* what, int index) {
        if (file_ != nullptr) std::fprintf(file_, "{\"ev\":\"%s\",\"index\":%d}\n", what, index);
    }
    void arm_grad_sync() { grad_sync_ = true; }

    std::string_view name() const noexcept override { return "recorder"; }
    vkml::Device device() const noexcept override { return vkml::Device::vulkan(9); }
    const vkml::DeviceCapabilities& capabilities() const noexcept override { return caps_; }
    vkml::Allocator& allocator() override { return alloc_; }
    bool supports(const vkml::Node&) const override { return true; }

    void compute(std::span<vkml::Node* const> nodes) override {
        if (file_ == nullptr) return;
        std::fprintf(file_, "{\"ev\":\"compute\",\"grad_sync\":%s,\"nodes\":[", grad_sync_ ? "true" : "false");
        grad_sync_ = false;
        bool first = true;
        for (vkml::Node* n : nodes) {
            if (vkml::is_view_op(n->op) || n->is_leaf()) continue;
            std::fprintf(file_, "%s{\"op\":%d,\"params\":\"", first ? "" : ",", static_cast<int>(n->op));
            first = false;
            for (std::byte b : n->params.raw) std::fprintf(file_, "%02x", static_cast<unsigned>(b));
            std::fprintf(file_, "\",\"out\":");
            tensor(*n);
            std::fprintf(file_, ",\"src\":[");
            for (int i = 0; i < n->n_src; ++i) {
                if (i) std::fputc(',', file_);
                tensor(*n->src[static_cast<size_t>(i)]);
            }
            std::fprintf(file_, "]}");
        }
        std::fprintf(file_, "]}\n");
    }
    void copy_from_host(vkml::Storage& dst, int64_t off, const void*, size_t nbytes) override {
        if (file_ != nullptr && nbytes != 0)
            std::fprintf(file_, "{\"ev\":\"h2d\",\"id\":%llu,\"off\":%lld,\"bytes\":%zu}\n", id_of(dst.data()),
                         static_cast<long long>(off), nbytes);
    }
    void copy_to_host(void* dst, const vkml::Storage& src, int64_t off, size_t nbytes) override {
        std::memset(dst, 0, nbytes);
        if (file_ != nullptr && nbytes != 0)
            std::fprintf(file_, "{\"ev\":\"d2h\",\"id\":%llu,\"off\":%lld,\"bytes\":%zu}\n", id_of(src.data()),
                         static_cast<long long>(off), nbytes);
    }
    void copy_device_to_device(std::span<const vkml::BufferCopy> copies) override {
        if (file_ == nullptr) return;
        std::fprintf(file_, "{\"ev\":\"d2d\",\"copies\":[");
        bool first = true;
        for (const vkml::BufferCopy& c : copies) {
            if (c.nbytes == 0) continue;
            std::fprintf(file_, "%s[%llu,%lld,%llu,%lld,%zu]", first ? "" : ",", id_of(c.dst->data()),
                         static_cast<long long>(c.dst_offset), id_of(c.src->data()),
                         static_cast<long long>(c.src_offset), c.nbytes);
            first = false;
        }
        std::fprintf(file_, "]}\n");
    }
    using vkml::Backend::copy_device_to_device;
    void synchronize() override {
        if (file_ != nullptr) std::fprintf(file_, "{\"ev\":\"sync\"}\n");
    }

private:
    class FakeAllocator final : public vkml::Allocator {
    public:
        explicit FakeAllocator(RecordingBackend* owner) : owner_(owner) {}
        std::shared_ptr<vkml::Storage> allocate(size_t nbytes) override {
            RecordingBackend* o = owner_;
            if (nbytes == 0) {
                return std::make_shared<vkml::Storage>(nullptr, 0, o->device(), vkml::Storage::Deleter{});
            }
            const uint64_t id = o->next_id_++;
            void* fake = reinterpret_cast<void*>(kArenaBase + (id << kArenaShift));
            if (o->file_ != nullptr)
                std::fprintf(o->file_, "{\"ev\":\"alloc\",\"id\":%llu,\"bytes\":%zu}\n",
                             static_cast<unsigned long long>(id), nbytes);
            live_ += nbytes;
            return std::make_shared<vkml::Storage>(fake, nbytes, o->device(), [o, id, this](void*, size_t n) {
                live_ -= n;
                if (o->file_ != nullptr)
                    std::fprintf(o->file_, "{\"ev\":\"free\",\"id\":%llu}\n", static_cast<unsigned long long>(id));
            });
        }
        std::string_view name() const noexcept override { return "recorder"; }
        vkml::Device device() const noexcept override { return vkml::Device::vulkan(9); }
        size_t live_bytes() const noexcept override { return live_; }

    private:
        RecordingBackend* owner_;
        size_t live_ = 0;
    };

    static unsigned long long id_of(const void* p) {
        return (reinterpret_cast<uint64_t>(p) - kArenaBase) >> kArenaShift;
    }
    void tensor(const vkml::Node& n) {
        const uint64_t addr = reinterpret_cast<uint64_t>(n.data());
        if (n.data() == nullptr) {
            std::fprintf(file_, "{\"id\":-1,\"off\":0");
        } else {
            std::fprintf(file_, "{\"id\":%llu,\"off\":%llu", static_cast<unsigned long long>((addr - kArenaBase) >> kArenaShift),
                         static_cast<unsigned long long>((addr - kArenaBase) & ((uint64_t(1) << kArenaShift) - 1)));
        }
        std::fprintf(file_, ",\"dtype\":%d,\"dims\":[", static_cast<int>(n.dtype));
        for (int i = 0; i < n.shape.ndim(); ++i) std::fprintf(file_, "%s%lld", i ? "," : "", static_cast<long long>(n.shape.dim(i)));
        std::fprintf(file_, "],\"strides\":[");
        for (int i = 0; i < n.shape.ndim(); ++i) std::fprintf(file_, "%s%lld", i ? "," : "", static_cast<long long>(n.shape.stride(i)));
        std::fprintf(file_, "]}");
    }

    vkml::DeviceCapabilities caps_;
    FakeAllocator alloc_;
    std::FILE* file_ = nullptr;
    uint64_t next_id_ = 0;
    bool grad_sync_ = false;
};

RecordingBackend& recorder() {
    static RecordingBackend* r = [] {
        auto* b = new RecordingBackend();  // process lifetime, like every backend
        vkml::register_backend(*b);
        return b;
    }();
    return *r;
}

// Tells the device that the next compute span is backward()'s: its sinks are the
// parameter gradients a data-parallel run all-reduces.
void before_backward(int device) {
    if (device == 2) recorder().arm_grad_sync();
#ifdef WITH_B200
    if (device == 1) vkml_b200::b200_backend(0).arm_grad_sync();
#endif
}

// Wall-clock time of every step of the last training run (forward, backward(), optimiser,
// loss.item()): how long the framework's own executor takes per step on the chosen device.
thread_local std::vector<double> g_step_seconds;
thread_local std::chrono::steady_clock::time_point g_step_begin;

void mark_step(int device, int index) {
    if (device == 2) recorder().mark("step", index);
    if (index == 0) g_step_seconds.clear();
    g_step_begin = std::chrono::steady_clock::now();
}

void end_step() {
    g_step_seconds.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - g_step_begin).count());
}

vkml::Device pick_device(int which) {
#ifdef WITH_B200
    if (which == 1) {
        return vkml_b200::b200_backend(0).device();
    }
#endif
    if (which == 2) {
        return recorder().device();
    }
    if (which != 0) {
        throw vkml::DeviceError("this build of the harness has no B200 adapter");
    }
    return vkml::Device::cpu();
}

struct Sgd {
    double lr, momentum;
    std::vector<vkml::Tensor> velocity;  // undefined until the first step

    // python/vkml/optim.py:97-128 (three batched passes) + :170-199 (SGD plan)
    void step(std::vector<vkml::Tensor>& params) {
        vkml::NoGradGuard no_grad;
        if (velocity.size() != params.size()) velocity.assign(params.size(), vkml::Tensor{});
        std::vector<vkml::Tensor> vel(params.size());
        std::vector<vkml::NodePtr> state;
        for (size_t i = 0; i < params.size(); ++i) {
            const vkml::Tensor g = params[i].grad();
            if (momentum == 0.0) continue;
            vel[i] = velocity[i].defined() ? vkml::scaled_add(velocity[i], g, momentum, 1.0) : g;
            state.push_back(vel[i].node());
        }
        if (!state.empty()) vkml::realize(state);
        std::vector<vkml::Tensor> values(params.size());
        std::vector<vkml::NodePtr> roots;
        for (size_t i = 0; i < params.size(); ++i) {
            vkml::Tensor direction = params[i].grad();
            if (momentum != 0.0) {
                velocity[i] = vkml::detach(vel[i]);
                direction = velocity[i];
            }
            values[i] = vkml::scaled_add(vkml::detach(params[i]), direction, 1.0, -lr);
            roots.push_back(values[i].node());
        }
        vkml::realize(roots);
        vkml::assign(params, values);
    }
};

// Host-side gradient exchange for the N-rank CPU oracle of data-parallel training: after
// backward(), every parameter gradient is brought to the host, handed to `hook` (which
// averages it across ranks, e.g. with a gloo all-reduce) and put back.
using GradHook = void (*)(float* data, int64_t count, void* user);
thread_local GradHook g_hook = nullptr;
thread_local void* g_hook_user = nullptr;

void exchange_grads(std::vector<vkml::Tensor>& params) {
    if (g_hook == nullptr) return;
    for (auto& p : params) {
        vkml::Tensor g = p.grad().contiguous();
        std::vector<float> host(static_cast<size_t>(g.numel()));
        g.to_host(host.data());
        g_hook(host.data(), g.numel(), g_hook_user);
        const std::vector<int64_t> dims = g.shape();
        p.set_grad(vkml::Tensor::from_host(host.data(), std::span<const int64_t>{dims}, vkml::DType::F32, g.device()));
    }
}

void zero_grad(std::vector<vkml::Tensor>& params) {
    for (auto& p : params) p.set_grad(vkml::Tensor{});
}

}  // namespace

extern "C" {

const char* vkml_ref_last_error(void) { return g_error.c_str(); }

int vkml_ref_has_b200(void) {
#ifdef WITH_B200
    return 1;
#else
    return 0;
#endif
}

// Per-step wall-clock seconds of the last vkml_ref_train_* call on this thread; returns how many
// steps were timed (at most `capacity` are copied).
int vkml_ref_step_seconds(double* out, int capacity) {
    const int n = static_cast<int>(g_step_seconds.size());
    for (int i = 0; i < n && i < capacity; ++i) out[i] = g_step_seconds[static_cast<size_t>(i)];
    return n;
}

// Install (or clear, with NULL) the host-side gradient exchange used by the trainers below.
void vkml_ref_set_grad_hook(void (*hook)(float*, int64_t, void*), void* user) {
    g_hook = hook;
    g_hook_user = user;
}

// Join a data-parallel job on the B200 adapter's context (NCCL communicator).
int vkml_ref_b200_dist_init(int rank, int world, const void* unique_id) {
#ifdef WITH_B200
    try {
        return b200_dist_init(vkml_b200::b200_backend(0).context(), rank, world, unique_id);
    } catch (const std::exception& e) {
        return status_of(e);
    }
#else
    (void)rank; (void)world; (void)unique_id;
    return B200_NOT_IMPLEMENTED;
#endif
}

// Start / stop writing the recording backend's log (device 2 of the trainers).
int vkml_ref_record_begin(const char* path) {
    try {
        recorder().open(path);
        return B200_OK;
    } catch (const std::exception& e) {
        return status_of(e);
    }
}

int vkml_ref_record_end(void) {
    recorder().close();
    return B200_OK;
}

int vkml_ref_compute(const b200_node* nodes, size_t n_nodes) {
    try {
        for (size_t i = 0; i < n_nodes; ++i) {
            const auto op = static_cast<vkml::OpKind>(nodes[i].op);
            if (vkml::is_view_op(op) || vkml::is_leaf_op(op)) continue;
            vkml::NodePtr node = rebuild(nodes[i]);
            vkml::Node* raw = node.get();
            vkml::cpu_backend().compute(std::span<vkml::Node* const>{&raw, 1});
        }
        return B200_OK;
    } catch (const std::exception& e) {
        return status_of(e);
    }
}

// Row slabs of A (axis 2) across `threads` host threads, each through the
// reference matmul kernel. node must be a rank-4 f32 matmul.
int vkml_ref_matmul_mt(const b200_node* node, int threads) {
    if (node == nullptr || node->op != B200_OP_MATMUL || threads < 1) return B200_INVALID_ARGUMENT;
    const int64_t m = node->out.dims[2];
    if (threads > m) threads = static_cast<int>(m > 0 ? m : 1);
    std::vector<int> rc(static_cast<size_t>(threads), B200_OK);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        pool.emplace_back([&, t] {
            const int64_t r0 = m * t / threads, r1 = m * (t + 1) / threads;
            if (r1 <= r0) return;
            b200_node slab = *node;
            slab.out.dims[2] = r1 - r0;
            slab.out.data = static_cast<char*>(node->out.data) + r0 * node->out.strides[2];
            slab.src[0].dims[2] = r1 - r0;
            slab.src[0].data = static_cast<char*>(node->src[0].data) + r0 * node->src[0].strides[2];
            rc[static_cast<size_t>(t)] = vkml_ref_compute(&slab, 1);
        });
    }
    for (auto& th : pool) th.join();
    for (int r : rc) if (r != B200_OK) return r;
    return B200_OK;
}

// MLP training run through the reference API (python/vkml/nn.py:253-295 Linear,
// ReLU between layers, cross_entropy, SGD).  `widths` = [in, h1, ..., out];
// `weights`/`biases` are concatenated per layer, weight l is [widths[l+1], widths[l]]
// row-major as nn.Linear stores it.  Every step consumes `batch` rows of `x`
// ([steps*batch, in]) and `y` (int64).  Writes the per-step loss and, at the end,
// the parameters back into `weights`/`biases`.
int vkml_ref_train_mlp(int device, const int64_t* widths, int n_layers, float* weights, float* biases,
                       const float* x, const int64_t* y, int64_t batch, int steps, double lr,
                       double momentum, float* losses) {
    try {
        const vkml::Device dev = pick_device(device);
        std::vector<vkml::Tensor> params;
        size_t wo = 0, bo = 0;
        for (int l = 0; l < n_layers; ++l) {
            const int64_t in = widths[l], out = widths[l + 1];
            params.push_back(vkml::Tensor::from_host(weights + wo, {out, in}, vkml::DType::F32, dev));
            params.push_back(vkml::Tensor::from_host(biases + bo, {out}, vkml::DType::F32, dev));
            wo += static_cast<size_t>(in * out);
            bo += static_cast<size_t>(out);
        }
        for (auto& p : params) p.set_requires_grad(true);
        Sgd opt{lr, momentum, {}};
        for (int s = 0; s < steps; ++s) {
            mark_step(device, s);
            const size_t at = device == 2 ? 0 : static_cast<size_t>(s);  // the recorder never reads the data
            vkml::Tensor h = vkml::Tensor::from_host(x + at * batch * widths[0], {batch, widths[0]},
                                                     vkml::DType::F32, dev);
            const vkml::Tensor labels = vkml::Tensor::from_host(y + at * batch, {batch}, vkml::DType::I64, dev);
            for (int l = 0; l < n_layers; ++l) {
                h = vkml::matmul(h, params[2 * l].transpose(-2, -1)) + params[2 * l + 1];
                if (l + 1 < n_layers) h = vkml::relu(h);
            }
            const vkml::Tensor loss = vkml::cross_entropy(h, labels);
            zero_grad(params);
            before_backward(device);
            vkml::backward(loss);
            exchange_grads(params);
            opt.step(params);
            losses[s] = loss.item();
            end_step();
        }
        wo = bo = 0;
        for (int l = 0; l < n_layers; ++l) {
            params[2 * l].to_host(weights + wo);
            params[2 * l + 1].to_host(biases + bo);
            wo += static_cast<size_t>(widths[l] * widths[l + 1]);
            bo += static_cast<size_t>(widths[l + 1]);
        }
        return B200_OK;
    } catch (const std::exception& e) {
        return status_of(e);
    }
}

// The CIFAR-style CNN: conv3x3(c1) ReLU pool2, conv3x3(c2) ReLU pool2,
// conv3x3(c3) ReLU pool2, Linear(c3*(hw/8)^2 -> classes); conv2d is the
// reference's im2col + matmul composition (src/api/ops.cpp:662-705).
// `params` holds, concatenated: w1[c1,cin,3,3] b1[c1] w2[c2,c1,3,3] b2 w3 b3 wf[classes,feat] bf.
int vkml_ref_train_cnn(int device, int64_t cin, int64_t hw, int64_t c1, int64_t c2, int64_t c3,
                       int64_t classes, float* params_flat, const float* x, const int64_t* y,
                       int64_t batch, int steps, double lr, double momentum, float* losses) {
    try {
        const vkml::Device dev = pick_device(device);
        const int64_t feat = c3 * (hw / 8) * (hw / 8);
        const std::vector<std::vector<int64_t>> shapes = {
            {c1, cin, 3, 3}, {c1}, {c2, c1, 3, 3}, {c2}, {c3, c2, 3, 3}, {c3}, {classes, feat}, {classes}};
        std::vector<vkml::Tensor> params;
        size_t off = 0;
        for (const auto& s : shapes) {
            int64_t n = 1;
            for (int64_t d : s) n *= d;
            params.push_back(vkml::Tensor::from_host(params_flat + off, std::span<const int64_t>{s}, vkml::DType::F32, dev));
            off += static_cast<size_t>(n);
        }
        for (auto& p : params) p.set_requires_grad(true);
        Sgd opt{lr, momentum, {}};
        for (int s = 0; s < steps; ++s) {
            mark_step(device, s);
            const size_t at = device == 2 ? 0 : static_cast<size_t>(s);
            vkml::Tensor h = vkml::Tensor::from_host(x + at * batch * cin * hw * hw, {batch, cin, hw, hw},
                                                     vkml::DType::F32, dev);
            const vkml::Tensor labels = vkml::Tensor::from_host(y + at * batch, {batch}, vkml::DType::I64, dev);
            for (int l = 0; l < 3; ++l) {
                h = vkml::conv2d(h, params[2 * l], params[2 * l + 1], {1, 1}, {1, 1});
                h = vkml::relu(h);
                h = vkml::max_pool2d(h, {2, 2});
            }
            h = h.reshape({batch, feat});
            h = vkml::matmul(h, params[6].transpose(-2, -1)) + params[7];
            const vkml::Tensor loss = vkml::cross_entropy(h, labels);
            zero_grad(params);
            before_backward(device);
            vkml::backward(loss);
            exchange_grads(params);
            opt.step(params);
            losses[s] = loss.item();
            end_step();
        }
        off = 0;
        for (size_t i = 0; i < params.size(); ++i) {
            params[i].to_host(params_flat + off);
            off += static_cast<size_t>(params[i].numel());
        }
        return B200_OK;
    } catch (const std::exception& e) {
        return status_of(e);
    }
}

// Cross-entropy forward and backward through the reference API (src/api/ops.cpp:417-441 and the
// autograd rules of src/autograd/autograd.cpp:528-546): loss = cross_entropy(logits, labels),
// backward(loss).  Returns the scalar loss and d loss / d logits ([b, c]).  The device sees
// exactly the node sequence the framework emits for this composite.
int vkml_ref_cross_entropy(int device, const float* logits, const int64_t* labels, int64_t b, int64_t c,
                           float* loss_out, float* grad_out) {
    try {
        const vkml::Device dev = pick_device(device);
        vkml::Tensor x = vkml::Tensor::from_host(logits, {b, c}, vkml::DType::F32, dev);
        const vkml::Tensor y = vkml::Tensor::from_host(labels, {b}, vkml::DType::I64, dev);
        x.set_requires_grad(true);
        const vkml::Tensor loss = vkml::cross_entropy(x, y);
        vkml::backward(loss);
        *loss_out = loss.item();
        x.grad().contiguous().to_host(grad_out);
        return B200_OK;
    } catch (const std::exception& e) {
        return status_of(e);
    }
}

}  // extern "C"
