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

#include <cstdio>
#include <cstring>
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

vkml::Device pick_device(int which) {
#ifdef WITH_B200
    if (which == 1) {
        return vkml_b200::b200_backend(0).device();
    }
#endif
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
            vkml::Tensor h = vkml::Tensor::from_host(x + static_cast<size_t>(s) * batch * widths[0],
                                                     {batch, widths[0]}, vkml::DType::F32, dev);
            const vkml::Tensor labels = vkml::Tensor::from_host(y + static_cast<size_t>(s) * batch, {batch},
                                                                vkml::DType::I64, dev);
            for (int l = 0; l < n_layers; ++l) {
                h = vkml::matmul(h, params[2 * l].transpose(-2, -1)) + params[2 * l + 1];
                if (l + 1 < n_layers) h = vkml::relu(h);
            }
            const vkml::Tensor loss = vkml::cross_entropy(h, labels);
            zero_grad(params);
            vkml::backward(loss);
            opt.step(params);
            losses[s] = loss.item();
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
            vkml::Tensor h = vkml::Tensor::from_host(x + static_cast<size_t>(s) * batch * cin * hw * hw,
                                                     {batch, cin, hw, hw}, vkml::DType::F32, dev);
            const vkml::Tensor labels = vkml::Tensor::from_host(y + static_cast<size_t>(s) * batch, {batch},
                                                                vkml::DType::I64, dev);
            for (int l = 0; l < 3; ++l) {
                h = vkml::conv2d(h, params[2 * l], params[2 * l + 1], {1, 1}, {1, 1});
                h = vkml::relu(h);
                h = vkml::max_pool2d(h, {2, 2});
            }
            h = h.reshape({batch, feat});
            h = vkml::matmul(h, params[6].transpose(-2, -1)) + params[7];
            const vkml::Tensor loss = vkml::cross_entropy(h, labels);
            zero_grad(params);
            vkml::backward(loss);
            opt.step(params);
            losses[s] = loss.item();
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

}  // extern "C"
