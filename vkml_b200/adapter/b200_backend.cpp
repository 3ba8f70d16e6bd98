#include "b200_backend.h"

#include "vkml_b200.h"

#include "vkml/util/env.h"
#include "vkml/util/error.h"
#include "vkml/util/observe.h"

#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace vkml_b200 {
namespace {

// The C ABI numbers ops and dtypes like vkML does; pin that at compile time.
static_assert(static_cast<int>(vkml::OpKind::Input) == B200_OP_INPUT);
static_assert(static_cast<int>(vkml::OpKind::Full) == B200_OP_FULL);
static_assert(static_cast<int>(vkml::OpKind::Unsqueeze) == B200_OP_UNSQUEEZE);
static_assert(static_cast<int>(vkml::OpKind::Contiguous) == B200_OP_CONTIGUOUS);
static_assert(static_cast<int>(vkml::OpKind::ScaledAdd) == B200_OP_SCALED_ADD);
static_assert(static_cast<int>(vkml::OpKind::NotEqual) == B200_OP_NOT_EQUAL);
static_assert(static_cast<int>(vkml::OpKind::Neg) == B200_OP_NEG);
static_assert(static_cast<int>(vkml::OpKind::Clamp) == B200_OP_CLAMP);
static_assert(static_cast<int>(vkml::OpKind::Sum) == B200_OP_SUM);
static_assert(static_cast<int>(vkml::OpKind::ArgMin) == B200_OP_ARGMIN);
static_assert(static_cast<int>(vkml::OpKind::Matmul) == B200_OP_MATMUL);
static_assert(static_cast<int>(vkml::OpKind::LogSoftmax) == B200_OP_LOG_SOFTMAX);
static_assert(static_cast<int>(vkml::OpKind::Im2Col) == B200_OP_IM2COL);
static_assert(static_cast<int>(vkml::OpKind::MaxPool2dBackward) == B200_OP_MAX_POOL2D_BACKWARD);
static_assert(static_cast<int>(vkml::OpKind::SliceBackward) == B200_OP_SLICE_BACKWARD);
static_assert(static_cast<int>(vkml::OpKind::Where) == B200_OP_WHERE);
static_assert(static_cast<int>(vkml::OpKind::Tril) == B200_OP_TRIL);
static_assert(static_cast<int>(vkml::OpKind::Count) == B200_OP_COUNT);
static_assert(static_cast<int>(vkml::DType::F32) == B200_F32);
static_assert(static_cast<int>(vkml::DType::F16) == B200_F16);
static_assert(static_cast<int>(vkml::DType::I32) == B200_I32);
static_assert(static_cast<int>(vkml::DType::I64) == B200_I64);
static_assert(static_cast<int>(vkml::DType::Bool) == B200_BOOL);
static_assert(vkml::kMaxDims == B200_MAX_DIMS);
static_assert(vkml::kMaxSrc == B200_MAX_SRC);
static_assert(vkml::kOpParamBytes == B200_PARAM_BYTES);

// Status code -> vkML exception (include/vkml/util/error.h:7-38).
[[noreturn]] void raise(int status, b200_ctx* ctx, const char* where) {
    std::string msg = std::string("b200 backend: ") + where + ": " + b200_status_name(status);
    if (ctx != nullptr) {
        const char* detail = b200_last_error(ctx);
        if (detail != nullptr && detail[0] != '\0') {
            msg += ": ";
            msg += detail;
        }
    }
    switch (status) {
        case B200_SHAPE_ERROR: throw vkml::ShapeError(msg);
        case B200_DTYPE_ERROR: throw vkml::DTypeError(msg);
        case B200_INDEX_ERROR: throw vkml::IndexError(msg);
        case B200_NOT_IMPLEMENTED: throw vkml::NotImplementedError(msg);
        case B200_OUT_OF_MEMORY: throw vkml::OutOfMemoryError(msg);
        case B200_DEVICE_ERROR:
        case B200_TIMEOUT: throw vkml::DeviceError(msg);
        default: throw vkml::InternalError(msg);
    }
}

void check(int status, b200_ctx* ctx, const char* where) {
    if (status != B200_OK) {
        raise(status, ctx, where);
    }
}

void flatten(const vkml::Node& n, b200_tensor& t) {
    t.data = const_cast<void*>(n.data());
    t.ndim = n.shape.ndim();
    t.dtype = static_cast<int32_t>(n.dtype);
    for (int i = 0; i < B200_MAX_DIMS; ++i) {
        t.dims[i] = i < t.ndim ? n.shape.dim(i) : 1;
        t.strides[i] = i < t.ndim ? n.shape.stride(i) : 0;
    }
}

void flatten(const vkml::Node& n, b200_node& d) {
    d.op = static_cast<uint32_t>(n.op);
    d.n_src = static_cast<uint32_t>(n.n_src);
    flatten(n, d.out);
    for (int i = 0; i < B200_MAX_SRC; ++i) {
        if (i < n.n_src && n.src[static_cast<size_t>(i)] != nullptr) {
            flatten(*n.src[static_cast<size_t>(i)], d.src[i]);
        } else {
            std::memset(&d.src[i], 0, sizeof(b200_tensor));
        }
    }
    std::memcpy(d.params, n.params.raw.data(), B200_PARAM_BYTES);
}

}  // namespace

// Allocator over the library's caching device allocator. The Storage deleter
// returns the block to the cache; the library recycles it in stream order, so a
// handle dropped while kernels are queued is safe (the role retire_later plays
// in src/backend/vulkan/vulkan_backend.cpp:934-984).
class B200Backend::DeviceAllocator final : public vkml::Allocator {
public:
    DeviceAllocator(b200_ctx* ctx, vkml::Device device) : ctx_(ctx), device_(device) {}

    [[nodiscard]] std::shared_ptr<vkml::Storage> allocate(size_t nbytes) override {
        if (nbytes == 0) {
            // a zero-size request yields a Storage with null data (allocator.h:41-43)
            return std::make_shared<vkml::Storage>(nullptr, 0, device_, vkml::Storage::Deleter{});
        }
        void* ptr = nullptr;
        check(b200_alloc(ctx_, nbytes, &ptr), ctx_, "allocate");
        b200_ctx* ctx = ctx_;
        return std::make_shared<vkml::Storage>(ptr, nbytes, device_,
                                               [ctx](void* p, size_t) { b200_free(ctx, p); });
    }
    [[nodiscard]] std::string_view name() const noexcept override { return "b200"; }
    [[nodiscard]] vkml::Device device() const noexcept override { return device_; }
    [[nodiscard]] size_t live_bytes() const noexcept override {
        b200_stats s{};
        b200_get_stats(ctx_, &s);
        return static_cast<size_t>(s.in_use_bytes);
    }

private:
    b200_ctx* ctx_;
    vkml::Device device_;
};

B200Backend::B200Backend(int cuda_ordinal, int device_index)
    : device_(vkml::Device::vulkan(device_index)) {
    const int rc = b200_create(cuda_ordinal, &ctx_);
    if (rc != B200_OK) {
        throw vkml::DeviceError(std::string("b200 backend: cannot open CUDA device ") +
                                std::to_string(cuda_ordinal) + ": " + b200_status_name(rc));
    }
    b200_caps c{};
    check(b200_get_caps(ctx_, &c), ctx_, "capabilities");
    name_ = std::string("b200:") + c.name;
    caps_.fp16_compute = false;  // f16 is a cast endpoint only
    caps_.fp64_compute = true;
    caps_.subgroup_ops = true;
    caps_.subgroup_size = c.warp_size;
    caps_.min_subgroup_size = c.warp_size;
    caps_.max_subgroup_size = c.warp_size;
    caps_.global_float_atomics = true;
    caps_.shared_float_atomics = true;
    caps_.cooperative_matrix = true;
    caps_.buffer_device_address = true;
    caps_.unified_memory = false;
    caps_.host_accessible_buffers = false;
    caps_.min_buffer_alignment = c.min_buffer_alignment;
    caps_.total_memory_bytes = c.total_memory_bytes;
    caps_.max_allocation_bytes = c.total_memory_bytes;
    caps_.max_workgroup_invocations = c.max_threads_per_block;
    caps_.shader_core_count = c.sm_count;
    caps_.max_shared_memory_bytes = c.max_shared_memory_bytes;
    caps_.asynchronous = true;
    allocator_ = std::make_unique<DeviceAllocator>(ctx_, device_);
    // The library reads its switches itself when the context is created; consulting them here
    // through vkML's one env reader (src/util/env.cpp:43-79) puts them into `configuration()`
    // beside vkML's own, with the values this process saw.
    for (const char* name : {"VKML_B200_GEMM_PRECISION", "VKML_B200_GEMM_OPERANDS", "VKML_B200_GEMM_STREAM",
                             "VKML_B200_GEMM_SCHEDULE", "VKML_B200_SHARE_PLANES", "VKML_B200_PDL",
                             "VKML_B200_LAZY_JOIN", "VKML_B200_HOIST_GRADIENTS", "VKML_B200_COMM_SMS",
                             "VKML_B200_FUSE", "VKML_B200_BUCKET", "VKML_B200_BUCKET_FLUSH_BYTES", "VKML_B200_COMM_TIMEOUT_MS", "VKML_B200_DIST_INIT_TIMEOUT_MS",
                             "VKML_B200_UPLOAD_THREADS", "VKML_B200_SPAN_GRAPHS"}) {
        (void)vkml::env_value(name);
    }
}

B200Backend::~B200Backend() {
    allocator_.reset();
    b200_destroy(ctx_);
}

vkml::Allocator& B200Backend::allocator() { return *allocator_; }

bool B200Backend::supports(const vkml::Node& node) const {
    if (vkml::is_view_op(node.op) || node.is_leaf()) {
        return true;
    }
    for (int i = 0; i < node.n_src; ++i) {
        if (node.src[static_cast<size_t>(i)] == nullptr) {
            return false;
        }
    }
    b200_node d{};
    flatten(node, d);
    return b200_supports(&d) != 0;
}

void B200Backend::compute(std::span<vkml::Node* const> nodes) {
    std::vector<b200_node> flat;
    flat.reserve(nodes.size());
    for (vkml::Node* n : nodes) {
        if (n == nullptr) {
            throw vkml::InternalError("b200 backend: null node in compute list");
        }
        if (vkml::is_view_op(n->op) || n->is_leaf()) {
            continue;  // resolved by the executor through aliasing (backend.h:34-45)
        }
        flat.emplace_back();
        flatten(*n, flat.back());
        if (n->op == vkml::OpKind::Matmul && vkml::observe::enabled()) {
            // a Decision, as the Vulkan backend publishes one per matmul (vulkan_backend.cpp:2363-2375):
            // which kernel runs decides the arithmetic, and is not derivable from the inputs alone
            char kernel[48] = "", why[128] = "";
            if (b200_matmul_kernel(ctx_, &flat.back(), kernel, sizeof(kernel), why, sizeof(why)) == B200_OK) {
                vkml::observe::publish({.site = "matmul.kernel",
                                        .op = "matmul",
                                        .chose = kernel,
                                        .instead_of = std::string_view(kernel) == "fp32_simt" ? "tcgen05_3xtf32" : "fp32_simt",
                                        .because = why,
                                        .required = n->shape.dim(n->shape.ndim() - 2),
                                        .available = 0});
            }
        }
    }
    uint32_t flags = B200_COMPUTE_DEFAULT;
    if (grad_sync_armed_) {
        flags |= B200_COMPUTE_GRAD_SYNC;
        grad_sync_armed_ = false;
    }
    check(b200_compute(ctx_, flat.data(), flat.size(), flags), ctx_, "compute");
}

void B200Backend::copy_from_host(vkml::Storage& dst, int64_t dst_offset, const void* src, size_t nbytes) {
    if (nbytes == 0) {
        return;
    }
    if (dst_offset < 0 || static_cast<size_t>(dst_offset) + nbytes > dst.nbytes()) {
        throw vkml::IndexError("b200 backend: copy_from_host range exceeds the storage");
    }
    check(b200_copy_from_host(ctx_, static_cast<std::byte*>(dst.data()) + dst_offset, src, nbytes), ctx_,
          "copy_from_host");
}

void B200Backend::copy_to_host(void* dst, const vkml::Storage& src, int64_t src_offset, size_t nbytes) {
    if (nbytes == 0) {
        return;
    }
    if (src_offset < 0 || static_cast<size_t>(src_offset) + nbytes > src.nbytes()) {
        throw vkml::IndexError("b200 backend: copy_to_host range exceeds the storage");
    }
    check(b200_copy_to_host(ctx_, dst, static_cast<const std::byte*>(src.data()) + src_offset, nbytes), ctx_,
          "copy_to_host");
}

void B200Backend::copy_device_to_device(std::span<const vkml::BufferCopy> copies) {
    std::vector<b200_copy> flat;
    flat.reserve(copies.size());
    for (const vkml::BufferCopy& c : copies) {
        if (c.nbytes == 0) {
            continue;
        }
        if (c.dst == nullptr || c.src == nullptr) {
            throw vkml::InternalError("b200 backend: null storage in copy_device_to_device");
        }
        if (c.dst_offset < 0 || static_cast<size_t>(c.dst_offset) + c.nbytes > c.dst->nbytes() ||
            c.src_offset < 0 || static_cast<size_t>(c.src_offset) + c.nbytes > c.src->nbytes()) {
            throw vkml::IndexError("b200 backend: copy_device_to_device range exceeds a storage");
        }
        flat.push_back(b200_copy{static_cast<std::byte*>(c.dst->data()) + c.dst_offset,
                                 static_cast<const std::byte*>(c.src->data()) + c.src_offset, c.nbytes});
    }
    check(b200_copy_device_to_device(ctx_, flat.data(), flat.size()), ctx_, "copy_device_to_device");
}

void B200Backend::synchronize() { check(b200_synchronize(ctx_), ctx_, "synchronize"); }

B200Backend& b200_backend(int index) {
    static std::mutex mu;
    // leaked on purpose: backends are process-lifetime objects (backend.h:132-137)
    static auto* registry = new std::unordered_map<int, B200Backend*>();
    const std::lock_guard<std::mutex> lock(mu);
    if (const auto it = registry->find(index); it != registry->end()) {
        return *it->second;
    }
    auto* backend = new B200Backend(index, index);
    registry->emplace(index, backend);
    vkml::register_backend(*backend);
    return *backend;
}

}  // namespace vkml_b200
