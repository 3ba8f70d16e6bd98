// vkML backend adapter for the B200 CUDA library.
//
// `B200Backend` derives from `vkml::Backend`
// (include/vkml/backend/api/backend.h:49-125) and forwards each virtual to the
// C ABI in vkml_b200.h; it is the only code that sees both vkML's C++ types
// and the C ABI.  It is compiled inside (or against) a vkML source tree: it
// includes vkML's public headers and nothing else of vkML.
//
// The backend registers under `Device::vulkan(index)` because vkML's
// `DeviceKind` has exactly two members, CPU and Vulkan
// (include/vkml/core/device.h:9-12), and every call site resolves a device
// through `backend_for(node.device)` (src/backend/api/backend.cpp:52-76): with
// this registration `V.device("vulkan:0")`, `module.to(device)`, `realize()`,
// `backward()` and the optimisers run on the B200 with no change to vkML.
#pragma once

#include "vkml/backend/api/backend.h"

#include <memory>
#include <string>

struct b200_ctx;

namespace vkml_b200 {

class B200Backend final : public vkml::Backend {
public:
    // Opens CUDA device `cuda_ordinal` and presents it as Device::vulkan(device_index).
    // Throws vkml::DeviceError if the device cannot be opened.
    B200Backend(int cuda_ordinal, int device_index);
    ~B200Backend() override;

    [[nodiscard]] std::string_view name() const noexcept override { return name_; }
    [[nodiscard]] vkml::Device device() const noexcept override { return device_; }
    [[nodiscard]] const vkml::DeviceCapabilities& capabilities() const noexcept override { return caps_; }
    [[nodiscard]] vkml::Allocator& allocator() override;
    [[nodiscard]] bool supports(const vkml::Node& node) const override;

    void compute(std::span<vkml::Node* const> nodes) override;
    void copy_from_host(vkml::Storage& dst, int64_t dst_offset, const void* src, size_t nbytes) override;
    void copy_to_host(void* dst, const vkml::Storage& src, int64_t src_offset, size_t nbytes) override;
    void copy_device_to_device(std::span<const vkml::BufferCopy> copies) override;
    using vkml::Backend::copy_device_to_device;
    void synchronize() override;

    // Data-parallel hook: when armed, the next compute() span all-reduces the
    // gradient buffers registered through the C ABI (b200_dist_mark_grad).
    void arm_grad_sync() noexcept { grad_sync_armed_ = true; }

    [[nodiscard]] b200_ctx* context() const noexcept { return ctx_; }

private:
    class DeviceAllocator;
    b200_ctx* ctx_ = nullptr;
    vkml::Device device_;
    std::string name_;
    vkml::DeviceCapabilities caps_;
    std::unique_ptr<DeviceAllocator> allocator_;
    bool grad_sync_armed_ = false;
};

// Process-lifetime backend for CUDA device `index`, created and registered with
// vkml::register_backend on first use: the counterpart of vkml::vulkan_backend(index)
// (src/backend/vulkan/vulkan_backend.cpp:2991).
B200Backend& b200_backend(int index = 0);

}  // namespace vkml_b200
