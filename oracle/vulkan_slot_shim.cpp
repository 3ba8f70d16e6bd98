// Lets vkML's own C++ tests reach the B200 through the two functions they call to obtain "the GPU
// device" (include/vkml/backend/vulkan/vulkan_backend.h:224,251): with this file linked in place
// of the Vulkan backend, `vkml::vulkan_available()` reports whether a CUDA device is visible and
// `vkml::vulkan_backend(i)` registers and returns the B200 adapter for device i.
// Test infrastructure (built by oracle/Makefile into oracle/_ref/).
#include "vkml/backend/vulkan/vulkan_backend.h"

#include "b200_backend.h"
#include "vkml_b200.h"

namespace vkml {

bool vulkan_available() {
    int n = 0;
    return b200_device_count(&n) == B200_OK && n > 0;
}

Backend& vulkan_backend(int index) { return vkml_b200::b200_backend(index); }

}  // namespace vkml
