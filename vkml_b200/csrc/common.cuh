// Shared device/host helpers for the B200 backend kernels.
#pragma once

#include "vkml_b200.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

namespace b200 {

constexpr int kMaxDims = B200_MAX_DIMS;

// SMs of the CURRENT device (a B200 has 148: 2 dies x 74); grids, wave counts and split
// decisions are sized in multiples of this.  Every entry point makes its context's device
// current before it launches, so the current device is the one the launch goes to.
inline int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Bits of the device status word (b200_ctx::d_status). Kernels never trap:
// they record the problem here, skip or clamp the access, and the host turns
// the word into a status code at the next synchronize.
enum DeviceStatusBits : uint32_t {
    kStatusIndexOutOfRange = 1u << 0,
    kStatusWaitTimedOut = 1u << 1,
    kStatusInternal = 1u << 2,
};

// Error carried from a launcher to the C-ABI layer.
struct Error {
    int status;
    std::string message;
};

[[noreturn]] inline void fail(int status, std::string message) {
    throw Error{status, std::move(message)};
}

#define B200_CUDA_CHECK(expr)                                                              \
    do {                                                                                   \
        cudaError_t err__ = (expr);                                                        \
        if (err__ != cudaSuccess) {                                                        \
            ::b200::fail(err__ == cudaErrorMemoryAllocation ? B200_OUT_OF_MEMORY           \
                                                            : B200_DEVICE_ERROR,           \
                         std::string(#expr) + ": " + cudaGetErrorString(err__));           \
        }                                                                                  \
    } while (0)

inline size_t dtype_size(int dt) {
    switch (dt) {
        case B200_F32: return 4;
        case B200_F16: return 2;
        case B200_I32: return 4;
        case B200_I64: return 8;
        case B200_BOOL: return 1;
        default: return 0;
    }
}

// A tensor view with ELEMENT strides, always padded to rank 4 by leading
// extents of 1 (so linear index decomposition is the same loop everywhere).
struct View {
    char* data;
    int64_t dim[kMaxDims];
    int64_t stride[kMaxDims];  // elements
    int64_t numel;
    int dtype;
    bool contiguous;
};

inline View make_view(const b200_tensor& t) {
    View v{};
    v.data = static_cast<char*>(t.data);
    v.dtype = t.dtype;
    const int64_t esz = static_cast<int64_t>(dtype_size(t.dtype));
    if (esz == 0) {
        fail(B200_DTYPE_ERROR, "unknown dtype " + std::to_string(t.dtype));
    }
    if (t.ndim < 0 || t.ndim > kMaxDims) {
        fail(B200_SHAPE_ERROR, "rank " + std::to_string(t.ndim) + " is outside 0..4");
    }
    const int pad = kMaxDims - t.ndim;
    v.numel = 1;
    for (int i = 0; i < kMaxDims; ++i) {
        if (i < pad) {
            v.dim[i] = 1;
            v.stride[i] = 0;
        } else {
            const int64_t d = t.dims[i - pad];
            const int64_t s = t.strides[i - pad];
            if (d < 0) {
                fail(B200_SHAPE_ERROR, "negative extent");
            }
            if (s % esz != 0) {
                fail(B200_NOT_IMPLEMENTED, "byte stride is not a multiple of the element size");
            }
            v.dim[i] = d;
            v.stride[i] = s / esz;
            v.numel *= d;
        }
    }
    // vkml::Shape::is_contiguous (src/core/shape.cpp:96-111): extents of 1 do
    // not constrain the layout; empty tensors are contiguous.
    v.contiguous = true;
    if (v.numel != 0) {
        int64_t expected = 1;
        for (int i = kMaxDims - 1; i >= 0; --i) {
            if (v.dim[i] == 1) {
                continue;
            }
            if (v.stride[i] != expected) {
                v.contiguous = false;
                break;
            }
            expected *= v.dim[i];
        }
    }
    return v;
}

template <typename T>
inline T get_params(const b200_node& n) {
    static_assert(sizeof(T) <= B200_PARAM_BYTES);
    T p;
    std::memcpy(&p, n.params, sizeof(T));
    return p;
}

// Byte-compatible mirrors of vkML's op parameter PODs (include/vkml/graph/op.h:226-318).
struct ReduceParams {
    uint32_t axes_mask;
    bool keepdim;
};
struct SliceParams {
    int32_t axis;
    int64_t start;
    int64_t stop;
    int64_t step;
};
struct AxisParams {
    int32_t axis;
};
struct ScaledAddParams {
    float alpha;
    float beta;
};
struct CastParams {
    uint8_t target;
};
struct TriParams {
    int32_t diagonal;
};
struct ClampParams {
    float lo;
    float hi;
    bool has_lo;
    bool has_hi;
};
struct FullParams {
    double value;
};
struct ArangeParams {
    double start;
    double step;
};
struct RandParams {
    uint64_t seed;
    uint64_t offset;
};
struct UnfoldParams {
    int32_t kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, image_h,
        image_w;
};

// Strides of up to 4 operands over one shared, collapsed iteration space; passed
// to kernels by value.
struct Layout4 {
    int64_t dim[kMaxDims];
    int64_t stride[4][kMaxDims];  // [operand][axis], elements
    int ndim;                      // collapsed rank (>= 1)
};

// Decompose a row-major linear index over `dim` into per-operand element offsets.
template <int N>
__device__ __forceinline__ void offsets_of(const Layout4& L, int64_t linear, int64_t (&off)[N]) {
#pragma unroll
    for (int o = 0; o < N; ++o) {
        off[o] = 0;
    }
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        if (a >= kMaxDims - L.ndim) {
            const int64_t extent = L.dim[a];
            int64_t idx;
            if (a == kMaxDims - L.ndim) {
                idx = linear;
            } else if (linear < (int64_t(1) << 31) && extent < (int64_t(1) << 31)) {
                const uint32_t q = static_cast<uint32_t>(linear) / static_cast<uint32_t>(extent);
                idx = static_cast<uint32_t>(linear) - q * static_cast<uint32_t>(extent);
                linear = q;
            } else {
                const int64_t q = linear / extent;
                idx = linear - q * extent;
                linear = q;
            }
#pragma unroll
            for (int o = 0; o < N; ++o) {
                off[o] += idx * L.stride[o][a];
            }
        }
    }
}

__device__ __forceinline__ int64_t view_offset(const int64_t* dim, const int64_t* stride,
                                               int64_t linear) {
    int64_t off = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        const int64_t extent = dim[a];
        const int64_t q = linear / extent;
        off += (linear - q * extent) * stride[a];
        linear = q;
    }
    return off;
}

// POD copy of a View's geometry for kernels that walk one tensor by linear index.
struct Geo {
    int64_t dim[kMaxDims];
    int64_t stride[kMaxDims];
};

inline Geo geo_of(const View& v) {
    Geo g;
    for (int i = 0; i < kMaxDims; ++i) {
        g.dim[i] = v.dim[i];
        g.stride[i] = v.stride[i];
    }
    return g;
}

__device__ __forceinline__ int64_t geo_offset(const Geo& g, int64_t linear) {
    return view_offset(g.dim, g.stride, linear);
}

// Index arithmetic is the whole cost of the strided kernels, and a 64-bit divide is
// several times a 32-bit one.  Kernels are therefore templated on the index type and
// the host picks uint32_t whenever every linear index and element offset fits.
template <typename I>
struct GeoT {
    I dim[kMaxDims];
    I stride[kMaxDims];
};

template <typename I>
inline GeoT<I> geo_t(const View& v) {
    GeoT<I> g;
    for (int i = 0; i < kMaxDims; ++i) {
        g.dim[i] = static_cast<I>(v.dim[i]);
        g.stride[i] = static_cast<I>(v.stride[i]);
    }
    return g;
}

template <typename I>
__device__ __forceinline__ I geo_off(const GeoT<I>& g, I linear) {
    I off = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        const I q = linear / g.dim[a];
        off += (linear - q * g.dim[a]) * g.stride[a];
        linear = q;
    }
    return off;
}

// True when a view can be walked with 32-bit unsigned indices: non-negative strides and
// both its element count and its largest element offset below 2^31.
inline bool fits32(const View& v) {
    if (v.numel >= (int64_t(1) << 31)) {
        return false;
    }
    int64_t last = 0;
    for (int i = 0; i < kMaxDims; ++i) {
        if (v.stride[i] < 0) {
            return false;
        }
        if (v.dim[i] > 0) {
            last += (v.dim[i] - 1) * v.stride[i];
        }
    }
    return last < (int64_t(1) << 31);
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Grid for a grid-stride loop over `work` items: enough blocks to cover the work,
// capped at a whole number of waves across the 148 SMs.
inline unsigned grid_for(int64_t work, int threads, int blocks_per_sm = 8) {
    const int64_t need = ceil_div(work, threads);
    const int64_t cap = int64_t(sm_count()) * blocks_per_sm;
    int64_t g = need < cap ? need : cap;
    if (g < 1) {
        g = 1;
    }
    return static_cast<unsigned>(g);
}

// Programmatic dependent launch.  Every kernel of the library starts with this pair: the first
// instruction lets the NEXT kernel of the stream be scheduled as soon as all blocks of this one
// are running (instead of after its last block has retired), the second holds this kernel until
// the PREVIOUS one has completed and its writes are visible.  Since the wait precedes every
// memory access, the stream keeps its in-order semantics; what overlaps is launch latency, block
// scheduling and the kernels' own set-up.  Without the launch attribute both are no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

// Division of a 31-bit unsigned number by a divisor known at launch time: one multiply-high
// and a shift instead of the ~20-instruction hardware sequence.  With p = 31 + ceil(log2 d)
// and m = ceil(2^p / d), floor(n / d) == (n * m) >> p for every n < 2^31.
struct FastDiv {
    uint32_t d = 1, mul = 0, shr = 0;
    FastDiv() = default;
    explicit FastDiv(uint32_t divisor) : d(divisor) {
        if (divisor > 1) {
            uint32_t lg = 0;
            while ((uint64_t(1) << lg) < divisor) ++lg;
            const uint32_t p = 31 + lg;
            mul = static_cast<uint32_t>(((uint64_t(1) << p) + divisor - 1) / divisor);
            shr = p - 32;
        }
    }
#ifdef __CUDACC__
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, mul) >> shr; }
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
#endif
};

}  // namespace b200
