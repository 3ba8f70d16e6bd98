// Memory-bound elementwise family: unary, binary, compare, where, scaled_add,
// cast, contiguous, full, arange, rand, triu/tril, cat, slice_backward.
//
// Arithmetic follows vkML's CPU backend (src/backend/cpu/kernels_elementwise.cpp,
// src/backend/cpu/kernels_movement.cpp) operation for operation; this file is
// compiled with -fmad=false so no multiply-add pair is contracted, which is what
// keeps scaled_add bit-identical to the composed mul/mul/add
// (kernels_elementwise.cpp:256-259).
//
// Three execution shapes, picked from the operand strides:
//   flat     -- every operand dense: 128-bit loads/stores, grid-stride.
//   strided  -- rank<=4 collapsed index walk; vectorised along the innermost axis
//               when every operand is unit-stride or broadcast (stride 0) there.
//   tiled    -- an operand whose unit stride lies on the second-innermost axis
//               (a transposed view) goes through a 64x65 shared-memory tile so
//               both the global read and the global write stay coalesced.
// Strided index arithmetic runs in 32 bits whenever every offset fits.
#include "context.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

namespace b200 {
namespace {

constexpr int kThreads = 256;

template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

// ---------------------------------------------------------------------------
// Functors. In0/In1/In2 and Out are the storage types; apply() is the CPU
// backend's lambda.
// ---------------------------------------------------------------------------

struct NoParams {};

#define UNARY_F32(NAME, EXPR)                                                      \
    struct NAME {                                                                   \
        static constexpr int NIN = 1;                                               \
        using In0 = float;                                                          \
        using In1 = float;                                                          \
        using In2 = float;                                                          \
        using Out = float;                                                          \
        using P = NoParams;                                                         \
        __device__ __forceinline__ static float apply(const P&, float x, float, float) { \
            return EXPR;                                                            \
        }                                                                           \
    };

__device__ __forceinline__ float sigmoid_ref(float x) {
    // kernels_elementwise.cpp:25-31: the branch keeps exp's argument non-positive.
    if (x >= 0.0F) {
        return 1.0F / (1.0F + expf(-x));
    }
    const float e = expf(x);
    return e / (1.0F + e);
}

__device__ __forceinline__ float sign_ref(float x) {
    return x > 0.0F ? 1.0F : (x < 0.0F ? -1.0F : 0.0F);  // NaN and -0 give +0 (:75-83)
}

UNARY_F32(FNeg, -x)
UNARY_F32(FAbs, fabsf(x))
UNARY_F32(FSign, sign_ref(x))
UNARY_F32(FSquare, x * x)
UNARY_F32(FSqrt, sqrtf(x))
UNARY_F32(FRsqrt, 1.0F / sqrtf(x))
UNARY_F32(FReciprocal, 1.0F / x)
UNARY_F32(FExp, expf(x))
UNARY_F32(FLog, logf(x))
UNARY_F32(FErf, erff(x))
UNARY_F32(FErfc, erfcf(x))
UNARY_F32(FSin, sinf(x))
UNARY_F32(FCos, cosf(x))
UNARY_F32(FTanh, tanhf(x))
UNARY_F32(FSigmoid, sigmoid_ref(x))
UNARY_F32(FRelu, (x <= 0.0F ? 0.0F : x))  // NaN propagates (:223-231)
UNARY_F32(FGelu, 0.5F * x * erfcf(-x * 0.70710678118654752440F))
UNARY_F32(FSilu, x * sigmoid_ref(x))

struct FClamp {
    static constexpr int NIN = 1;
    using In0 = float;
    using In1 = float;
    using In2 = float;
    using Out = float;
    using P = ClampParams;
    __device__ __forceinline__ static float apply(const P& p, float v, float, float) {
        if (p.has_lo && v < p.lo) {
            return p.lo;
        }
        if (p.has_hi && v > p.hi) {
            return p.hi;
        }
        return v;
    }
};

#define BINARY_F32(NAME, EXPR)                                                     \
    struct NAME {                                                                   \
        static constexpr int NIN = 2;                                               \
        using In0 = float;                                                          \
        using In1 = float;                                                          \
        using In2 = float;                                                          \
        using Out = float;                                                          \
        using P = NoParams;                                                         \
        __device__ __forceinline__ static float apply(const P&, float x, float y, float) { \
            return EXPR;                                                            \
        }                                                                           \
    };

BINARY_F32(FAdd, __fadd_rn(x, y))
BINARY_F32(FSub, __fsub_rn(x, y))
BINARY_F32(FMul, __fmul_rn(x, y))
BINARY_F32(FDiv, __fdiv_rn(x, y))
BINARY_F32(FPow, powf(x, y))
BINARY_F32(FMaximum, ((isnan(x) || isnan(y)) ? __int_as_float(0x7fc00000) : (x > y ? x : y)))
BINARY_F32(FMinimum, ((isnan(x) || isnan(y)) ? __int_as_float(0x7fc00000) : (x < y ? x : y)))

struct FScaledAdd {
    static constexpr int NIN = 2;
    using In0 = float;
    using In1 = float;
    using In2 = float;
    using Out = float;
    using P = ScaledAddParams;
    __device__ __forceinline__ static float apply(const P& p, float x, float y, float) {
        // two rounded products, then one rounded sum: never an FMA
        return __fadd_rn(__fmul_rn(x, p.alpha), __fmul_rn(y, p.beta));
    }
};

#define COMPARE_F32(NAME, EXPR)                                                    \
    struct NAME {                                                                   \
        static constexpr int NIN = 2;                                               \
        using In0 = float;                                                          \
        using In1 = float;                                                          \
        using In2 = float;                                                          \
        using Out = uint8_t;                                                        \
        using P = NoParams;                                                         \
        __device__ __forceinline__ static uint8_t apply(const P&, float x, float y, float) { \
            return (EXPR) ? 1 : 0;                                                  \
        }                                                                           \
    };

COMPARE_F32(FEqual, x == y)
COMPARE_F32(FLess, x < y)
COMPARE_F32(FGreater, x > y)
COMPARE_F32(FLessEqual, x <= y)
COMPARE_F32(FGreaterEqual, x >= y)
COMPARE_F32(FNotEqual, x != y)

struct FWhere {
    static constexpr int NIN = 3;
    using In0 = uint8_t;
    using In1 = float;
    using In2 = float;
    using Out = float;
    using P = NoParams;
    __device__ __forceinline__ static float apply(const P&, uint8_t c, float a, float b) {
        return c != 0 ? a : b;
    }
};

// Same-type copy by element width (Contiguous, and Cast with from == to).
template <typename T>
struct FCopy {
    static constexpr int NIN = 1;
    using In0 = T;
    using In1 = T;
    using In2 = T;
    using Out = T;
    using P = NoParams;
    __device__ __forceinline__ static T apply(const P&, T x, T, T) { return x; }
};

// fp32 -> fp16 bits, round to nearest even; NaN becomes a quiet NaN with the
// input's sign and an otherwise empty payload, as vkML's software conversion
// produces (src/core/dtype.cpp:47-70).
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
    if (isnan(f)) {
        return static_cast<uint16_t>(((__float_as_uint(f) >> 16) & 0x8000U) | 0x7E00U);
    }
    return __half_as_ushort(__float2half_rn(f));
}

template <typename From, typename To>
struct FCast {
    static constexpr int NIN = 1;
    using In0 = From;
    using In1 = From;
    using In2 = From;
    using Out = To;
    using P = NoParams;
    __device__ __forceinline__ static To apply(const P&, From x, From, From) {
        return static_cast<To>(x);
    }
};
struct FCastF32Bool {
    static constexpr int NIN = 1;
    using In0 = float;
    using In1 = float;
    using In2 = float;
    using Out = uint8_t;
    using P = NoParams;
    __device__ __forceinline__ static uint8_t apply(const P&, float x, float, float) {
        return x != 0.0F ? 1 : 0;
    }
};
struct FCastF32F16 {
    static constexpr int NIN = 1;
    using In0 = float;
    using In1 = float;
    using In2 = float;
    using Out = uint16_t;
    using P = NoParams;
    __device__ __forceinline__ static uint16_t apply(const P&, float x, float, float) {
        return f32_to_f16_bits(x);
    }
};
struct FCastF16F32 {
    static constexpr int NIN = 1;
    using In0 = uint16_t;
    using In1 = uint16_t;
    using In2 = uint16_t;
    using Out = float;
    using P = NoParams;
    __device__ __forceinline__ static float apply(const P&, uint16_t x, uint16_t, uint16_t) {
        return __half2float(__ushort_as_half(x));
    }
};
// F16 is storage, never arithmetic (src/backend/cpu/kernels_elementwise.cpp:89-99): the same
// functor, with every float operand widened from half bits on load and a float result narrowed
// once, round-to-nearest-even, on store.  What the widened-copy path computes, without the copies.
template <typename T>
using HalfIf = std::conditional_t<std::is_same_v<T, float>, uint16_t, T>;

template <typename F>
struct HalfIO {
    static constexpr int NIN = F::NIN;
    using In0 = HalfIf<typename F::In0>;
    using In1 = HalfIf<typename F::In1>;
    using In2 = HalfIf<typename F::In2>;
    using Out = HalfIf<typename F::Out>;
    using P = typename F::P;
    template <typename Want, typename Got>
    __device__ __forceinline__ static Want widen(Got x) {
        if constexpr (std::is_same_v<Want, float>) {
            return __half2float(__ushort_as_half(x));
        } else {
            return x;
        }
    }
    __device__ __forceinline__ static Out apply(const P& p, In0 a, In1 b, In2 c) {
        const auto r = F::apply(p, widen<typename F::In0>(a), widen<typename F::In1>(b), widen<typename F::In2>(c));
        if constexpr (std::is_same_v<typename F::Out, float>) {
            return f32_to_f16_bits(r);
        } else {
            return r;
        }
    }
};

template <typename To>
struct FCastBool {
    static constexpr int NIN = 1;
    using In0 = uint8_t;
    using In1 = uint8_t;
    using In2 = uint8_t;
    using Out = To;
    using P = NoParams;
    __device__ __forceinline__ static To apply(const P&, uint8_t x, uint8_t, uint8_t) {
        return x != 0 ? To(1) : To(0);
    }
};

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------

// Independent vectors in flight per thread: four, or two for the 8-wide vectors of
// the mixed-width ops so the kernel stays under 64 registers.
template <int VEC>
__host__ __device__ constexpr int unroll_for() {
    return VEC >= 8 ? 2 : 4;
}

template <typename F, int VEC>
__device__ __forceinline__ Vec<typename F::Out, VEC> apply_vec(const typename F::P& p,
                                                               const Vec<typename F::In0, VEC>& a,
                                                               const Vec<typename F::In1, VEC>& b,
                                                               const Vec<typename F::In2, VEC>& c) {
    Vec<typename F::Out, VEC> o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        o.v[k] = F::apply(p, a.v[k], b.v[k], c.v[k]);
    }
    return o;
}

// Every operand dense and aligned: VEC elements per vector, kUnroll vectors per
// thread per trip, all loads issued before the first use.
template <typename F, int VEC>
__global__ void __launch_bounds__(kThreads)
flat_kernel(typename F::Out* __restrict__ out, const typename F::In0* __restrict__ a,
            const typename F::In1* __restrict__ b, const typename F::In2* __restrict__ c,
            int64_t n, typename F::P p) {
    pdl_prologue();
    using VA = Vec<typename F::In0, VEC>;
    using VB = Vec<typename F::In1, VEC>;
    using VC = Vec<typename F::In2, VEC>;
    using VO = Vec<typename F::Out, VEC>;
    constexpr int kUnroll = unroll_for<VEC>();
    const int64_t nvec = n / VEC;
    const int64_t step = int64_t(gridDim.x) * kThreads * kUnroll;
    for (int64_t base = int64_t(blockIdx.x) * kThreads * kUnroll + threadIdx.x; base < nvec; base += step) {
        VA va[kUnroll];
        VB vb[kUnroll];
        VC vc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t i = base + int64_t(u) * kThreads;
            vb[u] = VB{};
            vc[u] = VC{};
            if (i < nvec) {
                va[u] = reinterpret_cast<const VA*>(a)[i];
                if constexpr (F::NIN >= 2) {
                    vb[u] = reinterpret_cast<const VB*>(b)[i];
                }
                if constexpr (F::NIN >= 3) {
                    vc[u] = reinterpret_cast<const VC*>(c)[i];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t i = base + int64_t(u) * kThreads;
            if (i < nvec) {
                reinterpret_cast<VO*>(out)[i] = apply_vec<F, VEC>(p, va[u], vb[u], vc[u]);
            }
        }
    }
    // tail (n % VEC elements) by the first threads of block 0
    if (blockIdx.x == 0) {
        const int64_t i = nvec * VEC + threadIdx.x;
        if (i < n) {
            typename F::In1 y{};
            typename F::In2 z{};
            if constexpr (F::NIN >= 2) {
                y = b[i];
            }
            if constexpr (F::NIN >= 3) {
                z = c[i];
            }
            out[i] = F::apply(p, a[i], y, z);
        }
    }
}

// Strides of up to three inputs over one collapsed iteration space, in index type I.
template <typename I>
struct LayoutT {
    I dim[kMaxDims];
    I stride[3][kMaxDims];
    int ndim;
};

template <typename I>
__device__ __forceinline__ void offsets3(const LayoutT<I>& L, I linear, I (&off)[3]) {
    off[0] = off[1] = off[2] = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        if (a >= kMaxDims - L.ndim) {
            I idx;
            if (a == kMaxDims - L.ndim) {
                idx = linear;
            } else {
                const I q = linear / L.dim[a];
                idx = linear - q * L.dim[a];
                linear = q;
            }
            off[0] += idx * L.stride[0][a];
            off[1] += idx * L.stride[1][a];
            off[2] += idx * L.stride[2][a];
        }
    }
}

template <typename T, int VEC, typename I>
__device__ __forceinline__ Vec<T, VEC> load_or_splat(const T* p, I off, I inner_stride) {
    Vec<T, VEC> v;
    if (VEC > 1 && inner_stride != 0) {
        v = *reinterpret_cast<const Vec<T, VEC>*>(p + off);
    } else {
        const T s = p[off];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            v.v[k] = s;
        }
    }
    return v;
}

// General strided walk; the output is dense.  With VEC > 1 the innermost extent has
// been divided by VEC and every input's innermost stride is VEC (unit stride: vector
// load) or 0 (broadcast: one load, splat).
template <typename F, int VEC, typename I>
__global__ void __launch_bounds__(kThreads)
strided_kernel(typename F::Out* __restrict__ out, const typename F::In0* __restrict__ a,
               const typename F::In1* __restrict__ b, const typename F::In2* __restrict__ c,
               I nvec, LayoutT<I> L, typename F::P p) {
    pdl_prologue();
    constexpr int kUnroll = unroll_for<VEC>();
    const int inner = kMaxDims - 1;
    const int64_t step = int64_t(gridDim.x) * kThreads * kUnroll;
    for (int64_t base = int64_t(blockIdx.x) * kThreads * kUnroll + threadIdx.x; base < int64_t(nvec);
         base += step) {
        Vec<typename F::In0, VEC> va[kUnroll];
        Vec<typename F::In1, VEC> vb[kUnroll];
        Vec<typename F::In2, VEC> vc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t i = base + int64_t(u) * kThreads;
            vb[u] = Vec<typename F::In1, VEC>{};
            vc[u] = Vec<typename F::In2, VEC>{};
            if (i < int64_t(nvec)) {
                I off[3];
                offsets3<I>(L, static_cast<I>(i), off);
                va[u] = load_or_splat<typename F::In0, VEC, I>(a, off[0], L.stride[0][inner]);
                if constexpr (F::NIN >= 2) {
                    vb[u] = load_or_splat<typename F::In1, VEC, I>(b, off[1], L.stride[1][inner]);
                }
                if constexpr (F::NIN >= 3) {
                    vc[u] = load_or_splat<typename F::In2, VEC, I>(c, off[2], L.stride[2][inner]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t i = base + int64_t(u) * kThreads;
            if (i < int64_t(nvec)) {
                reinterpret_cast<Vec<typename F::Out, VEC>*>(out)[i] = apply_vec<F, VEC>(p, va[u], vb[u], vc[u]);
            }
        }
    }
}

// Transposed operands. Iteration space [batch, R, C], output dense row-major.
// Each input is read either along C (its stride on C is 1 or 0) or, when
// `transposed` is set for it, along R -- its unit-stride axis -- into a padded
// 64x64 shared tile that is then read back along C.  16 elements per thread are in
// flight per phase; global reads and writes are both 256-byte runs.  4-byte types.
struct TileArgs {
    int64_t batch, rows, cols;
    int64_t sb[3], sr[3], sc[3];  // per-input element strides over (batch, R, C)
    int transposed[3];
    int vec;  // every pointer and pitch is 16-byte aligned: full tiles move as 128-bit vectors
};

constexpr int kTile = 64;

template <typename F>
__global__ void __launch_bounds__(256)
tiled_kernel(typename F::Out* __restrict__ out, const typename F::In0* __restrict__ a,
             const typename F::In1* __restrict__ b, const typename F::In2* __restrict__ c,
             TileArgs t, typename F::P p) {
    pdl_prologue();
    __shared__ typename F::In0 ta[kTile][kTile + 1];
    __shared__ typename F::In1 tb[kTile][kTile + 1];
    const int64_t tiles_c = (t.cols + kTile - 1) / kTile;
    const int64_t tiles_r = (t.rows + kTile - 1) / kTile;
    const int64_t n_tiles = tiles_c * tiles_r * t.batch;
    const int fast = threadIdx.x & 63;  // position along the unit-stride axis of the phase
    const int slow = threadIdx.x >> 6;  // 0..3
    // Tiles are numbered so that 16 consecutive ones form a 4x4 super-tile: blocks
    // that run at the same time then touch 1 KB runs of both the transposed source and
    // the destination instead of 256-byte fragments of 16 different DRAM pages.
    const int64_t super_c = (tiles_c + 3) / 4;
    const int64_t super_r = (tiles_r + 3) / 4;
    const int64_t n_slots = super_c * super_r * 16 * t.batch;
    (void)n_tiles;
    for (int64_t slot = blockIdx.x; slot < n_slots; slot += gridDim.x) {
        const int64_t within = slot & 15;
        const int64_t sup = slot >> 4;
        const int64_t sc_i = sup % super_c;
        const int64_t sr_i = (sup / super_c) % super_r;
        const int64_t bi = sup / (super_c * super_r);
        const int64_t tc = sc_i * 4 + (within & 3);
        const int64_t tr = sr_i * 4 + (within >> 2);
        if (tc >= tiles_c || tr >= tiles_r) {
            continue;  // block-uniform
        }
        const int64_t r0 = tr * kTile;
        const int64_t c0 = tc * kTile;
        const bool full = r0 + kTile <= t.rows && c0 + kTile <= t.cols;  // block-uniform
        if (full && t.vec) {
            // Full tile, everything 16-byte aligned.  A warp moves four 128-byte runs per
            // step: along R of a transposed input in phase 1 (8 lanes x 4 elements, 4
            // neighbouring columns), along C of the output and the other inputs in phase 2.
            // With the 65-word pitch both the scattered stores of phase 1 and the gathered
            // loads of phase 2 touch 32 different banks.
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            const int q = lane & 7, l4 = lane >> 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int wt = j * 8 + warp;
                const int rr = ((wt & 1) * 8 + q) * 4;
                const int cc = (wt >> 1) * 4 + l4;
                if (t.transposed[0]) {
                    const Vec<typename F::In0, 4> v = *reinterpret_cast<const Vec<typename F::In0, 4>*>(
                        a + bi * t.sb[0] + (c0 + cc) * t.sc[0] + (r0 + rr));
#pragma unroll
                    for (int e = 0; e < 4; ++e) ta[rr + e][cc] = v.v[e];
                }
                if constexpr (F::NIN >= 2) {
                    if (t.transposed[1]) {
                        const Vec<typename F::In1, 4> v = *reinterpret_cast<const Vec<typename F::In1, 4>*>(
                            b + bi * t.sb[1] + (c0 + cc) * t.sc[1] + (r0 + rr));
#pragma unroll
                        for (int e = 0; e < 4; ++e) tb[rr + e][cc] = v.v[e];
                    }
                }
            }
            // operands that are not transposed are read straight along C, in the phase-2 mapping;
            // their loads are issued here, before the barrier, so they travel together with the
            // transposed operand's instead of after it
            Vec<typename F::In0, 4> xd[4];
            Vec<typename F::In1, 4> yd[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int wt = j * 8 + warp;
                const int cc = ((wt & 1) * 8 + q) * 4;
                const int rr = (wt >> 1) * 4 + l4;
                xd[j] = Vec<typename F::In0, 4>{};
                yd[j] = Vec<typename F::In1, 4>{};
                if (!t.transposed[0]) {
                    const typename F::In0* src = a + bi * t.sb[0] + (r0 + rr) * t.sr[0];
                    if (t.sc[0] == 1) {
                        xd[j] = *reinterpret_cast<const Vec<typename F::In0, 4>*>(src + c0 + cc);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) xd[j].v[e] = src[0];
                    }
                }
                if constexpr (F::NIN >= 2) {
                    if (!t.transposed[1]) {
                        const typename F::In1* src = b + bi * t.sb[1] + (r0 + rr) * t.sr[1];
                        if (t.sc[1] == 1) {
                            yd[j] = *reinterpret_cast<const Vec<typename F::In1, 4>*>(src + c0 + cc);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) yd[j].v[e] = src[0];
                        }
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int wt = j * 8 + warp;
                const int cc = ((wt & 1) * 8 + q) * 4;
                const int rr = (wt >> 1) * 4 + l4;
                Vec<typename F::In0, 4> x = xd[j];
                Vec<typename F::In1, 4> y = yd[j];
                if (t.transposed[0]) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) x.v[e] = ta[rr][cc + e];
                }
                if constexpr (F::NIN >= 2) {
                    if (t.transposed[1]) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) y.v[e] = tb[rr][cc + e];
                    }
                }
                Vec<typename F::Out, 4> o;
#pragma unroll
                for (int e = 0; e < 4; ++e) o.v[e] = F::apply(p, x.v[e], y.v[e], typename F::In2{});
                *reinterpret_cast<Vec<typename F::Out, 4>*>(out + (bi * t.rows + r0 + rr) * t.cols + c0 + cc) = o;
            }
            __syncthreads();
            continue;
        }
        // phase 1: transposed inputs, threads run along R (their unit-stride axis)
        if (t.transposed[0]) {
            const typename F::In0* src = a + bi * t.sb[0] + (r0 + fast) * t.sr[0] + (c0 + slow) * t.sc[0];
            const int64_t step = 4 * t.sc[0];
            if (full) {
#pragma unroll
                for (int j = 0; j < kTile / 4; ++j) {
                    ta[fast][slow + 4 * j] = src[j * step];
                }
            } else if (r0 + fast < t.rows) {
#pragma unroll
                for (int j = 0; j < kTile / 4; ++j) {
                    if (c0 + slow + 4 * j < t.cols) {
                        ta[fast][slow + 4 * j] = src[j * step];
                    }
                }
            }
        }
        if constexpr (F::NIN >= 2) {
            if (t.transposed[1]) {
                const typename F::In1* src = b + bi * t.sb[1] + (r0 + fast) * t.sr[1] + (c0 + slow) * t.sc[1];
                const int64_t step = 4 * t.sc[1];
                if (full) {
#pragma unroll
                    for (int j = 0; j < kTile / 4; ++j) {
                        tb[fast][slow + 4 * j] = src[j * step];
                    }
                } else if (r0 + fast < t.rows) {
#pragma unroll
                    for (int j = 0; j < kTile / 4; ++j) {
                        if (c0 + slow + 4 * j < t.cols) {
                            tb[fast][slow + 4 * j] = src[j * step];
                        }
                    }
                }
            }
        }
        __syncthreads();
        // phase 2: threads run along C; row r0 + slow + 4j for j = 0..15
        typename F::Out* dst = out + (bi * t.rows + r0 + slow) * t.cols + c0 + fast;
        const int64_t dstep = 4 * t.cols;
        const typename F::In0* ap = a + bi * t.sb[0] + (r0 + slow) * t.sr[0] + (c0 + fast) * t.sc[0];
        const int64_t astep = 4 * t.sr[0];
        const typename F::In1* bp = nullptr;
        int64_t bstep = 0;
        if constexpr (F::NIN >= 2) {
            bp = b + bi * t.sb[1] + (r0 + slow) * t.sr[1] + (c0 + fast) * t.sc[1];
            bstep = 4 * t.sr[1];
        }
        const bool col_ok = c0 + fast < t.cols;
        typename F::In0 xs[kTile / 4];
        typename F::In1 ys[kTile / 4];
#pragma unroll
        for (int j = 0; j < kTile / 4; ++j) {
            const bool ok = full || (col_ok && r0 + slow + 4 * j < t.rows);
            xs[j] = typename F::In0{};
            ys[j] = typename F::In1{};
            if (ok) {
                xs[j] = t.transposed[0] ? ta[slow + 4 * j][fast] : ap[j * astep];
                if constexpr (F::NIN >= 2) {
                    ys[j] = t.transposed[1] ? tb[slow + 4 * j][fast] : bp[j * bstep];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kTile / 4; ++j) {
            if (full || (col_ok && r0 + slow + 4 * j < t.rows)) {
                dst[j * dstep] = F::apply(p, xs[j], ys[j], typename F::In2{});
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Layout analysis
// ---------------------------------------------------------------------------

// Collapse the shared iteration space of `n` views (all already broadcast to the
// same extents): drop extents of 1, merge neighbours that every operand walks as
// one run.
Layout4 collapse(const View* views, int n) {
    int64_t dim[kMaxDims];
    int64_t st[4][kMaxDims];
    int rank = 0;
    for (int a = 0; a < kMaxDims; ++a) {
        const int64_t d = views[0].dim[a];
        if (d == 1) {
            continue;
        }
        bool merged = false;
        if (rank > 0) {
            merged = true;
            for (int o = 0; o < n; ++o) {
                if (st[o][rank - 1] != views[o].stride[a] * d) {
                    merged = false;
                    break;
                }
            }
        }
        if (merged) {
            dim[rank - 1] *= d;
            for (int o = 0; o < n; ++o) {
                st[o][rank - 1] = views[o].stride[a];
            }
        } else {
            dim[rank] = d;
            for (int o = 0; o < n; ++o) {
                st[o][rank] = views[o].stride[a];
            }
            ++rank;
        }
    }
    if (rank == 0) {
        dim[0] = 1;
        for (int o = 0; o < n; ++o) {
            st[o][0] = 0;
        }
        rank = 1;
    }
    Layout4 L{};
    L.ndim = rank;
    for (int a = 0; a < kMaxDims; ++a) {
        L.dim[a] = 1;
        for (int o = 0; o < 4; ++o) {
            L.stride[o][a] = 0;
        }
    }
    for (int r = 0; r < rank; ++r) {
        const int a = kMaxDims - rank + r;
        L.dim[a] = dim[r];
        for (int o = 0; o < n; ++o) {
            L.stride[o][a] = st[o][r];
        }
    }
    return L;
}

template <typename I>
LayoutT<I> narrow(const Layout4& L) {
    LayoutT<I> r;
    r.ndim = L.ndim;
    for (int a = 0; a < kMaxDims; ++a) {
        r.dim[a] = static_cast<I>(L.dim[a]);
        for (int o = 0; o < 3; ++o) {
            r.stride[o][a] = static_cast<I>(L.stride[o][a]);
        }
    }
    return r;
}

template <typename T>
bool aligned_for(const void* p, int vec) {
    return reinterpret_cast<uintptr_t>(p) % (sizeof(T) * vec) == 0;
}

template <typename F, int VEC>
void launch_strided(b200_ctx* ctx, typename F::Out* o, const typename F::In0* a, const typename F::In1* b,
                    const typename F::In2* c, int64_t nvec, const Layout4& L, bool small_index,
                    const typename F::P& p) {
    const unsigned grid = grid_for(ceil_div(nvec, unroll_for<VEC>()), kThreads);
    if (small_index) {
        launch_kernel(ctx, strided_kernel<F, VEC, uint32_t>, grid, kThreads, 0, o, a, b, c, static_cast<uint32_t>(nvec), narrow<uint32_t>(L), p);
    } else {
        launch_kernel(ctx, strided_kernel<F, VEC, int64_t>, grid, kThreads, 0, o, a, b, c, nvec,
                                                                            narrow<int64_t>(L), p);
    }
}

template <typename F>
void run(b200_ctx* ctx, const b200_node& node, const typename F::P& p) {
    const View out = make_view(node.out);
    if (out.numel == 0) {
        return;
    }
    if (!out.contiguous) {
        fail(B200_NOT_IMPLEMENTED, "elementwise output must be contiguous");
    }
    if (static_cast<int>(node.n_src) < F::NIN) {
        fail(B200_INVALID_ARGUMENT, "elementwise node is missing a source");
    }
    View in[3];
    bool small_index = out.numel < (int64_t(1) << 31);
    for (int i = 0; i < F::NIN; ++i) {
        in[i] = make_view(node.src[i]);
        for (int a = 0; a < kMaxDims; ++a) {
            if (in[i].dim[a] != out.dim[a]) {
                fail(B200_SHAPE_ERROR, "elementwise operand extents differ from the output's");
            }
        }
        small_index = small_index && fits32(in[i]);
    }
    auto* o = reinterpret_cast<typename F::Out*>(out.data);
    auto* a = reinterpret_cast<const typename F::In0*>(in[0].data);
    auto* b = F::NIN >= 2 ? reinterpret_cast<const typename F::In1*>(in[1].data) : nullptr;
    auto* c = F::NIN >= 3 ? reinterpret_cast<const typename F::In2*>(in[2].data) : nullptr;
    const int64_t n = out.numel;

    bool dense = true;
    for (int i = 0; i < F::NIN; ++i) {
        dense = dense && in[i].contiguous;
    }
    // 16 bytes per vector of the NARROWEST type involved (capped at 8 elements)
    constexpr size_t kMinSize =
        std::min(std::min(sizeof(typename F::In0), sizeof(typename F::Out)),
                 std::min(F::NIN >= 2 ? sizeof(typename F::In1) : size_t(8),
                          F::NIN >= 3 ? sizeof(typename F::In2) : size_t(8)));
    constexpr int kVec = kMinSize >= 8 ? 2 : (kMinSize == 4 ? 4 : 8);
    if (dense) {
        bool al = aligned_for<typename F::Out>(o, kVec) && aligned_for<typename F::In0>(a, kVec);
        if (F::NIN >= 2) {
            al = al && aligned_for<typename F::In1>(b, kVec);
        }
        if (F::NIN >= 3) {
            al = al && aligned_for<typename F::In2>(c, kVec);
        }
        if (al) {
            launch_kernel(ctx, flat_kernel<F, kVec>, grid_for(ceil_div(n / kVec + 1, unroll_for<kVec>()), kThreads), kThreads, 0, o, a, b, c, n, p);
        } else {
            launch_kernel(ctx, flat_kernel<F, 1>, grid_for(ceil_div(n, unroll_for<1>()), kThreads), kThreads, 0, o, a, b, c, n,
                                                                                                   p);
        }
        ctx->count_launch();
        check_last_launch("elementwise flat");
        return;
    }

    Layout4 L = collapse(in, F::NIN);
    const int inner = kMaxDims - 1;

    // transposed-operand path: 4-byte types, <= 2 inputs, collapsed rank 2 or 3
    if constexpr (F::NIN <= 2 && sizeof(typename F::In0) == 4 && sizeof(typename F::In1) == 4 &&
                  sizeof(typename F::Out) == 4) {
        if (L.ndim >= 2 && L.ndim <= 3) {
            const int rax = kMaxDims - 2;
            bool any_t = false;
            bool ok = true;
            TileArgs t{};
            t.cols = L.dim[inner];
            t.rows = L.dim[rax];
            t.batch = L.ndim == 3 ? L.dim[kMaxDims - 3] : 1;
            for (int i = 0; i < F::NIN; ++i) {
                t.sc[i] = L.stride[i][inner];
                t.sr[i] = L.stride[i][rax];
                t.sb[i] = L.ndim == 3 ? L.stride[i][kMaxDims - 3] : 0;
                if (t.sc[i] == 1 || t.sc[i] == 0) {
                    t.transposed[i] = 0;
                } else if (t.sr[i] == 1) {
                    t.transposed[i] = 1;
                    any_t = true;
                } else {
                    ok = false;
                }
            }
            t.vec = t.cols % 4 == 0 && reinterpret_cast<uintptr_t>(o) % 16 == 0;
            const void* bases[3] = {a, b, c};
            for (int i = 0; i < F::NIN; ++i) {
                bool al = reinterpret_cast<uintptr_t>(bases[i]) % 16 == 0 && t.sb[i] % 4 == 0;
                if (t.transposed[i]) {
                    al = al && t.sc[i] % 4 == 0;
                } else if (t.sc[i] == 1) {
                    al = al && t.sr[i] % 4 == 0;
                }
                t.vec = t.vec && al;
            }
            if (ok && any_t && t.rows >= 8 && t.cols >= 8) {
                const int64_t tiles = ceil_div(ceil_div(t.rows, kTile), 4) * ceil_div(ceil_div(t.cols, kTile), 4) * 16 *
                                      t.batch;
                launch_kernel(ctx, tiled_kernel<F>, grid_for(tiles, 1, 8), 256, 0, o, a, b, c, t, p);
                ctx->count_launch();
                check_last_launch("elementwise tiled");
                return;
            }
        }
    }

    // vectorise along the innermost axis when every input is unit-stride or broadcast there
    bool vec_ok = L.dim[inner] % kVec == 0 && aligned_for<typename F::Out>(o, kVec);
    const void* ptrs[3] = {a, b, c};
    const size_t esz[3] = {sizeof(typename F::In0), sizeof(typename F::In1), sizeof(typename F::In2)};
    for (int i = 0; i < F::NIN && vec_ok; ++i) {
        const int64_t si = L.stride[i][inner];
        if (si == 0) {
            continue;
        }
        if (si != 1 || reinterpret_cast<uintptr_t>(ptrs[i]) % (esz[i] * kVec) != 0) {
            vec_ok = false;
            break;
        }
        for (int ax = kMaxDims - L.ndim; ax < inner; ++ax) {
            if (L.stride[i][ax] % kVec != 0) {
                vec_ok = false;
            }
        }
    }
    if (vec_ok) {
        Layout4 V = L;
        V.dim[inner] /= kVec;
        for (int i = 0; i < F::NIN; ++i) {
            V.stride[i][inner] *= kVec;
        }
        launch_strided<F, kVec>(ctx, o, a, b, c, n / kVec, V, small_index, p);
    } else {
        launch_strided<F, 1>(ctx, o, a, b, c, n, L, small_index, p);
    }
    ctx->count_launch();
    check_last_launch("elementwise strided");
}

// ---------------------------------------------------------------------------
// Creation and index-pattern ops (outputs are dense)
// ---------------------------------------------------------------------------

// 16-byte stores; the pointer comes from the allocator, so it is 512-byte aligned.
template <typename T>
__global__ void __launch_bounds__(kThreads) fill_kernel(T* __restrict__ out, int64_t n, T value) {
    pdl_prologue();
    constexpr int V = 16 / sizeof(T);
    Vec<T, V> v;
#pragma unroll
    for (int k = 0; k < V; ++k) {
        v.v[k] = value;
    }
    const bool aligned = reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const int64_t nvec = aligned ? n / V : 0;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        reinterpret_cast<Vec<T, V>*>(out)[i] = v;
    }
    for (int64_t i = nvec * V + int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        out[i] = value;
    }
}

// start + i*step evaluated in double with two roundings, then narrowed
// (kernels_movement.cpp:175-197).
template <typename T>
__global__ void __launch_bounds__(kThreads)
arange_kernel(T* __restrict__ out, int64_t n, double start, double step) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        out[i] = static_cast<T>(__dadd_rn(start, __dmul_rn(static_cast<double>(i), step)));
    }
}

// Philox4x32-10 keyed by the seed, counter = (index, offset); the first output
// word's top 24 bits scaled by 2^-24 (src/backend/cpu/philox.h:47-89).
__global__ void __launch_bounds__(kThreads)
rand_kernel(float* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t c0 = static_cast<uint32_t>(i), c1 = static_cast<uint32_t>(uint64_t(i) >> 32);
        uint32_t c2 = static_cast<uint32_t>(offset), c3 = static_cast<uint32_t>(offset >> 32);
        uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
        for (int r = 0; r < 10; ++r) {
            const uint32_t hi0 = __umulhi(0xD2511F53U, c0), lo0 = 0xD2511F53U * c0;
            const uint32_t hi1 = __umulhi(0xCD9E8D57U, c2), lo1 = 0xCD9E8D57U * c2;
            c0 = hi1 ^ c1 ^ k0;
            c1 = lo1;
            c2 = hi0 ^ c3 ^ k1;
            c3 = lo0;
            k0 += 0x9E3779B9U;
            k1 += 0xBB67AE85U;
        }
        out[i] = static_cast<float>(c0 >> 8) * (1.0F / 16777216.0F);
    }
}

// triu/tril over the last two axes (kernels_elementwise.cpp:326-352).
__global__ void __launch_bounds__(kThreads)
tri_kernel(float* __restrict__ out, const float* __restrict__ in, Geo gin, int64_t n, int64_t width,
           int64_t height, int diagonal, int upper) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t col = i % width;
        const int64_t row = (i / width) % height;
        const int64_t d = col - row;
        const bool keep = upper ? d >= diagonal : d <= diagonal;
        out[i] = keep ? in[geo_offset(gin, i)] : 0.0F;
    }
}

// Two-input concatenation along `axis` (kernels_movement.cpp:272-317).
template <typename T>
__global__ void __launch_bounds__(kThreads)
cat_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, Geo ga, Geo gb,
           int64_t n, int64_t inner, int64_t out_extent, int64_t a_extent, int64_t b_extent) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t rest = i % inner;
        const int64_t along = (i / inner) % out_extent;
        const int64_t outer = i / (inner * out_extent);
        if (along < a_extent) {
            out[i] = a[geo_offset(ga, (outer * a_extent + along) * inner + rest)];
        } else {
            out[i] = b[geo_offset(gb, (outer * b_extent + (along - a_extent)) * inner + rest)];
        }
    }
}

// Adjoint of a strided slice, pull form: every element of the zero-padded result
// looks up whether a gradient element lands on it (kernels_movement.cpp:226-262).
__global__ void __launch_bounds__(kThreads)
slice_backward_kernel(float* __restrict__ out, const float* __restrict__ g, Geo gout, Geo gg,
                      int64_t n, int axis, int64_t start, int64_t step) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i;
        int64_t goff = 0;
        bool hit = true;
#pragma unroll
        for (int a = kMaxDims - 1; a >= 0; --a) {
            const int64_t idx = rem % gout.dim[a];
            rem /= gout.dim[a];
            if (a == axis) {
                const int64_t rel = idx - start;
                if (rel < 0 || rel % step != 0 || rel / step >= gg.dim[a]) {
                    hit = false;
                } else {
                    goff += (rel / step) * gg.stride[a];
                }
            } else {
                goff += idx * gg.stride[a];
            }
        }
        out[i] = hit ? g[goff] : 0.0F;
    }
}

void run_full(b200_ctx* ctx, const b200_node& node) {
    const View out = make_view(node.out);
    const auto p = get_params<FullParams>(node);
    const int64_t n = out.numel;
    if (n == 0) {
        return;
    }
    const unsigned g = grid_for(ceil_div(n, 4), kThreads);
    switch (out.dtype) {
        case B200_F32:
            launch_kernel(ctx, fill_kernel<float>, g, kThreads, 0, reinterpret_cast<float*>(out.data), n,
                                                               static_cast<float>(p.value));
            break;
        case B200_F16: {
            // narrow on the host with the same rule as the device cast
            const float f = static_cast<float>(p.value);
            uint16_t bits;
            if (f != f) {
                uint32_t w;
                std::memcpy(&w, &f, 4);
                bits = static_cast<uint16_t>(((w >> 16) & 0x8000U) | 0x7E00U);
            } else {
                const __half h = __float2half_rn(f);
                std::memcpy(&bits, &h, 2);
            }
            launch_kernel(ctx, fill_kernel<uint16_t>, g, kThreads, 0, reinterpret_cast<uint16_t*>(out.data), n, bits);
            break;
        }
        case B200_I64:
            launch_kernel(ctx, fill_kernel<int64_t>, g, kThreads, 0, reinterpret_cast<int64_t*>(out.data), n, static_cast<int64_t>(p.value));
            break;
        case B200_I32:
            launch_kernel(ctx, fill_kernel<int32_t>, g, kThreads, 0, reinterpret_cast<int32_t*>(out.data), n, static_cast<int32_t>(p.value));
            break;
        case B200_BOOL:
            launch_kernel(ctx, fill_kernel<uint8_t>, g, kThreads, 0, reinterpret_cast<uint8_t*>(out.data), n, static_cast<uint8_t>(p.value != 0.0 ? 1 : 0));
            break;
        default: fail(B200_DTYPE_ERROR, "full: unsupported dtype");
    }
    ctx->count_launch();
    check_last_launch("full");
}

void run_cast(b200_ctx* ctx, const b200_node& node) {
    const int from = node.src[0].dtype;
    const int to = node.out.dtype;
    if (from == to) {
        switch (dtype_size(to)) {
            case 1: run<FCopy<uint8_t>>(ctx, node, {}); return;
            case 2: run<FCopy<uint16_t>>(ctx, node, {}); return;
            case 4: run<FCopy<uint32_t>>(ctx, node, {}); return;
            case 8: run<FCopy<uint64_t>>(ctx, node, {}); return;
        }
    }
    // the conversions vkML's CPU backend defines (kernels_movement.cpp:52-123)
    if (from == B200_F32 && to == B200_I32) return run<FCast<float, int32_t>>(ctx, node, {});
    if (from == B200_F32 && to == B200_I64) return run<FCast<float, int64_t>>(ctx, node, {});
    if (from == B200_F32 && to == B200_BOOL) return run<FCastF32Bool>(ctx, node, {});
    if (from == B200_F32 && to == B200_F16) return run<FCastF32F16>(ctx, node, {});
    if (from == B200_F16 && to == B200_F32) return run<FCastF16F32>(ctx, node, {});
    if (from == B200_I32 && to == B200_F32) return run<FCast<int32_t, float>>(ctx, node, {});
    if (from == B200_I32 && to == B200_I64) return run<FCast<int32_t, int64_t>>(ctx, node, {});
    if (from == B200_I64 && to == B200_F32) return run<FCast<int64_t, float>>(ctx, node, {});
    if (from == B200_I64 && to == B200_I32) return run<FCast<int64_t, int32_t>>(ctx, node, {});
    if (from == B200_BOOL && to == B200_F32) return run<FCastBool<float>>(ctx, node, {});
    if (from == B200_BOOL && to == B200_I64) return run<FCastBool<int64_t>>(ctx, node, {});
    fail(B200_DTYPE_ERROR, "cast: unsupported conversion");
}

void require_f32(const b200_node& node, const char* what) {
    if (node.out.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, std::string(what) + ": only f32 is implemented");
    }
}

// Every floating tensor of the node is F16 (and there is at least one).
bool all_half(const b200_node& node) {
    auto floating = [](int dt) { return dt == B200_F32 || dt == B200_F16; };
    bool any = false;
    if (floating(node.out.dtype)) {
        if (node.out.dtype != B200_F16) return false;
        any = true;
    }
    for (uint32_t s = 0; s < node.n_src && s < B200_MAX_SRC; ++s) {
        if (floating(node.src[s].dtype)) {
            if (node.src[s].dtype != B200_F16) return false;
            any = true;
        }
    }
    return any;
}

// The f32 functor F on f32 tensors, or on half storage through HalfIO.
template <typename F>
void run_float(b200_ctx* ctx, const b200_node& node, const typename F::P& p, const char* what) {
    if (all_half(node)) {
        run<HalfIO<F>>(ctx, node, p);
    } else {
        require_f32(node, what);
        run<F>(ctx, node, p);
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// Chains of tiny elementwise nodes: one block, one launch
// ---------------------------------------------------------------------------
// A loss prologue is a run of nodes of a few hundred elements each -- scalar fills, a division of
// scalars, broadcasts made contiguous, the labels cast to float, an arange, the one-hot comparison
// (src/api/ops.cpp:347-354,417-441) -- eleven launches that each cost more to start than to run.
// Here one block walks such a run node by node, in span order, with a block barrier between nodes
// (which also orders its own global writes before the next node's reads).  Every element goes
// through the functor the stand-alone kernel uses, so the values are the same bits.
namespace {

constexpr int kTinyNodes = 12;
constexpr int64_t kTinyElems = 4096;  // one block: beyond a few thousand elements a node is faster as its own launch
enum TinyKind : int {
    kTinyFull, kTinyArange, kTinyCopy4, kTinyCastI64, kTinyCastBool, kTinyNeg, kTinyAdd, kTinySub, kTinyMul, kTinyDiv, kTinyEqual
};

struct TinyNode {
    int kind;
    int numel;
    void* out;
    const void* src[2];
    int dim[kMaxDims];
    int stride[2][kMaxDims];  // elements
    float value;              // full
    double start, step;       // arange
};

struct TinyChain {
    int n;
    TinyNode node[kTinyNodes];
};

__global__ void __launch_bounds__(1024) tiny_chain_kernel(const __grid_constant__ TinyChain c) {
    pdl_prologue();
    const NoParams np{};
    for (int t = 0; t < c.n; ++t) {
        const TinyNode& nd = c.node[t];
        for (int i = threadIdx.x; i < nd.numel; i += blockDim.x) {
            int r = i, o0 = 0, o1 = 0;
#pragma unroll
            for (int a = kMaxDims - 1; a >= 0; --a) {
                const int q = r / nd.dim[a];
                const int idx = r - q * nd.dim[a];
                r = q;
                o0 += idx * nd.stride[0][a];
                o1 += idx * nd.stride[1][a];
            }
            const float* a32 = static_cast<const float*>(nd.src[0]);
            const float* b32 = static_cast<const float*>(nd.src[1]);
            float* out32 = static_cast<float*>(nd.out);
            switch (nd.kind) {
                case kTinyFull: out32[i] = nd.value; break;
                case kTinyArange: out32[i] = static_cast<float>(__dadd_rn(nd.start, __dmul_rn(static_cast<double>(i), nd.step))); break;
                case kTinyCopy4: static_cast<uint32_t*>(nd.out)[i] = static_cast<const uint32_t*>(nd.src[0])[o0]; break;
                case kTinyCastI64: out32[i] = FCast<int64_t, float>::apply(np, static_cast<const int64_t*>(nd.src[0])[o0], 0, 0); break;
                case kTinyCastBool: out32[i] = FCastBool<float>::apply(np, static_cast<const uint8_t*>(nd.src[0])[o0], 0, 0); break;
                case kTinyNeg: out32[i] = FNeg::apply(np, a32[o0], 0.0F, 0.0F); break;
                case kTinyAdd: out32[i] = FAdd::apply(np, a32[o0], b32[o1], 0.0F); break;
                case kTinySub: out32[i] = FSub::apply(np, a32[o0], b32[o1], 0.0F); break;
                case kTinyMul: out32[i] = FMul::apply(np, a32[o0], b32[o1], 0.0F); break;
                case kTinyDiv: out32[i] = FDiv::apply(np, a32[o0], b32[o1], 0.0F); break;
                case kTinyEqual: static_cast<uint8_t*>(nd.out)[i] = FEqual::apply(np, a32[o0], b32[o1], 0.0F); break;
                default: break;
            }
        }
        __syncthreads();
    }
}

// Fills `t` when the node is one the chain kernel serves as it stands.
bool tiny_node(const b200_node& node, TinyNode& t) {
    const View out = make_view(node.out);
    if (!out.contiguous || out.numel <= 0 || out.numel > kTinyElems || out.data == nullptr) return false;
    const int dt = out.dtype;
    int n_src = 0;
    int want[2] = {B200_F32, B200_F32};
    switch (node.op) {
        case B200_OP_FULL:
            if (dt != B200_F32) return false;
            t.kind = kTinyFull;
            t.value = static_cast<float>(get_params<FullParams>(node).value);
            break;
        case B200_OP_ARANGE: {
            if (dt != B200_F32) return false;
            const auto p = get_params<ArangeParams>(node);
            t.kind = kTinyArange;
            t.start = p.start;
            t.step = p.step;
            break;
        }
        case B200_OP_CONTIGUOUS:
            if (dtype_size(dt) != 4 || node.src[0].dtype != dt) return false;
            t.kind = kTinyCopy4;
            n_src = 1;
            want[0] = dt;
            break;
        case B200_OP_CAST:
            if (dt != B200_F32) return false;
            n_src = 1;
            if (node.src[0].dtype == B200_I64) { t.kind = kTinyCastI64; want[0] = B200_I64; }
            else if (node.src[0].dtype == B200_BOOL) { t.kind = kTinyCastBool; want[0] = B200_BOOL; }
            else return false;
            break;
        case B200_OP_NEG: t.kind = kTinyNeg; n_src = 1; if (dt != B200_F32) return false; break;
        case B200_OP_ADD: t.kind = kTinyAdd; n_src = 2; if (dt != B200_F32) return false; break;
        case B200_OP_SUB: t.kind = kTinySub; n_src = 2; if (dt != B200_F32) return false; break;
        case B200_OP_MUL: t.kind = kTinyMul; n_src = 2; if (dt != B200_F32) return false; break;
        case B200_OP_DIV: t.kind = kTinyDiv; n_src = 2; if (dt != B200_F32) return false; break;
        case B200_OP_EQUAL: t.kind = kTinyEqual; n_src = 2; if (dt != B200_BOOL) return false; break;
        default: return false;
    }
    if (static_cast<int>(node.n_src) < n_src) return false;
    t.numel = static_cast<int>(out.numel);
    t.out = out.data;
    t.src[0] = t.src[1] = nullptr;
    for (int a = 0; a < kMaxDims; ++a) {
        t.dim[a] = static_cast<int>(out.dim[a]);
        t.stride[0][a] = t.stride[1][a] = 0;
    }
    for (int s = 0; s < n_src; ++s) {
        if (node.src[s].dtype != want[s] || node.src[s].data == nullptr) return false;
        const View in = make_view(node.src[s]);
        for (int a = 0; a < kMaxDims; ++a) {
            if (in.dim[a] != out.dim[a]) return false;
            if (in.stride[a] < -(int64_t(1) << 30) || in.stride[a] > (int64_t(1) << 30)) return false;
            t.stride[s][a] = in.dim[a] > 1 ? static_cast<int>(in.stride[a]) : 0;
        }
        t.src[s] = in.data;
    }
    return true;
}

}  // namespace

// `seq`: consecutive nodes of a span.  Serves the leading run of tiny elementwise nodes (at least
// three of them) with one launch; returns how many it served.
size_t launch_tiny_chain(b200_ctx* ctx, const b200_node* const* seq, size_t avail) {
    TinyChain chain{};
    size_t n = 0;
    while (n < avail && n < static_cast<size_t>(kTinyNodes) && tiny_node(*seq[n], chain.node[n])) ++n;
    if (n < 3) return 0;
    chain.n = static_cast<int>(n);
    ProfScope scope(ctx, "fused.tiny_chain");
    launch_kernel(ctx, tiny_chain_kernel, 1u, 1024, 0, chain);
    ctx->count_launch();
    check_last_launch("chain of tiny elementwise nodes");
    return n;
}

void launch_elementwise(b200_ctx* ctx, const b200_node& node) {
    switch (node.op) {
        case B200_OP_FULL: run_full(ctx, node); return;
        case B200_OP_ARANGE: {
            const View out = make_view(node.out);
            const auto p = get_params<ArangeParams>(node);
            if (out.numel == 0) return;
            if (out.dtype == B200_F32) {
                launch_kernel(ctx, arange_kernel<float>, grid_for(out.numel, kThreads), kThreads, 0, reinterpret_cast<float*>(out.data), out.numel, p.start, p.step);
            } else if (out.dtype == B200_I64) {
                launch_kernel(ctx, arange_kernel<int64_t>, grid_for(out.numel, kThreads), kThreads, 0, reinterpret_cast<int64_t*>(out.data), out.numel, p.start, p.step);
            } else {
                fail(B200_DTYPE_ERROR, "arange: unsupported dtype");
            }
            ctx->count_launch();
            check_last_launch("arange");
            return;
        }
        case B200_OP_RAND: {
            require_f32(node, "rand");
            const View out = make_view(node.out);
            const auto p = get_params<RandParams>(node);
            if (out.numel == 0) return;
            launch_kernel(ctx, rand_kernel, grid_for(out.numel, kThreads), kThreads, 0, reinterpret_cast<float*>(out.data), out.numel, p.seed, p.offset);
            ctx->count_launch();
            check_last_launch("rand");
            return;
        }
        case B200_OP_CONTIGUOUS:
            if (node.src[0].dtype != node.out.dtype) {
                fail(B200_DTYPE_ERROR, "contiguous must not change dtype");
            }
            switch (dtype_size(node.out.dtype)) {
                case 1: run<FCopy<uint8_t>>(ctx, node, {}); return;
                case 2: run<FCopy<uint16_t>>(ctx, node, {}); return;
                case 4: run<FCopy<uint32_t>>(ctx, node, {}); return;
                case 8: run<FCopy<uint64_t>>(ctx, node, {}); return;
            }
            fail(B200_DTYPE_ERROR, "contiguous: unknown dtype");
        case B200_OP_CAST: run_cast(ctx, node); return;
        case B200_OP_TRIU:
        case B200_OP_TRIL: {
            require_f32(node, "triu/tril");
            const View out = make_view(node.out);
            const View in = make_view(node.src[0]);
            if (out.numel == 0) return;
            const auto p = get_params<TriParams>(node);
            launch_kernel(ctx, tri_kernel, grid_for(out.numel, kThreads), kThreads, 0, reinterpret_cast<float*>(out.data), reinterpret_cast<const float*>(in.data),
                geo_of(in), out.numel, out.dim[3], out.dim[2], p.diagonal,
                node.op == B200_OP_TRIU ? 1 : 0);
            ctx->count_launch();
            check_last_launch("tri");
            return;
        }
        case B200_OP_CAT: {
            const View out = make_view(node.out);
            const View a = make_view(node.src[0]);
            const View b = make_view(node.src[1]);
            if (out.numel == 0) return;
            const int axis = get_params<AxisParams>(node).axis + (kMaxDims - node.out.ndim);
            int64_t inner = 1;
            for (int i = axis + 1; i < kMaxDims; ++i) inner *= out.dim[i];
            const unsigned g = grid_for(out.numel, kThreads);
            if (dtype_size(out.dtype) == 4) {
                launch_kernel(ctx, cat_kernel<uint32_t>, g, kThreads, 0, reinterpret_cast<uint32_t*>(out.data), reinterpret_cast<const uint32_t*>(a.data),
                    reinterpret_cast<const uint32_t*>(b.data), geo_of(a), geo_of(b), out.numel, inner,
                    out.dim[axis], a.dim[axis], b.dim[axis]);
            } else {
                fail(B200_DTYPE_ERROR, "cat: only 4-byte dtypes are implemented");
            }
            ctx->count_launch();
            check_last_launch("cat");
            return;
        }
        case B200_OP_SLICE_BACKWARD: {
            require_f32(node, "slice_backward");
            const View out = make_view(node.out);
            const View g = make_view(node.src[0]);
            if (out.numel == 0) return;
            const auto p = get_params<SliceParams>(node);
            launch_kernel(ctx, slice_backward_kernel, grid_for(out.numel, kThreads), kThreads, 0, reinterpret_cast<float*>(out.data), reinterpret_cast<const float*>(g.data),
                geo_of(out), geo_of(g), out.numel, p.axis + (kMaxDims - node.out.ndim), p.start,
                p.step);
            ctx->count_launch();
            check_last_launch("slice_backward");
            return;
        }
        case B200_OP_WHERE: run_float<FWhere>(ctx, node, {}, "where"); return;
        case B200_OP_SCALED_ADD: run_float<FScaledAdd>(ctx, node, get_params<ScaledAddParams>(node), "scaled_add"); return;
        case B200_OP_CLAMP: run_float<FClamp>(ctx, node, get_params<ClampParams>(node), "clamp"); return;
        default: break;
    }

    if (node.op >= B200_OP_EQUAL && node.op <= B200_OP_NOT_EQUAL) {
        const bool half = node.src[0].dtype == B200_F16 && node.src[1].dtype == B200_F16;
        if (node.out.dtype != B200_BOOL || (!half && (node.src[0].dtype != B200_F32 || node.src[1].dtype != B200_F32))) {
            fail(B200_DTYPE_ERROR, "comparison: expects f32 (or f16) operands and a bool result");
        }
#define B200_COMPARE(F)                         \
    if (half) run<HalfIO<F>>(ctx, node, {});    \
    else run<F>(ctx, node, {});                 \
    return
        switch (node.op) {
            case B200_OP_EQUAL: B200_COMPARE(FEqual);
            case B200_OP_LESS: B200_COMPARE(FLess);
            case B200_OP_GREATER: B200_COMPARE(FGreater);
            case B200_OP_LESS_EQUAL: B200_COMPARE(FLessEqual);
            case B200_OP_GREATER_EQUAL: B200_COMPARE(FGreaterEqual);
            case B200_OP_NOT_EQUAL: B200_COMPARE(FNotEqual);
        }
#undef B200_COMPARE
    }

    switch (node.op) {
        case B200_OP_ADD: run_float<FAdd>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SUB: run_float<FSub>(ctx, node, {}, "elementwise"); return;
        case B200_OP_MUL: run_float<FMul>(ctx, node, {}, "elementwise"); return;
        case B200_OP_DIV: run_float<FDiv>(ctx, node, {}, "elementwise"); return;
        case B200_OP_POW: run_float<FPow>(ctx, node, {}, "elementwise"); return;
        case B200_OP_MAXIMUM: run_float<FMaximum>(ctx, node, {}, "elementwise"); return;
        case B200_OP_MINIMUM: run_float<FMinimum>(ctx, node, {}, "elementwise"); return;
        case B200_OP_NEG: run_float<FNeg>(ctx, node, {}, "elementwise"); return;
        case B200_OP_ABS: run_float<FAbs>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SIGN: run_float<FSign>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SQUARE: run_float<FSquare>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SQRT: run_float<FSqrt>(ctx, node, {}, "elementwise"); return;
        case B200_OP_RSQRT: run_float<FRsqrt>(ctx, node, {}, "elementwise"); return;
        case B200_OP_RECIPROCAL: run_float<FReciprocal>(ctx, node, {}, "elementwise"); return;
        case B200_OP_EXP: run_float<FExp>(ctx, node, {}, "elementwise"); return;
        case B200_OP_LOG: run_float<FLog>(ctx, node, {}, "elementwise"); return;
        case B200_OP_ERF: run_float<FErf>(ctx, node, {}, "elementwise"); return;
        case B200_OP_ERFC: run_float<FErfc>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SIN: run_float<FSin>(ctx, node, {}, "elementwise"); return;
        case B200_OP_COS: run_float<FCos>(ctx, node, {}, "elementwise"); return;
        case B200_OP_TANH: run_float<FTanh>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SIGMOID: run_float<FSigmoid>(ctx, node, {}, "elementwise"); return;
        case B200_OP_RELU: run_float<FRelu>(ctx, node, {}, "elementwise"); return;
        case B200_OP_GELU: run_float<FGelu>(ctx, node, {}, "elementwise"); return;
        case B200_OP_SILU: run_float<FSilu>(ctx, node, {}, "elementwise"); return;
        default: fail(B200_NOT_IMPLEMENTED, "elementwise: unhandled op");
    }
}

}  // namespace b200
