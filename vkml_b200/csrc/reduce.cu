// Reductions (sum, mean, max, min, argmax, argmin) and softmax / log_softmax.
//
// Semantics follow vkML's CPU backend (src/backend/cpu/kernels_reduce.cpp):
// an axis bitmask splits the input into kept and reduced axes
// (src/backend/cpu/reduce.cpp:11-30); max/min return NaN if any element is NaN
// (:128-158); argmax/argmin return the FIRST extremum under a strict compare,
// which ignores NaN (:160-192); mean is one sum and one divide, NaN when empty
// (:98-107).  Sums are folded in a fixed order (no atomics), so repeated runs
// are byte-identical; the order differs from the CPU's midpoint pairwise tree,
// which is why sums are compared under a backward-error bound, not bitwise.
//
// Three kernels, chosen from the strides:
//   group  -- a warp or a block per output walks the reduced index space with
//             consecutive lanes on consecutive reduced elements (rows, and the
//             [N,C,H,W]->[C] case where the kept axis sits in the middle).
//   thread -- one lane per output, lanes on consecutive outputs (column sums such
//             as [B,N]->[N], batch-axis sums, and very short rows).
//   Both split a long reduction across blocks into partials held in the
//   context's scratch buffer; the block that finishes last folds them in split
//   order inside the same launch.
#include "context.h"

#include <type_traits>

#include <cfloat>
#include <cmath>

namespace b200 {
namespace {

template <typename I>
struct RedGeoT {
    I kdim[kMaxDims], kstride[kMaxDims];  // kept axes (input strides), padded in front
    I rdim[kMaxDims], rstride[kMaxDims];  // reduced axes
    int krank, rrank;
    // multiply-high reciprocals of kdim / rdim, used by the 32-bit kernels (set_divisors)
    FastDiv kdiv[kMaxDims], rdiv[kMaxDims];
};

template <typename I>
void set_divisors(RedGeoT<I>& g) {
    for (int a = 0; a < kMaxDims; ++a) {
        g.kdiv[a] = FastDiv(static_cast<uint32_t>(g.kdim[a] > 0 ? g.kdim[a] : 1));
        g.rdiv[a] = FastDiv(static_cast<uint32_t>(g.rdim[a] > 0 ? g.rdim[a] : 1));
    }
}
using RedGeo = RedGeoT<int64_t>;

// Offset of the `linear`-th element of a row-major index space.  The outermost axis needs no
// division (what is left of `linear` is its index); 32-bit walks divide by multiply-high.
template <typename I>
__device__ __forceinline__ I walk(const I* dim, const I* stride, const FastDiv* div, int rank, I linear) {
    if (rank == 1) {
        return linear * stride[kMaxDims - 1];
    }
    I off = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        if (a > kMaxDims - rank) {
            I q;
            if constexpr (sizeof(I) == 4) {
                q = static_cast<I>(div[a].div(static_cast<uint32_t>(linear)));
            } else {
                q = linear / dim[a];
            }
            off += (linear - q * dim[a]) * stride[a];
            linear = q;
        } else if (a == kMaxDims - rank) {
            off += linear * stride[a];
        }
    }
    return off;
}

struct ArgAcc {
    float v;
    int64_t i;
};

// Product: the CPU backend multiplies in index order (kernels_reduce.cpp:118-126), and a product
// regrouped by a tree is a different answer, not a rounding difference (1e20 and 1e-20 alternating
// give 1 in order and inf once the large values are grouped) -- which is why vkML's own GPU
// backend declines it (vulkan_backend.cpp:1137-1154).  Here one thread per output walks the
// reduced axes in row-major order: sequential, bit-identical to the CPU, slow for long axes.
struct ProdP {
    using Acc = float;
    static constexpr bool kSequential = true;
    __device__ static Acc init() { return 1.0F; }
    __device__ static Acc step(Acc a, float v, int64_t) { return a * v; }
    __device__ static Acc merge(Acc a, Acc b) { return a * b; }
};
struct SumP {
    using Acc = float;
    __device__ static Acc init() { return 0.0F; }
    __device__ static Acc step(Acc a, float v, int64_t) { return a + v; }
    __device__ static Acc merge(Acc a, Acc b) { return a + b; }
};
struct MaxP {
    using Acc = float;
    __device__ static Acc init() { return -INFINITY; }
    __device__ static Acc step(Acc a, float v, int64_t) { return merge(a, v); }
    __device__ static Acc merge(Acc a, Acc b) {
        return (isnan(a) || isnan(b)) ? __int_as_float(0x7fc00000) : (b > a ? b : a);
    }
};
struct MinP {
    using Acc = float;
    __device__ static Acc init() { return INFINITY; }
    __device__ static Acc step(Acc a, float v, int64_t) { return merge(a, v); }
    __device__ static Acc merge(Acc a, Acc b) {
        return (isnan(a) || isnan(b)) ? __int_as_float(0x7fc00000) : (b < a ? b : a);
    }
};
// First index of the strict extremum. The identity (-inf, 0) reproduces the CPU
// loop's starting state, so an all -inf / all NaN run yields index 0.
struct ArgMaxP {
    using Acc = ArgAcc;
    __device__ static Acc init() { return {-INFINITY, 0}; }
    __device__ static Acc step(Acc a, float v, int64_t k) { return merge(a, Acc{v, k}); }
    __device__ static Acc merge(Acc a, Acc b) {
        if (b.v > a.v || (b.v == a.v && b.i < a.i)) {
            return b;
        }
        return a;
    }
};
struct ArgMinP {
    using Acc = ArgAcc;
    __device__ static Acc init() { return {INFINITY, 0}; }
    __device__ static Acc step(Acc a, float v, int64_t k) { return merge(a, Acc{v, k}); }
    __device__ static Acc merge(Acc a, Acc b) {
        if (b.v < a.v || (b.v == a.v && b.i < a.i)) {
            return b;
        }
        return a;
    }
};

__device__ __forceinline__ float shfl_down(float v, int d) {
    return __shfl_down_sync(0xffffffffU, v, d);
}
__device__ __forceinline__ ArgAcc shfl_down(ArgAcc v, int d) {
    ArgAcc r;
    r.v = __shfl_down_sync(0xffffffffU, v.v, d);
    r.i = __shfl_down_sync(0xffffffffU, v.i, d);
    return r;
}

template <typename P>
__device__ __forceinline__ typename P::Acc warp_fold(typename P::Acc a) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        a = P::merge(a, shfl_down(a, d));
    }
    return a;
}

// Result in thread 0 of the group. GROUP is 32 (a warp) or the whole block.
template <typename P, int GROUP>
__device__ __forceinline__ typename P::Acc group_fold(typename P::Acc a, typename P::Acc* smem) {
    a = warp_fold<P>(a);
    if constexpr (GROUP > 32) {
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;
        if (lane == 0) {
            smem[warp] = a;
        }
        __syncthreads();
        if (warp == 0) {
            a = lane < GROUP / 32 ? smem[lane] : P::init();
            a = warp_fold<P>(a);
        }
        __syncthreads();
    }
    return a;
}

enum Post { kPostNone = 0, kPostMean = 1 };

template <typename P>
__device__ __forceinline__ void write_result(void* out, int64_t o, typename P::Acc a, int post,
                                             int64_t n_red) {
    if constexpr (sizeof(typename P::Acc) == sizeof(float)) {
        float v = a;
        if (post == kPostMean) {
            v = n_red == 0 ? __int_as_float(0x7fc00000) : v / static_cast<float>(n_red);
        }
        static_cast<float*>(out)[o] = v;
    } else {
        static_cast<int64_t*>(out)[o] = a.i;
    }
}

constexpr int kMaxCounters = 4096;

// Splits of one output (or of one block of outputs) hand their partials to whichever
// block arrives LAST, which folds them in split order: one launch instead of two,
// and the order of the fold does not depend on which block that was.  The counter
// wraps back to zero on the last arrival (atomicInc with the split count as bound),
// so the counter array needs no clearing between launches.
__device__ __forceinline__ bool last_block_of(unsigned* counter, unsigned splits, int* flag_smem) {
    __threadfence();  // this block's partials are visible before the ticket is taken
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned ticket = atomicInc(counter, splits - 1);
        *flag_smem = ticket == splits - 1;
    }
    __syncthreads();
    const bool last = *flag_smem != 0;
    if (last) {
        __threadfence();  // and the other blocks' partials are visible to this one
    }
    return last;
}

// grid = (outputs / groups-per-block, splits). `partial` ([split][output]) non-null
// when splits > 1; then split s owns the units k with (k / (GROUP*U)) % splits == s, so
// the blocks of one launch sweep memory side by side instead of in distant chunks.
// With VEC4 the innermost reduced axis is a dense run whose length is a multiple of 4
// and every row start is 16-byte aligned: the reduced index space is walked in float4
// units (g.rdim / g.rstride of the innermost axis already divided / multiplied by 4).
template <typename P, int GROUP, bool VEC4, typename I, int U = 4>
__global__ void __launch_bounds__(256)
reduce_group_kernel(void* out, typename P::Acc* partial, unsigned* counters, const float* __restrict__ in,
                    RedGeoT<I> g, int64_t n_out, I n_units, int post, int64_t n_red) {
    pdl_prologue();
    __shared__ typename P::Acc smem[8];
    __shared__ int last_flag;
    constexpr int kGroups = 256 / GROUP;
    const int gid = threadIdx.x / GROUP;
    const int lane = threadIdx.x % GROUP;
    const int64_t o = int64_t(blockIdx.x) * kGroups + gid;
    const I split = blockIdx.y;
    const I splits = gridDim.y;
    typename P::Acc acc = P::init();
    const bool live = o < n_out;
    if (live) {
        const I base = walk<I>(g.kdim, g.kstride, g.kdiv, g.krank, static_cast<I>(o));
        // one accumulator per vector component: a thread that walks millions of elements (a mean over
        // 2^31 of them) then adds four chains a quarter as long, which keeps a float sum's rounding
        // error well inside the tolerance the CPU's pairwise sums set
        typename P::Acc acc4[4] = {P::init(), P::init(), P::init(), P::init()};
        for (int64_t kb64 = int64_t(split) * (GROUP * U) + lane; kb64 < int64_t(n_units);
             kb64 += int64_t(splits) * (GROUP * U)) {
            const I kb = static_cast<I>(kb64);
            if constexpr (VEC4) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const I k = kb + u * GROUP;
                    if (k < n_units) {
                        v[u] = *reinterpret_cast<const float4*>(in + base + walk<I>(g.rdim, g.rstride, g.rdiv, g.rrank, k));
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const I k = kb + u * GROUP;
                    if (k < n_units) {
                        // element index of v.x in reduced (row-major) order, for argmax / argmin
                        const int64_t e = int64_t(k) * 4;
                        acc4[0] = P::step(acc4[0], v[u].x, e);
                        acc4[1] = P::step(acc4[1], v[u].y, e + 1);
                        acc4[2] = P::step(acc4[2], v[u].z, e + 2);
                        acc4[3] = P::step(acc4[3], v[u].w, e + 3);
                    }
                }
            } else {
                float v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const I k = kb + u * GROUP;
                    if (k < n_units) {
                        v[u] = in[base + walk<I>(g.rdim, g.rstride, g.rdiv, g.rrank, k)];
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const I k = kb + u * GROUP;
                    if (k < n_units) {
                        acc = P::step(acc, v[u], int64_t(k));
                    }
                }
            }
        }
        if constexpr (VEC4) {
            acc = P::merge(P::merge(acc4[0], acc4[1]), P::merge(acc4[2], acc4[3]));
        }
    }
    acc = group_fold<P, GROUP>(acc, smem);
    if (partial == nullptr) {
        if (live && lane == 0) {
            write_result<P>(out, o, acc, post, n_red);
        }
        return;
    }
    // splits > 1 only with one output per block (GROUP == 256)
    if (live && lane == 0) {
        partial[int64_t(split) * n_out + o] = acc;
    }
    if (counters == nullptr || !last_block_of(counters + blockIdx.x, splits, &last_flag)) {
        return;
    }
    typename P::Acc total = P::init();
    for (I s = threadIdx.x; s < splits; s += 256) {
        total = P::merge(total, partial[int64_t(s) * n_out + o]);
    }
    total = group_fold<P, 256>(total, smem);
    if (threadIdx.x == 0) {
        write_result<P>(out, o, total, post, n_red);
    }
}

// One lane per (output, split); consecutive lanes own consecutive outputs, split s owns
// the reduced indices k with (k / U) % splits == s.
template <typename P, typename I>
__global__ void __launch_bounds__(256)
reduce_thread_kernel(void* out, typename P::Acc* partial, unsigned* counters, const float* __restrict__ in,
                     RedGeoT<I> g, int64_t n_out, I n_red, int post) {
    pdl_prologue();
    __shared__ int last_flag;
    constexpr int U = 4;
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const I split = blockIdx.y;
    const I splits = gridDim.y;
    const bool live = o < n_out;
    typename P::Acc acc = P::init();
    if (live) {
        const I base = walk<I>(g.kdim, g.kstride, g.kdiv, g.krank, static_cast<I>(o));
        for (int64_t kb64 = int64_t(split) * U; kb64 < int64_t(n_red); kb64 += int64_t(splits) * U) {
            const I kb = static_cast<I>(kb64);
            float v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    v[u] = in[base + walk<I>(g.rdim, g.rstride, g.rdiv, g.rrank, kb + u)];
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    acc = P::step(acc, v[u], int64_t(kb + u));
                }
            }
        }
    }
    if (partial == nullptr) {
        if (live) {
            write_result<P>(out, o, acc, post, int64_t(n_red));
        }
        return;
    }
    if (live) {
        partial[int64_t(split) * n_out + o] = acc;
    }
    if (counters == nullptr || !last_block_of(counters + blockIdx.x, splits, &last_flag)) {
        return;
    }
    if (live) {
        typename P::Acc total = P::init();
        for (I s0 = 0; s0 < splits; s0 += 8) {
            typename P::Acc q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    q[u] = partial[int64_t(s0 + u) * n_out + o];
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    total = P::merge(total, q[u]);
                }
            }
        }
        write_result<P>(out, o, total, post, int64_t(n_red));
    }
}

// Column sums with a dense kept axis: each lane owns FOUR adjacent outputs and reads one
// float4 per reduced index (float accumulators only: sum, mean, max, min).
template <typename P, typename I, int U = 8>
__global__ void __launch_bounds__(256)
reduce_thread4_kernel(float* out, float4* partial, unsigned* counters, const float* __restrict__ in,
                      RedGeoT<I> g, int64_t n_out4, I n_red, int post) {
    pdl_prologue();
    __shared__ int last_flag;
    const int64_t o4 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const I split = blockIdx.y;
    const I splits = gridDim.y;
    const bool live = o4 < n_out4;
    float acc[4] = {P::init(), P::init(), P::init(), P::init()};
    if (live) {
        const I base = walk<I>(g.kdim, g.kstride, g.kdiv, g.krank, static_cast<I>(o4));
        for (int64_t kb64 = int64_t(split) * U; kb64 < int64_t(n_red); kb64 += int64_t(splits) * U) {
            const I kb = static_cast<I>(kb64);
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    v[u] = *reinterpret_cast<const float4*>(in + base + walk<I>(g.rdim, g.rstride, g.rdiv, g.rrank, kb + u));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    acc[0] = P::step(acc[0], v[u].x, 0);
                    acc[1] = P::step(acc[1], v[u].y, 0);
                    acc[2] = P::step(acc[2], v[u].z, 0);
                    acc[3] = P::step(acc[3], v[u].w, 0);
                }
            }
        }
    }
    auto finish = [&](float v) {
        if (post == kPostMean) {
            return n_red == 0 ? __int_as_float(0x7fc00000) : v / static_cast<float>(n_red);
        }
        return v;
    };
    if (partial == nullptr) {
        if (live) {
            reinterpret_cast<float4*>(out)[o4] = make_float4(finish(acc[0]), finish(acc[1]), finish(acc[2]), finish(acc[3]));
        }
        return;
    }
    if (live) {
        partial[int64_t(split) * n_out4 + o4] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
    if (!last_block_of(counters + blockIdx.x, splits, &last_flag)) {
        return;
    }
    if (live) {
        // eight partial rows in flight at a time: they come from L2, and a loop that waits for one
        // load before it issues the next pays that latency per split.  The merges keep split order.
        float t[4] = {P::init(), P::init(), P::init(), P::init()};
        for (I s0 = 0; s0 < splits; s0 += 8) {
            float4 q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    q[u] = __ldcg(partial + int64_t(s0 + u) * n_out4 + o4);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    t[0] = P::merge(t[0], q[u].x);
                    t[1] = P::merge(t[1], q[u].y);
                    t[2] = P::merge(t[2], q[u].z);
                    t[3] = P::merge(t[3], q[u].w);
                }
            }
        }
        reinterpret_cast<float4*>(out)[o4] = make_float4(finish(t[0]), finish(t[1]), finish(t[2]), finish(t[3]));
    }
}

// Column sums with a dense kept axis, second form: a block is 64 output quads wide (1 KB of every
// row) and FOUR row-lanes deep.  Row-lane l of K-slice s takes the reduced indices
// (g * splits + s) * 32 + l * 8 + u, u < 8 -- eight vectors in flight per thread -- the four lanes
// meet in shared memory in lane order, and only then does the block hand a partial row to the
// last block of its column stripe.  Against one quad per thread and no row-lanes this needs a
// quarter of the K-slices for the same number of blocks: a quarter of the partial rows, and a
// fold that is two rounds of loads instead of five.
template <typename P, typename I>
__global__ void __launch_bounds__(256)
reduce_lanes4_kernel(float* out, float4* partial, unsigned* counters, const float* __restrict__ in,
                     RedGeoT<I> g, int64_t n_out4, I n_red, int post) {
    pdl_prologue();
    constexpr int U = 8;
    __shared__ float4 part[4][64];
    __shared__ int last_flag;
    const int q = threadIdx.x & 63;
    const int lane = threadIdx.x >> 6;
    const int64_t o4 = int64_t(blockIdx.x) * 64 + q;
    const I split = blockIdx.y;
    const I splits = gridDim.y;
    const bool live = o4 < n_out4;
    float acc[4] = {P::init(), P::init(), P::init(), P::init()};
    if (live) {
        const I base = walk<I>(g.kdim, g.kstride, g.kdiv, g.krank, static_cast<I>(o4));
        for (int64_t kb64 = int64_t(split) * (4 * U) + lane * U; kb64 < int64_t(n_red); kb64 += int64_t(splits) * (4 * U)) {
            const I kb = static_cast<I>(kb64);
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    v[u] = *reinterpret_cast<const float4*>(in + base + walk<I>(g.rdim, g.rstride, g.rdiv, g.rrank, kb + u));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < n_red) {
                    acc[0] = P::step(acc[0], v[u].x, 0);
                    acc[1] = P::step(acc[1], v[u].y, 0);
                    acc[2] = P::step(acc[2], v[u].z, 0);
                    acc[3] = P::step(acc[3], v[u].w, 0);
                }
            }
        }
    }
    part[lane][q] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    float t[4] = {P::init(), P::init(), P::init(), P::init()};
    if (lane == 0) {
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const float4 w = part[l][q];
            t[0] = P::merge(t[0], w.x);
            t[1] = P::merge(t[1], w.y);
            t[2] = P::merge(t[2], w.z);
            t[3] = P::merge(t[3], w.w);
        }
    }
    auto finish = [&](float v) {
        if (post == kPostMean) {
            return n_red == 0 ? __int_as_float(0x7fc00000) : v / static_cast<float>(n_red);
        }
        return v;
    };
    if (partial == nullptr) {
        if (lane == 0 && live) {
            reinterpret_cast<float4*>(out)[o4] = make_float4(finish(t[0]), finish(t[1]), finish(t[2]), finish(t[3]));
        }
        return;
    }
    if (lane == 0 && live) {
        partial[int64_t(split) * n_out4 + o4] = make_float4(t[0], t[1], t[2], t[3]);
    }
    if (!last_block_of(counters + blockIdx.x, splits, &last_flag)) {
        return;
    }
    if (lane == 0 && live) {
        float r[4] = {P::init(), P::init(), P::init(), P::init()};
        for (I s0 = 0; s0 < splits; s0 += 8) {
            float4 w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    w[u] = __ldcg(partial + int64_t(s0 + u) * n_out4 + o4);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (s0 + u < splits) {
                    r[0] = P::merge(r[0], w[u].x);
                    r[1] = P::merge(r[1], w[u].y);
                    r[2] = P::merge(r[2], w[u].z);
                    r[3] = P::merge(r[3], w[u].w);
                }
            }
        }
        reinterpret_cast<float4*>(out)[o4] = make_float4(finish(r[0]), finish(r[1]), finish(r[2]), finish(r[3]));
    }
}

// Fallback fold for launches with more blocks than counters. partial is [split][output].
template <typename P>
__global__ void __launch_bounds__(256)
reduce_finalize_kernel(void* out, const typename P::Acc* __restrict__ partial, int64_t n_out,
                       int splits, int post, int64_t n_red) {
    pdl_prologue();
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (o >= n_out) {
        return;
    }
    typename P::Acc acc = P::init();
    for (int s = 0; s < splits; ++s) {
        acc = P::merge(acc, partial[int64_t(s) * n_out + o]);
    }
    write_result<P>(out, o, acc, post, n_red);
}

// Pack an axis list (dims/strides) to the back of a rank-4 array, merging
// neighbours that form one run.
int pack_axes(const int64_t* d, const int64_t* s, int n, int64_t* dim, int64_t* stride) {
    int64_t td[kMaxDims], ts[kMaxDims];
    int r = 0;
    for (int i = 0; i < n; ++i) {
        if (d[i] == 1) {
            continue;
        }
        if (r > 0 && ts[r - 1] == s[i] * d[i]) {
            td[r - 1] *= d[i];
            ts[r - 1] = s[i];
        } else {
            td[r] = d[i];
            ts[r] = s[i];
            ++r;
        }
    }
    if (r == 0) {
        td[0] = 1;
        ts[0] = 0;
        r = 1;
    }
    for (int a = 0; a < kMaxDims; ++a) {
        dim[a] = 1;
        stride[a] = 0;
    }
    for (int i = 0; i < r; ++i) {
        dim[kMaxDims - r + i] = td[i];
        stride[kMaxDims - r + i] = ts[i];
    }
    return r;
}

template <typename I>
RedGeoT<I> narrow_geo(const RedGeo& g) {
    RedGeoT<I> r;
    r.krank = g.krank;
    r.rrank = g.rrank;
    for (int a = 0; a < kMaxDims; ++a) {
        r.kdim[a] = static_cast<I>(g.kdim[a]);
        r.kstride[a] = static_cast<I>(g.kstride[a]);
        r.rdim[a] = static_cast<I>(g.rdim[a]);
        r.rstride[a] = static_cast<I>(g.rstride[a]);
    }
    set_divisors(r);
    return r;
}

template <typename P, typename = void>
struct is_sequential : std::false_type {};
template <typename P>
struct is_sequential<P, std::void_t<decltype(P::kSequential)>> : std::bool_constant<P::kSequential> {};

template <typename P, typename I>
void launch_reduce_kernels(b200_ctx* ctx, const View& out, const float* src, const RedGeo& g64, int64_t n_out,
                           int64_t n_red, int post) {
    using Acc = typename P::Acc;
    RedGeoT<I> g = narrow_geo<I>(g64);
    if constexpr (is_sequential<P>::value) {
        // one thread per output, the reduced index space in order, no slices to regroup
        dim3 grid(static_cast<unsigned>(ceil_div(n_out, 256)), 1);
        launch_kernel(ctx, reduce_thread_kernel<P, I>, grid, 256, 0, out.data, static_cast<Acc*>(nullptr),
                      static_cast<unsigned*>(nullptr), src, g, n_out, static_cast<I>(n_red), post);
        ctx->count_launch();
        check_last_launch("reduce (sequential)");
        return;
    }
    const int64_t r_inner = g64.rstride[kMaxDims - 1];
    const int64_t k_inner = g64.kstride[kMaxDims - 1];
    const bool column = (n_red <= 16) || (k_inner == 1 && r_inner != 1 && n_out >= 32);

    if (column) {
        int64_t splits = 1;
        if (n_red >= 64) {
            splits = ceil_div(int64_t(sm_count()) * 2048, n_out);
            splits = std::min<int64_t>(splits, n_red / 16);
            splits = std::max<int64_t>(1, std::min<int64_t>(splits, 1024));
        }
        if constexpr (sizeof(Acc) == sizeof(float)) {
            // four adjacent outputs per lane when the kept axis is dense and everything is 16-byte aligned
            const int64_t k_run = g64.kdim[kMaxDims - 1];
            bool v4 = k_inner == 1 && k_run % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(out.data) % 16 == 0 && n_out >= 1024;
            for (int a = 0; a < kMaxDims && v4; ++a) {
                if (g64.rdim[a] > 1 && g64.rstride[a] % 4 != 0) v4 = false;
                if (a < kMaxDims - 1 && g64.kdim[a] > 1 && g64.kstride[a] % 4 != 0) v4 = false;
            }
            const int64_t n_out4 = n_out / 4;
            const int64_t bx = ceil_div(n_out4, 256);
            if (v4 && bx <= kMaxCounters) {
                int64_t sp = 1;
                if (n_red >= 64) {
                    // eight vectors per thread in flight, so half as many K-slices (and half the
                    // partial rows the last block has to fold) keep the memory system as busy
                    // (measured at 2048x8192: 17 us with 512, 20 with 1024, 24 with 2048 -- more slices
                    // only add partial rows and a longer fold)
                    sp = ceil_div(int64_t(sm_count()) * 512, n_out4);
                    sp = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(sp, n_red / 16), 1024));
                }
                RedGeoT<I> g4 = g;
                g4.kdim[kMaxDims - 1] = static_cast<I>(k_run / 4);
                set_divisors(g4);
                g4.kstride[kMaxDims - 1] = 4;
                const int64_t bx64 = ceil_div(n_out4, 64);
                if (n_red >= 128 && bx64 <= kMaxCounters) {
                    // three blocks per SM is what the kernel's registers allow: one full wave (measured at
                    // 2048 x 8192: 16.6 us with two per SM, 15.4 with three, 17.2 with four; 17.0 before)
                    int lanes_per_sm = 0;
                    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&lanes_per_sm, reduce_lanes4_kernel<P, I>, 256, 0) != cudaSuccess ||
                        lanes_per_sm < 1) {
                        cudaGetLastError();
                        lanes_per_sm = 3;
                    }
                    int64_t sl = int64_t(sm_count()) * lanes_per_sm / bx64;  // every block resident at once
                    sl = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(sl, n_red / 64), 256));
                    float4* part4 = nullptr;
                    if (sl > 1) {
                        part4 = static_cast<float4*>(ctx->ensure_workspace(sizeof(float4) * n_out4 * sl));
                    }
                    dim3 gridl(static_cast<unsigned>(bx64), static_cast<unsigned>(sl));
                    launch_kernel(ctx, reduce_lanes4_kernel<P, I>, gridl, 256, 0, reinterpret_cast<float*>(out.data), part4,
                                  ctx->d_counters, src, g4, n_out4, static_cast<I>(n_red), post);
                    ctx->count_launch();
                    check_last_launch("reduce (row lanes)");
                    return;
                }
                float4* part = nullptr;
                if (sp > 1) {
                    part = static_cast<float4*>(ctx->ensure_workspace(sizeof(float4) * n_out4 * sp));
                }
                dim3 grid4(static_cast<unsigned>(bx), static_cast<unsigned>(sp));
                launch_kernel(ctx, reduce_thread4_kernel<P, I>, grid4, 256, 0, reinterpret_cast<float*>(out.data), part, ctx->d_counters, src, g4, n_out4, static_cast<I>(n_red),
                    post);
                ctx->count_launch();
                check_last_launch("reduce (thread x4)");
                return;
            }
        }
        const int64_t blocks_x = ceil_div(n_out, 256);
        Acc* partial = nullptr;
        unsigned* counters = nullptr;
        if (splits > 1) {
            partial = static_cast<Acc*>(ctx->ensure_workspace(sizeof(Acc) * n_out * splits));
            counters = blocks_x <= kMaxCounters ? ctx->d_counters : nullptr;
        }
        dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(splits));
        launch_kernel(ctx, reduce_thread_kernel<P, I>, grid, 256, 0, out.data, partial, counters, src, g, n_out,
                                                                  static_cast<I>(n_red), post);
        ctx->count_launch();
        if (splits > 1 && counters == nullptr) {
            launch_kernel(ctx, reduce_finalize_kernel<P>, static_cast<unsigned>(blocks_x), 256, 0, out.data, partial, n_out, static_cast<int>(splits), post, n_red);
            ctx->count_launch();
        }
        check_last_launch("reduce (thread)");
        return;
    }

    // float4 walk: innermost reduced run dense, a multiple of 4 long, every start aligned
    const int64_t inner_run = g64.rdim[kMaxDims - 1];
    bool vec4 = r_inner == 1 && inner_run % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0;
    for (int a = 0; a < kMaxDims && vec4; ++a) {
        if (g64.kdim[a] > 1 && g64.kstride[a] % 4 != 0) vec4 = false;
        if (a < kMaxDims - 1 && g64.rdim[a] > 1 && g64.rstride[a] % 4 != 0) vec4 = false;
    }
    int64_t n_units = n_red;
    if (vec4) {
        g.rdim[kMaxDims - 1] = static_cast<I>(inner_run / 4);
        set_divisors(g);
        g.rstride[kMaxDims - 1] = 4;
        n_units = n_red / 4;
    }
    const bool warp = n_units <= 1024 && n_out >= 1024;
    const int64_t groups_per_block = warp ? 8 : 1;
    int64_t splits = 1;
    if (!warp && n_out < int64_t(sm_count()) * 8 && n_units >= 4096) {
        // as many K-slices as keep every block of the launch resident at once: a launch that
        // spills into a second, partial wave pays for it (64 outputs on 148 SMs with five
        // blocks each: 14.3 us with 11 slices = 704 blocks, 16.7 us with 12 = 768)
        int per_sm = 0;
        const cudaError_t occ = vec4
            ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reduce_group_kernel<P, 256, true, I, 8>, 256, 0)
            : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reduce_group_kernel<P, 256, false, I>, 256, 0);
        if (occ != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            per_sm = 4;
        }
        splits = std::max<int64_t>(1, int64_t(sm_count()) * per_sm / n_out);
        splits = std::min<int64_t>(splits, n_units / 2048);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 65535));
    }
    const int64_t blocks_x = ceil_div(n_out, groups_per_block);
    Acc* partial = nullptr;
    unsigned* counters = nullptr;
    if (splits > 1) {
        partial = static_cast<Acc*>(ctx->ensure_workspace(sizeof(Acc) * n_out * splits));
        counters = blocks_x <= kMaxCounters ? ctx->d_counters : nullptr;
    }
    dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(splits));
    const I nu = static_cast<I>(n_units);
    if (warp) {
        if (vec4) {
            launch_kernel(ctx, reduce_group_kernel<P, 32, true, I>, grid, 256, 0, out.data, partial, counters, src, g,
                                                                               n_out, nu, post, n_red);
        } else {
            launch_kernel(ctx, reduce_group_kernel<P, 32, false, I>, grid, 256, 0, out.data, partial, counters, src, g,
                                                                                n_out, nu, post, n_red);
        }
    } else {
        if (vec4 && splits > 1) {
            // short runs per block: all of a thread's loads at once
            launch_kernel(ctx, reduce_group_kernel<P, 256, true, I, 8>, grid, 256, 0, out.data, partial, counters, src, g,
                                                                                n_out, nu, post, n_red);
        } else if (vec4) {
            launch_kernel(ctx, reduce_group_kernel<P, 256, true, I>, grid, 256, 0, out.data, partial, counters, src, g,
                                                                                n_out, nu, post, n_red);
        } else {
            launch_kernel(ctx, reduce_group_kernel<P, 256, false, I>, grid, 256, 0, out.data, partial, counters, src,
                                                                                 g, n_out, nu, post, n_red);
        }
    }
    ctx->count_launch();
    if (splits > 1 && counters == nullptr) {
        launch_kernel(ctx, reduce_finalize_kernel<P>, static_cast<unsigned>(ceil_div(n_out, 256)), 256, 0, out.data, partial, n_out, static_cast<int>(splits), post, n_red);
        ctx->count_launch();
    }
    check_last_launch("reduce (group)");
}

template <typename P>
void run_reduce(b200_ctx* ctx, const View& out, const View& in, uint32_t mask4, int post) {
    int64_t kd[kMaxDims], ks[kMaxDims], rd[kMaxDims], rs[kMaxDims];
    int nk = 0, nr = 0;
    int64_t n_out = 1, n_red = 1;
    for (int a = 0; a < kMaxDims; ++a) {
        if (mask4 & (1U << a)) {
            rd[nr] = in.dim[a];
            rs[nr] = in.stride[a];
            n_red *= in.dim[a];
            ++nr;
        } else {
            kd[nk] = in.dim[a];
            ks[nk] = in.stride[a];
            n_out *= in.dim[a];
            ++nk;
        }
    }
    if (n_out != out.numel) {
        fail(B200_SHAPE_ERROR, "reduction output extent does not match the kept axes");
    }
    if (n_out == 0) {
        return;
    }
    RedGeo g{};
    g.krank = pack_axes(kd, ks, nk, g.kdim, g.kstride);
    g.rrank = pack_axes(rd, rs, nr, g.rdim, g.rstride);
    const float* src = reinterpret_cast<const float*>(in.data);
    if (fits32(in) && n_out < (int64_t(1) << 31) && n_red < (int64_t(1) << 31)) {
        launch_reduce_kernels<P, uint32_t>(ctx, out, src, g, n_out, n_red, post);
    } else {
        launch_reduce_kernels<P, int64_t>(ctx, out, src, g, n_out, n_red, post);
    }
}

// ---------------------------------------------------------------------------
// softmax / log_softmax along one axis (kernels_reduce.cpp:206-245):
// peak = max x; denom = sum exp(x - peak); y = exp(x - peak)/denom, or
// (x - peak) - log(denom).
// ---------------------------------------------------------------------------

struct SoftGeo {
    int64_t kdim[kMaxDims], kstride_in[kMaxDims], kstride_out[kMaxDims];
    int krank;
    int64_t n_axis, axis_stride_in, axis_stride_out;
};

__device__ __forceinline__ void soft_bases(const SoftGeo& g, int64_t row, int64_t& bi, int64_t& bo) {
    bi = 0;
    bo = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        if (a >= kMaxDims - g.krank) {
            const int64_t q = row / g.kdim[a];
            const int64_t idx = row - q * g.kdim[a];
            bi += idx * g.kstride_in[a];
            bo += idx * g.kstride_out[a];
            row = q;
        }
    }
}

// Short rows: one lane per row, the row re-read from L1.
template <bool LOG>
__global__ void __launch_bounds__(256)
softmax_thread_kernel(float* __restrict__ out, const float* __restrict__ in, SoftGeo g,
                      int64_t n_rows) {
    pdl_prologue();
    const int64_t row = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (row >= n_rows) {
        return;
    }
    int64_t bi, bo;
    soft_bases(g, row, bi, bo);
    float peak = -INFINITY;
    for (int64_t k = 0; k < g.n_axis; ++k) {
        peak = fmaxf(peak, in[bi + k * g.axis_stride_in]);
    }
    float denom = 0.0F;
    for (int64_t k = 0; k < g.n_axis; ++k) {
        denom += expf(in[bi + k * g.axis_stride_in] - peak);
    }
    const float lg = logf(denom);
    for (int64_t k = 0; k < g.n_axis; ++k) {
        const float shifted = in[bi + k * g.axis_stride_in] - peak;
        out[bo + k * g.axis_stride_out] = LOG ? shifted - lg : expf(shifted) / denom;
    }
}

__device__ __forceinline__ float block_all_max(float v, float* smem) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, d));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (nw == 1) {
        return v;
    }
    if (lane == 0) {
        smem[warp] = v;
    }
    __syncthreads();
    v = lane < nw ? smem[lane] : -INFINITY;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, d));
    }
    __syncthreads();
    return v;
}

__device__ __forceinline__ float block_all_sum(float v, float* smem) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        v += __shfl_xor_sync(0xffffffffU, v, d);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (nw == 1) {
        return v;
    }
    if (lane == 0) {
        smem[warp] = v;
    }
    __syncthreads();
    v = lane < nw ? smem[lane] : 0.0F;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        v += __shfl_xor_sync(0xffffffffU, v, d);
    }
    __syncthreads();
    return v;
}

// One block per row. The row is read from HBM once into shared memory when
// `staged` (dynamic shared memory = n_axis floats), so the op moves the
// algorithmic 8 bytes per element; otherwise passes 2 and 3 re-read it.
template <bool LOG>
__global__ void softmax_block_kernel(float* __restrict__ out, const float* __restrict__ in, SoftGeo g,
                                     int64_t n_rows, int staged, int vec4) {
    pdl_prologue();
    extern __shared__ float row_cache[];
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
        int64_t bi, bo;
        soft_bases(g, row, bi, bo);
        const float* x = in + bi;
        float* y = out + bo;
        const int64_t n = g.n_axis;
        const int64_t si = g.axis_stride_in, so = g.axis_stride_out;

        float peak = -INFINITY;
        if (vec4) {
            const float4* x4 = reinterpret_cast<const float4*>(x);
            for (int64_t k = threadIdx.x; k < n / 4; k += blockDim.x) {
                const float4 v = x4[k];
                if (staged) {
                    reinterpret_cast<float4*>(row_cache)[k] = v;
                }
                peak = fmaxf(fmaxf(peak, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
            }
        } else {
            for (int64_t k = threadIdx.x; k < n; k += blockDim.x) {
                const float v = x[k * si];
                if (staged) {
                    row_cache[k] = v;
                }
                peak = fmaxf(peak, v);
            }
        }
        peak = block_all_max(peak, red);  // also orders the row_cache writes

        float denom = 0.0F;
        for (int64_t k = threadIdx.x; k < n; k += blockDim.x) {
            const float v = staged ? row_cache[k] : x[k * si];
            denom += expf(v - peak);
        }
        denom = block_all_sum(denom, red);
        const float lg = logf(denom);

        if (vec4) {
            float4* y4 = reinterpret_cast<float4*>(y);
            for (int64_t k = threadIdx.x; k < n / 4; k += blockDim.x) {
                const float4 v = staged ? reinterpret_cast<const float4*>(row_cache)[k]
                                        : reinterpret_cast<const float4*>(x)[k];
                float4 r;
                const float a = v.x - peak, b = v.y - peak, c = v.z - peak, d = v.w - peak;
                r.x = LOG ? a - lg : expf(a) / denom;
                r.y = LOG ? b - lg : expf(b) / denom;
                r.z = LOG ? c - lg : expf(c) / denom;
                r.w = LOG ? d - lg : expf(d) / denom;
                y4[k] = r;
            }
        } else {
            for (int64_t k = threadIdx.x; k < n; k += blockDim.x) {
                const float shifted = (staged ? row_cache[k] : x[k * si]) - peak;
                y[k * so] = LOG ? shifted - lg : expf(shifted) / denom;
            }
        }
        __syncthreads();  // row_cache is reused by the next row
    }
}

// Rows that fit in registers: GROUP threads (a warp, or the whole block) own one row,
// each thread keeps ITEMS units (float4 when VEC4, else scalars read through the axis
// stride), so the row is read from memory exactly once and written once.
template <bool LOG, int GROUP, int ITEMS, bool VEC4>
__global__ void __launch_bounds__(GROUP == 32 ? 256 : GROUP)
softmax_reg_kernel(float* __restrict__ out, const float* __restrict__ in, SoftGeo g, int64_t n_rows) {
    pdl_prologue();
    constexpr int kBlock = GROUP == 32 ? 256 : GROUP;
    constexpr int kRows = kBlock / GROUP;
    constexpr int W = VEC4 ? 4 : 1;
    __shared__ float red[32];
    const int lane = threadIdx.x % GROUP;
    const int64_t n_units = VEC4 ? g.n_axis / 4 : g.n_axis;
    for (int64_t row0 = int64_t(blockIdx.x) * kRows; row0 < n_rows; row0 += int64_t(gridDim.x) * kRows) {
        const int64_t row = row0 + threadIdx.x / GROUP;
        const bool live = row < n_rows;
        int64_t bi = 0, bo = 0;
        if (live) {
            soft_bases(g, row, bi, bo);
        }
        float v[ITEMS * W];
        float peak = -INFINITY;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int64_t u = lane + int64_t(i) * GROUP;
            if (live && u < n_units) {
                if constexpr (VEC4) {
                    const float4 t = reinterpret_cast<const float4*>(in + bi)[u];
                    v[4 * i] = t.x;
                    v[4 * i + 1] = t.y;
                    v[4 * i + 2] = t.z;
                    v[4 * i + 3] = t.w;
                } else {
                    v[i] = in[bi + u * g.axis_stride_in];
                }
            } else {
#pragma unroll
                for (int w = 0; w < W; ++w) {
                    v[W * i + w] = -INFINITY;
                }
            }
#pragma unroll
            for (int w = 0; w < W; ++w) {
                peak = fmaxf(peak, v[W * i + w]);
            }
        }
        if constexpr (GROUP == 32) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                peak = fmaxf(peak, __shfl_xor_sync(0xffffffffU, peak, d));
            }
        } else {
            peak = block_all_max(peak, red);
        }
        // slots past the row hold -inf: exp(-inf - peak) = 0 adds nothing (a row of all
        // -inf gives NaN everywhere, as on the CPU)
        float denom = 0.0F;
#pragma unroll
        for (int i = 0; i < ITEMS * W; ++i) {
            const float e = expf(v[i] - peak);
            denom += e;
            if (!LOG) {
                v[i] = e;
            }
        }
        if constexpr (GROUP == 32) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                denom += __shfl_xor_sync(0xffffffffU, denom, d);
            }
        } else {
            denom = block_all_sum(denom, red);
        }
        const float lg = logf(denom);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int64_t u = lane + int64_t(i) * GROUP;
            if (live && u < n_units) {
                float r[W];
#pragma unroll
                for (int w = 0; w < W; ++w) {
                    r[w] = LOG ? (v[W * i + w] - peak) - lg : v[W * i + w] / denom;
                }
                if constexpr (VEC4) {
                    reinterpret_cast<float4*>(out + bo)[u] = make_float4(r[0], r[1], r[2], r[3]);
                } else {
                    out[bo + u * g.axis_stride_out] = r[0];
                }
            }
        }
    }
}

// Long dense rows (2049 .. 8192 float4 units), one 1024-thread block per SM, persistent over rows.
// The row in flight lives in registers, as in softmax_reg_kernel, but it arrives through shared
// memory: while a row is reduced, normalised and stored, the bulk-copy engine already fetches the
// block's next row (cp.async.bulk + mbarrier), so the SM's loads and stores overlap instead of
// alternating.  The wait is bounded: on expiry the kernel records kStatusWaitTimedOut and returns.
__device__ __forceinline__ uint32_t sm_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

template <bool LOG>
__global__ void __launch_bounds__(1024, 1)
softmax_bulk_kernel(float* __restrict__ out, const float* __restrict__ in, SoftGeo g, int64_t n_rows,
                    uint32_t* status) {
    pdl_prologue();
    constexpr int ITEMS = 8;
    extern __shared__ __align__(128) unsigned char row_buf[];
    __shared__ float red[32];
    __shared__ __align__(8) unsigned long long bar;
    const int tid = threadIdx.x;
    const int64_t n_units = g.n_axis / 4;
    const uint32_t row_bytes = static_cast<uint32_t>(g.n_axis) * 4u;
    const uint32_t sbar = sm_u32(&bar), sdst = sm_u32(row_buf);
    auto fetch = [&](int64_t row) {  // thread 0 only
        int64_t bi, bo;
        soft_bases(g, row, bi, bo);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sbar), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(sdst), "l"(reinterpret_cast<uint64_t>(in + bi)), "r"(row_bytes), "r"(sbar)
                     : "memory");
    };
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sbar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    int64_t row = blockIdx.x;
    if (tid == 0 && row < n_rows) {
        fetch(row);
    }
    uint32_t phase = 0;
    for (; row < n_rows; row += gridDim.x) {
        // bounded wait for the row (4 s on the global timer, consulted every 1024 polls)
        int ok = 1;
        {
            unsigned long long start = 0;
            uint32_t spins = 0;
            for (;;) {
                uint32_t done;
                asm volatile(
                    "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                    : "=r"(done)
                    : "r"(sbar), "r"(phase)
                    : "memory");
                if (done) break;
                if ((++spins & 0x3ff) == 0) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                    if (start == 0) {
                        start = now;
                    } else if (now - start > 4000000000ULL) {
                        ok = 0;
                        break;
                    }
                }
            }
        }
        phase ^= 1u;
        float v[ITEMS * 4];
        float peak = -INFINITY;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int64_t u = tid + int64_t(i) * 1024;
            if (ok && u < n_units) {
                const float4 t = reinterpret_cast<const float4*>(row_buf)[u];
                v[4 * i] = t.x;
                v[4 * i + 1] = t.y;
                v[4 * i + 2] = t.z;
                v[4 * i + 3] = t.w;
            } else {
#pragma unroll
                for (int w = 0; w < 4; ++w) v[4 * i + w] = -INFINITY;
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) peak = fmaxf(peak, v[4 * i + w]);
        }
        // every thread holds its part of the row: the buffer may take the next one
        if (!__syncthreads_and(ok)) {
            if (tid == 0) atomicOr(status, kStatusWaitTimedOut);
            return;
        }
        const int64_t next = row + gridDim.x;
        if (tid == 0 && next < n_rows) {
            // order the threads' generic-proxy reads of the buffer before the async-proxy refill
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fetch(next);
        }
        peak = block_all_max(peak, red);
        float denom = 0.0F;
#pragma unroll
        for (int i = 0; i < ITEMS * 4; ++i) {
            const float e = expf(v[i] - peak);
            denom += e;
            if (!LOG) {
                v[i] = e;
            }
        }
        denom = block_all_sum(denom, red);
        const float lg = logf(denom);
        int64_t bi, bo;
        soft_bases(g, row, bi, bo);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int64_t u = tid + int64_t(i) * 1024;
            if (u < n_units) {
                float r[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    r[w] = LOG ? (v[4 * i + w] - peak) - lg : v[4 * i + w] / denom;
                }
                reinterpret_cast<float4*>(out + bo)[u] = make_float4(r[0], r[1], r[2], r[3]);
            }
        }
    }
}

template <bool LOG>
void launch_softmax_bulk(b200_ctx* ctx, float* dst, const float* src, const SoftGeo& g, int64_t n_rows) {
    const size_t smem = static_cast<size_t>(g.n_axis) * sizeof(float);
    // the limit is a per-device attribute of the kernel and a process may hold several contexts:
    // set it at every launch (it is a cheap host-side call)
    B200_CUDA_CHECK(cudaFuncSetAttribute(softmax_bulk_kernel<LOG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         160 * 1024));
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(n_rows, sm_count()));
    launch_kernel(ctx, softmax_bulk_kernel<LOG>, grid, 1024, smem, dst, src, g, n_rows, ctx->d_status);
    ctx->count_launch();
    check_last_launch("softmax (bulk prefetch)");
}

template <bool LOG, int GROUP, int ITEMS, bool VEC4>
void launch_softmax_reg(b200_ctx* ctx, float* dst, const float* src, const SoftGeo& g, int64_t n_rows) {
    constexpr int kBlock = GROUP == 32 ? 256 : GROUP;
    constexpr int kRows = kBlock / GROUP;
    const int64_t blocks = ceil_div(n_rows, kRows);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(blocks, int64_t(sm_count()) * (2048 / kBlock) * 4));
    launch_kernel(ctx, softmax_reg_kernel<LOG, GROUP, ITEMS, VEC4>, grid, kBlock, 0, dst, src, g, n_rows);
    ctx->count_launch();
    check_last_launch("softmax (registers)");
}

template <bool LOG>
void run_softmax(b200_ctx* ctx, const View& out, const View& in, int axis4) {
    SoftGeo g{};
    int64_t kd[kMaxDims], ksi[kMaxDims], kso[kMaxDims];
    int nk = 0;
    int64_t n_rows = 1;
    for (int a = 0; a < kMaxDims; ++a) {
        if (a == axis4 || in.dim[a] == 1) {
            continue;
        }
        kd[nk] = in.dim[a];
        ksi[nk] = in.stride[a];
        kso[nk] = out.stride[a];
        n_rows *= in.dim[a];
        ++nk;
    }
    for (int a = 0; a < kMaxDims; ++a) {
        g.kdim[a] = 1;
        g.kstride_in[a] = 0;
        g.kstride_out[a] = 0;
    }
    for (int i = 0; i < nk; ++i) {
        g.kdim[kMaxDims - nk + i] = kd[i];
        g.kstride_in[kMaxDims - nk + i] = ksi[i];
        g.kstride_out[kMaxDims - nk + i] = kso[i];
    }
    g.krank = nk == 0 ? 1 : nk;
    g.n_axis = in.dim[axis4];
    g.axis_stride_in = in.stride[axis4];
    g.axis_stride_out = out.stride[axis4];
    if (out.numel == 0) {
        return;
    }
    const float* src = reinterpret_cast<const float*>(in.data);
    float* dst = reinterpret_cast<float*>(out.data);

    if (g.n_axis <= 32) {
        launch_kernel(ctx, softmax_thread_kernel<LOG>, static_cast<unsigned>(ceil_div(n_rows, 256)), 256, 0, dst, src, g, n_rows);
        ctx->count_launch();
        check_last_launch("softmax (thread)");
        return;
    }
    {
        bool v4 = g.axis_stride_in == 1 && g.axis_stride_out == 1 && g.n_axis % 4 == 0 &&
                  reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
        for (int a = 0; a < kMaxDims && v4; ++a) {
            if (g.kdim[a] > 1 && (g.kstride_in[a] % 4 != 0 || g.kstride_out[a] % 4 != 0)) {
                v4 = false;
            }
        }
        const int64_t n = g.n_axis;
        if (v4) {
            const int64_t u = n / 4;
            if (u <= 64) return launch_softmax_reg<LOG, 32, 2, true>(ctx, dst, src, g, n_rows);
            if (u <= 256) return launch_softmax_reg<LOG, 32, 8, true>(ctx, dst, src, g, n_rows);
            if (u <= 2048) return launch_softmax_reg<LOG, 256, 8, true>(ctx, dst, src, g, n_rows);
            // enough rows to keep every SM busy with more than one: prefetch the next row while
            // the current one is processed
            if (u <= 8192 && n_rows >= 2 * int64_t(sm_count())) return launch_softmax_bulk<LOG>(ctx, dst, src, g, n_rows);
            if (u <= 8192) return launch_softmax_reg<LOG, 1024, 8, true>(ctx, dst, src, g, n_rows);
        } else {
            if (n <= 256) return launch_softmax_reg<LOG, 32, 8, false>(ctx, dst, src, g, n_rows);
            if (n <= 1024) return launch_softmax_reg<LOG, 32, 32, false>(ctx, dst, src, g, n_rows);
            if (n <= 8192) return launch_softmax_reg<LOG, 256, 32, false>(ctx, dst, src, g, n_rows);
            if (n <= 32768) return launch_softmax_reg<LOG, 1024, 32, false>(ctx, dst, src, g, n_rows);
        }
    }
    // longer rows: staged in shared memory, or re-read when even that does not fit
    int threads = 128;
    if (g.n_axis > 512) threads = 256;
    if (g.n_axis > 4096) threads = 512;
    if (g.n_axis > 16384) threads = 1024;
    const size_t row_bytes = static_cast<size_t>(g.n_axis) * sizeof(float);
    const int staged = row_bytes <= 160 * 1024 ? 1 : 0;
    bool vec4 = g.axis_stride_in == 1 && g.axis_stride_out == 1 && g.n_axis % 4 == 0 &&
                reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
    for (int a = 0; a < kMaxDims && vec4; ++a) {
        if (g.kdim[a] > 1 && (g.kstride_in[a] % 4 != 0 || g.kstride_out[a] % 4 != 0)) {
            vec4 = false;
        }
    }
    const size_t smem = staged ? row_bytes : 0;
    if (smem > 48 * 1024) {
        // per device, so per launch (see launch_softmax_bulk)
        B200_CUDA_CHECK(cudaFuncSetAttribute(softmax_block_kernel<LOG>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    }
    // resident blocks per SM: limited by shared memory and by 2048 threads
    int per_sm = 2048 / threads;
    if (smem > 0) {
        per_sm = std::min<int>(per_sm, static_cast<int>((200 * 1024) / (smem + 1024)));
    }
    per_sm = std::max(per_sm, 1);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(n_rows, int64_t(sm_count()) * per_sm));
    launch_kernel(ctx, softmax_block_kernel<LOG>, grid, threads, smem, dst, src, g, n_rows, staged,
                                                                   vec4 ? 1 : 0);
    ctx->count_launch();
    check_last_launch("softmax (block)");
}

}  // namespace

void launch_reduce(b200_ctx* ctx, const b200_node& node) {
    const View out = make_view(node.out);
    const View in = make_view(node.src[0]);
    if (in.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, "reduce: only f32 input is implemented");
    }
    if (!out.contiguous) {
        fail(B200_NOT_IMPLEMENTED, "reduction output must be contiguous");
    }
    const auto p = get_params<ReduceParams>(node);
    const int nd = node.src[0].ndim;
    uint32_t mask = p.axes_mask != 0 ? p.axes_mask : (nd <= 0 ? 0U : (1U << nd) - 1U);
    const uint32_t mask4 = mask << (kMaxDims - nd);  // axes are padded in front
    const bool arg = node.op == B200_OP_ARGMAX || node.op == B200_OP_ARGMIN;
    if (arg ? out.dtype != B200_I64 : out.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, "reduce: unexpected output dtype");
    }
    switch (node.op) {
        case B200_OP_SUM: run_reduce<SumP>(ctx, out, in, mask4, kPostNone); return;
        case B200_OP_MEAN: run_reduce<SumP>(ctx, out, in, mask4, kPostMean); return;
        case B200_OP_MAX: run_reduce<MaxP>(ctx, out, in, mask4, kPostNone); return;
        case B200_OP_MIN: run_reduce<MinP>(ctx, out, in, mask4, kPostNone); return;
        case B200_OP_PROD: run_reduce<ProdP>(ctx, out, in, mask4, kPostNone); return;
        case B200_OP_ARGMAX: run_reduce<ArgMaxP>(ctx, out, in, mask4, kPostNone); return;
        case B200_OP_ARGMIN: run_reduce<ArgMinP>(ctx, out, in, mask4, kPostNone); return;
        default: fail(B200_NOT_IMPLEMENTED, "reduce: unhandled op");
    }
}

void launch_softmax(b200_ctx* ctx, const b200_node& node) {
    const View out = make_view(node.out);
    const View in = make_view(node.src[0]);
    if (in.dtype != B200_F32 || out.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, "softmax: only f32 is implemented");
    }
    const int axis = get_params<AxisParams>(node).axis;
    if (axis < 0 || axis >= node.src[0].ndim) {
        fail(B200_SHAPE_ERROR, "softmax: axis out of range");
    }
    const int axis4 = axis + (kMaxDims - node.src[0].ndim);
    if (node.op == B200_OP_LOG_SOFTMAX) {
        run_softmax<true>(ctx, out, in, axis4);
    } else {
        run_softmax<false>(ctx, out, in, axis4);
    }
}

}  // namespace b200

// ---------------------------------------------------------------------------
// Column sum that allocates nothing (b200_sum_columns_f32_noalloc).
//
// For callers that must not touch the device allocator at all: code running inside a
// latency-critical loop or a host callback, a process whose memory budget was fixed at
// start-up, a plug-in that was handed a stream and buffers but no permission to call
// cudaMalloc.  It is the split column reduction used for bias gradients
// (reduce_thread_kernel + last-block fold), with the partial sums and arrival counters
// kept in a fixed array that is part of the library image instead of the context's
// growable scratch buffer.
//
// The array costs its full size on every GPU the library is loaded on, until the process
// exits.  Every call uses the same array and it keeps what the previous call left there:
// the counters are cleared at the start of each call (stream-ordered), the partial planes
// are fully written before they are read.  Two calls that run on the GPU at the same time
// (different streams, or different host threads on different streams) would share it and
// corrupt each other: callers serialise them.
// ---------------------------------------------------------------------------

namespace b200 {
namespace {

constexpr size_t kNoAllocCounterBytes = size_t(kMaxCounters) * sizeof(unsigned);  // 16 KiB
constexpr size_t kNoAllocPartialBytes = size_t(B200_NOALLOC_MAX_COLUMNS) * sizeof(float);  // 4 MiB
constexpr size_t kNoAllocScratchBytes = kNoAllocCounterBytes + kNoAllocPartialBytes;

// Inside device code this name is the array; inside host code it is only a handle the
// runtime can look up -- never an address a kernel may be given.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device, looked up once per device.
int noalloc_scratch(void** out, std::string& why) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        why = "cannot identify the current CUDA device";
        return B200_DEVICE_ERROR;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            why = std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(err);
            return B200_DEVICE_ERROR;
        }
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return B200_OK;
}

void put_error(char* error, size_t error_len, const std::string& msg) {
    if (error != nullptr && error_len > 0) {
        std::snprintf(error, error_len, "%s", msg.c_str());
    }
}

template <typename I>
void launch_noalloc(const float* in, float* out, int64_t rows, int64_t cols, int64_t pitch, int64_t splits,
                    float* partial, unsigned* counters, cudaStream_t stream) {
    RedGeoT<I> g{};
    for (int a = 0; a < kMaxDims; ++a) {
        g.kdim[a] = g.rdim[a] = 1;
        g.kstride[a] = g.rstride[a] = 0;
    }
    g.krank = g.rrank = 1;
    g.kdim[kMaxDims - 1] = static_cast<I>(cols);
    g.kstride[kMaxDims - 1] = 1;
    g.rdim[kMaxDims - 1] = static_cast<I>(rows);
    g.rstride[kMaxDims - 1] = static_cast<I>(pitch);
    set_divisors(g);
    dim3 grid(static_cast<unsigned>(ceil_div(cols, 256)), static_cast<unsigned>(splits));
    reduce_thread_kernel<SumP, I><<<grid, 256, 0, stream>>>(out, splits > 1 ? partial : nullptr,
                                                             splits > 1 ? counters : nullptr, in, g, cols,
                                                             static_cast<I>(rows), kPostNone);
}

}  // namespace
}  // namespace b200

extern "C" int b200_sum_columns_f32_noalloc(const float* in, int64_t rows, int64_t cols, int64_t row_pitch,
                                            float* out, void* stream, char* error, size_t error_len) {
    using namespace b200;
    if (error != nullptr && error_len > 0) {
        error[0] = '\0';
    }
    if (rows < 0 || cols < 0 || row_pitch < 0 || (cols > 0 && out == nullptr) ||
        (rows > 0 && cols > 0 && in == nullptr)) {
        put_error(error, error_len, "b200_sum_columns_f32_noalloc: null pointer or negative extent");
        return B200_INVALID_ARGUMENT;
    }
    if (cols > B200_NOALLOC_MAX_COLUMNS) {
        put_error(error, error_len,
                  "b200_sum_columns_f32_noalloc: " + std::to_string(cols) + " columns exceed the fixed scratch array (" +
                      std::to_string(B200_NOALLOC_MAX_COLUMNS) + " columns); use b200_compute with a sum node instead");
        return B200_INVALID_ARGUMENT;
    }
    if (rows > 1 && row_pitch < cols) {
        put_error(error, error_len, "b200_sum_columns_f32_noalloc: row_pitch is smaller than the row length");
        return B200_INVALID_ARGUMENT;
    }
    if (cols == 0) {
        return B200_OK;
    }
    void* scratch = nullptr;
    std::string why;
    const int rc = noalloc_scratch(&scratch, why);
    if (rc != B200_OK) {
        put_error(error, error_len, "b200_sum_columns_f32_noalloc: " + why);
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned* counters = static_cast<unsigned*>(scratch);
    float* partial = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kNoAllocCounterBytes);

    // as many splits as fill the machine, as few as fit the partial planes
    int64_t splits = 1;
    if (rows >= 64) {
        splits = ceil_div(int64_t(sm_count()) * 2048, cols);
        splits = std::min<int64_t>(splits, rows / 16);
        splits = std::min<int64_t>(splits, B200_NOALLOC_MAX_COLUMNS / cols);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 1024));
    }
    if (splits > 1) {
        // the arrival counters must start at zero whatever an earlier call left behind
        const cudaError_t err = cudaMemsetAsync(counters, 0, kNoAllocCounterBytes, s);
        if (err != cudaSuccess) {
            cudaGetLastError();
            put_error(error, error_len, std::string("b200_sum_columns_f32_noalloc: ") + cudaGetErrorString(err));
            return B200_DEVICE_ERROR;
        }
    }
    const bool small = rows < (int64_t(1) << 31) && cols < (int64_t(1) << 31) &&
                       (rows == 0 ? 0 : (rows - 1) * row_pitch + cols) < (int64_t(1) << 31);
    if (small) {
        launch_noalloc<uint32_t>(in, out, rows, cols, row_pitch, splits, partial, counters, s);
    } else {
        launch_noalloc<int64_t>(in, out, rows, cols, row_pitch, splits, partial, counters, s);
    }
    const cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        cudaGetLastError();
        put_error(error, error_len, std::string("b200_sum_columns_f32_noalloc: launch failed: ") + cudaGetErrorString(err));
        return B200_DEVICE_ERROR;
    }
    return B200_OK;
}
