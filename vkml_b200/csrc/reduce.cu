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
//   context's scratch buffer; `finalize` folds the partials in split order.
#include "context.h"

#include <cfloat>
#include <cmath>

namespace b200 {
namespace {

struct RedGeo {
    int64_t kdim[kMaxDims], kstride[kMaxDims];  // kept axes (input strides), padded in front
    int64_t rdim[kMaxDims], rstride[kMaxDims];  // reduced axes
    int krank, rrank;
};

__device__ __forceinline__ int64_t walk(const int64_t* dim, const int64_t* stride, int rank,
                                        int64_t linear) {
    if (rank == 1) {
        return linear * stride[kMaxDims - 1];
    }
    int64_t off = 0;
#pragma unroll
    for (int a = kMaxDims - 1; a >= 0; --a) {
        if (a >= kMaxDims - rank) {
            const int64_t q = linear / dim[a];
            off += (linear - q * dim[a]) * stride[a];
            linear = q;
        }
    }
    return off;
}

struct ArgAcc {
    float v;
    int64_t i;
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

// grid = (outputs / groups-per-block, splits). `partial` non-null when splits > 1.
template <typename P, int GROUP, bool VEC4>
__global__ void __launch_bounds__(256)
reduce_group_kernel(void* out, typename P::Acc* partial, const float* __restrict__ in, RedGeo g,
                    int64_t n_out, int64_t n_red, int64_t chunk, int post) {
    __shared__ typename P::Acc smem[8];
    constexpr int kGroups = 256 / GROUP;
    const int gid = threadIdx.x / GROUP;
    const int lane = threadIdx.x % GROUP;
    const int64_t o = int64_t(blockIdx.x) * kGroups + gid;
    const int64_t split = blockIdx.y;
    typename P::Acc acc = P::init();
    const bool live = o < n_out;
    if (live) {
        const int64_t base = walk(g.kdim, g.kstride, g.krank, o);
        const int64_t k0 = split * chunk;
        const int64_t k1 = min(k0 + chunk, n_red);
        if constexpr (VEC4) {
            // reduced run is dense and 16-byte aligned; chunk is a multiple of 4
            const float4* p = reinterpret_cast<const float4*>(in + base);
            for (int64_t k = k0 / 4 + lane; k < k1 / 4; k += GROUP) {
                const float4 v = p[k];
                acc = P::step(acc, v.x, 4 * k);
                acc = P::step(acc, v.y, 4 * k + 1);
                acc = P::step(acc, v.z, 4 * k + 2);
                acc = P::step(acc, v.w, 4 * k + 3);
            }
        } else {
            for (int64_t k = k0 + lane; k < k1; k += GROUP) {
                acc = P::step(acc, in[base + walk(g.rdim, g.rstride, g.rrank, k)], k);
            }
        }
    }
    acc = group_fold<P, GROUP>(acc, smem);
    if (live && lane == 0) {
        if (partial != nullptr) {
            partial[o * gridDim.y + split] = acc;
        } else {
            write_result<P>(out, o, acc, post, n_red);
        }
    }
}

// One lane per (output, split); consecutive lanes own consecutive outputs.
template <typename P>
__global__ void __launch_bounds__(256)
reduce_thread_kernel(void* out, typename P::Acc* partial, const float* __restrict__ in, RedGeo g,
                     int64_t n_out, int64_t n_red, int64_t chunk, int post) {
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t split = blockIdx.y;
    if (o >= n_out) {
        return;
    }
    const int64_t base = walk(g.kdim, g.kstride, g.krank, o);
    const int64_t k0 = split * chunk;
    const int64_t k1 = min(k0 + chunk, n_red);
    typename P::Acc acc = P::init();
    if (g.rrank == 1) {
        const int64_t s = g.rstride[kMaxDims - 1];
        const float* p = in + base + k0 * s;
        for (int64_t k = k0; k < k1; ++k, p += s) {
            acc = P::step(acc, *p, k);
        }
    } else {
        for (int64_t k = k0; k < k1; ++k) {
            acc = P::step(acc, in[base + walk(g.rdim, g.rstride, g.rrank, k)], k);
        }
    }
    if (partial != nullptr) {
        partial[o * gridDim.y + split] = acc;
    } else {
        write_result<P>(out, o, acc, post, n_red);
    }
}

template <typename P>
__global__ void __launch_bounds__(256)
reduce_finalize_kernel(void* out, const typename P::Acc* __restrict__ partial, int64_t n_out,
                       int splits, int post, int64_t n_red) {
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (o >= n_out) {
        return;
    }
    typename P::Acc acc = P::init();
    for (int s = 0; s < splits; ++s) {
        acc = P::merge(acc, partial[o * splits + s]);
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
    using Acc = typename P::Acc;

    const int64_t r_inner = g.rstride[kMaxDims - 1];
    const int64_t k_inner = g.kstride[kMaxDims - 1];
    const bool column = (n_red <= 16) || (k_inner == 1 && r_inner != 1 && n_out >= 32);

    if (column) {
        int64_t splits = 1;
        if (n_red >= 64) {
            splits = ceil_div(int64_t(kSmCount) * 1024, n_out);
            splits = std::min<int64_t>(splits, n_red / 32);
            splits = std::max<int64_t>(1, std::min<int64_t>(splits, 1024));
        }
        const int64_t chunk = ceil_div(n_red, splits);
        splits = n_red == 0 ? 1 : ceil_div(n_red, chunk);
        Acc* partial = nullptr;
        if (splits > 1) {
            partial = static_cast<Acc*>(ctx->ensure_workspace(sizeof(Acc) * n_out * splits));
        }
        dim3 grid(static_cast<unsigned>(ceil_div(n_out, 256)), static_cast<unsigned>(splits));
        reduce_thread_kernel<P><<<grid, 256, 0, ctx->stream>>>(out.data, partial, src, g, n_out, n_red,
                                                             chunk, post);
        ctx->count_launch();
        if (splits > 1) {
            reduce_finalize_kernel<P><<<static_cast<unsigned>(ceil_div(n_out, 256)), 256, 0,
                                        ctx->stream>>>(out.data, partial, n_out,
                                                       static_cast<int>(splits), post, n_red);
            ctx->count_launch();
        }
        check_last_launch("reduce (thread)");
        return;
    }

    const bool warp = n_red <= 1024 && n_out >= 1024;
    const int64_t groups_per_block = warp ? 8 : 1;
    int64_t splits = 1;
    if (!warp) {
        const int64_t blocks = n_out;
        if (blocks < int64_t(kSmCount) * 4 && n_red >= 16384) {
            splits = ceil_div(int64_t(kSmCount) * 4, blocks);
            splits = std::min<int64_t>(splits, n_red / 8192);
            splits = std::max<int64_t>(1, std::min<int64_t>(splits, 65535));
        }
    }
    int64_t chunk = ceil_div(n_red, splits);
    chunk = ceil_div(chunk, 4) * 4;
    splits = n_red == 0 ? 1 : ceil_div(n_red, chunk);
    Acc* partial = nullptr;
    if (splits > 1) {
        partial = static_cast<Acc*>(ctx->ensure_workspace(sizeof(Acc) * n_out * splits));
    }
    // dense, aligned rows take the 128-bit path
    bool vec4 = g.rrank == 1 && r_inner == 1 && n_red % 4 == 0 &&
                reinterpret_cast<uintptr_t>(src) % 16 == 0;
    for (int a = 0; a < kMaxDims && vec4; ++a) {
        if (g.kdim[a] > 1 && g.kstride[a] % 4 != 0) {
            vec4 = false;
        }
    }
    dim3 grid(static_cast<unsigned>(ceil_div(n_out, groups_per_block)), static_cast<unsigned>(splits));
    if (warp) {
        if (vec4) {
            reduce_group_kernel<P, 32, true><<<grid, 256, 0, ctx->stream>>>(out.data, partial, src, g,
                                                                            n_out, n_red, chunk, post);
        } else {
            reduce_group_kernel<P, 32, false><<<grid, 256, 0, ctx->stream>>>(
                out.data, partial, src, g, n_out, n_red, chunk, post);
        }
    } else {
        if (vec4) {
            reduce_group_kernel<P, 256, true><<<grid, 256, 0, ctx->stream>>>(
                out.data, partial, src, g, n_out, n_red, chunk, post);
        } else {
            reduce_group_kernel<P, 256, false><<<grid, 256, 0, ctx->stream>>>(
                out.data, partial, src, g, n_out, n_red, chunk, post);
        }
    }
    ctx->count_launch();
    if (splits > 1) {
        reduce_finalize_kernel<P><<<static_cast<unsigned>(ceil_div(n_out, 256)), 256, 0, ctx->stream>>>(
            out.data, partial, n_out, static_cast<int>(splits), post, n_red);
        ctx->count_launch();
    }
    check_last_launch("reduce (group)");
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
        softmax_thread_kernel<LOG><<<static_cast<unsigned>(ceil_div(n_rows, 256)), 256, 0,
                                     ctx->stream>>>(dst, src, g, n_rows);
        ctx->count_launch();
        check_last_launch("softmax (thread)");
        return;
    }
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
        static bool raised[2] = {false, false};
        if (!raised[LOG ? 1 : 0]) {
            B200_CUDA_CHECK(cudaFuncSetAttribute(softmax_block_kernel<LOG>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 160 * 1024));
            raised[LOG ? 1 : 0] = true;
        }
    }
    // resident blocks per SM: limited by shared memory and by 2048 threads
    int per_sm = 2048 / threads;
    if (smem > 0) {
        per_sm = std::min<int>(per_sm, static_cast<int>((200 * 1024) / (smem + 1024)));
    }
    per_sm = std::max(per_sm, 1);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(n_rows, int64_t(kSmCount) * per_sm));
    softmax_block_kernel<LOG><<<grid, threads, smem, ctx->stream>>>(dst, src, g, n_rows, staged,
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
