// Window and index movement ops: im2col, col2im, max_pool2d (+backward),
// index_select, scatter_add.
//
// Every kernel is one thread per OUTPUT element and accumulates in the same
// order as vkML's CPU backend (src/backend/cpu/kernels_movement.cpp), so
// results are bit-identical: col2im and max_pool2d_backward pull their window
// terms in (ki, kj) order (:501-542, :629-680); scatter_add folds the sources
// of one destination in ascending index position (:381-429); max_pool2d takes
// the first maximum under a strict compare (:557-580).  Inputs may be strided
// views; outputs are dense.
#include "context.h"

namespace b200 {
namespace {

constexpr int kThreads = 256;

struct Win {
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int64_t image_h, image_w, out_h, out_w, channels;
};

// window_of (kernels_movement.cpp:438-447)
Win make_win(const UnfoldParams& p, int64_t channels_times_patch) {
    auto span = [](int64_t extent, int k, int s, int pad, int d) {
        return (extent + 2LL * pad - (static_cast<int64_t>(d) * (k - 1) + 1)) / s + 1;
    };
    Win w;
    w.kh = p.kernel_h;
    w.kw = p.kernel_w;
    w.sh = p.stride_h;
    w.sw = p.stride_w;
    w.ph = p.pad_h;
    w.pw = p.pad_w;
    w.dh = p.dilation_h;
    w.dw = p.dilation_w;
    w.image_h = p.image_h;
    w.image_w = p.image_w;
    w.out_h = span(p.image_h, p.kernel_h, p.stride_h, p.pad_h, p.dilation_h);
    w.out_w = span(p.image_w, p.kernel_w, p.stride_w, p.pad_w, p.dilation_w);
    w.channels = channels_times_patch / (static_cast<int64_t>(p.kernel_h) * p.kernel_w);
    return w;
}

template <bool DENSE>
__device__ __forceinline__ float load_lin(const float* p, const Geo& g, int64_t linear) {
    return DENSE ? p[linear] : p[geo_offset(g, linear)];
}

// out[n, c*kh*kw + ki*kw + kj, oh*out_w + ow] = in[n, c, h, x] or 0 outside.
template <bool DENSE>
__global__ void __launch_bounds__(kThreads)
im2col_kernel(float* __restrict__ out, const float* __restrict__ in, Geo gin, Win w, int64_t rows,
              int64_t total) {
    const int64_t positions = w.out_h * w.out_w;
    const int64_t patch = int64_t(w.kh) * w.kw;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t pos = i % positions;
        const int64_t row = (i / positions) % rows;
        const int64_t n = i / (positions * rows);
        const int64_t c = row / patch;
        const int64_t ki = (row % patch) / w.kw;
        const int64_t kj = (row % patch) % w.kw;
        const int64_t oh = pos / w.out_w;
        const int64_t ow = pos % w.out_w;
        const int64_t h = oh * w.sh - w.ph + ki * w.dh;
        const int64_t x = ow * w.sw - w.pw + kj * w.dw;
        float v = 0.0F;
        if (h >= 0 && h < w.image_h && x >= 0 && x < w.image_w) {
            v = load_lin<DENSE>(in, gin, ((n * w.channels + c) * w.image_h + h) * w.image_w + x);
        }
        out[i] = v;
    }
}

template <bool DENSE>
__global__ void __launch_bounds__(kThreads)
col2im_kernel(float* __restrict__ out, const float* __restrict__ cols, Geo gcols, Win w,
              int64_t rows, int64_t total) {
    const int64_t positions = w.out_h * w.out_w;
    const int64_t patch = int64_t(w.kh) * w.kw;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t x = i % w.image_w;
        const int64_t h = (i / w.image_w) % w.image_h;
        const int64_t c = (i / (w.image_w * w.image_h)) % w.channels;
        const int64_t n = i / (w.image_w * w.image_h * w.channels);
        float acc = 0.0F;
        for (int ki = 0; ki < w.kh; ++ki) {
            const int64_t top = h + w.ph - int64_t(ki) * w.dh;
            if (top < 0 || top % w.sh != 0) {
                continue;
            }
            const int64_t oh = top / w.sh;
            if (oh >= w.out_h) {
                continue;
            }
            for (int kj = 0; kj < w.kw; ++kj) {
                const int64_t left = x + w.pw - int64_t(kj) * w.dw;
                if (left < 0 || left % w.sw != 0) {
                    continue;
                }
                const int64_t ow = left / w.sw;
                if (ow >= w.out_w) {
                    continue;
                }
                const int64_t row = c * patch + int64_t(ki) * w.kw + kj;
                acc += load_lin<DENSE>(cols, gcols, (n * rows + row) * positions + oh * w.out_w + ow);
            }
        }
        out[i] = acc;
    }
}

// First strict maximum of one window; -1 if nothing beat -inf.
template <bool DENSE>
__device__ __forceinline__ int argmax_in_window(const float* in, const Geo& gin, const Win& w,
                                                int64_t base, int64_t oh, int64_t ow, float& best) {
    best = -INFINITY;
    int best_offset = -1;
    for (int ki = 0; ki < w.kh; ++ki) {
        const int64_t h = oh * w.sh - w.ph + int64_t(ki) * w.dh;
        if (h < 0 || h >= w.image_h) {
            continue;
        }
        for (int kj = 0; kj < w.kw; ++kj) {
            const int64_t x = ow * w.sw - w.pw + int64_t(kj) * w.dw;
            if (x < 0 || x >= w.image_w) {
                continue;
            }
            const float v = load_lin<DENSE>(in, gin, base + h * w.image_w + x);
            if (v > best) {
                best = v;
                best_offset = ki * w.kw + kj;
            }
        }
    }
    return best_offset;
}

template <bool DENSE>
__global__ void __launch_bounds__(kThreads)
max_pool2d_kernel(float* __restrict__ out, const float* __restrict__ in, Geo gin, Win w,
                  int64_t out_h, int64_t out_w, int64_t total, uint32_t* status) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t ow = i % out_w;
        const int64_t oh = (i / out_w) % out_h;
        const int64_t plane = i / (out_w * out_h);
        float best;
        const int off = argmax_in_window<DENSE>(in, gin, w, plane * w.image_h * w.image_w, oh, ow, best);
        if (off < 0) {
            // the CPU backend asserts here: a window with no element above -inf
            atomicOr(status, kStatusInternal);
            best = __int_as_float(0x7fc00000);
        }
        out[i] = best;
    }
}

template <bool DENSE_IN, bool DENSE_G>
__global__ void __launch_bounds__(kThreads)
max_pool2d_backward_kernel(float* __restrict__ out, const float* __restrict__ grad,
                           const float* __restrict__ in, Geo ggrad, Geo gin, Win w, int64_t out_h,
                           int64_t out_w, int64_t total) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t x = i % w.image_w;
        const int64_t h = (i / w.image_w) % w.image_h;
        const int64_t plane = i / (w.image_w * w.image_h);
        const int64_t base = plane * w.image_h * w.image_w;
        float acc = 0.0F;
        for (int ki = 0; ki < w.kh; ++ki) {
            const int64_t top = h + w.ph - int64_t(ki) * w.dh;
            if (top < 0 || top % w.sh != 0) {
                continue;
            }
            const int64_t oh = top / w.sh;
            if (oh >= out_h) {
                continue;
            }
            for (int kj = 0; kj < w.kw; ++kj) {
                const int64_t left = x + w.pw - int64_t(kj) * w.dw;
                if (left < 0 || left % w.sw != 0) {
                    continue;
                }
                const int64_t ow = left / w.sw;
                if (ow >= out_w) {
                    continue;
                }
                float best;
                if (argmax_in_window<DENSE_IN>(in, gin, w, base, oh, ow, best) == ki * w.kw + kj) {
                    acc += load_lin<DENSE_G>(grad, ggrad, (plane * out_h + oh) * out_w + ow);
                }
            }
        }
        out[i] = acc;
    }
}

// out[outer, k, rest] = a[outer, idx[k], rest]  (kernels_movement.cpp:339-369).
// An out-of-range index is recorded in the status word and clamped; the host
// reports it as an index error at the next synchronize.
template <typename T>
__global__ void __launch_bounds__(kThreads)
index_select_kernel(T* __restrict__ out, const T* __restrict__ a, const int64_t* __restrict__ idx,
                    Geo ga, Geo gidx, int64_t inner, int64_t extent, int64_t a_extent, int64_t total,
                    uint32_t* status) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t rest = i % inner;
        const int64_t k = (i / inner) % extent;
        const int64_t outer = i / (inner * extent);
        int64_t j = idx[geo_offset(gidx, k)];
        if (j < 0 || j >= a_extent) {
            atomicOr(status, kStatusIndexOutOfRange);
            j = j < 0 ? 0 : a_extent - 1;
        }
        out[i] = a[geo_offset(ga, (outer * a_extent + j) * inner + rest)];
    }
}

// out[outer, j, rest] = sum over k with idx[k] == j of src[outer, k, rest], k ascending.
__global__ void __launch_bounds__(kThreads)
scatter_add_kernel(float* __restrict__ out, const float* __restrict__ src,
                   const int64_t* __restrict__ idx, Geo gsrc, Geo gidx, int64_t inner,
                   int64_t src_extent, int64_t out_extent, int64_t total, uint32_t* status) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t rest = i % inner;
        const int64_t j = (i / inner) % out_extent;
        const int64_t outer = i / (inner * out_extent);
        float acc = 0.0F;
        for (int64_t k = 0; k < src_extent; ++k) {
            const int64_t t = idx[geo_offset(gidx, k)];
            if (t == j) {
                acc += src[geo_offset(gsrc, (outer * src_extent + k) * inner + rest)];
            }
        }
        out[i] = acc;
    }
}

// Flags any index outside [0, extent): scatter_add's pull form would otherwise
// just never match it.
__global__ void __launch_bounds__(kThreads)
index_range_kernel(const int64_t* __restrict__ idx, Geo gidx, int64_t n, int64_t extent,
                   uint32_t* status) {
    const int64_t k = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (k < n) {
        const int64_t t = idx[geo_offset(gidx, k)];
        if (t < 0 || t >= extent) {
            atomicOr(status, kStatusIndexOutOfRange);
        }
    }
}

void require_f32(const View& v, const char* what) {
    if (v.dtype != B200_F32) {
        fail(B200_DTYPE_ERROR, std::string(what) + ": only f32 is implemented");
    }
}

void require_dense(const View& v, const char* what) {
    if (!v.contiguous) {
        fail(B200_NOT_IMPLEMENTED, std::string(what) + ": output must be contiguous");
    }
}

}  // namespace

void launch_movement(b200_ctx* ctx, const b200_node& node) {
    const View out = make_view(node.out);
    const int64_t total = out.numel;
    const unsigned grid = grid_for(total, kThreads);
    float* o = reinterpret_cast<float*>(out.data);

    switch (node.op) {
        case B200_OP_IM2COL: {
            const View in = make_view(node.src[0]);
            require_f32(out, "im2col");
            require_f32(in, "im2col");
            require_dense(out, "im2col");
            if (node.out.ndim != 3) fail(B200_SHAPE_ERROR, "im2col: output must be [N, C*kh*kw, L]");
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), node.out.dims[1]);
            if (w.out_h * w.out_w != node.out.dims[2] ||
                in.numel != node.out.dims[0] * w.channels * w.image_h * w.image_w) {
                fail(B200_SHAPE_ERROR, "im2col: geometry does not match the tensors");
            }
            const float* src = reinterpret_cast<const float*>(in.data);
            if (in.contiguous) {
                im2col_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(o, src, geo_of(in), w,
                                                                       node.out.dims[1], total);
            } else {
                im2col_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(o, src, geo_of(in), w,
                                                                        node.out.dims[1], total);
            }
            break;
        }
        case B200_OP_COL2IM: {
            const View cols = make_view(node.src[0]);
            require_f32(out, "col2im");
            require_f32(cols, "col2im");
            require_dense(out, "col2im");
            if (node.src[0].ndim != 3) fail(B200_SHAPE_ERROR, "col2im: input must be [N, C*kh*kw, L]");
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), node.src[0].dims[1]);
            if (w.out_h * w.out_w != node.src[0].dims[2] ||
                total != node.src[0].dims[0] * w.channels * w.image_h * w.image_w) {
                fail(B200_SHAPE_ERROR, "col2im: geometry does not match the tensors");
            }
            const float* src = reinterpret_cast<const float*>(cols.data);
            if (cols.contiguous) {
                col2im_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(o, src, geo_of(cols), w,
                                                                       node.src[0].dims[1], total);
            } else {
                col2im_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(o, src, geo_of(cols), w,
                                                                        node.src[0].dims[1], total);
            }
            break;
        }
        case B200_OP_MAX_POOL2D: {
            const View in = make_view(node.src[0]);
            require_f32(out, "max_pool2d");
            require_f32(in, "max_pool2d");
            require_dense(out, "max_pool2d");
            if (node.out.ndim != 4) fail(B200_SHAPE_ERROR, "max_pool2d: output must be rank 4");
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), 1);
            const float* src = reinterpret_cast<const float*>(in.data);
            if (in.contiguous) {
                max_pool2d_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(
                    o, src, geo_of(in), w, out.dim[2], out.dim[3], total, ctx->d_status);
            } else {
                max_pool2d_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(
                    o, src, geo_of(in), w, out.dim[2], out.dim[3], total, ctx->d_status);
            }
            break;
        }
        case B200_OP_MAX_POOL2D_BACKWARD: {
            const View grad = make_view(node.src[0]);
            const View in = make_view(node.src[1]);
            require_f32(out, "max_pool2d_backward");
            require_f32(in, "max_pool2d_backward");
            require_f32(grad, "max_pool2d_backward");
            require_dense(out, "max_pool2d_backward");
            if (node.out.ndim != 4 || node.src[0].ndim != 4) {
                fail(B200_SHAPE_ERROR, "max_pool2d_backward: tensors must be rank 4");
            }
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), 1);
            const float* g = reinterpret_cast<const float*>(grad.data);
            const float* src = reinterpret_cast<const float*>(in.data);
            if (in.contiguous && grad.contiguous) {
                max_pool2d_backward_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(
                    o, g, src, geo_of(grad), geo_of(in), w, grad.dim[2], grad.dim[3], total);
            } else {
                max_pool2d_backward_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(
                    o, g, src, geo_of(grad), geo_of(in), w, grad.dim[2], grad.dim[3], total);
            }
            break;
        }
        case B200_OP_INDEX_SELECT: {
            const View a = make_view(node.src[0]);
            const View idx = make_view(node.src[1]);
            require_dense(out, "index_select");
            if (idx.dtype != B200_I64) fail(B200_DTYPE_ERROR, "index_select: index must be i64");
            if (a.dtype != out.dtype) fail(B200_DTYPE_ERROR, "index_select must not change dtype");
            if (total == 0) return;
            const int axis = get_params<AxisParams>(node).axis + (kMaxDims - node.out.ndim);
            if (axis < 0 || axis >= kMaxDims) fail(B200_SHAPE_ERROR, "index_select: bad axis");
            int64_t inner = 1;
            for (int i = axis + 1; i < kMaxDims; ++i) inner *= out.dim[i];
            const auto* ip = reinterpret_cast<const int64_t*>(idx.data);
            if (dtype_size(out.dtype) == 4) {
                index_select_kernel<uint32_t><<<grid, kThreads, 0, ctx->stream>>>(
                    reinterpret_cast<uint32_t*>(out.data), reinterpret_cast<const uint32_t*>(a.data), ip,
                    geo_of(a), geo_of(idx), inner, out.dim[axis], a.dim[axis], total, ctx->d_status);
            } else if (dtype_size(out.dtype) == 8) {
                index_select_kernel<uint64_t><<<grid, kThreads, 0, ctx->stream>>>(
                    reinterpret_cast<uint64_t*>(out.data), reinterpret_cast<const uint64_t*>(a.data), ip,
                    geo_of(a), geo_of(idx), inner, out.dim[axis], a.dim[axis], total, ctx->d_status);
            } else {
                fail(B200_DTYPE_ERROR, "index_select: unsupported element width");
            }
            break;
        }
        case B200_OP_SCATTER_ADD: {
            const View src = make_view(node.src[0]);
            const View idx = make_view(node.src[1]);
            require_f32(out, "scatter_add");
            require_f32(src, "scatter_add");
            require_dense(out, "scatter_add");
            if (idx.dtype != B200_I64) fail(B200_DTYPE_ERROR, "scatter_add: index must be i64");
            if (total == 0) return;
            const int axis = get_params<AxisParams>(node).axis + (kMaxDims - node.out.ndim);
            if (axis < 0 || axis >= kMaxDims) fail(B200_SHAPE_ERROR, "scatter_add: bad axis");
            int64_t inner = 1;
            for (int i = axis + 1; i < kMaxDims; ++i) inner *= out.dim[i];
            const auto* ip = reinterpret_cast<const int64_t*>(idx.data);
            const int64_t n_idx = src.dim[axis];
            if (n_idx > 0 && src.numel > 0) {
                index_range_kernel<<<static_cast<unsigned>(ceil_div(n_idx, kThreads)), kThreads, 0,
                                     ctx->stream>>>(ip, geo_of(idx), n_idx, out.dim[axis],
                                                    ctx->d_status);
                ctx->count_launch();
            }
            scatter_add_kernel<<<grid, kThreads, 0, ctx->stream>>>(
                o, reinterpret_cast<const float*>(src.data), ip, geo_of(src), geo_of(idx), inner,
                src.numel == 0 ? 0 : n_idx, out.dim[axis], total, ctx->d_status);
            break;
        }
        default: fail(B200_NOT_IMPLEMENTED, "movement: unhandled op");
    }
    ctx->count_launch();
    check_last_launch("movement");
}

}  // namespace b200
