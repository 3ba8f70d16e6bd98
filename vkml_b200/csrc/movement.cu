// Window and index movement ops: im2col, col2im, max_pool2d (+backward),
// index_select, scatter_add.
//
// Every kernel is one thread per OUTPUT element (or per pooling window) and
// accumulates in the same order as vkML's CPU backend
// (src/backend/cpu/kernels_movement.cpp), so results are bit-identical: col2im and
// max_pool2d_backward pull their window terms in (ki, kj) order (:501-542,
// :629-680); scatter_add folds the sources of one destination in ascending index
// position (:381-429); max_pool2d takes the first maximum under a strict compare
// (:557-580).  Inputs may be strided views; outputs are dense.
//
// These ops move 8-40 bytes per element, so index arithmetic decides the speed:
// the block owns one (image, row) or one plane, the per-thread work is one 32-bit
// divide, and the unit-stride / non-overlapping-window cases are compiled without
// any divide by the window stride.  Tensors too large for 32-bit indices take the
// generic 64-bit kernels.
#include "context.h"

namespace b200 {
namespace {

constexpr int kThreads = 256;

struct Win {
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int image_h, image_w, out_h, out_w;
    int64_t channels;
};

// window_of (kernels_movement.cpp:438-447)
Win make_win(const UnfoldParams& p, int64_t channels_times_patch) {
    auto span = [](int64_t extent, int k, int s, int pad, int d) {
        return (extent + 2LL * pad - (static_cast<int64_t>(d) * (k - 1) + 1)) / s + 1;
    };
    if (p.kernel_h <= 0 || p.kernel_w <= 0 || p.stride_h <= 0 || p.stride_w <= 0 || p.dilation_h <= 0 ||
        p.dilation_w <= 0 || p.image_h < 0 || p.image_w < 0) {
        fail(B200_SHAPE_ERROR, "window geometry must be positive");
    }
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
    w.out_h = static_cast<int>(span(p.image_h, p.kernel_h, p.stride_h, p.pad_h, p.dilation_h));
    w.out_w = static_cast<int>(span(p.image_w, p.kernel_w, p.stride_w, p.pad_w, p.dilation_w));
    w.channels = channels_times_patch / (static_cast<int64_t>(p.kernel_h) * p.kernel_w);
    return w;
}

// Element strides of a rank-4 [N, C, H, W] (or [N, R, L] padded) view.
struct Strides4 {
    int64_t s[4];
};

Strides4 strides_of(const View& v) {
    Strides4 r;
    for (int i = 0; i < 4; ++i) r.s[i] = v.stride[i];
    return r;
}

// ---------------------------------------------------------------------------
// im2col: out[n, c*kh*kw + ki*kw + kj, oh*out_w + ow] = in[n, c, h, x] or 0 outside.
// One block per (n, c, chunk of positions) writes all kh*kw rows of that channel:
// the rows re-read the same input plane, so it is fetched from HBM once.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
im2col_kernel(float* __restrict__ out, const float* __restrict__ in, Strides4 is, Win w, int positions,
              int chunks) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned nc = b / chunks;  // n * channels + c
    const unsigned c = nc % static_cast<unsigned>(w.channels);
    const unsigned n = nc / static_cast<unsigned>(w.channels);
    const int pos = chunk * blockDim.x + threadIdx.x;
    if (pos >= positions) {
        return;
    }
    const int oh = pos / w.out_w;
    const int ow = pos - oh * w.out_w;
    const float* plane = in + int64_t(n) * is.s[0] + int64_t(c) * is.s[1];
    float* dst = out + int64_t(nc) * (w.kh * w.kw) * positions + pos;
    const int h0 = oh * w.sh - w.ph;
    const int x0 = ow * w.sw - w.pw;
    for (int ki = 0; ki < w.kh; ++ki) {
        const int h = h0 + ki * w.dh;
        const bool row_ok = h >= 0 && h < w.image_h;
        for (int kj = 0; kj < w.kw; ++kj) {
            const int x = x0 + kj * w.dw;
            float v = 0.0F;
            if (row_ok && x >= 0 && x < w.image_w) {
                v = plane[int64_t(h) * is.s[2] + int64_t(x) * is.s[3]];
            }
            dst[int64_t(ki * w.kw + kj) * positions] = v;
        }
    }
}

// ---------------------------------------------------------------------------
// col2im: pull form, one thread per image element, one block per chunk of a plane.
// UNIT: stride 1 and dilation 1 in both directions (no divide by the stride);
// KH, KW > 0: window extents known at compile time, taps fully unrolled.
// ---------------------------------------------------------------------------
template <bool UNIT, int KH, int KW>
__global__ void __launch_bounds__(kThreads)
col2im_kernel(float* __restrict__ out, const float* __restrict__ cols, Strides4 cs, Win w, int chunks) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned plane = b / chunks;  // n * channels + c
    const unsigned c = plane % static_cast<unsigned>(w.channels);
    const unsigned n = plane / static_cast<unsigned>(w.channels);
    const int hw = chunk * blockDim.x + threadIdx.x;
    if (hw >= w.image_h * w.image_w) {
        return;
    }
    const int h = hw / w.image_w;
    const int x = hw - h * w.image_w;
    const int kh = KH > 0 ? KH : w.kh;
    const int kw = KW > 0 ? KW : w.kw;
    const float* base = cols + int64_t(n) * cs.s[1] + int64_t(c) * (kh * kw) * cs.s[2];
    float acc = 0.0F;
#pragma unroll
    for (int ki = 0; ki < kh; ++ki) {
        const int top = h + w.ph - (UNIT ? ki : ki * w.dh);
        int oh = top;
        bool ok_h = top >= 0;
        if (!UNIT) {
            ok_h = ok_h && top % w.sh == 0;
            oh = top / w.sh;
        }
        ok_h = ok_h && oh < w.out_h;
#pragma unroll
        for (int kj = 0; kj < kw; ++kj) {
            const int left = x + w.pw - (UNIT ? kj : kj * w.dw);
            int ow = left;
            bool ok = ok_h && left >= 0;
            if (!UNIT) {
                ok = ok && left % w.sw == 0;
                ow = left / w.sw;
            }
            ok = ok && ow < w.out_w;
            if (ok) {
                acc += base[int64_t(ki * kw + kj) * cs.s[2] + int64_t(oh * w.out_w + ow) * cs.s[3]];
            }
        }
    }
    out[int64_t(plane) * (w.image_h * w.image_w) + hw] = acc;
}

// ---------------------------------------------------------------------------
// Dense fast paths of the convolution pipeline: contiguous [N,C,H,W] images and
// [N, C*kh*kw, L] columns, unit stride and dilation, output rows a multiple of four wide.
// A block owns `group` consecutive (n, c) planes, stages them in shared memory with
// 128-bit loads and writes 128-bit vectors; all index arithmetic is 32-bit with
// multiply-high divisions.  Same values in the same order as the generic kernels.
// ---------------------------------------------------------------------------
struct DenseGeo {
    int h, w, ph, pw, oh, ow, kh, kw;
    int padded_w, padded_plane;  // im2col: (w + 2 pw), (h + 2 ph) * padded_w
    int group, planes;
    int vec_in;                  // the staged source can be read as 128-bit vectors
};

template <int KH, int KW>
__global__ void __launch_bounds__(kThreads)
im2col_dense_kernel(float* __restrict__ out, const float* __restrict__ in, DenseGeo g, FastDiv div_w4,
                    FastDiv div_w, FastDiv div_h, FastDiv div_l4, FastDiv div_ow) {
    pdl_prologue();
    extern __shared__ __align__(16) float tile[];  // group x (h + 2 ph) x (w + 2 pw), zero border
    const int kh = KH > 0 ? KH : g.kh, kw = KW > 0 ? KW : g.kw;
    const int first = blockIdx.x * g.group;
    const int count = min(g.group, g.planes - first);
    const int plane = g.h * g.w;
    for (int i = threadIdx.x; i < count * g.padded_plane; i += kThreads) {
        tile[i] = 0.0F;
    }
    __syncthreads();
    const float* src = in + int64_t(first) * plane;
    if (g.vec_in) {
        const int n4 = count * plane / 4;
        for (int i = threadIdx.x; i < n4; i += kThreads) {
            const float4 v = reinterpret_cast<const float4*>(src)[i];
            uint32_t row, x4, pl, h;
            div_w4.divmod(static_cast<uint32_t>(i), row, x4);  // row counts across the group's planes
            div_h.divmod(row, pl, h);
            float* d = tile + pl * g.padded_plane + (h + g.ph) * g.padded_w + g.pw + 4 * x4;
            d[0] = v.x;
            d[1] = v.y;
            d[2] = v.z;
            d[3] = v.w;
        }
    } else {
        for (int i = threadIdx.x; i < count * plane; i += kThreads) {
            uint32_t row, x, pl, h;
            div_w.divmod(static_cast<uint32_t>(i), row, x);
            div_h.divmod(row, pl, h);
            tile[pl * g.padded_plane + (h + g.ph) * g.padded_w + g.pw + x] = src[i];
        }
    }
    __syncthreads();
    const int l = g.oh * g.ow;
    const int l4 = l / 4;
    float* dst = out + int64_t(first) * (kh * kw) * l;
    for (int i = threadIdx.x; i < count * l4; i += kThreads) {
        uint32_t pl, p4, oh, ow;
        div_l4.divmod(static_cast<uint32_t>(i), pl, p4);
        div_ow.divmod(4 * p4, oh, ow);
        // tap (ki, kj) of output position (oh, ow) is padded-plane element (oh + ki, ow + kj)
        const float* sp = tile + pl * g.padded_plane + oh * g.padded_w + ow;
        float* o = dst + pl * (kh * kw) * l + 4 * p4;
#pragma unroll
        for (int ki = 0; ki < kh; ++ki) {
#pragma unroll
            for (int kj = 0; kj < kw; ++kj) {
                const float* t = sp + ki * g.padded_w + kj;
                *reinterpret_cast<float4*>(o + (ki * kw + kj) * l) = make_float4(t[0], t[1], t[2], t[3]);
            }
        }
    }
}

template <int KH, int KW>
__global__ void __launch_bounds__(kThreads)
col2im_dense_kernel(float* __restrict__ out, const float* __restrict__ cols, DenseGeo g, FastDiv div_hw4,
                    FastDiv div_w) {
    pdl_prologue();
    extern __shared__ __align__(16) float tile[];  // group x (kh kw) x L: this block's slice of the columns
    const int kh = KH > 0 ? KH : g.kh, kw = KW > 0 ? KW : g.kw;
    const int kk = kh * kw;
    const int l = g.oh * g.ow;
    const int first = blockIdx.x * g.group;
    const int count = min(g.group, g.planes - first);
    const float4* src = reinterpret_cast<const float4*>(cols + int64_t(first) * kk * l);
    const int n4 = count * kk * l / 4;
    for (int i = threadIdx.x; i < n4; i += kThreads) {
        reinterpret_cast<float4*>(tile)[i] = src[i];
    }
    __syncthreads();
    const int hw = g.h * g.w;
    const int hw4 = hw / 4;
    float* dst = out + int64_t(first) * hw;
    for (int i = threadIdx.x; i < count * hw4; i += kThreads) {
        uint32_t pl, p4, h, x;
        div_hw4.divmod(static_cast<uint32_t>(i), pl, p4);
        div_w.divmod(4 * p4, h, x);
        const float* t = tile + pl * kk * l;
        float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
        // (ki, kj) order, as the pull loop of the CPU backend.  A tap outside the column
        // image adds +0.0, which leaves a sum that started at +0.0 unchanged bit for bit.
#pragma unroll
        for (int ki = 0; ki < kh; ++ki) {
            const int oh = static_cast<int>(h) + g.ph - ki;
            const bool ok_h = oh >= 0 && oh < g.oh;
#pragma unroll
            for (int kj = 0; kj < kw; ++kj) {
                const int ow0 = static_cast<int>(x) + g.pw - kj;
                const float* r = t + (ki * kw + kj) * l + oh * g.ow + ow0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const bool ok = ok_h && ow0 + e >= 0 && ow0 + e < g.ow;
                    float v = 0.0F;
                    if (ok) {
                        v = r[e];
                    }
                    acc[e] += v;
                }
            }
        }
        *reinterpret_cast<float4*>(dst + pl * hw + 4 * p4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
}

// The 3x3, padding 1 case (every convolution of the CNN benchmark): same staging, but the four
// outputs of a thread read each tap plane as one aligned 128-bit vector plus, for the two shifted
// taps, one neighbouring word, and the image-edge tests collapse to three conditions per thread
// (first column, last column, row in range).  Same sum order: (ki, kj) ascending, +0.0 for taps
// outside the column image.
__global__ void __launch_bounds__(kThreads)
col2im_dense_3x3p1_kernel(float* __restrict__ out, const float* __restrict__ cols, DenseGeo g, FastDiv div_hw4,
                          FastDiv div_w) {
    pdl_prologue();
    extern __shared__ __align__(16) float tile[];  // group x 9 x L
    const int l = g.oh * g.ow;                     // == h * w here
    const int first = blockIdx.x * g.group;
    const int count = min(g.group, g.planes - first);
    const float4* src = reinterpret_cast<const float4*>(cols + int64_t(first) * 9 * l);
    const int n4 = count * 9 * l / 4;
    for (int i = threadIdx.x; i < n4; i += kThreads) {
        reinterpret_cast<float4*>(tile)[i] = src[i];
    }
    __syncthreads();
    const int hw = g.h * g.w;
    const int hw4 = hw / 4;
    float* dst = out + int64_t(first) * hw;
    for (int i = threadIdx.x; i < count * hw4; i += kThreads) {
        uint32_t pl, p4, h, x;
        div_hw4.divmod(static_cast<uint32_t>(i), pl, p4);
        div_w.divmod(4 * p4, h, x);
        const float* t = tile + pl * 9 * l;
        const bool has_left = x > 0;                                   // column x - 1 exists
        const bool has_right = static_cast<int>(x) + 4 < g.ow;         // column x + 4 exists
        float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
        for (int ki = 0; ki < 3; ++ki) {
            const int oh = static_cast<int>(h) + 1 - ki;
            const bool ok_h = oh >= 0 && oh < g.oh;
            const float* row = t + (ki * 3) * l + oh * g.ow + static_cast<int>(x);  // tap (ki, 0), column x
            float4 a = make_float4(0.0F, 0.0F, 0.0F, 0.0F), b = a, c = a;
            float a_next = 0.0F, c_prev = 0.0F;
            if (ok_h) {
                a = *reinterpret_cast<const float4*>(row);           // kj = 0 reads columns x+1 .. x+4
                b = *reinterpret_cast<const float4*>(row + l);       // kj = 1 reads columns x   .. x+3
                c = *reinterpret_cast<const float4*>(row + 2 * l);   // kj = 2 reads columns x-1 .. x+2
                if (has_right) a_next = row[4];
                if (has_left) c_prev = row[2 * l - 1];
            }
            // kj = 0
            acc[0] += a.y;
            acc[1] += a.z;
            acc[2] += a.w;
            acc[3] += a_next;
            // kj = 1
            acc[0] += b.x;
            acc[1] += b.y;
            acc[2] += b.z;
            acc[3] += b.w;
            // kj = 2
            acc[0] += c_prev;
            acc[1] += c.x;
            acc[2] += c.y;
            acc[3] += c.z;
        }
        *reinterpret_cast<float4*>(dst + pl * hw + 4 * p4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
}

// 2x2 pooling with stride 2 over dense planes whose width is a multiple of eight: one thread
// per four windows, rows read as two 128-bit vectors, first strict maximum in (ki, kj) order.
__global__ void __launch_bounds__(kThreads)
max_pool2d_dense2_kernel(float* __restrict__ out, const float* __restrict__ in, int h, int w, int out_h,
                         uint32_t items, FastDiv div_ow4, FastDiv div_oh, uint32_t* status) {
    pdl_prologue();
    const uint32_t step = gridDim.x * kThreads;
    const int out_w = w / 2;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < items; i += step) {
        uint32_t prow, ow4, plane, oh;
        div_ow4.divmod(i, prow, ow4);   // prow = plane * out_h + oh
        div_oh.divmod(prow, plane, oh);
        const float* top = in + (int64_t(plane) * h + 2 * oh) * w + 8 * ow4;
        float v[2][8];
#pragma unroll
        for (int ki = 0; ki < 2; ++ki) {
            const float4 lo = *reinterpret_cast<const float4*>(top + ki * w);
            const float4 hi = *reinterpret_cast<const float4*>(top + ki * w + 4);
            v[ki][0] = lo.x; v[ki][1] = lo.y; v[ki][2] = lo.z; v[ki][3] = lo.w;
            v[ki][4] = hi.x; v[ki][5] = hi.y; v[ki][6] = hi.z; v[ki][7] = hi.w;
        }
        float best[4];
        bool missing = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float m = -INFINITY;
            bool any = false;
#pragma unroll
            for (int ki = 0; ki < 2; ++ki) {
#pragma unroll
                for (int kj = 0; kj < 2; ++kj) {
                    if (v[ki][2 * j + kj] > m) {
                        m = v[ki][2 * j + kj];
                        any = true;
                    }
                }
            }
            if (!any) {
                missing = true;  // the CPU backend asserts here: no element above -inf
                m = __int_as_float(0x7fc00000);
            }
            best[j] = m;
        }
        if (missing) {
            atomicOr(status, kStatusInternal);
        }
        *reinterpret_cast<float4*>(out + int64_t(prow) * out_w + 4 * ow4) =
            make_float4(best[0], best[1], best[2], best[3]);
    }
}

// Its adjoint under the same conditions (image exactly 2 out_h x 2 out_w): the thread that
// owns four windows writes their 2 x 8 patch, the gradient (as 0 + g) at each window's first
// maximum and zero elsewhere.
// With WHERE, the `where(mask, x, y)` that ReLU's backward rule puts behind the pooling's adjoint
// (src/autograd/autograd.cpp:397-409) is served from the same registers: one of x / y is this
// kernel's own result, the other a tensor filled with one value (read from its first element).
struct PoolWhere {
    float* out;            // the where node's result
    const uint8_t* mask;   // dense, the shape of the image
    const float* constant; // first element of the filled operand
    int result_is_x;       // the pooling gradient is where's x (taken where the mask is set)
};

template <bool WHERE>
__global__ void __launch_bounds__(kThreads)
max_pool2d_backward_dense2_kernel(float* __restrict__ out, const float* __restrict__ grad,
                                  const float* __restrict__ in, int w, uint32_t items, FastDiv div_ow4,
                                  PoolWhere pw) {
    pdl_prologue();
    const uint32_t step = gridDim.x * kThreads;
    const int out_w = w / 2;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < items; i += step) {
        uint32_t prow, ow4;
        div_ow4.divmod(i, prow, ow4);   // prow = plane * out_h + oh; image row 2 * prow (h == 2 out_h)
        const int64_t base = int64_t(prow) * 2 * w + 8 * ow4;
        float v[2][8];
#pragma unroll
        for (int ki = 0; ki < 2; ++ki) {
            const float4 lo = *reinterpret_cast<const float4*>(in + base + ki * w);
            const float4 hi = *reinterpret_cast<const float4*>(in + base + ki * w + 4);
            v[ki][0] = lo.x; v[ki][1] = lo.y; v[ki][2] = lo.z; v[ki][3] = lo.w;
            v[ki][4] = hi.x; v[ki][5] = hi.y; v[ki][6] = hi.z; v[ki][7] = hi.w;
        }
        const float4 g4 = *reinterpret_cast<const float4*>(grad + int64_t(prow) * out_w + 4 * ow4);
        const float g[4] = {0.0F + g4.x, 0.0F + g4.y, 0.0F + g4.z, 0.0F + g4.w};
        float r[2][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float m = -INFINITY;
            int best = -1;
#pragma unroll
            for (int ki = 0; ki < 2; ++ki) {
#pragma unroll
                for (int kj = 0; kj < 2; ++kj) {
                    if (v[ki][2 * j + kj] > m) {
                        m = v[ki][2 * j + kj];
                        best = ki * 2 + kj;
                    }
                }
            }
#pragma unroll
            for (int ki = 0; ki < 2; ++ki) {
#pragma unroll
                for (int kj = 0; kj < 2; ++kj) {
                    r[ki][2 * j + kj] = (ki * 2 + kj == best) ? g[j] : 0.0F;
                }
            }
        }
#pragma unroll
        for (int ki = 0; ki < 2; ++ki) {
            *reinterpret_cast<float4*>(out + base + ki * w) = make_float4(r[ki][0], r[ki][1], r[ki][2], r[ki][3]);
            *reinterpret_cast<float4*>(out + base + ki * w + 4) = make_float4(r[ki][4], r[ki][5], r[ki][6], r[ki][7]);
        }
        if (WHERE) {
            const float c = *pw.constant;
#pragma unroll
            for (int ki = 0; ki < 2; ++ki) {
                const uint2 m8 = *reinterpret_cast<const uint2*>(pw.mask + base + ki * w);
                float s[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool set = (((j < 4 ? m8.x : m8.y) >> (8 * (j & 3))) & 0xffu) != 0;
                    s[j] = (set == (pw.result_is_x != 0)) ? r[ki][j] : c;
                }
                *reinterpret_cast<float4*>(pw.out + base + ki * w) = make_float4(s[0], s[1], s[2], s[3]);
                *reinterpret_cast<float4*>(pw.out + base + ki * w + 4) = make_float4(s[4], s[5], s[6], s[7]);
            }
        }
    }
}

// First strict maximum of one window; -1 if nothing beat -inf.
__device__ __forceinline__ int argmax_in_window(const float* plane, int64_t sh_, int64_t sw_, const Win& w,
                                                int oh, int ow, float& best) {
    best = -INFINITY;
    int best_offset = -1;
    for (int ki = 0; ki < w.kh; ++ki) {
        const int h = oh * w.sh - w.ph + ki * w.dh;
        if (h < 0 || h >= w.image_h) {
            continue;
        }
        for (int kj = 0; kj < w.kw; ++kj) {
            const int x = ow * w.sw - w.pw + kj * w.dw;
            if (x < 0 || x >= w.image_w) {
                continue;
            }
            const float v = plane[int64_t(h) * sh_ + int64_t(x) * sw_];
            if (v > best) {
                best = v;
                best_offset = ki * w.kw + kj;
            }
        }
    }
    return best_offset;
}

// One thread per output element, one block per chunk of an output plane.
__global__ void __launch_bounds__(kThreads)
max_pool2d_kernel(float* __restrict__ out, const float* __restrict__ in, Strides4 is, Win w, int out_h,
                  int out_w, int channels, int chunks, uint32_t* status) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned plane = b / chunks;
    const unsigned c = plane % channels;
    const unsigned n = plane / channels;
    const int p = chunk * blockDim.x + threadIdx.x;
    if (p >= out_h * out_w) {
        return;
    }
    const int oh = p / out_w;
    const int ow = p - oh * out_w;
    float best;
    const int off = argmax_in_window(in + int64_t(n) * is.s[0] + int64_t(c) * is.s[1], is.s[2], is.s[3], w, oh, ow,
                                     best);
    if (off < 0) {
        // the CPU backend asserts here: a window with no element above -inf
        atomicOr(status, kStatusInternal);
        best = __int_as_float(0x7fc00000);
    }
    out[int64_t(plane) * (out_h * out_w) + p] = best;
}

// Non-overlapping windows (stride == kernel, no padding or dilation): one thread per
// window with compile-time extents, rows read as one KW-wide vector when aligned.
template <int KH, int KW>
__global__ void __launch_bounds__(kThreads)
max_pool2d_tiled_kernel(float* __restrict__ out, const float* __restrict__ in, Strides4 is, int out_h, int out_w,
                        int channels, int chunks, int vec_ok, uint32_t* status) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned plane = b / chunks;
    const unsigned c = plane % channels;
    const unsigned n = plane / channels;
    const int p = chunk * blockDim.x + threadIdx.x;
    if (p >= out_h * out_w) {
        return;
    }
    const int oh = p / out_w;
    const int ow = p - oh * out_w;
    const float* src = in + int64_t(n) * is.s[0] + int64_t(c) * is.s[1] + int64_t(oh * KH) * is.s[2] +
                       int64_t(ow * KW) * is.s[3];
    float best = -INFINITY;
    bool any = false;
#pragma unroll
    for (int ki = 0; ki < KH; ++ki) {
        float v[KW];
        if (KW == 2 && vec_ok) {
            const float2 t = *reinterpret_cast<const float2*>(src + int64_t(ki) * is.s[2]);
            v[0] = t.x;
            v[KW - 1] = t.y;
        } else {
#pragma unroll
            for (int kj = 0; kj < KW; ++kj) {
                v[kj] = src[int64_t(ki) * is.s[2] + int64_t(kj) * is.s[3]];
            }
        }
#pragma unroll
        for (int kj = 0; kj < KW; ++kj) {
            if (v[kj] > best) {
                best = v[kj];
                any = true;
            }
        }
    }
    if (!any) {
        atomicOr(status, kStatusInternal);
        best = __int_as_float(0x7fc00000);
    }
    out[int64_t(plane) * (out_h * out_w) + p] = best;
}

// Pull form of the pooling adjoint (any geometry): every input element sums the
// gradients of the windows whose first maximum it is, in (ki, kj) order.
__global__ void __launch_bounds__(kThreads)
max_pool2d_backward_kernel(float* __restrict__ out, const float* __restrict__ grad, const float* __restrict__ in,
                           Strides4 gs, Strides4 is, Win w, int out_h, int out_w, int channels, int chunks) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned plane = b / chunks;
    const unsigned c = plane % channels;
    const unsigned n = plane / channels;
    const int hw = chunk * blockDim.x + threadIdx.x;
    if (hw >= w.image_h * w.image_w) {
        return;
    }
    const int h = hw / w.image_w;
    const int x = hw - h * w.image_w;
    const float* in_plane = in + int64_t(n) * is.s[0] + int64_t(c) * is.s[1];
    const float* g_plane = grad + int64_t(n) * gs.s[0] + int64_t(c) * gs.s[1];
    float acc = 0.0F;
    for (int ki = 0; ki < w.kh; ++ki) {
        const int top = h + w.ph - ki * w.dh;
        if (top < 0 || top % w.sh != 0) {
            continue;
        }
        const int oh = top / w.sh;
        if (oh >= out_h) {
            continue;
        }
        for (int kj = 0; kj < w.kw; ++kj) {
            const int left = x + w.pw - kj * w.dw;
            if (left < 0 || left % w.sw != 0) {
                continue;
            }
            const int ow = left / w.sw;
            if (ow >= out_w) {
                continue;
            }
            float best;
            if (argmax_in_window(in_plane, is.s[2], is.s[3], w, oh, ow, best) == ki * w.kw + kj) {
                acc += g_plane[int64_t(oh) * gs.s[2] + int64_t(ow) * gs.s[3]];
            }
        }
    }
    out[int64_t(plane) * (w.image_h * w.image_w) + hw] = acc;
}

// Non-overlapping windows (stride == kernel, no padding, no dilation): every input
// element lies in at most one window, so one thread per WINDOW finds the first
// maximum once and writes its kh x kw patch: the gradient at the maximum (as
// 0 + g, the value the pull form accumulates), zero elsewhere.  Rows and columns
// past the last whole window belong to no window and are written as zero by the
// threads of the extra, partial windows.
template <int KH, int KW>
__global__ void __launch_bounds__(kThreads)
max_pool2d_backward_tiled_kernel(float* __restrict__ out, const float* __restrict__ grad,
                                 const float* __restrict__ in, Strides4 gs, Strides4 is, Win w, int out_h,
                                 int out_w, int cover_h, int cover_w, int channels, int chunks) {
    pdl_prologue();
    const unsigned b = blockIdx.x;
    const unsigned chunk = b % chunks;
    const unsigned plane = b / chunks;
    const unsigned c = plane % channels;
    const unsigned n = plane / channels;
    const int p = chunk * blockDim.x + threadIdx.x;
    if (p >= cover_h * cover_w) {
        return;
    }
    const int oh = p / cover_w;
    const int ow = p - oh * cover_w;
    const float* in_plane = in + int64_t(n) * is.s[0] + int64_t(c) * is.s[1];
    float* out_plane = out + int64_t(plane) * (w.image_h * w.image_w);
    const bool real = oh < out_h && ow < out_w;
    int best_offset = -1;
    float g = 0.0F;
    if (real) {
        float best = -INFINITY;
#pragma unroll
        for (int ki = 0; ki < KH; ++ki) {
#pragma unroll
            for (int kj = 0; kj < KW; ++kj) {
                const float v = in_plane[int64_t(oh * KH + ki) * is.s[2] + int64_t(ow * KW + kj) * is.s[3]];
                if (v > best) {
                    best = v;
                    best_offset = ki * KW + kj;
                }
            }
        }
        g = 0.0F + grad[int64_t(n) * gs.s[0] + int64_t(c) * gs.s[1] + int64_t(oh) * gs.s[2] + int64_t(ow) * gs.s[3]];
    }
#pragma unroll
    for (int ki = 0; ki < KH; ++ki) {
        const int h = oh * KH + ki;
        if (h >= w.image_h) {
            continue;
        }
#pragma unroll
        for (int kj = 0; kj < KW; ++kj) {
            const int x = ow * KW + kj;
            if (x < w.image_w) {
                out_plane[h * w.image_w + x] = (ki * KW + kj == best_offset) ? g : 0.0F;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// index_select / scatter_add
// ---------------------------------------------------------------------------

// out[outer, k, rest] = a[outer, idx[k], rest]  (kernels_movement.cpp:339-369).
// An out-of-range index is recorded in the status word and clamped; the host
// reports it as an index error at the next synchronize.
template <typename T, typename I>
__global__ void __launch_bounds__(kThreads)
index_select_kernel(T* __restrict__ out, const T* __restrict__ a, const int64_t* __restrict__ idx, GeoT<I> ga,
                    I idx_stride, I inner, I extent, I a_extent, I total, uint32_t* status) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t li = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; li < int64_t(total); li += stride) {
        const I i = static_cast<I>(li);
        const I q = i / inner;
        const I rest = i - q * inner;
        const I outer = q / extent;
        const I k = q - outer * extent;
        int64_t j = idx[k * idx_stride];
        if (j < 0 || j >= int64_t(a_extent)) {
            atomicOr(status, kStatusIndexOutOfRange);
            j = j < 0 ? 0 : int64_t(a_extent) - 1;
        }
        out[i] = a[geo_off<I>(ga, (outer * a_extent + static_cast<I>(j)) * inner + rest)];
    }
}

// Dense source rows of 16-byte multiples: one thread per 16 bytes, four independent
// index -> row -> vector chains in flight per thread, divisions by multiply-high.
__global__ void __launch_bounds__(kThreads)
index_select_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ a, const int64_t* __restrict__ idx,
                         int64_t idx_stride, FastDiv div_inner16, FastDiv div_extent, unsigned a_extent,
                         unsigned total16, uint32_t* status) {
    pdl_prologue();
    constexpr int U = 4;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const unsigned inner16 = div_inner16.d;
    for (int64_t base = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; base < int64_t(total16); base += U * stride) {
        int64_t j[U];
        uint32_t outer[U], rest[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t li = base + u * stride;
            live[u] = li < int64_t(total16);
            j[u] = 0;
            outer[u] = rest[u] = 0;
            if (live[u]) {
                uint32_t q, k;
                div_inner16.divmod(static_cast<uint32_t>(li), q, rest[u]);
                div_extent.divmod(q, outer[u], k);
                j[u] = idx[int64_t(k) * idx_stride];
            }
        }
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live[u]) {
                if (j[u] < 0 || j[u] >= int64_t(a_extent)) {
                    atomicOr(status, kStatusIndexOutOfRange);
                    j[u] = j[u] < 0 ? 0 : int64_t(a_extent) - 1;
                }
                v[u] = a[(int64_t(outer[u]) * a_extent + j[u]) * inner16 + rest[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live[u]) {
                out[base + u * stride] = v[u];
            }
        }
    }
}

// out[outer, j, rest] = sum over k with idx[k] == j of src[outer, k, rest], k ascending.
template <typename I>
__global__ void __launch_bounds__(kThreads)
scatter_add_kernel(float* __restrict__ out, const float* __restrict__ src, const int64_t* __restrict__ idx,
                   GeoT<I> gsrc, I idx_stride, I inner, I src_extent, I out_extent, I total) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t li = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; li < int64_t(total); li += stride) {
        const I i = static_cast<I>(li);
        const I q = i / inner;
        const I rest = i - q * inner;
        const I outer = q / out_extent;
        const int64_t j = int64_t(q - outer * out_extent);
        float acc = 0.0F;
        for (I k = 0; k < src_extent; ++k) {
            if (idx[k * idx_stride] == j) {
                acc += src[geo_off<I>(gsrc, (outer * src_extent + k) * inner + rest)];
            }
        }
        out[i] = acc;
    }
}

// ---- scatter_add for long index lists -------------------------------------
// The pull form above reads every index for every output element: exact, in the reference's
// order, and O(outputs x indices) -- an Embedding backward over a 50 000-row table with 8192
// indices would be 4e11 index reads.  Here the indices are bucketed by destination first:
//   1. count the sources of every destination,
//   2. exclusive scan -> where each destination's list starts,
//   3. place every k into its destination's list AT ITS RANK among the earlier k with the same
//      destination, so every list is in ascending k: the rank inside a chunk of 512 indices comes
//      from comparing the chunk's indices in shared memory (all chunks in parallel), the rank
//      before the chunk from a per-destination cursor that one block advances chunk by chunk,
//   4. every output element adds the sources of its list in list order.
// Same sums in the same order as the pull form, bit for bit; each source element is read once.
constexpr int kScatterChunk = 512;

__global__ void __launch_bounds__(kThreads)
scatter_count_kernel(int* __restrict__ count, const int64_t* __restrict__ idx, int64_t idx_stride, int n,
                     int64_t extent) {
    pdl_prologue();
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < n) {
        const int64_t t = idx[k * idx_stride];
        if (t >= 0 && t < extent) {
            atomicAdd(count + t, 1);  // integer counts: the result does not depend on the order
        }
    }
}

// One block: offsets[j] = number of sources of destinations < j; offsets[extent] = their total.
// cursor[j] starts as a copy of offsets[j].  Eight consecutive destinations per thread and step.
__global__ void __launch_bounds__(1024)
scatter_scan_kernel(int* __restrict__ offsets, int* __restrict__ cursor, const int* __restrict__ count, int extent) {
    pdl_prologue();
    constexpr int PER = 8;
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < extent; base += 1024 * PER) {
        const int j0 = base + threadIdx.x * PER;
        int c[PER];
        int mine = 0;
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            c[u] = j0 + u < extent ? count[j0 + u] : 0;
            mine += c[u];
        }
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffU, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffU, w, d);
                if (lane >= d) w += up;
            }
            warp_sums[lane] = w;  // inclusive over the warps
        }
        __syncthreads();
        int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - mine;
        const int block_total = warp_sums[31];
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            if (j0 + u < extent) {
                offsets[j0 + u] = before;
                cursor[j0 + u] = before;
            }
            before += c[u];
        }
        __syncthreads();
        if (threadIdx.x == 0) carry += block_total;
        __syncthreads();
    }
    if (threadIdx.x == 0) offsets[extent] = carry;
}

// rank[k] = how many EARLIER indices of k's chunk have k's destination, bit 30 set when no LATER
// index of the chunk has it; -1 for an index out of range.  All chunks at once.
__global__ void __launch_bounds__(kScatterChunk)
scatter_rank_kernel(int* __restrict__ rank, const int64_t* __restrict__ idx, int64_t idx_stride, int n,
                    int64_t extent) {
    pdl_prologue();
    __shared__ int keys[kScatterChunk];
    const int k = blockIdx.x * kScatterChunk + threadIdx.x;
    int key = -1;
    if (k < n) {
        const int64_t t = idx[k * idx_stride];
        if (t >= 0 && t < extent) key = static_cast<int>(t);
    }
    keys[threadIdx.x] = key;
    __syncthreads();
    if (k >= n) return;
    int before = 0, later = 0;
    if (key >= 0) {
        const int me = static_cast<int>(threadIdx.x);
#pragma unroll 8
        for (int t = 0; t < kScatterChunk; ++t) {
            const int same = keys[t] == key;   // every lane reads the same word: a broadcast
            before += same & (t < me);
            later |= same & (t > me);
        }
    }
    rank[k] = key < 0 ? -1 : (before | (later ? 0 : (1 << 30)));
}

// One block walks the chunks in order: an index goes to its destination's cursor plus its rank
// inside the chunk, and the chunk's last index of a destination moves that cursor on.
__global__ void __launch_bounds__(kScatterChunk)
scatter_place_kernel(int* __restrict__ perm, int* __restrict__ cursor, const int* __restrict__ rank,
                     const int64_t* __restrict__ idx, int64_t idx_stride, int n) {
    pdl_prologue();
    for (int k0 = 0; k0 < n; k0 += kScatterChunk) {
        const int k = k0 + static_cast<int>(threadIdx.x);
        const int r = k < n ? rank[k] : -1;
        int64_t key = 0;
        int start = 0;
        if (r >= 0) {
            key = idx[k * idx_stride];
            start = __ldcg(cursor + key);  // written by this block's earlier steps only
        }
        __syncthreads();
        if (r >= 0) {
            const int pos = start + (r & ((1 << 30) - 1));
            perm[pos] = k;
            if (r >> 30) __stcg(cursor + key, pos + 1);
        }
        __syncthreads();
    }
}

template <typename I>
__global__ void __launch_bounds__(kThreads)
scatter_gather_kernel(float* __restrict__ out, const float* __restrict__ src, const int* __restrict__ perm,
                      const int* __restrict__ offsets, GeoT<I> gsrc, I inner, I src_extent, I out_extent, I total) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t li = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; li < int64_t(total); li += stride) {
        const I i = static_cast<I>(li);
        const I q = i / inner;
        const I rest = i - q * inner;
        const I outer = q / out_extent;
        const I j = q - outer * out_extent;
        const int t0 = offsets[j], t1 = offsets[j + 1];
        float acc = 0.0F;
        for (int t = t0; t < t1; ++t) {
            acc += src[geo_off<I>(gsrc, (outer * src_extent + static_cast<I>(perm[t])) * inner + rest)];
        }
        out[i] = acc;
    }
}

// Dense source, rows of 16-byte multiples: four adjacent elements per thread and four such items
// in flight, so the (list bounds -> source index -> source row) chains of different items overlap.
__global__ void __launch_bounds__(kThreads)
scatter_gather4_kernel(float4* __restrict__ out, const float4* __restrict__ src, const int* __restrict__ perm,
                       const int* __restrict__ offsets, FastDiv div_inner4, FastDiv div_extent, unsigned src_extent,
                       unsigned total4) {
    pdl_prologue();
    constexpr int U = 4;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const unsigned inner4 = div_inner4.d;
    for (int64_t base = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; base < int64_t(total4); base += U * stride) {
        int t0[U], t1[U];
        uint32_t outer[U], rest[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t li = base + u * stride;
            t0[u] = t1[u] = 0;
            outer[u] = rest[u] = 0;
            if (li < int64_t(total4)) {
                uint32_t q, j;
                div_inner4.divmod(static_cast<uint32_t>(li), q, rest[u]);
                div_extent.divmod(q, outer[u], j);
                t0[u] = offsets[j];
                t1[u] = offsets[j + 1];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t li = base + u * stride;
            if (li < int64_t(total4)) {
                float4 acc = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
                for (int t = t0[u]; t < t1[u]; ++t) {
                    const float4 v = src[(int64_t(outer[u]) * src_extent + perm[t]) * inner4 + rest[u]];
                    acc.x += v.x;
                    acc.y += v.y;
                    acc.z += v.z;
                    acc.w += v.w;
                }
                out[li] = acc;
            }
        }
    }
}

// Flags any index outside [0, extent): scatter_add's pull form would otherwise
// just never match it.
__global__ void __launch_bounds__(kThreads)
index_range_kernel(const int64_t* __restrict__ idx, int64_t idx_stride, int64_t n, int64_t extent,
                   uint32_t* status) {
    pdl_prologue();
    const int64_t k = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (k < n) {
        const int64_t t = idx[k * idx_stride];
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

// Block size for a per-plane loop of `n` items: a whole number of warps, at most 256.
int block_for(int64_t n) {
    if (n >= 256) return 256;
    return static_cast<int>(std::max<int64_t>(32, (n + 31) / 32 * 32));
}

void check_grid(int64_t blocks, const char* what) {
    if (blocks <= 0 || blocks > 0x7fffffffLL) {
        fail(B200_NOT_IMPLEMENTED, std::string(what) + ": tensor too large for one launch");
    }
}

// The index tensor of index_select / scatter_add is one-dimensional (any stride).
int64_t index_stride(const View& idx) {
    int64_t stride = 0;
    int live = 0;
    for (int i = 0; i < kMaxDims; ++i) {
        if (idx.dim[i] > 1) {
            stride = idx.stride[i];
            ++live;
        }
    }
    if (live > 1) {
        fail(B200_SHAPE_ERROR, "index tensor must be one-dimensional");
    }
    return stride;
}

}  // namespace

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Planes per block of the dense convolution kernels: enough for two vector items per thread,
// within the shared-memory allowance, and never so many that the grid cannot fill the machine.
int planes_per_block(int64_t items_per_plane, int64_t bytes_per_plane, int64_t byte_limit, int64_t planes) {
    int64_t group = ceil_div(int64_t(2) * kThreads, std::max<int64_t>(items_per_plane, 1));
    group = std::min(group, std::max<int64_t>(byte_limit / std::max<int64_t>(bytes_per_plane, 1), 1));
    group = std::min(group, std::max<int64_t>(planes / (int64_t(sm_count()) * 8), 1));
    return static_cast<int>(std::max<int64_t>(group, 1));
}

constexpr int kDenseSmemLimit = 96 * 1024;

template <typename K>
void allow_large_smem(K kernel) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmemLimit));
}

// max_pool2d_backward followed by where(mask, x, y) with one of x / y the pooling gradient and the
// other a tensor filled with one value: one launch when the pooling is the dense 2x2 case, false otherwise.
bool launch_pool_backward_where(b200_ctx* ctx, const b200_node& pool, const b200_node& where, int result_is_x,
                                const void* constant) {
    const View out = make_view(pool.out);
    const View grad = make_view(pool.src[0]);
    const View in = make_view(pool.src[1]);
    const View wout = make_view(where.out);
    const View mask = make_view(where.src[0]);
    if (out.dtype != B200_F32 || in.dtype != B200_F32 || grad.dtype != B200_F32 || wout.dtype != B200_F32 ||
        mask.dtype != B200_BOOL || pool.out.ndim != 4 || pool.src[0].ndim != 4 || pool.src[1].ndim != 4) {
        return false;
    }
    if (!out.contiguous || !in.contiguous || !grad.contiguous || !wout.contiguous || !mask.contiguous ||
        wout.numel != out.numel || mask.numel != out.numel) {
        return false;
    }
    const Win w = make_win(get_params<UnfoldParams>(pool), 1);
    const int out_h = static_cast<int>(grad.dim[2]), out_w = static_cast<int>(grad.dim[3]);
    const int64_t planes = out.dim[0] * out.dim[1];
    const int64_t total = out.numel;
    const bool dense2 = w.sh == 2 && w.sw == 2 && w.kh == 2 && w.kw == 2 && w.ph == 0 && w.pw == 0 && w.dh == 1 && w.dw == 1 &&
                        in.dim[2] == w.image_h && in.dim[3] == w.image_w && out.dim[2] == w.image_h && out.dim[3] == w.image_w &&
                        in.dim[0] == out.dim[0] && in.dim[1] == out.dim[1] && grad.dim[0] == out.dim[0] && grad.dim[1] == out.dim[1] &&
                        w.image_w % 8 == 0 && w.image_h % 2 == 0 && out_h * 2 == w.image_h && out_w * 2 == w.image_w &&
                        total > 0 && total / 16 < (int64_t(1) << 31);
    const auto aligned = [](const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
    if (!dense2 || !aligned(out.data, 16) || !aligned(in.data, 16) || !aligned(grad.data, 16) || !aligned(wout.data, 16) ||
        !aligned(mask.data, 8)) {
        return false;
    }
    const uint32_t items = static_cast<uint32_t>(planes * out_h * (out_w / 4));
    PoolWhere pw{reinterpret_cast<float*>(wout.data), reinterpret_cast<const uint8_t*>(mask.data),
                 static_cast<const float*>(constant), result_is_x};
    ProfScope scope(ctx, "fused.pool_backward_where");
    launch_kernel(ctx, max_pool2d_backward_dense2_kernel<true>, grid_for(items, kThreads), kThreads, 0,
                  reinterpret_cast<float*>(out.data), reinterpret_cast<const float*>(grad.data),
                  reinterpret_cast<const float*>(in.data), w.image_w, items, FastDiv(static_cast<uint32_t>(out_w / 4)), pw);
    ctx->count_launch();
    check_last_launch("max_pool2d_backward + where");
    return true;
}

void launch_movement(b200_ctx* ctx, const b200_node& node) {
    const View out = make_view(node.out);
    const int64_t total = out.numel;
    float* o = reinterpret_cast<float*>(out.data);
    constexpr int64_t kMax32 = int64_t(1) << 31;

    switch (node.op) {
        case B200_OP_IM2COL: {
            const View in = make_view(node.src[0]);
            require_f32(out, "im2col");
            require_f32(in, "im2col");
            require_dense(out, "im2col");
            if (node.out.ndim != 3 || node.src[0].ndim != 4) {
                fail(B200_SHAPE_ERROR, "im2col: expects [N,C,H,W] -> [N, C*kh*kw, L]");
            }
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), node.out.dims[1]);
            const int64_t rows = node.out.dims[1], positions = node.out.dims[2], n = node.out.dims[0];
            if (int64_t(w.out_h) * w.out_w != positions || in.dim[0] != n || in.dim[1] != w.channels ||
                in.dim[2] != w.image_h || in.dim[3] != w.image_w || rows != w.channels * w.kh * w.kw) {
                fail(B200_SHAPE_ERROR, "im2col: geometry does not match the tensors");
            }
            if (positions >= kMax32 || rows >= kMax32) fail(B200_NOT_IMPLEMENTED, "im2col: extent too large");
            {
                const bool unit = w.sh == 1 && w.sw == 1 && w.dh == 1 && w.dw == 1;
                const int64_t planes = n * w.channels;
                const int64_t padded_w = w.image_w + 2 * int64_t(w.pw);
                const int64_t padded_plane = (w.image_h + 2 * int64_t(w.ph)) * padded_w;
                const int64_t taps = int64_t(w.kh) * w.kw;
                if (unit && in.contiguous && w.out_w % 4 == 0 && aligned16(o) && w.ph >= 0 && w.pw >= 0 &&
                    padded_plane * 4 <= 48 * 1024 && planes < kMax32 && taps * positions < (kMax32 >> 8)) {
                    DenseGeo g{};
                    g.h = w.image_h; g.w = w.image_w; g.ph = w.ph; g.pw = w.pw;
                    g.oh = w.out_h; g.ow = w.out_w; g.kh = w.kh; g.kw = w.kw;
                    g.padded_w = static_cast<int>(padded_w);
                    g.padded_plane = static_cast<int>(padded_plane);
                    g.planes = static_cast<int>(planes);
                    g.group = planes_per_block(positions / 4, padded_plane * 4, 48 * 1024, planes);
                    g.group = static_cast<int>(std::min<int64_t>(g.group, (kMax32 >> 2) / (taps * positions)));
                    g.vec_in = w.image_w % 4 == 0 && aligned16(in.data);
                    const unsigned grid = static_cast<unsigned>(ceil_div(planes, g.group));
                    const size_t smem = size_t(g.group) * padded_plane * 4;
                    const FastDiv div_w4(g.vec_in ? w.image_w / 4 : 1), div_w(w.image_w), div_h(w.image_h),
                        div_l4(static_cast<uint32_t>(positions / 4)), div_ow(w.out_w);
                    const float* src = reinterpret_cast<const float*>(in.data);
                    if (w.kh == 3 && w.kw == 3) {
                        launch_kernel(ctx, im2col_dense_kernel<3, 3>, grid, kThreads, smem, o, src, g, div_w4, div_w, div_h,
                                                                                         div_l4, div_ow);
                    } else {
                        launch_kernel(ctx, im2col_dense_kernel<0, 0>, grid, kThreads, smem, o, src, g, div_w4, div_w, div_h,
                                                                                         div_l4, div_ow);
                    }
                    break;
                }
            }
            const int block = block_for(positions);
            const int64_t chunks = ceil_div(positions, block);
            check_grid(n * w.channels * chunks, "im2col");
            launch_kernel(ctx, im2col_kernel, static_cast<unsigned>(n * w.channels * chunks), block, 0, o, reinterpret_cast<const float*>(in.data), strides_of(in), w, static_cast<int>(positions),
                static_cast<int>(chunks));
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
            const int64_t n = node.src[0].dims[0];
            const int64_t plane = int64_t(w.image_h) * w.image_w;
            if (int64_t(w.out_h) * w.out_w != node.src[0].dims[2] || total != n * w.channels * plane ||
                node.src[0].dims[1] != w.channels * w.kh * w.kw) {
                fail(B200_SHAPE_ERROR, "col2im: geometry does not match the tensors");
            }
            if (plane >= kMax32 || w.channels >= kMax32) fail(B200_NOT_IMPLEMENTED, "col2im: extent too large");
            const float* src = reinterpret_cast<const float*>(cols.data);
            const bool unit = w.sh == 1 && w.sw == 1 && w.dh == 1 && w.dw == 1;
            {
                const int64_t planes = n * w.channels;
                const int64_t l = int64_t(w.out_h) * w.out_w;
                const int64_t taps = int64_t(w.kh) * w.kw;
                const int64_t plane_bytes = taps * l * 4;
                if (unit && cols.contiguous && (taps * l) % 4 == 0 && w.image_w % 4 == 0 && aligned16(o) &&
                    aligned16(src) && plane_bytes <= kDenseSmemLimit && planes < kMax32 && l > 0) {
                    DenseGeo g{};
                    g.h = w.image_h; g.w = w.image_w; g.ph = w.ph; g.pw = w.pw;
                    g.oh = w.out_h; g.ow = w.out_w; g.kh = w.kh; g.kw = w.kw;
                    g.planes = static_cast<int>(planes);
                    g.group = planes_per_block(plane / 4, plane_bytes, 36 * 1024, planes);
                    const unsigned grid = static_cast<unsigned>(ceil_div(planes, g.group));
                    const size_t smem = size_t(g.group) * plane_bytes;
                    const FastDiv div_hw4(static_cast<uint32_t>(plane / 4)), div_w(w.image_w);
                    static const bool once = [] {
                        allow_large_smem(col2im_dense_kernel<3, 3>);
                        allow_large_smem(col2im_dense_kernel<0, 0>);
                        return true;
                    }();
                    (void)once;
                    if (w.kh == 3 && w.kw == 3 && w.ph == 1 && w.pw == 1 && l % 4 == 0 && w.out_w % 4 == 0 &&
                        w.out_h == w.image_h && w.out_w == w.image_w) {
                        static const bool once3 = [] {
                            allow_large_smem(col2im_dense_3x3p1_kernel);
                            return true;
                        }();
                        (void)once3;
                        launch_kernel(ctx, col2im_dense_3x3p1_kernel, grid, kThreads, smem, o, src, g, div_hw4, div_w);
                    } else if (w.kh == 3 && w.kw == 3) {
                        launch_kernel(ctx, col2im_dense_kernel<3, 3>, grid, kThreads, smem, o, src, g, div_hw4, div_w);
                    } else {
                        launch_kernel(ctx, col2im_dense_kernel<0, 0>, grid, kThreads, smem, o, src, g, div_hw4, div_w);
                    }
                    break;
                }
            }
            const int block = block_for(plane);
            const int64_t chunks = ceil_div(plane, block);
            check_grid(n * w.channels * chunks, "col2im");
            const unsigned grid = static_cast<unsigned>(n * w.channels * chunks);
            if (unit && w.kh == 3 && w.kw == 3) {
                launch_kernel(ctx, col2im_kernel<true, 3, 3>, grid, block, 0, o, src, strides_of(cols), w,
                                                                           static_cast<int>(chunks));
            } else if (unit) {
                launch_kernel(ctx, col2im_kernel<true, 0, 0>, grid, block, 0, o, src, strides_of(cols), w,
                                                                           static_cast<int>(chunks));
            } else {
                launch_kernel(ctx, col2im_kernel<false, 0, 0>, grid, block, 0, o, src, strides_of(cols), w,
                                                                            static_cast<int>(chunks));
            }
            break;
        }
        case B200_OP_MAX_POOL2D: {
            const View in = make_view(node.src[0]);
            require_f32(out, "max_pool2d");
            require_f32(in, "max_pool2d");
            require_dense(out, "max_pool2d");
            if (node.out.ndim != 4 || node.src[0].ndim != 4) {
                fail(B200_SHAPE_ERROR, "max_pool2d: tensors must be rank 4");
            }
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), 1);
            if (in.dim[2] != w.image_h || in.dim[3] != w.image_w || in.dim[0] != out.dim[0] ||
                in.dim[1] != out.dim[1]) {
                fail(B200_SHAPE_ERROR, "max_pool2d: geometry does not match the tensors");
            }
            const int64_t plane = out.dim[2] * out.dim[3];
            if (plane >= kMax32 || out.dim[1] >= kMax32) fail(B200_NOT_IMPLEMENTED, "max_pool2d: extent too large");
            const int block = block_for(plane);
            const int64_t chunks = ceil_div(plane, block);
            check_grid(out.dim[0] * out.dim[1] * chunks, "max_pool2d");
            const bool tiled = w.sh == w.kh && w.sw == w.kw && w.ph == 0 && w.pw == 0 && w.dh == 1 && w.dw == 1 &&
                               ((w.kh == 2 && w.kw == 2) || (w.kh == 3 && w.kw == 3));
            if (tiled && w.kh == 2 && in.contiguous && w.image_w % 8 == 0 && aligned16(in.data) && aligned16(o) &&
                total / 4 < kMax32 && out.dim[0] * out.dim[1] * w.image_h < kMax32) {
                const uint32_t items = static_cast<uint32_t>(total / 4);
                const FastDiv div_ow4(static_cast<uint32_t>(out.dim[3] / 4)), div_oh(static_cast<uint32_t>(out.dim[2]));
                launch_kernel(ctx, max_pool2d_dense2_kernel, grid_for(items, kThreads), kThreads, 0, o, reinterpret_cast<const float*>(in.data), w.image_h, w.image_w, static_cast<int>(out.dim[2]), items,
                    div_ow4, div_oh, ctx->d_status);
                break;
            }
            if (tiled) {
                const unsigned grid = static_cast<unsigned>(out.dim[0] * out.dim[1] * chunks);
                const float* src = reinterpret_cast<const float*>(in.data);
                const int vec_ok = in.stride[3] == 1 && in.stride[2] % 2 == 0 && in.stride[1] % 2 == 0 &&
                                   in.stride[0] % 2 == 0 && reinterpret_cast<uintptr_t>(src) % 8 == 0;
                if (w.kh == 2) {
                    launch_kernel(ctx, max_pool2d_tiled_kernel<2, 2>, grid, block, 0, o, src, strides_of(in), static_cast<int>(out.dim[2]), static_cast<int>(out.dim[3]),
                        static_cast<int>(out.dim[1]), static_cast<int>(chunks), vec_ok, ctx->d_status);
                } else {
                    launch_kernel(ctx, max_pool2d_tiled_kernel<3, 3>, grid, block, 0, o, src, strides_of(in), static_cast<int>(out.dim[2]), static_cast<int>(out.dim[3]),
                        static_cast<int>(out.dim[1]), static_cast<int>(chunks), 0, ctx->d_status);
                }
                break;
            }
            launch_kernel(ctx, max_pool2d_kernel, static_cast<unsigned>(out.dim[0] * out.dim[1] * chunks), block, 0, o, reinterpret_cast<const float*>(in.data), strides_of(in), w, static_cast<int>(out.dim[2]),
                static_cast<int>(out.dim[3]), static_cast<int>(out.dim[1]), static_cast<int>(chunks), ctx->d_status);
            break;
        }
        case B200_OP_MAX_POOL2D_BACKWARD: {
            const View grad = make_view(node.src[0]);
            const View in = make_view(node.src[1]);
            require_f32(out, "max_pool2d_backward");
            require_f32(in, "max_pool2d_backward");
            require_f32(grad, "max_pool2d_backward");
            require_dense(out, "max_pool2d_backward");
            if (node.out.ndim != 4 || node.src[0].ndim != 4 || node.src[1].ndim != 4) {
                fail(B200_SHAPE_ERROR, "max_pool2d_backward: tensors must be rank 4");
            }
            if (total == 0) return;
            const Win w = make_win(get_params<UnfoldParams>(node), 1);
            if (in.dim[2] != w.image_h || in.dim[3] != w.image_w || out.dim[2] != w.image_h ||
                out.dim[3] != w.image_w || in.dim[0] != out.dim[0] || in.dim[1] != out.dim[1] ||
                grad.dim[0] != out.dim[0] || grad.dim[1] != out.dim[1]) {
                fail(B200_SHAPE_ERROR, "max_pool2d_backward: geometry does not match the tensors");
            }
            const int out_h = static_cast<int>(grad.dim[2]), out_w = static_cast<int>(grad.dim[3]);
            const int64_t planes = out.dim[0] * out.dim[1];
            const float* g = reinterpret_cast<const float*>(grad.data);
            const float* src = reinterpret_cast<const float*>(in.data);
            const bool tiled = w.sh == w.kh && w.sw == w.kw && w.ph == 0 && w.pw == 0 && w.dh == 1 && w.dw == 1 &&
                               ((w.kh == 2 && w.kw == 2) || (w.kh == 3 && w.kw == 3));
            if (out.dim[1] >= kMax32 || int64_t(w.image_h) * w.image_w >= kMax32) {
                fail(B200_NOT_IMPLEMENTED, "max_pool2d_backward: extent too large");
            }
            if (tiled && w.kh == 2 && in.contiguous && grad.contiguous && w.image_w % 8 == 0 && w.image_h % 2 == 0 &&
                out_h * 2 == w.image_h && out_w * 2 == w.image_w && aligned16(src) && aligned16(g) && aligned16(o) &&
                total / 16 < kMax32) {
                const uint32_t items = static_cast<uint32_t>(planes * out_h * (out_w / 4));
                const FastDiv div_ow4(static_cast<uint32_t>(out_w / 4));
                launch_kernel(ctx, max_pool2d_backward_dense2_kernel<false>, grid_for(items, kThreads), kThreads, 0, o, g, src, w.image_w, items, div_ow4, PoolWhere{});
                break;
            }
            if (tiled) {
                const int cover_h = static_cast<int>(ceil_div(w.image_h, w.kh));
                const int cover_w = static_cast<int>(ceil_div(w.image_w, w.kw));
                const int64_t per_plane = int64_t(cover_h) * cover_w;
                const int block = block_for(per_plane);
                const int64_t chunks = ceil_div(per_plane, block);
                check_grid(planes * chunks, "max_pool2d_backward");
                const unsigned grid = static_cast<unsigned>(planes * chunks);
                if (w.kh == 2) {
                    launch_kernel(ctx, max_pool2d_backward_tiled_kernel<2, 2>, grid, block, 0, o, g, src, strides_of(grad), strides_of(in), w, out_h, out_w, cover_h, cover_w,
                        static_cast<int>(out.dim[1]), static_cast<int>(chunks));
                } else {
                    launch_kernel(ctx, max_pool2d_backward_tiled_kernel<3, 3>, grid, block, 0, o, g, src, strides_of(grad), strides_of(in), w, out_h, out_w, cover_h, cover_w,
                        static_cast<int>(out.dim[1]), static_cast<int>(chunks));
                }
            } else {
                const int64_t per_plane = int64_t(w.image_h) * w.image_w;
                const int block = block_for(per_plane);
                const int64_t chunks = ceil_div(per_plane, block);
                check_grid(planes * chunks, "max_pool2d_backward");
                launch_kernel(ctx, max_pool2d_backward_kernel, static_cast<unsigned>(planes * chunks), block, 0, o, g, src, strides_of(grad), strides_of(in), w, out_h, out_w, static_cast<int>(out.dim[1]),
                    static_cast<int>(chunks));
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
            const int64_t istride = index_stride(idx);
            const size_t esz = dtype_size(out.dtype);
            const int64_t row_bytes = inner * static_cast<int64_t>(esz);
            const bool small = total < kMax32 && fits32(a) && idx.numel < kMax32 && istride >= 0 &&
                               istride * idx.numel < kMax32;
            if (a.contiguous && row_bytes % 16 == 0 && small && reinterpret_cast<uintptr_t>(a.data) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(out.data) % 16 == 0) {
                const int64_t total16 = total * static_cast<int64_t>(esz) / 16;
                launch_kernel(ctx, index_select_rows_kernel, grid_for(ceil_div(total16, 4), kThreads), kThreads, 0,
                              reinterpret_cast<uint4*>(out.data), reinterpret_cast<const uint4*>(a.data), ip, istride,
                              FastDiv(static_cast<uint32_t>(row_bytes / 16)),
                              FastDiv(static_cast<uint32_t>(out.dim[axis])), static_cast<unsigned>(a.dim[axis]),
                              static_cast<unsigned>(total16), ctx->d_status);
                break;
            }
            const unsigned grid = grid_for(total, kThreads);
#define B200_INDEX_SELECT(T, I)                                                                              \
    launch_kernel(ctx, index_select_kernel<T, I>, grid, kThreads, 0, \
        reinterpret_cast<T*>(out.data), reinterpret_cast<const T*>(a.data), ip, geo_t<I>(a),                 \
        static_cast<I>(istride), static_cast<I>(inner), static_cast<I>(out.dim[axis]),                       \
        static_cast<I>(a.dim[axis]), static_cast<I>(total), ctx->d_status)
            if (esz == 4) {
                if (small) B200_INDEX_SELECT(uint32_t, uint32_t);
                else B200_INDEX_SELECT(uint32_t, int64_t);
            } else if (esz == 8) {
                if (small) B200_INDEX_SELECT(uint64_t, uint32_t);
                else B200_INDEX_SELECT(uint64_t, int64_t);
            } else {
                fail(B200_DTYPE_ERROR, "index_select: unsupported element width");
            }
#undef B200_INDEX_SELECT
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
            const int64_t istride = index_stride(idx);
            const int64_t n_idx = src.numel == 0 ? 0 : src.dim[axis];
            if (n_idx > 0) {
                launch_kernel(ctx, index_range_kernel, static_cast<unsigned>(ceil_div(n_idx, kThreads)), kThreads, 0, ip, istride, n_idx, out.dim[axis], ctx->d_status);
                ctx->count_launch();
            }
            const unsigned grid = grid_for(total, kThreads);
            const float* sp = reinterpret_cast<const float*>(src.data);
            const bool small = total < kMax32 && fits32(src) && istride >= 0 && istride * std::max<int64_t>(n_idx, 1) < kMax32;
            const int64_t extent = out.dim[axis];
            // (worth its five small launches and its one-block scan over the destinations only when the
            // pull form's outputs x indices reads are many and the destination axis is not enormous)
            if (n_idx >= 256 && n_idx < (int64_t(1) << 30) && extent <= (int64_t(1) << 26) &&
                double(total) * double(n_idx) >= 1e8) {
                // bucket the indices by destination first (see above): five small launches and the gather
                const size_t ints = static_cast<size_t>(3 * extent + 1 + 2 * n_idx);
                int* count = static_cast<int*>(ctx->ensure_workspace(ints * sizeof(int) + 16));
                int* offsets = count + extent;  // extent + 1 entries
                int* cursor = offsets + extent + 1;
                int* perm = cursor + extent;
                int* rank = perm + n_idx;
                B200_CUDA_CHECK(cudaMemsetAsync(count, 0, static_cast<size_t>(extent) * sizeof(int), ctx->stream));
                const int n = static_cast<int>(n_idx);
                launch_kernel(ctx, scatter_count_kernel, static_cast<unsigned>(ceil_div(n_idx, kThreads)), kThreads, 0, count, ip, istride, n, extent);
                launch_kernel(ctx, scatter_scan_kernel, 1u, 1024, 0, offsets, cursor, static_cast<const int*>(count), static_cast<int>(extent));
                launch_kernel(ctx, scatter_rank_kernel, static_cast<unsigned>(ceil_div(n_idx, kScatterChunk)), kScatterChunk, 0, rank, ip, istride, n, extent);
                launch_kernel(ctx, scatter_place_kernel, 1u, kScatterChunk, 0, perm, cursor, static_cast<const int*>(rank), ip, istride, n);
                ctx->count_launch(4);
                if (src.contiguous && inner % 4 == 0 && total / 4 < kMax32 && reinterpret_cast<uintptr_t>(sp) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(o) % 16 == 0) {
                    const unsigned total4 = static_cast<unsigned>(total / 4);
                    launch_kernel(ctx, scatter_gather4_kernel, grid_for(ceil_div(int64_t(total4), 4), kThreads), kThreads, 0, reinterpret_cast<float4*>(o),
                                  reinterpret_cast<const float4*>(sp), static_cast<const int*>(perm), static_cast<const int*>(offsets),
                                  FastDiv(static_cast<uint32_t>(inner / 4)), FastDiv(static_cast<uint32_t>(extent)),
                                  static_cast<unsigned>(n_idx), total4);
                } else if (small) {
                    launch_kernel(ctx, scatter_gather_kernel<uint32_t>, grid, kThreads, 0, o, sp, static_cast<const int*>(perm), static_cast<const int*>(offsets),
                        geo_t<uint32_t>(src), static_cast<uint32_t>(inner), static_cast<uint32_t>(n_idx), static_cast<uint32_t>(extent), static_cast<uint32_t>(total));
                } else {
                    launch_kernel(ctx, scatter_gather_kernel<int64_t>, grid, kThreads, 0, o, sp, static_cast<const int*>(perm), static_cast<const int*>(offsets),
                        geo_t<int64_t>(src), inner, n_idx, extent, total);
                }
            } else if (small) {
                launch_kernel(ctx, scatter_add_kernel<uint32_t>, grid, kThreads, 0, o, sp, ip, geo_t<uint32_t>(src), static_cast<uint32_t>(istride), static_cast<uint32_t>(inner),
                    static_cast<uint32_t>(n_idx), static_cast<uint32_t>(out.dim[axis]), static_cast<uint32_t>(total));
            } else {
                launch_kernel(ctx, scatter_add_kernel<int64_t>, grid, kThreads, 0, o, sp, ip, geo_t<int64_t>(src), istride, inner, n_idx, out.dim[axis], total);
            }
            break;
        }
        default: fail(B200_NOT_IMPLEMENTED, "movement: unhandled op");
    }
    ctx->count_launch();
    check_last_launch("movement");
}

}  // namespace b200
