// In-span fusion: node sequences vkML's autograd and loss builders always emit, served by one
// kernel each.
//
// A backend must leave every node's value in that node's own buffer (include/vkml/backend/api/
// backend.h:34-45: later spans may read any of them), so a fused kernel still WRITES what the
// separate kernels wrote; what it saves is launches and the re-reading of intermediates.  The
// values are the ones the separate kernels produce: same functions, same rounding, one thread per
// element (the one reduction below states its order).
//
//   * Linear / conv epilogue with its ReLU-backward mask:
//       [add(x, bias)]  [full(0)  less_equal(y, 0)  full(0)]  [relu(y)]
//     (src/api/ops.cpp: bias add as a broadcast view; src/autograd/autograd.cpp:397-409: the
//     mask of ReLU's backward rule) in whichever of its forms a span holds -- all five nodes
//     (5 launches and 33 bytes per element become 1 launch and 21), add + relu, or the mask alone;
//   * one-hot mask of cross_entropy:  equal(labels, arange)  cast(bool->f32)  mul(w, mask)
//     (src/api/ops.cpp:347-354,417-441);
//   * backward of log_softmax:  exp(l)  sum(g, axis=-1, keepdim)  mul(exp, sum)  sub(g, mul)
//     (src/autograd/autograd.cpp:528-546), one block per row;
//   * max_pool2d_backward followed by the where() of ReLU's backward rule: served by the pooling
//     kernel itself (movement.cu, launch_pool_backward_where);
//   * the optimiser's spans: independent scaled_add nodes, one per parameter tensor
//     (python/vkml/optim.py), served by one multi-tensor launch.
//
// A group is taken only when its nodes are consecutive in execution order (the scaled_add group
// may jump over nodes it is independent of), every operand has the
// layout the kernel reads (dense outputs, a bias that is one contiguous vector), and none of its
// members is a gradient that a data-parallel span all-reduces.  VKML_B200_FUSE=0 turns it off.
#include "context.h"

namespace b200 {
namespace {

constexpr int kThreads = 256;

int64_t numel_of(const b200_tensor& t) {
    int64_t n = 1;
    for (int d = 0; d < t.ndim; ++d) n *= t.dims[d];
    return n;
}

bool dense_tensor(const b200_tensor& t) {
    int64_t expected = static_cast<int64_t>(dtype_size(t.dtype));
    for (int i = t.ndim - 1; i >= 0; --i) {
        if (t.dims[i] == 1) continue;
        if (t.strides[i] != expected) return false;
        expected *= t.dims[i];
    }
    return true;
}

bool same_shape(const b200_tensor& a, const b200_tensor& b) {
    if (a.ndim != b.ndim) return false;
    for (int d = 0; d < a.ndim; ++d) {
        if (a.dims[d] != b.dims[d]) return false;
    }
    return true;
}

// `src` is exactly the buffer `out` describes (same address, extents and strides).
bool reads(const b200_tensor& src, const b200_tensor& out) {
    if (src.data != out.data || src.dtype != out.dtype || !same_shape(src, out)) return false;
    for (int d = 0; d < src.ndim; ++d) {
        if (src.dims[d] != 1 && src.strides[d] != out.strides[d]) return false;
    }
    return true;
}

double full_value(const b200_node& n) {
    double v;
    std::memcpy(&v, n.params, sizeof(double));
    return v;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// ---------------------------------------------------------------------------
// [add(x, bias)]  [full  less_equal(y, full)  full]  [relu(y)]      (y = the sum, or x itself)
// ---------------------------------------------------------------------------

struct BiasGroup {
    const float* x;
    const float* bias;  // null: no add, y = x
    float* add;
    float* full_a;      // null: no mask part
    uint8_t* mask;
    float* full_b;
    float* relu;        // null: no relu
    float value_a, value_b;
    int64_t n4;           // quads
    uint32_t inner4;      // quads that share one bias element (0: the bias runs along the quad)
    uint32_t count;       // bias elements
};

__global__ void __launch_bounds__(kThreads) bias_relu_group_kernel(BiasGroup g) {
    pdl_prologue();
    const int64_t step = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < g.n4; i += step) {
        float4 s = reinterpret_cast<const float4*>(g.x)[i];
        if (g.bias != nullptr) {
            float4 b;
            if (g.inner4 != 0) {
                const float v = g.bias[(i / g.inner4) % g.count];
                b = make_float4(v, v, v, v);
            } else {
                b = reinterpret_cast<const float4*>(g.bias)[i % (g.count / 4)];
            }
            s.x = __fadd_rn(s.x, b.x);
            s.y = __fadd_rn(s.y, b.y);
            s.z = __fadd_rn(s.z, b.z);
            s.w = __fadd_rn(s.w, b.w);
            reinterpret_cast<float4*>(g.add)[i] = s;
        }
        if (g.full_a != nullptr) {
            reinterpret_cast<float4*>(g.full_a)[i] = make_float4(g.value_a, g.value_a, g.value_a, g.value_a);
            reinterpret_cast<float4*>(g.full_b)[i] = make_float4(g.value_b, g.value_b, g.value_b, g.value_b);
            uchar4 m;
            m.x = s.x <= g.value_a ? 1 : 0;  // false for NaN, as the CPU's comparison
            m.y = s.y <= g.value_a ? 1 : 0;
            m.z = s.z <= g.value_a ? 1 : 0;
            m.w = s.w <= g.value_a ? 1 : 0;
            reinterpret_cast<uchar4*>(g.mask)[i] = m;
        }
        if (g.relu != nullptr) {
            // relu(x) = x <= 0 ? 0 : x, so a NaN goes through (src/backend/cpu/kernels_elementwise.cpp:223-231)
            float4 r;
            r.x = s.x <= 0.0F ? 0.0F : s.x;
            r.y = s.y <= 0.0F ? 0.0F : s.y;
            r.z = s.z <= 0.0F ? 0.0F : s.z;
            r.w = s.w <= 0.0F ? 0.0F : s.w;
            reinterpret_cast<float4*>(g.relu)[i] = r;
        }
    }
}

// The bias operand of `add`: a broadcast view of ONE contiguous vector, i.e. exactly one axis
// with extent > 1 carries a stride, and that stride is one element.
bool bias_layout(const b200_tensor& b, int64_t& inner, int64_t& count) {
    int axis = -1;
    for (int d = 0; d < b.ndim; ++d) {
        if (b.dims[d] > 1 && b.strides[d] != 0) {
            if (axis >= 0) return false;
            axis = d;
        }
    }
    if (axis < 0 || b.strides[axis] != 4) return false;
    count = b.dims[axis];
    inner = 1;
    for (int d = axis + 1; d < b.ndim; ++d) inner *= b.dims[d];
    return true;
}

// The forms this group takes in a recorded step: all five nodes (a hidden Linear layer), without
// the relu (the layer before the loss, whose relu is emitted later), add + relu alone (a
// convolution, whose mask nodes come with the backward pass) and the mask alone.
size_t fuse_bias_group(b200_ctx* ctx, const b200_node* const* seq, size_t avail) {
    BiasGroup g{};
    size_t at = 0;
    const b200_tensor* y = nullptr;  // what the mask compares and the relu reads
    if (seq[0]->op == B200_OP_ADD) {
        const b200_node& add = *seq[0];
        if (add.out.dtype != B200_F32 || add.n_src != 2 || add.src[0].dtype != B200_F32 || add.src[1].dtype != B200_F32) return 0;
        if (!dense_tensor(add.src[0]) || !same_shape(add.src[0], add.out) || !same_shape(add.src[1], add.out)) return 0;
        int64_t inner = 0, count = 0;
        if (!bias_layout(add.src[1], inner, count)) return 0;
        const bool along = inner == 1 && count % 4 == 0 && aligned16(add.src[1].data);
        if (!along && inner % 4 != 0) return 0;
        if (inner / 4 >= (int64_t(1) << 31) || count >= (int64_t(1) << 31)) return 0;
        if (!aligned16(add.src[0].data) || !aligned16(add.out.data)) return 0;
        g.x = static_cast<const float*>(add.src[0].data);
        g.bias = static_cast<const float*>(add.src[1].data);
        g.add = static_cast<float*>(add.out.data);
        g.inner4 = along ? 0u : static_cast<uint32_t>(inner / 4);
        g.count = static_cast<uint32_t>(count);
        y = &add.out;
        at = 1;
    }
    if (avail >= at + 3 && seq[at]->op == B200_OP_FULL && seq[at + 1]->op == B200_OP_LESS_EQUAL &&
        seq[at + 2]->op == B200_OP_FULL) {
        const b200_node& fa = *seq[at];
        const b200_node& le = *seq[at + 1];
        const b200_node& fb = *seq[at + 2];
        const b200_tensor& cmp = y != nullptr ? *y : le.src[0];
        const bool ok = fa.out.dtype == B200_F32 && fb.out.dtype == B200_F32 && le.out.dtype == B200_BOOL && le.n_src == 2 &&
                        cmp.dtype == B200_F32 && dense_tensor(cmp) && same_shape(fa.out, cmp) && same_shape(fb.out, cmp) &&
                        same_shape(le.out, cmp) && reads(le.src[0], cmp) && reads(le.src[1], fa.out) &&
                        aligned16(cmp.data) && aligned16(fa.out.data) && aligned16(fb.out.data) &&
                        reinterpret_cast<uintptr_t>(le.out.data) % 4 == 0;
        if (ok) {
            if (y == nullptr) {
                y = &le.src[0];
                g.x = static_cast<const float*>(le.src[0].data);
            }
            g.full_a = static_cast<float*>(fa.out.data);
            g.mask = static_cast<uint8_t*>(le.out.data);
            g.full_b = static_cast<float*>(fb.out.data);
            g.value_a = static_cast<float>(full_value(fa));
            g.value_b = static_cast<float>(full_value(fb));
            at += 3;
        }
    }
    if (y == nullptr) return 0;
    if (avail > at && seq[at]->op == B200_OP_RELU && seq[at]->out.dtype == B200_F32 && seq[at]->n_src == 1 &&
        reads(seq[at]->src[0], *y) && same_shape(seq[at]->out, *y) && aligned16(seq[at]->out.data)) {
        g.relu = static_cast<float*>(seq[at]->out.data);
        ++at;
    }
    if (at < 2) return 0;  // a lone add: nothing to fuse
    const int64_t n = numel_of(*y);
    if (n == 0 || n % 4 != 0) return 0;
    g.n4 = n / 4;
    const char* label = g.bias != nullptr ? (g.full_a != nullptr ? (g.relu != nullptr ? "fused.bias_mask_relu" : "fused.bias_mask")
                                                                 : "fused.bias_relu")
                                          : "fused.mask";
    ProfScope scope(ctx, label);
    launch_kernel(ctx, bias_relu_group_kernel, grid_for(g.n4, kThreads), kThreads, 0, g);
    ctx->count_launch();
    check_last_launch("fused bias / mask / relu");
    return at;
}

// ---------------------------------------------------------------------------
// equal(a, b) + cast(bool -> f32) + mul(w, mask)
// ---------------------------------------------------------------------------

struct OneHotGroup {
    const float* a;
    const float* b;
    const float* w;
    uint8_t* eq;
    float* mask;
    float* out;
    int64_t rows, cols;
    int64_t a_row, a_col, b_row, b_col;  // element strides of the compared operands (0 = broadcast)
};

__global__ void __launch_bounds__(kThreads) one_hot_group_kernel(OneHotGroup g) {
    pdl_prologue();
    const int64_t n = g.rows * g.cols;
    const int64_t step = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
        const int64_t r = i / g.cols, c = i - r * g.cols;
        const bool hit = g.a[r * g.a_row + c * g.a_col] == g.b[r * g.b_row + c * g.b_col];
        const float m = hit ? 1.0F : 0.0F;
        g.eq[i] = hit ? 1 : 0;
        g.mask[i] = m;
        g.out[i] = __fmul_rn(g.w[i], m);
    }
}

size_t fuse_one_hot(b200_ctx* ctx, const b200_node* const* seq, size_t avail) {
    if (avail < 3) return 0;
    const b200_node& eq = *seq[0];
    const b200_node& cast = *seq[1];
    const b200_node& mul = *seq[2];
    if (eq.op != B200_OP_EQUAL || cast.op != B200_OP_CAST || mul.op != B200_OP_MUL) return 0;
    if (eq.out.ndim != 2 || eq.out.dtype != B200_BOOL || cast.out.dtype != B200_F32 || mul.out.dtype != B200_F32) return 0;
    if (eq.n_src != 2 || eq.src[0].dtype != B200_F32 || eq.src[1].dtype != B200_F32 || mul.n_src != 2) return 0;
    if (!same_shape(eq.src[0], eq.out) || !same_shape(eq.src[1], eq.out)) return 0;
    if (!reads(cast.src[0], eq.out) || !same_shape(cast.out, eq.out) || !same_shape(mul.out, eq.out)) return 0;
    int w_at = -1;
    if (reads(mul.src[1], cast.out)) w_at = 0;
    else if (reads(mul.src[0], cast.out)) w_at = 1;
    if (w_at < 0) return 0;
    const b200_tensor& w = mul.src[w_at];
    if (w.dtype != B200_F32 || !same_shape(w, mul.out) || !dense_tensor(w)) return 0;
    for (int s = 0; s < 2; ++s) {
        for (int d = 0; d < 2; ++d) {
            if (eq.src[s].strides[d] % 4 != 0 || eq.src[s].strides[d] < 0) return 0;
        }
    }
    if (numel_of(eq.out) == 0) return 0;
    OneHotGroup g{};
    g.a = static_cast<const float*>(eq.src[0].data);
    g.b = static_cast<const float*>(eq.src[1].data);
    g.w = static_cast<const float*>(w.data);
    g.eq = static_cast<uint8_t*>(eq.out.data);
    g.mask = static_cast<float*>(cast.out.data);
    g.out = static_cast<float*>(mul.out.data);
    g.rows = eq.out.dims[0];
    g.cols = eq.out.dims[1];
    g.a_row = eq.src[0].dims[0] > 1 ? eq.src[0].strides[0] / 4 : 0;
    g.a_col = eq.src[0].dims[1] > 1 ? eq.src[0].strides[1] / 4 : 0;
    g.b_row = eq.src[1].dims[0] > 1 ? eq.src[1].strides[0] / 4 : 0;
    g.b_col = eq.src[1].dims[1] > 1 ? eq.src[1].strides[1] / 4 : 0;
    ProfScope scope(ctx, "fused.one_hot_mul");
    launch_kernel(ctx, one_hot_group_kernel, grid_for(g.rows * g.cols, kThreads), kThreads, 0, g);
    ctx->count_launch();
    check_last_launch("fused one-hot");
    return 3;
}

// ---------------------------------------------------------------------------
// backward of log_softmax: exp(l), sum(g, -1, keepdim), exp * sum, g - exp * sum
// ---------------------------------------------------------------------------

struct LsmBackward {
    const float* l;   // log-probabilities [rows, cols]
    const float* gr;  // upstream gradient [rows, cols]
    float* e;         // exp(l)
    float* s;         // row sums of gr [rows]
    float* es;        // e * s
    float* out;       // gr - e * s
    int64_t rows, cols;
};

// One block per row.  The row sum is taken in a fixed order -- each thread adds its strided
// elements in index order, the 32 lanes of a warp are folded by a butterfly, the warps in warp
// order -- so repeated runs give identical bytes.
__global__ void __launch_bounds__(kThreads) lsm_backward_kernel(LsmBackward g) {
    pdl_prologue();
    __shared__ float partial[kThreads / 32];
    __shared__ float total;
    for (int64_t r = blockIdx.x; r < g.rows; r += gridDim.x) {
        const float* gr = g.gr + r * g.cols;
        float acc = 0.0F;
        for (int64_t c = threadIdx.x; c < g.cols; c += kThreads) acc = __fadd_rn(acc, gr[c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = partial[0];
            for (int w = 1; w < kThreads / 32; ++w) t = __fadd_rn(t, partial[w]);
            total = t;
            g.s[r] = t;
        }
        __syncthreads();
        const float s = total;
        const float* l = g.l + r * g.cols;
        for (int64_t c = threadIdx.x; c < g.cols; c += kThreads) {
            const float e = expf(l[c]);
            const float es = __fmul_rn(e, s);
            g.e[r * g.cols + c] = e;
            g.es[r * g.cols + c] = es;
            g.out[r * g.cols + c] = __fsub_rn(gr[c], es);
        }
        __syncthreads();
    }
}

size_t fuse_lsm_backward(b200_ctx* ctx, const b200_node* const* seq, size_t avail) {
    if (avail < 4) return 0;
    const b200_node& ex = *seq[0];
    const b200_node& sum = *seq[1];
    const b200_node& mul = *seq[2];
    const b200_node& sub = *seq[3];
    if (ex.op != B200_OP_EXP || sum.op != B200_OP_SUM || mul.op != B200_OP_MUL || sub.op != B200_OP_SUB) return 0;
    if (ex.out.ndim != 2 || ex.out.dtype != B200_F32 || !dense_tensor(ex.src[0]) || ex.src[0].dtype != B200_F32) return 0;
    const int64_t rows = ex.out.dims[0], cols = ex.out.dims[1];
    if (rows == 0 || cols == 0 || (cols < 64 && rows > 8192)) return 0;  // (many tiny rows: a block per row would idle)
    const b200_tensor& gr = sum.src[0];
    if (gr.dtype != B200_F32 || !same_shape(gr, ex.out) || !dense_tensor(gr)) return 0;
    uint32_t mask = 0;
    uint8_t keepdim = 0;
    std::memcpy(&mask, sum.params, 4);
    std::memcpy(&keepdim, sum.params + 4, 1);
    if (mask != 2u || keepdim == 0 || sum.out.ndim != 2 || sum.out.dims[0] != rows || sum.out.dims[1] != 1) return 0;
    // mul(exp, sum broadcast along the row), sub(g, mul)
    if (mul.n_src != 2 || !reads(mul.src[0], ex.out) || !same_shape(mul.out, ex.out)) return 0;
    const b200_tensor& sb = mul.src[1];
    if (sb.data != sum.out.data || sb.ndim != 2 || sb.dims[0] != rows || sb.dims[1] != cols || sb.strides[1] != 0 ||
        (rows > 1 && sb.strides[0] != 4)) {
        return 0;
    }
    if (sub.n_src != 2 || !reads(sub.src[0], gr) || !reads(sub.src[1], mul.out) || !same_shape(sub.out, ex.out)) return 0;
    LsmBackward g{};
    g.l = static_cast<const float*>(ex.src[0].data);
    g.gr = static_cast<const float*>(gr.data);
    g.e = static_cast<float*>(ex.out.data);
    g.s = static_cast<float*>(sum.out.data);
    g.es = static_cast<float*>(mul.out.data);
    g.out = static_cast<float*>(sub.out.data);
    g.rows = rows;
    g.cols = cols;
    ProfScope scope(ctx, "fused.log_softmax_backward");
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, int64_t(sm_count()) * 8));
    launch_kernel(ctx, lsm_backward_kernel, grid, kThreads, 0, g);
    ctx->count_launch();
    check_last_launch("fused log_softmax backward");
    return 4;
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// scaled_add over several tensors: the optimiser's spans
// ---------------------------------------------------------------------------
// An optimiser step reaches the backend as spans of nothing but scaled_add nodes, one per parameter
// tensor (python/vkml/optim.py: the velocity update of every parameter in one span, the parameter
// update in the next).  The nodes are independent, so one launch serves them all: every block takes
// one 4096-element tile of one tensor.  Same arithmetic as the single-tensor kernel (two rounded
// products, one rounded sum).
constexpr int kGroupTensors = 16;
constexpr int kGroupTile = 4096;

struct ScaledAddGroup {
    float* out[kGroupTensors];
    const float* a[kGroupTensors];
    const float* b[kGroupTensors];
    int64_t count[kGroupTensors];
    float alpha[kGroupTensors], beta[kGroupTensors];
    uint32_t first_block[kGroupTensors + 1];
    uint32_t vec_mask;  // bit t: tensor t may be walked in 16-byte quads
    int n;
};

__global__ void __launch_bounds__(kThreads) scaled_add_group_kernel(const __grid_constant__ ScaledAddGroup g) {
    pdl_prologue();
    int t = 0;
    while (t + 1 < g.n && blockIdx.x >= g.first_block[t + 1]) ++t;
    const int64_t base = int64_t(blockIdx.x - g.first_block[t]) * kGroupTile;
    const int64_t count = g.count[t];
    const float alpha = g.alpha[t], beta = g.beta[t];
    if ((g.vec_mask >> t) & 1u) {
        const float4* __restrict__ a = reinterpret_cast<const float4*>(g.a[t] + base);
        const float4* __restrict__ b = reinterpret_cast<const float4*>(g.b[t] + base);
        float4* __restrict__ o = reinterpret_cast<float4*>(g.out[t] + base);
        const int quads = static_cast<int>(min(int64_t(kGroupTile), count - base) / 4);
        float4 x[4], y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = threadIdx.x + u * kThreads;
            if (q < quads) {
                x[u] = a[q];
                y[u] = b[q];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = threadIdx.x + u * kThreads;
            if (q < quads) {
                float4 r;
                r.x = __fadd_rn(__fmul_rn(x[u].x, alpha), __fmul_rn(y[u].x, beta));
                r.y = __fadd_rn(__fmul_rn(x[u].y, alpha), __fmul_rn(y[u].y, beta));
                r.z = __fadd_rn(__fmul_rn(x[u].z, alpha), __fmul_rn(y[u].z, beta));
                r.w = __fadd_rn(__fmul_rn(x[u].w, alpha), __fmul_rn(y[u].w, beta));
                o[q] = r;
            }
        }
    } else {
        const int n = static_cast<int>(min(int64_t(kGroupTile), count - base));
        for (int i = threadIdx.x; i < n; i += kThreads) {
            g.out[t][base + i] = __fadd_rn(__fmul_rn(g.a[t][base + i], alpha), __fmul_rn(g.b[t][base + i], beta));
        }
    }
}

bool overlaps(const void* p, size_t pn, const void* q, size_t qn) {
    const char* a = static_cast<const char*>(p);
    const char* b = static_cast<const char*>(q);
    return a < b + qn && b < a + pn;
}

}  // namespace

// `seq`: the next nodes of a span in execution order, the first a scaled_add.  Picks the scaled_add
// nodes over dense f32 tensors among them that are independent of every other node of `seq` up to
// the last one picked (none writes what another reads or writes, so running them first changes
// nothing), marks them in `picked` and serves them with one launch.  Returns how many it served
// (0: fewer than two qualified).
size_t launch_scaled_add_group(b200_ctx* ctx, const b200_node* const* seq, size_t avail, bool* picked) {
    ScaledAddGroup g{};
    uint64_t blocks = 0;
    size_t n = 0;
    auto bytes_of = [](const b200_tensor& t) {
        // the span of addresses the tensor can touch (strided views included)
        int64_t hi = static_cast<int64_t>(dtype_size(t.dtype));
        for (int d = 0; d < t.ndim; ++d) {
            if (t.dims[d] > 1) hi += (t.dims[d] - 1) * std::abs(t.strides[d]);
        }
        return static_cast<size_t>(hi);
    };
    auto independent = [&](const b200_node& x, const b200_node& y) {
        // x and y may run in either order: neither writes what the other reads or writes
        for (uint32_t s = 0; s < y.n_src && s < B200_MAX_SRC; ++s) {
            if (y.src[s].data != nullptr && overlaps(x.out.data, bytes_of(x.out), y.src[s].data, bytes_of(y.src[s]))) return false;
        }
        for (uint32_t s = 0; s < x.n_src && s < B200_MAX_SRC; ++s) {
            if (x.src[s].data != nullptr && overlaps(y.out.data, bytes_of(y.out), x.src[s].data, bytes_of(x.src[s]))) return false;
        }
        return !overlaps(x.out.data, bytes_of(x.out), y.out.data, bytes_of(y.out));
    };
    for (size_t k = 0; k < avail; ++k) picked[k] = false;
    for (size_t k = 0; k < avail && n < static_cast<size_t>(kGroupTensors); ++k) {
        const b200_node& node = *seq[k];
        if (node.op != B200_OP_SCALED_ADD || node.n_src != 2) continue;
        const b200_tensor& o = node.out;
        bool ok = o.dtype == B200_F32 && dense_tensor(o) && o.data != nullptr;
        for (int s = 0; s < 2 && ok; ++s) {
            ok = node.src[s].dtype == B200_F32 && same_shape(node.src[s], o) && dense_tensor(node.src[s]) &&
                 node.src[s].data != nullptr;
        }
        for (int d = 0; d < o.ndim && ok; ++d) ok = o.strides[d] >= 0;
        for (size_t e = 0; e < k && ok; ++e) ok = independent(node, *seq[e]);  // members and the nodes it jumps over
        const int64_t count = numel_of(o);
        ok = ok && blocks + static_cast<uint64_t>((count + kGroupTile - 1) / kGroupTile) < (uint64_t(1) << 31);
        if (!ok) continue;
        const ScaledAddParams prm = get_params<ScaledAddParams>(node);
        g.out[n] = static_cast<float*>(o.data);
        g.a[n] = static_cast<const float*>(node.src[0].data);
        g.b[n] = static_cast<const float*>(node.src[1].data);
        g.count[n] = count;
        g.alpha[n] = prm.alpha;
        g.beta[n] = prm.beta;
        g.first_block[n] = static_cast<uint32_t>(blocks);
        if (count % 4 == 0 && aligned16(g.out[n]) && aligned16(g.a[n]) && aligned16(g.b[n])) g.vec_mask |= 1u << n;
        blocks += static_cast<uint64_t>((count + kGroupTile - 1) / kGroupTile);
        picked[k] = true;
        ++n;
    }
    if (n < 2) {
        for (size_t k = 0; k < avail; ++k) picked[k] = false;
        return 0;
    }
    g.first_block[n] = static_cast<uint32_t>(blocks);
    g.n = static_cast<int>(n);
    ProfScope scope(ctx, "fused.scaled_add_group");
    launch_kernel(ctx, scaled_add_group_kernel, static_cast<unsigned>(blocks), kThreads, 0, g);
    ctx->count_launch();
    check_last_launch("fused scaled_add group");
    return n;
}

// Tries every pattern at the head of `seq` (the span's remaining computed nodes, in execution
// order); returns how many nodes one fused launch served, or 0.
size_t launch_fused(b200_ctx* ctx, const b200_node* const* seq, size_t avail) {
    if (size_t n = fuse_bias_group(ctx, seq, avail)) return n;
    if (size_t n = fuse_one_hot(ctx, seq, avail)) return n;
    if (size_t n = fuse_lsm_backward(ctx, seq, avail)) return n;
    return 0;
}

}  // namespace b200
