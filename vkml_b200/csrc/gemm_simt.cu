// fp32 GEMM on the CUDA cores: the path for shapes the tensor-core kernel
// does not take (tiny or ragged problems such as the 64x10 logits of the MNIST
// MLP or conv1's K = 27) and for B200_GEMM_FP32.
//
// 64x64 output tile, K in steps of 16, 256 threads with a 4x4 register block, products
// rounded before they are summed (no fused multiply-add: this is the exactness path);
// operands are read through their element strides, the staging index order is
// picked per operand so the global reads follow whichever axis has unit stride
// (a transposed view is read along its own rows).  A long K with too few tiles
// to fill 148 SMs is split across blockIdx.z into partial sums in the context's
// scratch buffer and folded in split order (deterministic, no atomics), the
// role gemm_split_k_reduce.comp plays in vkML's Vulkan backend.
#include "gemm.h"

namespace b200 {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmProblem p, float* __restrict__ dst, int64_t k_chunk, int64_t split_stride) {
    pdl_prologue();
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];

    const int64_t tiles_n = (p.n + BN - 1) / BN;
    const int64_t tiles_m = (p.m + BM - 1) / BM;
    int64_t t = blockIdx.x;
    const int64_t tn = t % tiles_n;
    t /= tiles_n;
    const int64_t tm = t % tiles_m;
    t /= tiles_m;
    const int64_t i1 = t % p.b1;
    const int64_t i0 = t / p.b1;

    const float* A = p.a + i0 * p.a_s[0] + i1 * p.a_s[1];
    const float* B = p.b + i0 * p.b_s[0] + i1 * p.b_s[1];
    const int64_t m0 = tm * BM, n0 = tn * BN;
    const int64_t k_begin = int64_t(blockIdx.z) * k_chunk;
    const int64_t k_end = min(k_begin + k_chunk, p.k);

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const bool a_k_fast = p.a_s[3] == 1 || p.a_s[2] != 1;  // read A along k unless m is the unit axis
    const bool b_n_fast = p.b_s[3] == 1 || p.b_s[2] != 1;  // read B along n unless k is the unit axis

    float acc[4][4] = {};

    // The next K-block travels from global memory to registers while the current one is
    // multiplied out of shared memory, so the load latency is paid once per tile, not per block.
    float ra[4], rb[4];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = tid + 256 * j;
            const int mm = a_k_fast ? (e >> 4) : (e & 63);
            const int ka = a_k_fast ? (e & 15) : (e >> 6);
            const int64_t gm = m0 + mm, gka = k0 + ka;
            ra[j] = (gm < p.m && gka < k_end) ? A[gm * p.a_s[2] + gka * p.a_s[3]] : 0.0F;
            const int nn = b_n_fast ? (e & 63) : (e >> 4);
            const int kb = b_n_fast ? (e >> 6) : (e & 15);
            const int64_t gn = n0 + nn, gkb = k0 + kb;
            rb[j] = (gn < p.n && gkb < k_end) ? B[gkb * p.b_s[2] + gn * p.b_s[3]] : 0.0F;
        }
    };
    fetch(k_begin);
    for (int64_t k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = tid + 256 * j;
            As[a_k_fast ? (e & 15) : (e >> 6)][a_k_fast ? (e >> 4) : (e & 63)] = ra[j];
            Bs[b_n_fast ? (e >> 6) : (e & 15)][b_n_fast ? (e & 63) : (e >> 4)] = rb[j];
        }
        __syncthreads();
        if (k0 + BK < k_end) {
            fetch(k0 + BK);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float a[4] = {av.x, av.y, av.z, av.w};
            const float b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // a rounded product, then a rounded add -- never a fused multiply-add.  vkML's
                    // kernels round every product (shaders/gemm_reg.comp:215 `precise`; the CPU
                    // backend multiplies, then sums), and its adversarial inputs tell the two apart:
                    // alternating +-1e7 sums to exactly zero only if each 1e14 is rounded before it
                    // is added, and an overflowing product must become an infinity of its own sign
                    // so that +inf and -inf meet as NaN (tests/python/test_invariants.py:496-531).
                    acc[i][j] = __fadd_rn(__fmul_rn(a[i], b[j]), acc[i][j]);
                }
            }
        }
        __syncthreads();
    }

    float* C = dst + int64_t(blockIdx.z) * split_stride + ((i0 * p.b1) + i1) * p.m * p.n;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn < p.n) {
                C[gm * p.n + gn] = acc[i][j];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
split_fold_kernel(float* __restrict__ out, const float* __restrict__ partial, int64_t n, int splits) {
    pdl_prologue();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) {
            acc += partial[int64_t(s) * n + i];
        }
        out[i] = acc;
    }
}

}  // namespace

void gemm_simt(b200_ctx* ctx, const GemmProblem& p) {
    const int64_t batches = p.b0 * p.b1;
    const int64_t out_elems = batches * p.m * p.n;
    if (out_elems == 0) {
        return;
    }
    if (p.k == 0) {
        B200_CUDA_CHECK(cudaMemsetAsync(p.out, 0, sizeof(float) * out_elems, ctx->stream));
        return;
    }
    const int64_t tiles = batches * ceil_div(p.m, BM) * ceil_div(p.n, BN);
    if (tiles > 0x7fffffffLL) {
        fail(B200_NOT_IMPLEMENTED, "matmul: too many output tiles for one launch");
    }
    int64_t splits = 1;
    // few tiles and a long K: spread K over the idle SMs in chunks of at least 48 (three
    // K-blocks, enough for the register prefetch to overlap anything)
    if (tiles < sm_count() && p.k >= 192) {
        splits = std::min<int64_t>(ceil_div(2 * sm_count(), tiles), p.k / 48);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 64));
    }
    int64_t k_chunk = ceil_div(ceil_div(p.k, splits), BK) * BK;
    splits = ceil_div(p.k, k_chunk);
    float* dst = p.out;
    if (splits > 1) {
        dst = static_cast<float*>(ctx->ensure_workspace(sizeof(float) * out_elems * splits));
    }
    dim3 grid(static_cast<unsigned>(tiles), 1, static_cast<unsigned>(splits));
    ProfScope scope(ctx, "matmul.fp32_simt");
    launch_kernel(ctx, gemm_simt_kernel, grid, 256, 0, p, dst, k_chunk, out_elems);
    ctx->count_launch();
    if (splits > 1) {
        launch_kernel(ctx, split_fold_kernel, grid_for(out_elems, 256), 256, 0, p.out, dst, out_elems,
                                                                           static_cast<int>(splits));
        ctx->count_launch();
    }
    check_last_launch("matmul (simt)");
}

}  // namespace b200
