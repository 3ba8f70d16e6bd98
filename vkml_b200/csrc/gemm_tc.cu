// fp32 GEMM on the Blackwell tensor cores: tcgen05.mma (kind::tf32) with TMEM
// accumulators, operands staged by TMA, 3xTF32 split emulation.
//
// Arithmetic.  Each fp32 operand x is split into hi = tf32(x) (round to
// nearest) and lo = tf32(x - hi); the product a*b is accumulated in fp32 as
//     a_lo*b_hi + a_hi*b_lo + a_hi*b_hi          (small terms first)
// by three tensor-core MMAs into ONE TMEM accumulator.  The dropped a_lo*b_lo
// term is ~2^-22 relative, so the result carries fp32-grade error.  With
// B200_GEMM_TF32 only a_hi*b_hi is issued (plain TF32, explicit opt-in).
//
// Data layout.  A pre-pass (split_kernel) reads the operands through their own
// strides -- transposed views, broadcast batches, slices: whatever the graph
// hands over -- and writes K-major planes into the context's scratch buffer:
//     A_hi, A_lo : [batches_a * M][Kp]     B_hi, B_lo : [batches_b * N][Kp]
// with Kp = K rounded up to 32 and zero-filled, so every TMA tile is a legal,
// 128-byte-aligned box regardless of the caller's pitches.  A broadcast batch
// (both batch strides 0) is stored once.
//
// Main kernel: persistent, one CTA per SM, 6 warps:
//     warp 0   TMA producer: per K-block of 32 floats, 4 boxes
//              (A_hi, A_lo: 128 rows; B_hi, B_lo: BN rows) into a ring of
//              128B-swizzled shared-memory stages, completion on an mbarrier;
//     warp 1   allocates TMEM, one elected lane issues the tcgen05.mma
//              instructions (M=128, N=BN, K=8 each) and commits stage release /
//              accumulator-ready onto mbarriers;
//     warps 2-5  epilogue: tcgen05.ld the 128 x BN fp32 accumulator (each warp
//              its own 32-lane quarter), store to C with bounds checks.
// Two accumulators live in TMEM so the epilogue of tile i overlaps the MMAs of
// tile i+1.  Tiles are walked in groups of 16 M-tiles so the CTAs running at one
// time share operand panels in L2.  A long K with few tiles is split across CTAs
// into fp32 partial planes that a second kernel folds in split order
// (deterministic, no atomics).
//
// Every wait on an mbarrier is bounded: when the limit runs out the kernel
// records kStatusWaitTimedOut in the context's status word, all roles leave
// their loops, TMEM is freed and the kernel returns; the host reports
// B200_TIMEOUT at the next synchronize.
#include "gemm.h"

#include <cuda.h>  // CUtensorMap and the cuTensorMapEncodeTiled prototype (types only)

namespace b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 32;          // floats per K-block = one 128-byte swizzle row
constexpr int UMMA_K = 8;       // tf32
constexpr int kThreads = 192;
constexpr int kGroupM = 16;
constexpr uint64_t kWaitLimitNs = 4000000000ULL;  // 4 s

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait. Returns false (and raises the abort flag) when the limit ran out
// or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* status) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const uint64_t start = global_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ff) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            if (global_ns() - start > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimedOut);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are exactly one
// 128-byte swizzle row (32 floats): 8-row groups are 1024 bytes apart (the
// stride-dimension offset); the leading-dimension offset is unused because the
// K extent of one instruction (32 bytes) lies inside the swizzle row.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, bits 0-13
    d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride-dimension byte offset, bits 32-45
    d |= static_cast<uint64_t>(1) << 46;                     // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                     // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor: D = f32, A = B = tf32, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// Operand split pre-pass
// ---------------------------------------------------------------------------

__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    float fh = __uint_as_float(h);
    if (isinf(fh) && !isinf(x)) {
        fh = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);  // rounding overflowed: truncate instead
    }
    float fl = 0.0F;
    if (isfinite(x)) {
        uint32_t l;
        const float rest = x - fh;  // exact
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
        fl = __uint_as_float(l);
    }
    hi = fh;
    lo = fl;
}

struct SplitArgs {
    const float* src;
    float* hi;
    float* lo;           // null: single-pass TF32
    int64_t b1;          // inner batch extent (outer is implied by the grid)
    int64_t rows, k, kp;
    int64_t s_b0, s_b1, s_r, s_k;  // element strides of src
    int64_t n_batches;
};

// One 32x32 (rows x k) tile per block iteration; reads follow whichever of the
// two axes has unit stride, writes are always along k (dense planes).
__global__ void __launch_bounds__(256) split_kernel(SplitArgs a) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t tiles_k = a.kp / 32;
    const int64_t tiles_r = (a.rows + 31) / 32;
    const int64_t n_tiles = tiles_k * tiles_r * a.n_batches;
    const bool k_fast = a.s_k == 1 || a.s_r != 1;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t tk = t % tiles_k;
        const int64_t tr = (t / tiles_k) % tiles_r;
        const int64_t b = t / (tiles_k * tiles_r);
        const float* src = a.src + (b / a.b1) * a.s_b0 + (b % a.b1) * a.s_b1;
        const int64_t r0 = tr * 32, k0 = tk * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int rr, kk;
            if (k_fast) {
                kk = tx;
                rr = ty + 8 * j;
            } else {
                rr = tx;
                kk = ty + 8 * j;
            }
            const int64_t r = r0 + rr, k = k0 + kk;
            tile[rr][kk] = (r < a.rows && k < a.k) ? src[r * a.s_r + k * a.s_k] : 0.0F;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int rr = ty + 8 * j;
            const int64_t r = r0 + rr;
            if (r < a.rows) {
                float hi, lo;
                split_tf32(tile[rr][tx], hi, lo);
                const int64_t o = (b * a.rows + r) * a.kp + k0 + tx;
                a.hi[o] = hi;
                if (a.lo != nullptr) {
                    a.lo[o] = lo;
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------

struct TcArgs {
    float* out;            // C, or the partial planes when splits > 1
    int64_t m, n;
    int64_t batches;       // B0*B1
    int64_t a_batch_rows;  // rows between consecutive batches in the A planes (0: broadcast)
    int64_t b_batch_rows;
    int64_t k_blocks;      // Kp / 32
    int64_t kb_per_split;
    int splits;
    int64_t split_stride;  // elements between partial planes
    int64_t tiles_m, tiles_n;
    uint32_t* status;
};

template <int BN, int STAGES>
struct Smem {
    static constexpr int kABytes = BM * BK * 4;  // one A plane tile
    static constexpr int kBBytes = BN * BK * 4;
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

template <int BN, int STAGES, bool THREE_PASS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
               const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
               TcArgs g) {
    using S = Smem<BN, STAGES>;
    constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr uint32_t kIdesc = make_idesc(BM, BN);
    constexpr uint32_t kStageTx = THREE_PASS ? S::kStageBytes : (S::kABytes + S::kBBytes);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * S::kStageBytes;
    // barrier slots (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;

    const int64_t tiles_per_batch = g.tiles_m * g.tiles_n;
    const int64_t n_units = tiles_per_batch * g.batches * g.splits;

    // unit -> (split, batch, m tile, n tile); M-tiles walked in groups of kGroupM
    auto decode = [&](int64_t u, int& split, int64_t& batch, int64_t& tm, int64_t& tn) {
        split = static_cast<int>(u % g.splits);
        int64_t t = u / g.splits;
        batch = t / tiles_per_batch;
        t -= batch * tiles_per_batch;
        const int64_t group_size = int64_t(kGroupM) * g.tiles_n;
        const int64_t group = t / group_size;
        const int64_t first_m = group * kGroupM;
        const int64_t rows_in_group = min(int64_t(kGroupM), g.tiles_m - first_m);
        const int64_t in_group = t - group * group_size;
        tm = first_m + in_group % rows_in_group;
        tn = in_group / rows_in_group;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                int split;
                int64_t batch, tm, tn;
                decode(u, split, batch, tm, tn);
                const int a_row = static_cast<int>(batch * g.a_batch_rows + tm * BM);
                const int b_row = static_cast<int>(batch * g.b_batch_rows + tn * BN);
                const int64_t kb0 = int64_t(split) * g.kb_per_split;
                const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
                for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_p, g.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t stage = base + s * S::kStageBytes;
                    const int kc = static_cast<int>(kb * BK);
                    mbar_arrive_expect_tx(full_bar(s), kStageTx);
                    tma_load_2d(stage, &map_a_hi, full_bar(s), kc, a_row);
                    tma_load_2d(stage + 2 * S::kABytes, &map_b_hi, full_bar(s), kc, b_row);
                    if (THREE_PASS) {
                        tma_load_2d(stage + S::kABytes, &map_a_lo, full_bar(s), kc, a_row);
                        tma_load_2d(stage + 2 * S::kABytes + S::kBBytes, &map_b_lo, full_bar(s), kc, b_row);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            uint32_t tile_it = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++tile_it) {
                int split;
                int64_t batch, tm, tn;
                decode(u, split, batch, tm, tn);
                const int acc = tile_it & 1;
                const uint32_t aph = (tile_it >> 1) & 1;
                if (!mbar_wait(acc_empty(acc), aph ^ 1, abort_p, g.status)) {
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int64_t kb0 = int64_t(split) * g.kb_per_split;
                const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
                for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full_bar(s), ph, abort_p, g.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t stage = base + s * S::kStageBytes;
                    const uint64_t a_hi = smem_desc_sw128(stage);
                    const uint64_t a_lo = smem_desc_sw128(stage + S::kABytes);
                    const uint64_t b_hi = smem_desc_sw128(stage + 2 * S::kABytes);
                    const uint64_t b_lo = smem_desc_sw128(stage + 2 * S::kABytes + S::kBBytes);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t adv = static_cast<uint64_t>((kk * UMMA_K * 4) >> 4);  // +32 bytes per step
                        const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
                        if (THREE_PASS) {
                            umma_tf32(d_tmem, a_lo + adv, b_hi + adv, kIdesc, first);
                            umma_tf32(d_tmem, a_hi + adv, b_lo + adv, kIdesc, 1u);
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, kIdesc, 1u);
                        } else {
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, kIdesc, first);
                        }
                    }
                    umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
                }
                if (ok) {
                    umma_commit(acc_full(acc));
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
        uint32_t tile_it = 0;
        bool ok = true;
        for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++tile_it) {
            int split;
            int64_t batch, tm, tn;
            decode(u, split, batch, tm, tn);
            const int acc = tile_it & 1;
            const uint32_t aph = (tile_it >> 1) & 1;
            if (!mbar_wait(acc_full(acc), aph, abort_p, g.status)) {
                break;
            }
            tc_fence_after();
            const int64_t row = tm * BM + quarter * 32 + lane;
            const int64_t col0 = tn * BN;
            float* dst = g.out + int64_t(split) * g.split_stride + (batch * g.m + row) * g.n + col0;
            const bool row_ok = row < g.m;
            const bool vec_ok = (g.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0) &&
                                ((g.split_stride % 4) == 0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                if (col0 + c * 32 >= g.n) {
                    break;  // uniform across the warp
                }
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + c * 32, r);
                if (row_ok) {
                    float* p = dst + c * 32;
                    const int64_t left = g.n - (col0 + c * 32);
                    if (vec_ok && left >= 32) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float4 v;
                            v.x = __uint_as_float(r[4 * j]);
                            v.y = __uint_as_float(r[4 * j + 1]);
                            v.z = __uint_as_float(r[4 * j + 2]);
                            v.w = __uint_as_float(r[4 * j + 3]);
                            reinterpret_cast<float4*>(p)[j] = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < left) {
                                p[j] = __uint_as_float(r[j]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(acc_empty(acc));
            }
        }
    }

    __syncthreads();
    if (abort_flag != 0) {
        // give copies that may still be in flight time to land before the CTA retires
        for (int i = 0; i < 200; ++i) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

__global__ void __launch_bounds__(256)
fold_partials_kernel(float* __restrict__ out, const float* __restrict__ partial, int64_t n, int splits) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) {
            acc += partial[int64_t(s) * n + i];
        }
        out[i] = acc;
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return static_cast<EncodeTiledFn>(nullptr);
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// K-major plane [rows][kp] of f32, boxes of 32 floats x box_rows, 128-byte swizzle.
CUtensorMap make_map(float* plane, int64_t rows, int64_t kp, int box_rows) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kp), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kp) * sizeof(float)};
    const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, plane, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        fail(B200_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc));
    }
    return m;
}

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

template <int BN, int STAGES>
void launch_main(b200_ctx* ctx, bool three_pass, const CUtensorMap& ah, const CUtensorMap& al,
                 const CUtensorMap& bh, const CUtensorMap& bl, const TcArgs& g, int grid) {
    using S = Smem<BN, STAGES>;
    if (three_pass) {
        B200_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        gemm_tc_kernel<BN, STAGES, true><<<grid, kThreads, S::kTotal, ctx->stream>>>(ah, al, bh, bl, g);
    } else {
        B200_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        gemm_tc_kernel<BN, STAGES, false><<<grid, kThreads, S::kTotal, ctx->stream>>>(ah, al, bh, bl, g);
    }
}

}  // namespace

bool gemm_tc_eligible(const b200_ctx* ctx, const GemmProblem& p) {
    if (ctx->prop.major != 10 || encode_tiled() == nullptr) {
        return false;
    }
    const int64_t batches = p.b0 * p.b1;
    if (p.m < 32 || p.n < 16 || p.k < 32 || batches < 1) {
        return false;
    }
    const double flops = 2.0 * double(p.m) * double(p.n) * double(p.k) * double(batches);
    if (flops < double(1 << 25)) {
        return false;  // launch-bound either way: the single CUDA-core kernel is cheaper than split + GEMM
    }
    // TMA coordinates are 32-bit
    const int64_t kp = align_up(p.k, BK);
    if (kp >= (int64_t(1) << 31) || batches * p.m >= (int64_t(1) << 31) || batches * p.n >= (int64_t(1) << 31)) {
        return false;
    }
    return true;
}

void gemm_tc(b200_ctx* ctx, const GemmProblem& p, bool three_pass) {
    const int64_t batches = p.b0 * p.b1;
    const int64_t kp = align_up(p.k, BK);
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    const bool b_bcast = (p.b_s[0] == 0 || p.b0 == 1) && (p.b_s[1] == 0 || p.b1 == 1);
    const int64_t nb_a = a_bcast ? 1 : batches;
    const int64_t nb_b = b_bcast ? 1 : batches;

    int bn = 64;
    if (p.n > 64) bn = 128;
    if (p.n > 128 && p.m * p.n * batches >= int64_t(128) * 256 * kSmCount) bn = 256;
    const int64_t tiles_m = ceil_div(p.m, BM);
    const int64_t tiles_n = ceil_div(p.n, bn);
    const int64_t tiles = tiles_m * tiles_n * batches;
    const int64_t k_blocks = kp / BK;

    // split K when the tiles alone cannot fill the machine
    int64_t splits = 1;
    if (tiles < kSmCount && k_blocks >= 16) {
        splits = std::min<int64_t>(ceil_div(kSmCount, tiles), k_blocks / 8);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 64));
    }
    int64_t kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);

    const int64_t planes = three_pass ? 2 : 1;
    const int64_t a_plane = align_up(nb_a * p.m * kp * 4, 1024);
    const int64_t b_plane = align_up(nb_b * p.n * kp * 4, 1024);
    const int64_t out_elems = batches * p.m * p.n;
    const int64_t partial_bytes = splits > 1 ? align_up(out_elems * splits * 4, 1024) : 0;
    char* ws = static_cast<char*>(
        ctx->ensure_workspace(static_cast<size_t>(planes * (a_plane + b_plane) + partial_bytes + 1024)));
    ws = reinterpret_cast<char*>(align_up(reinterpret_cast<int64_t>(ws), 1024));
    float* a_hi = reinterpret_cast<float*>(ws);
    float* a_lo = three_pass ? reinterpret_cast<float*>(ws + a_plane) : nullptr;
    float* b_hi = reinterpret_cast<float*>(ws + planes * a_plane);
    float* b_lo = three_pass ? reinterpret_cast<float*>(ws + planes * a_plane + b_plane) : nullptr;
    float* partial = splits > 1 ? reinterpret_cast<float*>(ws + planes * (a_plane + b_plane)) : nullptr;

    // ---- operand split ----
    {
        SplitArgs s{};
        s.src = p.a;
        s.hi = a_hi;
        s.lo = a_lo;
        s.b1 = a_bcast ? 1 : p.b1;
        s.rows = p.m;
        s.k = p.k;
        s.kp = kp;
        s.s_b0 = a_bcast ? 0 : p.a_s[0];
        s.s_b1 = a_bcast ? 0 : p.a_s[1];
        s.s_r = p.a_s[2];
        s.s_k = p.a_s[3];
        s.n_batches = nb_a;
        const int64_t t = (kp / 32) * ceil_div(p.m, 32) * nb_a;
        {
            ProfScope scope(ctx, "matmul.split_a");
            split_kernel<<<grid_for(t, 1, 16), 256, 0, ctx->stream>>>(s);
        }
        ctx->count_launch();
        s.src = p.b;
        s.hi = b_hi;
        s.lo = b_lo;
        s.b1 = b_bcast ? 1 : p.b1;
        s.rows = p.n;
        s.s_b0 = b_bcast ? 0 : p.b_s[0];
        s.s_b1 = b_bcast ? 0 : p.b_s[1];
        s.s_r = p.b_s[3];
        s.s_k = p.b_s[2];
        s.n_batches = nb_b;
        const int64_t t2 = (kp / 32) * ceil_div(p.n, 32) * nb_b;
        ProfScope scope(ctx, "matmul.split_b");
        split_kernel<<<grid_for(t2, 1, 16), 256, 0, ctx->stream>>>(s);
        ctx->count_launch();
        check_last_launch("matmul (operand split)");
    }

    // ---- main kernel ----
    const CUtensorMap ah = make_map(a_hi, nb_a * p.m, kp, BM);
    const CUtensorMap al = three_pass ? make_map(a_lo, nb_a * p.m, kp, BM) : ah;
    const CUtensorMap bh = make_map(b_hi, nb_b * p.n, kp, bn);
    const CUtensorMap bl = three_pass ? make_map(b_lo, nb_b * p.n, kp, bn) : bh;

    TcArgs g{};
    g.out = splits > 1 ? partial : p.out;
    g.m = p.m;
    g.n = p.n;
    g.batches = batches;
    g.a_batch_rows = a_bcast ? 0 : p.m;
    g.b_batch_rows = b_bcast ? 0 : p.n;
    g.k_blocks = k_blocks;
    g.kb_per_split = kb_per_split;
    g.splits = static_cast<int>(splits);
    g.split_stride = out_elems;
    g.tiles_m = tiles_m;
    g.tiles_n = tiles_n;
    g.status = ctx->d_status;
    const int grid = static_cast<int>(std::min<int64_t>(tiles * splits, ctx->prop.multiProcessorCount));
    {
        ProfScope scope(ctx, three_pass ? "matmul.tcgen05_3xtf32" : "matmul.tcgen05_tf32");
        if (bn == 256) {
            launch_main<256, 2>(ctx, three_pass, ah, al, bh, bl, g, grid);
        } else if (bn == 128) {
            launch_main<128, 3>(ctx, three_pass, ah, al, bh, bl, g, grid);
        } else {
            launch_main<64, 4>(ctx, three_pass, ah, al, bh, bl, g, grid);
        }
    }
    ctx->count_launch();
    check_last_launch("matmul (tcgen05)");

    if (splits > 1) {
        ProfScope scope(ctx, "matmul.fold");
        fold_partials_kernel<<<grid_for(out_elems, 256), 256, 0, ctx->stream>>>(p.out, partial, out_elems,
                                                                              static_cast<int>(splits));
        ctx->count_launch();
        check_last_launch("matmul (fold)");
    }
}

}  // namespace b200
