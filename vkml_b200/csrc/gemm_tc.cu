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
// (both batch strides 0) is stored once.  An operand whose M (or N) axis is the
// contiguous one -- a transposed view as A, a row-major [K,N] matrix as B -- is
// NOT transposed: its planes keep the [Kp][M or N] layout and the MMA reads them
// through MN-major descriptors, so the split is a dense 128-bit pass.
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

// Shared-memory matrix descriptors, 128-byte swizzle, 32-bit elements.
//
// K-major tile ([rows][32 floats], one swizzle row per matrix row): 8-row groups are 1024
// bytes apart (stride-dimension offset); the leading-dimension offset is unused because the
// K extent of one instruction (8 floats = 32 bytes) lies inside the swizzle row.  One K step
// advances the start address by 32 bytes.
//
// MN-major tile (the operand is stored with its M or N axis contiguous, as a row-major
// [K][N] matrix is for B): the tile is a row of "atoms", each 32 K-rows of 128 bytes (32
// floats along MN).  32-bit operands must use the 128-byte swizzle with 32-byte atomicity
// here (layout type 1, TMA mode SWIZZLE_128B_ATOM_32B): the pattern repeats every 4 K-rows,
// so the stride-dimension offset is 512 bytes; the next atom along MN starts kMnAtomBytes
// later (leading-dimension offset).  One K step (8 K-rows) advances the start by 1024 bytes.
constexpr uint32_t kMnAtomBytes = BK * 128;  // 32 K-rows x 128 bytes

__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);   // start address, bits 0-13
    d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;         // leading-dimension byte offset, bits 16-29
    d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;         // stride-dimension byte offset, bits 32-45
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version for sm_100
    d |= static_cast<uint64_t>(layout_type) << 61;            // 2: 128-byte swizzle, 1: same with 32-byte atoms
    return d;
}

template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    return MN_MAJOR ? smem_desc(smem_addr, kMnAtomBytes, 512, 1) : smem_desc(smem_addr, 0, 1024, 2);
}

// Instruction descriptor: D = f32, A = B = tf32, M x N tile, operand majors as given.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_mn, bool b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (a_mn ? (1u << 15) : 0u) | (b_mn ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
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
    int64_t out_rows;    // plane rows per batch (>= rows; the extra rows are written as zero)
};

// Source rows dense along K and 16-byte aligned: one thread per four K-elements, 128-bit
// loads and stores, no shared memory.
__global__ void __launch_bounds__(256) split_rows_kernel(SplitArgs a) {
    const int64_t kp4 = a.kp / 4;
    const int64_t total = kp4 * a.out_rows * a.n_batches;
    const int64_t step = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t k4 = i % kp4;
        const int64_t rb = i / kp4;
        const int64_t r = rb % a.out_rows;
        const int64_t b = rb / a.out_rows;
        const int64_t k = k4 * 4;
        float4 v = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
        if (r < a.rows) {
            const float* src = a.src + (b / a.b1) * a.s_b0 + (b % a.b1) * a.s_b1 + r * a.s_r;
            if (k + 3 < a.k) {
                v = *reinterpret_cast<const float4*>(src + k);
            } else {
                if (k < a.k) v.x = src[k];
                if (k + 1 < a.k) v.y = src[k + 1];
                if (k + 2 < a.k) v.z = src[k + 2];
            }
        }
        float4 h, l;
        split_tf32(v.x, h.x, l.x);
        split_tf32(v.y, h.y, l.y);
        split_tf32(v.z, h.z, l.z);
        split_tf32(v.w, h.w, l.w);
        const int64_t o = rb * a.kp + k;
        *reinterpret_cast<float4*>(a.hi + o) = h;
        if (a.lo != nullptr) {
            *reinterpret_cast<float4*>(a.lo + o) = l;
        }
    }
}

// General layouts, 64x64 (rows x k) tiles through shared memory: global reads follow
// whichever of the two axes has unit stride (so a row-major [K,N] operand is read along N
// and written K-major, i.e. transposed), writes are always dense along k.  16 elements per
// thread in flight in each phase.
constexpr int kSplitTile = 64;

__global__ void __launch_bounds__(256) split_kernel(SplitArgs a) {
    __shared__ float tile[kSplitTile][kSplitTile + 1];  // [row][k]
    const int fast = threadIdx.x & 63, slow = threadIdx.x >> 6;
    const int64_t tiles_k = a.kp / kSplitTile + (a.kp % kSplitTile != 0);
    const int64_t tiles_r = (a.rows + kSplitTile - 1) / kSplitTile;
    const int64_t n_tiles = tiles_k * tiles_r * a.n_batches;
    const bool k_fast = a.s_k == 1 || a.s_r != 1;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t tk = t % tiles_k;
        const int64_t tr = (t / tiles_k) % tiles_r;
        const int64_t b = t / (tiles_k * tiles_r);
        const float* src = a.src + (b / a.b1) * a.s_b0 + (b % a.b1) * a.s_b1;
        const int64_t r0 = tr * kSplitTile, k0 = tk * kSplitTile;
        const bool full = r0 + kSplitTile <= a.rows && k0 + kSplitTile <= a.k;
        if (k_fast) {
            const float* p = src + (r0 + slow) * a.s_r + (k0 + fast) * a.s_k;
            const int64_t step = 4 * a.s_r;
#pragma unroll
            for (int j = 0; j < kSplitTile / 4; ++j) {
                const bool ok = full || (r0 + slow + 4 * j < a.rows && k0 + fast < a.k);
                tile[slow + 4 * j][fast] = ok ? p[j * step] : 0.0F;
            }
        } else {
            const float* p = src + (r0 + fast) * a.s_r + (k0 + slow) * a.s_k;
            const int64_t step = 4 * a.s_k;
#pragma unroll
            for (int j = 0; j < kSplitTile / 4; ++j) {
                const bool ok = full || (r0 + fast < a.rows && k0 + slow + 4 * j < a.k);
                tile[fast][slow + 4 * j] = ok ? p[j * step] : 0.0F;
            }
        }
        __syncthreads();
        if (k0 + fast < a.kp) {
            float* hi = a.hi + (b * a.rows + r0 + slow) * a.kp + k0 + fast;
            float* lo = a.lo != nullptr ? a.lo + (b * a.rows + r0 + slow) * a.kp + k0 + fast : nullptr;
            const int64_t ostep = 4 * a.kp;
#pragma unroll
            for (int j = 0; j < kSplitTile / 4; ++j) {
                if (full || r0 + slow + 4 * j < a.rows) {
                    float h, l;
                    split_tf32(tile[slow + 4 * j][fast], h, l);
                    hi[j * ostep] = h;
                    if (lo != nullptr) {
                        lo[j * ostep] = l;
                    }
                }
            }
        }
        __syncthreads();
    }
}

void launch_split(b200_ctx* ctx, const SplitArgs& s, const char* label) {
    ProfScope scope(ctx, label);
    const bool rows_dense = s.s_k == 1 && s.s_r % 4 == 0 && s.s_b0 % 4 == 0 && s.s_b1 % 4 == 0 &&
                            reinterpret_cast<uintptr_t>(s.src) % 16 == 0;
    if (rows_dense) {
        const int64_t total = (s.kp / 4) * s.out_rows * s.n_batches;
        split_rows_kernel<<<grid_for(ceil_div(total, 2), 256), 256, 0, ctx->stream>>>(s);
    } else {
        const int64_t tiles = ceil_div(s.kp, kSplitTile) * ceil_div(s.rows, kSplitTile) * s.n_batches;
        split_kernel<<<grid_for(tiles, 1, 8), 256, 0, ctx->stream>>>(s);
    }
    ctx->count_launch();
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

template <int BN, int STAGES, bool THREE_PASS, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
               const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
               TcArgs g) {
    using S = Smem<BN, STAGES>;
    constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr uint32_t kIdesc = make_idesc(BM, BN, A_MN, B_MN);
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
                // K-major plane: coordinates (k, plane row); MN-major plane: (m or n, plane K-row)
                const int a_base = static_cast<int>(batch * g.a_batch_rows);
                const int b_base = static_cast<int>(batch * g.b_batch_rows);
                const int m0 = static_cast<int>(tm * BM), n0 = static_cast<int>(tn * BN);
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
                    const uint32_t bar = full_bar(s);
                    mbar_arrive_expect_tx(bar, kStageTx);
                    auto load_a = [&](uint32_t dst, const CUtensorMap* map) {
                        if (A_MN) {
#pragma unroll
                            for (int atom = 0; atom < BM / 32; ++atom) {
                                tma_load_2d(dst + atom * kMnAtomBytes, map, bar, m0 + 32 * atom, a_base + kc);
                            }
                        } else {
                            tma_load_2d(dst, map, bar, kc, a_base + m0);
                        }
                    };
                    auto load_b = [&](uint32_t dst, const CUtensorMap* map) {
                        if (B_MN) {
#pragma unroll
                            for (int atom = 0; atom < BN / 32; ++atom) {
                                tma_load_2d(dst + atom * kMnAtomBytes, map, bar, n0 + 32 * atom, b_base + kc);
                            }
                        } else {
                            tma_load_2d(dst, map, bar, kc, b_base + n0);
                        }
                    };
                    load_a(stage, &map_a_hi);
                    load_b(stage + 2 * S::kABytes, &map_b_hi);
                    if (THREE_PASS) {
                        load_a(stage + S::kABytes, &map_a_lo);
                        load_b(stage + 2 * S::kABytes + S::kBBytes, &map_b_lo);
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
                    const uint64_t a_hi = operand_desc<A_MN>(stage);
                    const uint64_t a_lo = operand_desc<A_MN>(stage + S::kABytes);
                    const uint64_t b_hi = operand_desc<B_MN>(stage + 2 * S::kABytes);
                    const uint64_t b_lo = operand_desc<B_MN>(stage + 2 * S::kABytes + S::kBBytes);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // one K step: +32 bytes inside the swizzle row (K-major), +8 K-rows (MN-major)
                        const uint64_t adv_a = static_cast<uint64_t>((A_MN ? kk * 1024 : kk * UMMA_K * 4) >> 4);
                        const uint64_t adv_b = static_cast<uint64_t>((B_MN ? kk * 1024 : kk * UMMA_K * 4) >> 4);
                        const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
                        if (THREE_PASS) {
                            umma_tf32(d_tmem, a_lo + adv_a, b_hi + adv_b, kIdesc, first);
                            umma_tf32(d_tmem, a_hi + adv_a, b_lo + adv_b, kIdesc, 1u);
                            umma_tf32(d_tmem, a_hi + adv_a, b_hi + adv_b, kIdesc, 1u);
                        } else {
                            umma_tf32(d_tmem, a_hi + adv_a, b_hi + adv_b, kIdesc, first);
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

// Plane [rows][pitch] of f32 (pitch in floats, a multiple of 4), boxes of 32 floats x box_rows,
// 128-byte swizzle.  K-major planes: pitch = Kp, rows = matrix rows, box_rows = tile rows.
// MN-major planes: pitch = padded M or N, rows = batches * Kp, box_rows = 32 K-rows.
CUtensorMap make_map(float* plane, int64_t rows, int64_t pitch, int box_rows, bool mn_major) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(pitch), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch) * sizeof(float)};
    const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, plane, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        fail(B200_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc));
    }
    return m;
}

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

template <int BN, int STAGES, bool THREE, bool A_MN, bool B_MN>
void launch_one(b200_ctx* ctx, const CUtensorMap& ah, const CUtensorMap& al, const CUtensorMap& bh,
                const CUtensorMap& bl, const TcArgs& g, int grid) {
    using S = Smem<BN, STAGES>;
    auto kernel = gemm_tc_kernel<BN, STAGES, THREE, A_MN, B_MN>;
    B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    kernel<<<grid, kThreads, S::kTotal, ctx->stream>>>(ah, al, bh, bl, g);
}

template <int BN, int STAGES>
void launch_main(b200_ctx* ctx, bool three_pass, bool a_mn, bool b_mn, const CUtensorMap& ah,
                 const CUtensorMap& al, const CUtensorMap& bh, const CUtensorMap& bl, const TcArgs& g, int grid) {
#define B200_TC_CASE(T, A, B)                                                     \
    if (three_pass == T && a_mn == A && b_mn == B) {                              \
        launch_one<BN, STAGES, T, A, B>(ctx, ah, al, bh, bl, g, grid);            \
        return;                                                                   \
    }
    B200_TC_CASE(true, false, false)
    B200_TC_CASE(true, false, true)
    B200_TC_CASE(true, true, false)
    B200_TC_CASE(true, true, true)
    B200_TC_CASE(false, false, false)
    B200_TC_CASE(false, false, true)
    B200_TC_CASE(false, true, false)
    B200_TC_CASE(false, true, true)
#undef B200_TC_CASE
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

    // Tile width: 128x256 tiles are the most efficient per tile (measured 5.5 % better than two
    // 128x128 tiles), but the persistent grid runs whole waves of 148 tiles, so the narrower
    // tile wins whenever it wastes less of the last wave (M=2048, N=8192: 4 waves of 256-wide
    // tiles against 7 half-cost waves of 128-wide ones).
    int bn = 64;
    if (p.n > 64) bn = 128;
    if (p.n > 128 && p.m * p.n * batches >= int64_t(128) * 256 * kSmCount) {
        const int64_t tm = ceil_div(p.m, BM);
        const double cost256 = double(ceil_div(tm * ceil_div(p.n, 256) * batches, kSmCount));
        const double cost128 = double(ceil_div(tm * ceil_div(p.n, 128) * batches, kSmCount)) * 0.5275;
        bn = cost128 < cost256 ? 128 : 256;
    }
    if (ctx->gemm_bn_override == 64 || ctx->gemm_bn_override == 128 || ctx->gemm_bn_override == 256) {
        bn = ctx->gemm_bn_override;
    }
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

    // An operand whose M (or N) axis is the contiguous one is consumed MN-major by the tensor
    // core: its planes keep the source's [K][MN] layout (padded to [Kp][MN rounded up to 4]) and
    // the split is a dense 128-bit pass.  Everything else becomes a K-major plane [MN][Kp].
    auto dense16 = [](const float* ptr, int64_t s_other, int64_t sb0, int64_t sb1, bool bcast) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && s_other % 4 == 0 &&
               (bcast || (sb0 % 4 == 0 && sb1 % 4 == 0));
    };
    const bool a_mn = p.a_s[2] == 1 && p.a_s[3] != 1 && dense16(p.a, p.a_s[3], p.a_s[0], p.a_s[1], a_bcast);
    const bool b_mn = p.b_s[3] == 1 && p.b_s[2] != 1 && dense16(p.b, p.b_s[2], p.b_s[0], p.b_s[1], b_bcast);
    const int64_t mp = align_up(p.m, 4), np = align_up(p.n, 4);

    const int64_t planes = three_pass ? 2 : 1;
    const int64_t a_plane = align_up(nb_a * (a_mn ? kp * mp : p.m * kp) * 4, 1024);
    const int64_t b_plane = align_up(nb_b * (b_mn ? kp * np : p.n * kp) * 4, 1024);
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
        // `rows` x `k` below are the plane's (outer, inner) axes: (M, K) for a K-major plane,
        // (K, M) for an MN-major one
        SplitArgs s{};
        s.src = p.a;
        s.hi = a_hi;
        s.lo = a_lo;
        s.b1 = a_bcast ? 1 : p.b1;
        s.s_b0 = a_bcast ? 0 : p.a_s[0];
        s.s_b1 = a_bcast ? 0 : p.a_s[1];
        s.n_batches = nb_a;
        if (a_mn) {
            s.rows = p.k;
            s.out_rows = kp;
            s.k = p.m;
            s.kp = mp;
            s.s_r = p.a_s[3];
            s.s_k = 1;
        } else {
            s.rows = s.out_rows = p.m;
            s.k = p.k;
            s.kp = kp;
            s.s_r = p.a_s[2];
            s.s_k = p.a_s[3];
        }
        launch_split(ctx, s, "matmul.split_a");
        s.src = p.b;
        s.hi = b_hi;
        s.lo = b_lo;
        s.b1 = b_bcast ? 1 : p.b1;
        s.s_b0 = b_bcast ? 0 : p.b_s[0];
        s.s_b1 = b_bcast ? 0 : p.b_s[1];
        s.n_batches = nb_b;
        if (b_mn) {
            s.rows = p.k;
            s.out_rows = kp;
            s.k = p.n;
            s.kp = np;
            s.s_r = p.b_s[2];
            s.s_k = 1;
        } else {
            s.rows = s.out_rows = p.n;
            s.k = p.k;
            s.kp = kp;
            s.s_r = p.b_s[3];
            s.s_k = p.b_s[2];
        }
        launch_split(ctx, s, "matmul.split_b");
        check_last_launch("matmul (operand split)");
    }

    // ---- main kernel ----
    auto map_of = [&](float* plane, bool mn, int64_t nb, int64_t extent, int64_t extent_p, int tile) {
        return mn ? make_map(plane, nb * kp, extent_p, BK, true) : make_map(plane, nb * extent, kp, tile, false);
    };
    const CUtensorMap ah = map_of(a_hi, a_mn, nb_a, p.m, mp, BM);
    const CUtensorMap al = three_pass ? map_of(a_lo, a_mn, nb_a, p.m, mp, BM) : ah;
    const CUtensorMap bh = map_of(b_hi, b_mn, nb_b, p.n, np, bn);
    const CUtensorMap bl = three_pass ? map_of(b_lo, b_mn, nb_b, p.n, np, bn) : bh;

    TcArgs g{};
    g.out = splits > 1 ? partial : p.out;
    g.m = p.m;
    g.n = p.n;
    g.batches = batches;
    g.a_batch_rows = a_bcast ? 0 : (a_mn ? kp : p.m);  // plane rows between consecutive batches
    g.b_batch_rows = b_bcast ? 0 : (b_mn ? kp : p.n);
    g.k_blocks = k_blocks;
    g.kb_per_split = kb_per_split;
    g.splits = static_cast<int>(splits);
    g.split_stride = out_elems;
    g.tiles_m = tiles_m;
    g.tiles_n = tiles_n;
    g.status = ctx->d_status;
    int sms = ctx->prop.multiProcessorCount;
    if (ctx->in_grad_sync_span && ctx->comm_pending) {
        sms = std::max(sms - ctx->comm_sms, sms / 2);  // leave room for the all-reduce kernels
    }
    const int grid = static_cast<int>(std::min<int64_t>(tiles * splits, sms));
    {
        ProfScope scope(ctx, three_pass ? "matmul.tcgen05_3xtf32" : "matmul.tcgen05_tf32");
        if (bn == 256) {
            launch_main<256, 2>(ctx, three_pass, a_mn, b_mn, ah, al, bh, bl, g, grid);
        } else if (bn == 128) {
            launch_main<128, 3>(ctx, three_pass, a_mn, b_mn, ah, al, bh, bl, g, grid);
        } else {
            launch_main<64, 4>(ctx, three_pass, a_mn, b_mn, ah, al, bh, bl, g, grid);
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
