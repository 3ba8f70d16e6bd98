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
constexpr int kProducerThreads = 256;  // direct-operand variant: two groups of four warps
constexpr int kThreadsDirect = kThreads + kProducerThreads;
constexpr int kGroupM = 16;
constexpr int kEpiPitch = 36;   // words per row of the epilogue's staging patch (16-byte aligned rows)
constexpr int kSchedRing = 4;  // published-but-unconsumed tile numbers per CTA
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

// The same test, but the hardware may park the thread for up to `hint_ns` while the phase is
// still open (it is woken when the phase completes).  For the many warps that wait for one
// event, a parked warp leaves the issue slots and the shared-memory pipe to the warps that work.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
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
                                          uint32_t* status, uint64_t limit_ns = kWaitLimitNs) {
    // The clock is only consulted every 1024 polls (reading %globaltimer costs far more than a
    // poll, and the converter warps wait here once per K-block), so the limit is the stated time
    // plus at most 1024 polls.
    uint64_t start = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ff) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            const uint64_t now = global_ns();
            if (start == 0) {
                start = now;
            } else if (now - start > limit_ns) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimedOut);
                return false;
            }
        }
    }
    return true;
}

// Bounded wait for the warps of a many-waiter role: parked polls, the clock read every 64 of them.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 uint32_t* status) {
    uint64_t start = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait_parked(bar, parity, 2000u)) {
        if ((++spins & 0x3f) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            const uint64_t now = global_ns();
            if (start == 0) {
                start = now;
            } else if (now - start > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(status, kStatusWaitTimedOut);
                return false;
            }
        }
    }
    return true;
}

// One block that waits, through the very mbar_wait the GEMM kernels use, on a barrier nobody will
// ever arrive on: the wait runs out after `limit_ns`, records kStatusWaitTimedOut and the kernel
// returns by itself.  Nothing is in flight, nothing faults; it exists so that the path from a
// bounded device wait to B200_TIMEOUT on the host can be exercised.
__global__ void wait_probe_kernel(uint32_t* status, uint64_t limit_ns) {
    __shared__ uint64_t barrier;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&barrier), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        (void)mbar_wait(smem_u32(&barrier), 0, &abort_flag, status, limit_ns);
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
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

// The same split on the integer pipe.  Conversion instructions issue at a quarter of the rate of
// integer adds, and a K-block of a 128x256 tile needs 24576 of them; adding half a TF32 ulp to
// the magnitude and clearing the 13 low bits is the same round-to-nearest, ties-away rounding
// (a mantissa carry runs into the exponent as it should).  Infinity, NaN and a rounding that
// overflows take the reference routine.
__device__ __forceinline__ void split_tf32_fast(float x, float& hi, float& lo) {
    const uint32_t b = __float_as_uint(x);
    const uint32_t h = (b + 0x1000u) & 0xFFFFE000u;
    if ((h << 1) >= 0xFF000000u) {  // x is infinite or NaN, or hi overflowed
        split_tf32(x, hi, lo);
        return;
    }
    const float fh = __uint_as_float(h);
    const uint32_t r = __float_as_uint(x - fh);  // exact
    hi = fh;
    lo = __uint_as_float((r + 0x1000u) & 0xFFFFE000u);
}

// The same split without a branch, for the converter warps of the streamed-operand kernel: two
// warps per scheduler cannot hide a taken-or-not decision per element, and sixteen independent
// elements interleave only if they are one basic block.  hi on the integer pipe (add half a TF32
// ulp, clear 13 bits; where that reaches the infinity exponent -- x is infinite, NaN, or finite
// but rounds past the largest TF32 -- truncate instead, keeping a NaN a NaN), lo = tf32(x - hi)
// on the conversion pipe, forced to zero for a non-finite x.  Same values as split_tf32.
__device__ __forceinline__ void split_tf32_select(float x, uint32_t& hi, uint32_t& lo) {
    const uint32_t b = __float_as_uint(x);
    uint32_t h = (b + 0x1000u) & 0xFFFFE000u;
    const bool nonfinite = (b & 0x7F800000u) == 0x7F800000u;
    const bool over = nonfinite || (h & 0x7F800000u) == 0x7F800000u;  // (a NaN's carry can leave the exponent)
    const bool is_nan = nonfinite && (b & 0x007FFFFFu) != 0u;
    h = over ? (b & 0xFFFFE000u) : h;
    h = is_nan ? (h | 0x00400000u) : h;
    const float rest = x - __uint_as_float(h);  // exact for a finite x
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    hi = h;
    lo = nonfinite ? 0u : l;
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
    pdl_prologue();
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
    pdl_prologue();
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
        launch_kernel(ctx, split_rows_kernel, grid_for(ceil_div(total, 2), 256), 256, 0, s);
    } else {
        const int64_t tiles = ceil_div(s.kp, kSplitTile) * ceil_div(s.rows, kSplitTile) * s.n_batches;
        launch_kernel(ctx, split_kernel, grid_for(tiles, 1, 8), 256, 0, s);
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
    int group_m;           // M-tiles walked together before moving along N (L2 reuse of the B tiles)
    uint32_t* status;
    // Dynamic tile order: null = every CTA walks units blockIdx.x, +gridDim.x, ... ; otherwise a
    // zeroed counter from which CTAs draw their units after the first, so a CTA that starts late
    // or shares its SM with another kernel (an all-reduce) simply takes fewer tiles.
    unsigned int* sched;
};

// Direct-operand variant: TMA brings the fp32 operand tiles themselves into the `hi` slots of a
// stage (through tensor maps over the caller's matrices: same swizzles, zero fill past the
// edges), eight converter warps split them in place into hi and lo, and only then is the stage
// handed to the MMA warp.  No plane ever exists in HBM: the kernel reads 4 bytes per operand
// element instead of 8, and the split pre-pass (4 read + 8 written) disappears.  It costs
// shared-memory bandwidth (one more read and write of every tile), so it is for products the
// plane scheme would leave waiting on HBM, not for the large compute-bound ones.
struct DirectArgs {
    int64_t b1;          // inner batch extent
    int a_bcast, b_bcast;
};

template <int BN, int STAGES>
struct Smem {
    static constexpr int kABytes = BM * BK * 4;  // one A plane tile
    static constexpr int kBBytes = BN * BK * 4;
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

template <int BN, int STAGES, bool THREE_PASS, bool A_MN, bool B_MN, bool DIRECT>
__global__ void __launch_bounds__(DIRECT ? kThreadsDirect : kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
               const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
               TcArgs g, DirectArgs da) {
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
    // dynamic tile order: the producer publishes each next unit through a small ring
    auto sched_full = [&](int r) { return bars + 8u * (2 * STAGES + 4 + r); };
    auto sched_empty = [&](int r) { return bars + 8u * (2 * STAGES + 4 + kSchedRing + r); };
    auto raw_bar = [&](int s) { return bars + 8u * (2 * STAGES + 4 + 2 * kSchedRing + s); };  // direct: fp32 tile landed
    __shared__ int sched_ring[kSchedRing];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) float epi_patch[4][32][kEpiPitch];  // one transposing patch per epilogue warp

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            // TMA: one arrival with the byte count; direct: every thread of a producer group
            mbar_init(full_bar(s), DIRECT ? kProducerThreads : 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(raw_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4);
        }
        for (int r = 0; r < kSchedRing; ++r) {
            mbar_init(sched_full(r), 1);
            mbar_init(sched_empty(r), 5);  // the MMA thread and the four epilogue warps
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
    // barriers and tensor memory are set up: only now wait for the previous kernel (the operand
    // split, usually), so this kernel's set-up runs under that kernel's tail
    pdl_prologue();

    const int64_t tiles_per_batch = g.tiles_m * g.tiles_n;
    const int64_t n_units = tiles_per_batch * g.batches * g.splits;

    // unit -> (split, batch, m tile, n tile); M-tiles walked in groups of kGroupM
    auto decode = [&](int64_t u, int& split, int64_t& batch, int64_t& tm, int64_t& tn) {
        split = static_cast<int>(u % g.splits);
        int64_t t = u / g.splits;
        batch = t / tiles_per_batch;
        t -= batch * tiles_per_batch;
        const int64_t group_size = int64_t(g.group_m) * g.tiles_n;
        const int64_t group = t / group_size;
        const int64_t first_m = group * g.group_m;
        const int64_t rows_in_group = min(int64_t(g.group_m), g.tiles_m - first_m);
        const int64_t in_group = t - group * group_size;
        tm = first_m + in_group % rows_in_group;
        tn = in_group / rows_in_group;
    };

    const bool dynamic = g.sched != nullptr;
    // unit after the t-th one of this CTA, for the MMA thread and the epilogue warps (-1: none)
    auto next_unit = [&](int64_t u, uint32_t t, bool single_thread) -> int64_t {
        if (!dynamic) {
            u += gridDim.x;
            return u < n_units ? u : -1;
        }
        const int r = t % kSchedRing;
        if (!mbar_wait(sched_full(r), (t / kSchedRing) & 1, abort_p, g.status)) {
            return -1;
        }
        const int v = *reinterpret_cast<volatile int*>(&sched_ring[r]);
        if (!single_thread) {
            __syncwarp();
        }
        if (single_thread || lane == 0) {
            mbar_arrive(sched_empty(r));
        }
        return v;
    };

    if (DIRECT && warp >= 6) {
        // ---------------- converters: split the fp32 tiles of each stage in place ----------------
        const int tc = static_cast<int>(threadIdx.x) - kThreads;  // 0 .. kProducerThreads-1
        uint32_t it = 0;
        bool ok = true;
        for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            int split;
            int64_t batch, tm, tn;
            decode(u, split, batch, tm, tn);
            const int64_t kb0 = int64_t(split) * g.kb_per_split;
            const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
            for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(raw_bar(s), ph, abort_p, g.status)) {
                    ok = false;
                    break;
                }
                // The split is elementwise, so the tile's swizzle is irrelevant here: every float
                // of a hi slot becomes hi in place and lo at the same offset of the lo slot.  All
                // of a thread's vectors are loaded before any is stored, so the shared-memory
                // latency is paid once per stage.
                uint8_t* stage_ptr = smem_raw + (base - smem_u32(smem_raw)) + s * S::kStageBytes;
                constexpr int NA = S::kABytes / 16 / kProducerThreads;
                constexpr int NB = S::kBBytes / 16 / kProducerThreads;
                static_assert(NA >= 1 && NB >= 1, "tile smaller than the converter group");
                float4 v[NA + NB];
                float4* a_hi = reinterpret_cast<float4*>(stage_ptr) + tc;
                float4* a_lo = reinterpret_cast<float4*>(stage_ptr + S::kABytes) + tc;
                float4* b_hi = reinterpret_cast<float4*>(stage_ptr + 2 * S::kABytes) + tc;
                float4* b_lo = reinterpret_cast<float4*>(stage_ptr + 2 * S::kABytes + S::kBBytes) + tc;
#pragma unroll
                for (int j = 0; j < NA; ++j) v[j] = a_hi[j * kProducerThreads];
#pragma unroll
                for (int j = 0; j < NB; ++j) v[NA + j] = b_hi[j * kProducerThreads];
#pragma unroll
                for (int j = 0; j < NA + NB; ++j) {
                    float4 h, l;
                    split_tf32_fast(v[j].x, h.x, l.x);
                    split_tf32_fast(v[j].y, h.y, l.y);
                    split_tf32_fast(v[j].z, h.z, l.z);
                    split_tf32_fast(v[j].w, h.w, l.w);
                    float4* hi = j < NA ? a_hi + j * kProducerThreads : b_hi + (j - NA) * kProducerThreads;
                    float4* lo = j < NA ? a_lo + j * kProducerThreads : b_lo + (j - NA) * kProducerThreads;
                    *hi = h;
                    if (THREE_PASS) {
                        *lo = l;
                    }
                }
                // generic-proxy stores must be visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(full_bar(s));
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            uint32_t t = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u >= 0 && u < n_units && ok; ++t) {
                // draw the next unit now; its value is needed only after this tile's loads
                int64_t nxt = u + gridDim.x;
                if (dynamic) {
                    nxt = int64_t(gridDim.x) + atomicAdd(g.sched, 1u);
                }
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
                    if (DIRECT) {
                        // fp32 tiles of the caller's matrices into the hi slots; coordinates are
                        // (unit-stride axis, other axis, inner batch, outer batch)
                        const uint32_t rbar = raw_bar(s);
                        mbar_arrive_expect_tx(rbar, S::kABytes + S::kBBytes);
                        const int64_t bo = batch / da.b1, bi = batch - bo * da.b1;
                        const int a1 = da.a_bcast ? 0 : static_cast<int>(bi), a0 = da.a_bcast ? 0 : static_cast<int>(bo);
                        const int b1c = da.b_bcast ? 0 : static_cast<int>(bi), b0c = da.b_bcast ? 0 : static_cast<int>(bo);
                        if (A_MN) {
#pragma unroll
                            for (int atom = 0; atom < BM / 32; ++atom) {
                                tma_load_4d(stage + atom * kMnAtomBytes, &map_a_hi, rbar, m0 + 32 * atom, kc, a1, a0);
                            }
                        } else {
                            tma_load_4d(stage, &map_a_hi, rbar, kc, m0, a1, a0);
                        }
                        const uint32_t bdst = stage + 2 * S::kABytes;
                        if (B_MN) {
#pragma unroll
                            for (int atom = 0; atom < BN / 32; ++atom) {
                                tma_load_4d(bdst + atom * kMnAtomBytes, &map_b_hi, rbar, n0 + 32 * atom, kc, b1c, b0c);
                            }
                        } else {
                            tma_load_4d(bdst, &map_b_hi, rbar, kc, n0, b1c, b0c);
                        }
                        continue;
                    }
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
                if (dynamic && ok) {
                    const int r = t % kSchedRing;
                    if (!mbar_wait(sched_empty(r), ((t / kSchedRing) & 1) ^ 1, abort_p, g.status)) {
                        break;
                    }
                    *reinterpret_cast<volatile int*>(&sched_ring[r]) = nxt < n_units ? static_cast<int>(nxt) : -1;
                    mbar_arrive(sched_full(r));
                }
                u = nxt;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            uint32_t tile_it = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u >= 0 && u < n_units && ok; u = next_unit(u, tile_it, true), ++tile_it) {
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
        for (int64_t u = blockIdx.x; u >= 0 && u < n_units && ok; u = next_unit(u, tile_it, false), ++tile_it) {
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
            const bool warp_rows_live = tm * BM + quarter * 32 < g.m;  // else nothing of this warp's is stored
#pragma unroll 2
            for (int c = 0; c < BN / 32; ++c) {
                if (col0 + c * 32 >= g.n || !warp_rows_live) {
                    break;  // uniform across the warp
                }
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + c * 32, r);
                const int64_t left = g.n - (col0 + c * 32);
                if (vec_ok && left >= 32) {
                    // Each lane holds 32 columns of ITS row, so storing from here makes every warp
                    // instruction touch 32 different rows (32 wavefronts for 512 bytes).  The chunk
                    // goes through a 32 x 36-word patch of shared memory instead and leaves as four
                    // 128-byte row segments per instruction; both the row-wise writes and the
                    // quarter-warp-per-row reads of the patch are conflict-free.
                    float* patch = &epi_patch[quarter][0][0];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 v;
                        v.x = __uint_as_float(r[4 * j]);
                        v.y = __uint_as_float(r[4 * j + 1]);
                        v.z = __uint_as_float(r[4 * j + 2]);
                        v.w = __uint_as_float(r[4 * j + 3]);
                        *reinterpret_cast<float4*>(patch + lane * kEpiPitch + 4 * j) = v;
                    }
                    __syncwarp();
                    const int sub = lane >> 3, seg = lane & 7;
                    const int64_t row_base = tm * BM + quarter * 32;
                    float* tile_dst = g.out + int64_t(split) * g.split_stride + (batch * g.m + row_base) * g.n + col0 +
                                      c * 32 + seg * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = i * 4 + sub;
                        if (row_base + rl < g.m) {
                            const float4 v = *reinterpret_cast<const float4*>(patch + rl * kEpiPitch + seg * 4);
                            *reinterpret_cast<float4*>(tile_dst + int64_t(rl) * g.n) = v;
                        }
                    }
                    __syncwarp();
                    continue;
                }
                if (row_ok) {
                    // ragged right edge, or an output that cannot take 128-bit stores
                    float* p = dst + c * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < left) {
                            p[j] = __uint_as_float(r[j]);
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

// ---------------------------------------------------------------------------
// Streamed-operand kernel: products bound by HBM, not by the tensor pipe
// ---------------------------------------------------------------------------
//
// C[b][m][n] = sum_k W[b][m][k] * S[b][k][n] with a SMALL W (few rows: a skinny left operand,
// convolution weights broadcast over the batch) and a LARGE S whose n axis is contiguous
// (a row-major [K][N] matrix, the column tensor of a convolution).  The plane scheme reads S,
// writes its two TF32 planes and reads them again -- five times S's bytes -- which is what
// bounds such a product.  Here S crosses HBM exactly once, as fp32:
//
//   * the product is computed transposed, D[n][m] = sum_k S[k][n] W[m][k], so that S is the
//     tensor core's A operand, and A may come from TENSOR MEMORY instead of shared memory;
//   * two producer warps: one brings [32 k][128 n] fp32 tiles of S (tensor map over the caller's
//     own matrix, zero fill past the edges) into a ring of 6 to 8 slots, the other the matching
//     K-blocks of W's planes into a ring of 4.  The rings are separate because their lifetimes
//     are: S's slot is free again as soon as the converters have read it, W's stays until the
//     MMAs that read it have finished.  (Measured: the deeper ring for S changes no time -- the
//     loop is bound by the rate at which tcgen05.mma instructions issue, about 98 cycles each
//     with A in tensor memory, twelve per K-block -- so its depth is headroom, not a tuning knob.)
//   * sixteen converter warps read their lane's column of the S tile (lane = n, conflict-free),
//     split every value into hi/lo in registers and put both into tensor memory with
//     tcgen05.st -- 64 columns per stage: the streamed operand never touches shared memory
//     again and no converted copy of it exists anywhere;
//   * warp 1 issues tcgen05.mma with A = [tmem] (128 lanes x 8 columns per K-step) and B = W's
//     plane tile in shared memory, three passes into one fp32 accumulator as above;
//   * warps 2-5 read the accumulator (lane = n, columns = m): for every m one warp instruction
//     stores 32 consecutive n, 128 bytes, straight from registers.
//
// S may also lie with its K axis contiguous (the transposed view of an [N][K] matrix: a Linear
// layer's weight in the forward product, the column tensor in a convolution's weight gradient).
// Then the tile is [128 n][32 k], fetched with the 128-byte swizzle so that a lane reading its own
// row (lane = n) meets no bank conflict, and everything after the converter is unchanged.
//
// W may have more rows than one accumulator holds: its 128-row chunks are separate units that run
// side by side on neighbouring SMs, so S's tile is fetched from HBM once and from L2 after that.
//
// When N is shorter than 128 and W is broadcast over the batch, one tile spans several batches
// (lanes = batch x n).  K is split across CTAs when the tiles alone cannot fill the machine;
// the warp that arrives last at its quarter of a tile folds the partial planes in split order in
// the same launch (deterministic, no atomics on data).
constexpr int kStreamStages = 4;          // W's ring in shared memory and S's ring in tensor memory
constexpr int kStreamConverters = 16;     // converter warps: four per tensor-memory lane quarter, 8 K columns each
constexpr int kStreamThreads = (7 + kStreamConverters) * 32;  // + two TMA warps, MMA and four epilogue warps
constexpr int kStreamTileBytes = BK * 128 * 4;  // one fp32 tile of S: 32 K-rows x 128 lanes
constexpr uint32_t kStreamTmemCols = 512;
constexpr int kStreamCounters = 1024;     // arrival counters of the in-kernel split-K fold: 4 per tile
constexpr int kStreamCounterBase = 4096 + 64;  // their place behind b200_ctx::d_counters

struct StreamArgs {
    float* out;            // C, or the partial planes when splits > 1
    float* folded;         // C when splits > 1 (target of the in-kernel fold)
    int64_t m, n;          // per batch
    int64_t batches;
    int64_t w_batch_rows;  // rows between consecutive batches in W's planes (0: broadcast)
    int64_t k_blocks, kb_per_split;
    int splits;
    int64_t split_stride;  // elements between partial planes
    int64_t tiles_m, tiles_n;
    int nt;                // n extent of one batch inside a tile (128, or N when N < 128)
    int bpt;               // batches per tile (nt * bpt == 128 when bpt > 1)
    int64_t batch_groups;  // ceil(batches / bpt)
    uint32_t* status;
    unsigned int* counters;
};


__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

template <int BNW>
struct StreamSmem {
    static constexpr int kWBytes = BNW * BK * 4;  // one plane tile of W
    static constexpr int kWStage = 2 * kWBytes;   // hi and lo
    static constexpr int kSlots = BNW <= 64 ? 8 : 6;  // fp32 tiles of S in flight (besides the 4 in tensor memory)
    static constexpr int kWBase = kSlots * kStreamTileBytes;
    static constexpr int kBars = kWBase + kStreamStages * kWStage;
    static constexpr int kTotal = kBars + 256 + 1024;
};

template <int BNW, bool THREE_PASS, bool W_MN, bool S_KM>
__global__ void __launch_bounds__(kStreamThreads, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_w_hi,
                   const __grid_constant__ CUtensorMap map_w_lo, StreamArgs g) {
    using S = StreamSmem<BNW>;
    constexpr int STAGES = kStreamStages;
    constexpr uint32_t kIdesc = make_idesc(BM, BNW, false, W_MN);
    constexpr int SLOTS = S::kSlots;
    constexpr uint32_t kWTx = (THREE_PASS ? 2 : 1) * S::kWBytes;
    constexpr uint32_t kStageCol0 = 2 * BNW;  // tensor-memory columns: two accumulators, then the S stages
    static_assert(8 * (2 * SLOTS + 3 * STAGES + 4) <= 256, "barrier block");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::kBars;
    auto full_bar = [&](int s) { return bars + 8u * s; };                    // W's planes landed
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };        // the stage's MMAs are done
    auto conv_bar = [&](int s) { return bars + 8u * (2 * STAGES + s); };     // S is in tensor memory
    auto acc_full = [&](int a) { return bars + 8u * (3 * STAGES + a); };
    auto acc_empty = [&](int a) { return bars + 8u * (3 * STAGES + 2 + a); };
    auto s_full = [&](int j) { return bars + 8u * (3 * STAGES + 4 + j); };            // an fp32 tile of S landed
    auto s_empty = [&](int j) { return bars + 8u * (3 * STAGES + 4 + SLOTS + j); };   // the converters have read it
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(conv_bar(s), kStreamConverters);  // one arrival per converter warp
        }
        for (int j = 0; j < SLOTS; ++j) {
            mbar_init(s_full(j), 1);
            mbar_init(s_empty(j), kStreamConverters);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kStreamTmemCols);
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;
    pdl_prologue();

    const int64_t n_units = g.tiles_m * g.splits * g.tiles_n * g.batch_groups;
    // unit -> (m tile, K split, n tile, batch group): the m tiles of one S tile run side by side
    auto decode = [&](int64_t u, int64_t& tm, int& split, int64_t& tn, int64_t& bg) {
        tm = u % g.tiles_m;
        int64_t t = u / g.tiles_m;
        split = static_cast<int>(t % g.splits);
        t /= g.splits;
        tn = t % g.tiles_n;
        bg = t / g.tiles_n;
    };

    if (warp == kStreamThreads / 32 - 1) {
        // ---------------- TMA producer of S ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                int64_t tm, tn, bg;
                int split;
                decode(u, tm, split, tn, bg);
                const int batch0 = static_cast<int>(bg * g.bpt);
                const int n0 = static_cast<int>(tn * g.nt);
                const int64_t kb0 = int64_t(split) * g.kb_per_split;
                const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
                for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const int j = it % SLOTS;
                    const uint32_t ph = (it / SLOTS) & 1;
                    if (!mbar_wait(s_empty(j), ph ^ 1, abort_p, g.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t slot = base + j * kStreamTileBytes;
                    const uint32_t bar = s_full(j);
                    const int kc = static_cast<int>(kb * BK);
                    mbar_arrive_expect_tx(bar, kStreamTileBytes);
                    if (S_KM) {
                        tma_load_3d(slot, &map_s, bar, kc, n0, batch0);  // [128 n][32 k], k contiguous
                    } else {
                        tma_load_3d(slot, &map_s, bar, n0, kc, batch0);  // [32 k][128 n], n contiguous
                    }
                }
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer of W's planes ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                int64_t tm, tn, bg;
                int split;
                decode(u, tm, split, tn, bg);
                const int batch0 = static_cast<int>(bg * g.bpt);
                const int m0 = static_cast<int>(tm * BNW);
                const int w_base = static_cast<int>(batch0 * g.w_batch_rows);
                const int64_t kb0 = int64_t(split) * g.kb_per_split;
                const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
                for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_p, g.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t stage = base + S::kWBase + s * S::kWStage;
                    const uint32_t bar = full_bar(s);
                    const int kc = static_cast<int>(kb * BK);
                    mbar_arrive_expect_tx(bar, kWTx);
                    auto load_w = [&](uint32_t dst, const CUtensorMap* map) {
                        if (W_MN) {
#pragma unroll
                            for (int atom = 0; atom < BNW / 32; ++atom) {
                                tma_load_2d(dst + atom * kMnAtomBytes, map, bar, m0 + 32 * atom, w_base + kc);
                            }
                        } else {
                            tma_load_2d(dst, map, bar, kc, w_base + m0);
                        }
                    };
                    load_w(stage, &map_w_hi);
                    if (THREE_PASS) {
                        load_w(stage + S::kWBytes, &map_w_lo);
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
                int64_t tm, tn, bg;
                int split;
                decode(u, tm, split, tn, bg);
                const int acc = tile_it & 1;
                const uint32_t aph = (tile_it >> 1) & 1;
                if (!mbar_wait(acc_empty(acc), aph ^ 1, abort_p, g.status)) {
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BNW;
                const int64_t kb0 = int64_t(split) * g.kb_per_split;
                const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
                for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full_bar(s), ph, abort_p, g.status) ||
                        !mbar_wait(conv_bar(s), ph, abort_p, g.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t stage = base + S::kWBase + s * S::kWStage;
                    const uint64_t w_hi = operand_desc<W_MN>(stage);
                    const uint64_t w_lo = operand_desc<W_MN>(stage + S::kWBytes);
                    const uint32_t s_hi = tmem_base + kStageCol0 + s * 64;
                    const uint32_t s_lo = s_hi + 32;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t adv_w = static_cast<uint64_t>((W_MN ? kk * 1024 : kk * UMMA_K * 4) >> 4);
                        const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
                        if (THREE_PASS) {
                            umma_tf32_ts(d_tmem, s_lo + kk * UMMA_K, w_hi + adv_w, kIdesc, first);
                            umma_tf32_ts(d_tmem, s_hi + kk * UMMA_K, w_lo + adv_w, kIdesc, 1u);
                            umma_tf32_ts(d_tmem, s_hi + kk * UMMA_K, w_hi + adv_w, kIdesc, 1u);
                        } else {
                            umma_tf32_ts(d_tmem, s_hi + kk * UMMA_K, w_hi + adv_w, kIdesc, first);
                        }
                    }
                    umma_commit(empty_bar(s));  // W's stage and S's tensor-memory stage are both free then
                }
                if (ok) {
                    umma_commit(acc_full(acc));
                }
            }
        }
    } else if (warp < 6) {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;
        const int l = quarter * 32 + lane;  // tensor-memory lane = position along (batch, n) of the tile
        const int bl = l / g.nt;
        const int nn = l - bl * g.nt;
        uint32_t tile_it = 0;
        for (int64_t u = blockIdx.x; u < n_units; u += gridDim.x, ++tile_it) {
            int64_t tm, tn, bg;
            int split;
            decode(u, tm, split, tn, bg);
            const int acc = tile_it & 1;
            const uint32_t aph = (tile_it >> 1) & 1;
            if (!mbar_wait(acc_full(acc), aph, abort_p, g.status)) {
                break;
            }
            tc_fence_after();
            const int64_t batch = bg * g.bpt + bl;
            const int64_t n = tn * g.nt + nn;
            const bool lane_ok = batch < g.batches && n < g.n;
            const int64_t m0 = tm * BNW;
            const int64_t col = (batch * g.m) * g.n + n;  // + m * N
            float* dst = g.out + int64_t(split) * g.split_stride + col;
#pragma unroll 1
            for (int c = 0; c < BNW / 32; ++c) {
                if (m0 + c * 32 >= g.m) {
                    break;  // uniform
                }
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BNW + c * 32, r);
                if (lane_ok) {
                    // one row of C per store: 32 lanes, 128 contiguous bytes.  The row pointer is
                    // stepped, not recomputed -- a 64-bit multiply per store would cost this
                    // single warp more than the store does.
                    const int64_t left = g.m - (m0 + c * 32);
                    float* p = dst + (m0 + c * 32) * g.n;
                    if (left >= 32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            *p = __uint_as_float(r[j]);
                            p += g.n;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < left) {
                                *p = __uint_as_float(r[j]);
                                p += g.n;
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
            if (g.splits > 1) {
                // Split K: each epilogue warp owns 32 lanes of the tile in every K-slice.  The warp
                // that completes its lanes' last slice folds the slices, in split order -- a
                // per-warp arrival counter, so no warp ever waits for another one.
                __threadfence();
                __syncwarp();
                unsigned old = 0;
                if (lane == 0) {
                    const int64_t tile = (bg * g.tiles_n + tn) * g.tiles_m + tm;
                    old = atomicInc(g.counters + tile * 4 + quarter, static_cast<unsigned>(g.splits - 1));
                }
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == static_cast<unsigned>(g.splits - 1)) {
                    __threadfence();
                    if (lane_ok) {
                        // Eight rows and up to four K-slices at a time, all 32 loads issued before
                        // the first add: the partial planes come from L2, and a chain that waits for
                        // one load before issuing the next would pay that latency per element.  The
                        // adds keep the split order.
                        const int64_t rows = min(int64_t(BNW), g.m - m0);
                        const float* __restrict__ part = g.out + col + m0 * g.n;
                        float* __restrict__ dstf = g.folded + col + m0 * g.n;
                        for (int64_t j0 = 0; j0 < rows; j0 += 8) {
                            float sum[8];
                            for (int sp0 = 0; sp0 < g.splits; sp0 += 4) {
                                float t[4][8];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        t[q][j] = (sp0 + q < g.splits && j0 + j < rows)
                                                      ? __ldcg(part + int64_t(sp0 + q) * g.split_stride + (j0 + j) * g.n)
                                                      : 0.0F;
                                    }
                                }
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    if (sp0 + q < g.splits) {
#pragma unroll
                                        for (int j = 0; j < 8; ++j) {
                                            sum[j] = (sp0 + q == 0) ? t[q][j] : sum[j] + t[q][j];
                                        }
                                    }
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (j0 + j < rows) dstf[(j0 + j) * g.n] = sum[j];
                            }
                        }
                    }
                }
            }
        }
    } else if (warp < 6 + kStreamConverters) {
        // ---------------- converters (warps 6..21): S tile -> hi / lo in tensor memory ----------------
        // Sixteen warps, four per tensor-memory lane quarter, each taking 8 of the stage's 32 K
        // columns: the split is ~7 instructions per element on 4096 elements per K-block, and it is
        // this loop, not HBM, that a thin set of warps would make the limit.
        const int quarter = warp & 3;
        const int part = (warp - 6) >> 2;  // which 8 of the stage's 32 K columns
        const int l = quarter * 32 + lane;
        const int bl = l / g.nt;
        const int nn = l - bl * g.nt;
        const uint32_t first_off = S_KM ? static_cast<uint32_t>(l * 128)
                                        : static_cast<uint32_t>(((bl * BK + part * 8) * g.nt + nn) * 4);
        const uint32_t k_step = static_cast<uint32_t>(g.nt * 4);
        // K-major tile: the row of lane l is 128 bytes, its 16-byte chunks permuted by the 128-byte
        // swizzle (chunk ^ (row & 7)); this warp's eight K values are chunks 2*part and 2*part + 1
        const uint32_t chunk0 = static_cast<uint32_t>(((2 * part) ^ (l & 7)) * 16);
        const uint32_t chunk1 = static_cast<uint32_t>(((2 * part + 1) ^ (l & 7)) * 16);
        const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        for (int64_t u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            int64_t tm, tn, bg;
            int split;
            decode(u, tm, split, tn, bg);
            const int64_t kb0 = int64_t(split) * g.kb_per_split;
            const int64_t kb1 = min(kb0 + g.kb_per_split, g.k_blocks);
            for (int64_t kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const int j = it % SLOTS;
                const uint32_t sph = (it / SLOTS) & 1;
                // the tile has landed, and the MMAs that read this tensor-memory stage last are done
                if (!mbar_wait_parked(s_full(j), sph, abort_p, g.status) ||
                    !mbar_wait(empty_bar(s), ph ^ 1, abort_p, g.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint8_t* tile = base_ptr + j * kStreamTileBytes + first_off;
                float v[8];
                uint32_t top = 0;
                if (S_KM) {
                    const float4 q0 = *reinterpret_cast<const float4*>(tile + chunk0);
                    const float4 q1 = *reinterpret_cast<const float4*>(tile + chunk1);
                    v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w;
                    v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        v[j] = *reinterpret_cast<const float*>(tile + j * k_step);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    top = max(top, __float_as_uint(v[j]) << 1);
                }
                uint32_t hi[8], lo[8];
                if (top < 0xFEFFE000u) {
                    // every value is finite and rounds inside the TF32 range: add half a TF32 ulp,
                    // clear 13 bits (round to nearest, ties away), lo = tf32(x - hi)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        hi[j] = (__float_as_uint(v[j]) + 0x1000u) & 0xFFFFE000u;
                        const float rest = v[j] - __uint_as_float(hi[j]);
                        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo[j]) : "f"(rest));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        split_tf32_select(v[j], hi[j], lo[j]);  // infinities, NaNs, values that round past the range
                    }
                }
                const uint32_t t_hi = tmem_base + lane_field + kStageCol0 + s * 64 + part * 8;
                tmem_st8(t_hi, hi);
                if (THREE_PASS) {
                    tmem_st8(t_hi + 32, lo);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(conv_bar(s));
                    mbar_arrive(s_empty(j));  // the values are in registers and tensor memory: the slot may be refilled
                }
            }
        }
    }

    __syncthreads();
    if (abort_flag != 0) {
        for (int i = 0; i < 200; ++i) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kStreamTmemCols);
    }
}

__global__ void __launch_bounds__(256)
fold_partials_kernel(float* __restrict__ out, const float* __restrict__ partial, int64_t n, int splits) {
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

// The caller's own matrix as a 4-D tensor: (unit-stride axis, the other matrix axis, inner
// batch, outer batch), f32, boxes of 32 floats x box_rows, zero fill outside.  A broadcast
// batch axis is given extent 1 and always addressed at coordinate 0.
CUtensorMap make_raw_map(const float* base, int64_t cols, int64_t rows, int64_t pitch, int64_t b1, int64_t s_b1,
                         int64_t b0, int64_t s_b0, int box_rows, bool mn_major) {
    CUtensorMap m;
    const int64_t plane = std::max<int64_t>(rows * pitch, 4);
    if (b1 <= 1 || s_b1 == 0) {
        b1 = 1;
        s_b1 = plane;
    }
    if (b0 <= 1 || s_b0 == 0) {
        b0 = 1;
        s_b0 = std::max(plane, s_b1 * b1);
    }
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                                static_cast<cuuint64_t>(b1), static_cast<cuuint64_t>(b0)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(pitch) * sizeof(float),
                                   static_cast<cuuint64_t>(s_b1) * sizeof(float),
                                   static_cast<cuuint64_t>(s_b0) * sizeof(float)};
    const cuuint32_t box[4] = {BK, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUresult rc = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides,
                                       box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        fail(B200_INTERNAL_ERROR, "cuTensorMapEncodeTiled (operand map) failed with code " + std::to_string(rc));
    }
    return m;
}

template <int BN, int STAGES, bool THREE, bool A_MN, bool B_MN>
void launch_one(b200_ctx* ctx, const CUtensorMap& ah, const CUtensorMap& al, const CUtensorMap& bh,
                const CUtensorMap& bl, const TcArgs& g, int grid, const DirectArgs* direct) {
    using S = Smem<BN, STAGES>;
    if (direct != nullptr) {
        auto kernel = gemm_tc_kernel<BN, STAGES, THREE, A_MN, B_MN, true>;
        B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        launch_kernel(ctx, kernel, grid, kThreadsDirect, S::kTotal, ah, al, bh, bl, g, *direct);
        return;
    }
    auto kernel = gemm_tc_kernel<BN, STAGES, THREE, A_MN, B_MN, false>;
    B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    launch_kernel(ctx, kernel, grid, kThreads, S::kTotal, ah, al, bh, bl, g, DirectArgs{});
}

template <int BN, int STAGES>
void launch_main(b200_ctx* ctx, bool three_pass, bool a_mn, bool b_mn, const CUtensorMap& ah,
                 const CUtensorMap& al, const CUtensorMap& bh, const CUtensorMap& bl, const TcArgs& g, int grid,
                 const DirectArgs* direct = nullptr) {
#define B200_TC_CASE(T, A, B)                                                     \
    if (three_pass == T && a_mn == A && b_mn == B) {                              \
        launch_one<BN, STAGES, T, A, B>(ctx, ah, al, bh, bl, g, grid, direct);    \
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


// One matmul operand, described by the matrix it is in memory.
struct Operand {
    PlaneKey key{};
    bool mn = false;     // consumed MN-major (the M or N axis is the contiguous one)
    bool dense = false;  // unit stride along one axis, everything else 16-byte aligned
    bool cached = false;
    int64_t nb = 1, rows = 0, cols = 0, rows_pad = 0, cols_pad = 0;
    size_t plane_bytes = 0;
    const char* src_begin = nullptr;
    const char* src_end = nullptr;
    float* hi = nullptr;
    float* lo = nullptr;
    SplitArgs split{};
};

// `s_mn` / `s_k` are the element strides along the operand's M (or N) axis and along K.
// An operand whose M (or N) axis is contiguous keeps its [K][MN] layout and is consumed
// MN-major; everything else becomes a K-major plane [MN][Kp].  Planes of densely readable
// sources are padded to 32 rows and 32 columns of zeros, so the same plane serves a later use
// of the same memory in the other orientation.
Operand plan_operand(const float* ptr, int64_t s_b0, int64_t s_b1, int64_t s_mn, int64_t s_k, int64_t mn_extent,
                     int64_t k_extent, bool bcast, const GemmProblem& p) {
    Operand o;
    const int64_t sb0 = bcast ? 0 : s_b0, sb1 = bcast ? 0 : s_b1;
    const bool aligned = reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && sb0 % 4 == 0 && sb1 % 4 == 0;
    o.mn = s_mn == 1 && s_k != 1 && aligned && s_k % 4 == 0;
    o.nb = bcast ? 1 : p.b0 * p.b1;
    int64_t s_r, s_c;
    if (o.mn) {
        o.rows = k_extent;
        o.cols = mn_extent;
        s_r = s_k;
        s_c = 1;
    } else {
        o.rows = mn_extent;
        o.cols = k_extent;
        s_r = s_mn;
        s_c = s_k;
    }
    const bool dense = s_c == 1 && s_r % 4 == 0 && aligned;  // the 128-bit split kernel's condition
    o.dense = dense;
    o.rows_pad = dense ? align_up(o.rows, 32) : o.rows;
    o.cols_pad = align_up(o.cols, 32);
    o.plane_bytes = static_cast<size_t>(align_up(o.nb * o.rows_pad * o.cols_pad * 4, 1024));
    const int64_t b1 = bcast ? 1 : p.b1;
    o.key.src = ptr;
    const int64_t kv[8] = {o.rows, o.cols, s_r, s_c, b1, sb0, sb1, o.nb};
    for (int i = 0; i < 8; ++i) o.key.v[i] = kv[i];
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    const int64_t b0 = bcast ? 1 : p.b0;
    const int64_t span = (b0 - 1) * mag(sb0) + (b1 - 1) * mag(sb1) + (o.rows - 1) * mag(s_r) + (o.cols - 1) * mag(s_c) + 1;
    o.src_begin = reinterpret_cast<const char*>(ptr);
    o.src_end = o.src_begin + span * 4;
    o.split.src = ptr;
    o.split.b1 = b1;
    o.split.s_b0 = sb0;
    o.split.s_b1 = sb1;
    o.split.n_batches = o.nb;
    o.split.rows = o.rows;
    o.split.out_rows = o.rows_pad;
    o.split.k = o.cols;
    o.split.kp = o.cols_pad;
    o.split.s_r = s_r;
    o.split.s_k = s_c;
    return o;
}

// Whether reading the operands directly beats splitting them into planes first.  Measured: the
// in-kernel split is bound by shared-memory traffic (the converter's loads and stores contend
// with the tensor core's operand reads) at about 147 TFLOP/s of algorithmic work -- 7.5 ms against
// 4.5 ms at 8192^3, 0.32 against 0.31 ms at 512 x 65536 x 512 -- while the plane scheme moves each
// operand five times (read, two planes written, two planes read).  It pays where that traffic is
// what the product costs and nobody else in the span uses the planes: the CNN's first
// weight gradient, g[256][64x1024] . cols^T[256][1024x27], 74 us against 105; the CNN's head,
// 19 against 24 us.
bool direct_pays(const b200_ctx* ctx, const GemmProblem& p, int64_t batches, const Operand& oa, const Operand& ob) {
    auto shared = [&](const Operand& o) {
        const auto it = ctx->plane_uses.find(o.key);
        return it != ctx->plane_uses.end() && it->second >= 2;
    };
    if (shared(oa) || shared(ob)) return false;
    const double flops = 2.0 * double(p.m) * double(p.n) * double(p.k) * double(batches);
    const double operand_bytes = double(oa.plane_bytes) + double(ob.plane_bytes);
    return flops / 147e12 < 4.0 * operand_bytes / 6.5e12;
}

size_t plane_cache_limit(const b200_ctx* ctx) {
    return std::min<size_t>(size_t(16) << 30, ctx->prop.totalGlobalMem / 8);
}

void release_use(b200_ctx* ctx, const Operand& o) {
    if (!o.cached) return;
    auto it = ctx->plane_cache.find(o.key);
    if (it == ctx->plane_cache.end()) return;
    if (--it->second.uses_left <= 0) {
        ctx->scratch.release(it->second.hi);
        ctx->plane_cache_bytes -= it->second.bytes;
        ctx->plane_cache.erase(it);
    }
}

// ---- streamed-operand kernel: eligibility and launch ----

struct StreamPlan {
    bool ok = false;
    bool s_km = false;         // S's K axis is the contiguous one
    int nt = 128, bpt = 1, bnw = 64;
    int64_t pitch = 0;         // elements between consecutive rows of S (K rows, or N rows when s_km)
    int64_t batch_stride = 0;  // elements between consecutive batches of S
};

// The product qualifies when its right operand can be read by TMA as it lies in memory (n or k
// contiguous, 16-byte pitches, batches one constant stride apart) and the product is bound by
// memory rather than by the tensor pipe: a left operand of at most 256 rows (the streamed operand
// is then worth 128 flops per byte at most, and one pass over it beats reading it once, writing
// two planes and reading those), or a short K (at most 256: the result outweighs the operands --
// the column gradient of a convolution -- and re-reading S's few tiles from L2 for every 128 rows
// of W costs less than the plane passes).
StreamPlan plan_stream(const b200_ctx* ctx, const GemmProblem& p) {
    StreamPlan sp;
    if (ctx->gemm_stream == 0 || (ctx->gemm_stream < 0 && ctx->gemm_operands >= 0)) {
        return sp;  // switched off, or another operand scheme was asked for by name
    }
    const int64_t batches = p.b0 * p.b1;
    // (VKML_B200_GEMM_STREAM=1 lifts the size rule: every product whose layout allows it, for A/B runs)
    if ((ctx->gemm_stream < 1 && p.m > 256 && (p.k > 256 || p.m > 4096)) || p.n < 32 || batches < 1) return sp;
    if (p.b_s[3] == 1 && p.b_s[2] % 4 == 0 && p.b_s[2] >= p.n) {
        sp.s_km = false;
        sp.pitch = p.b_s[2];
    } else if (p.b_s[2] == 1 && p.b_s[3] % 4 == 0 && p.b_s[3] >= p.k && p.n >= 128) {
        sp.s_km = true;
        sp.pitch = p.b_s[3];
    } else {
        return sp;
    }
    if (reinterpret_cast<uintptr_t>(p.b) % 16 != 0) return sp;
    int64_t sb = std::max<int64_t>((sp.s_km ? p.n : p.k) * sp.pitch, 4);
    if (batches > 1) {
        if (p.b0 == 1) sb = p.b_s[1];
        else if (p.b1 == 1) sb = p.b_s[0];
        else if (p.b_s[0] == p.b1 * p.b_s[1]) sb = p.b_s[1];
        else return sp;
        if (sb <= 0 || sb % 4 != 0) return sp;
    }
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    if (p.n >= 128) {
        sp.nt = 128;
        sp.bpt = 1;
    } else if ((p.n == 32 || p.n == 64) && a_bcast && batches % (128 / p.n) == 0) {
        sp.nt = static_cast<int>(p.n);  // a tile spans several batches: lanes = batch x n
        sp.bpt = static_cast<int>(128 / p.n);
    } else {
        return sp;
    }
    if (batches >= (int64_t(1) << 31) || p.n >= (int64_t(1) << 31) || sb * 4 >= (int64_t(1) << 40)) return sp;
    sp.bnw = p.m <= 64 ? 64 : 128;
    sp.batch_stride = sb;
    sp.ok = true;
    return sp;
}

CUtensorMap make_stream_map(const float* base, int64_t n, int64_t k, int64_t pitch, int64_t batches,
                            int64_t batch_stride, int nt, int bpt, bool s_km) {
    CUtensorMap m;
    // n contiguous: tiles of [32 k][nt n] as they lie; k contiguous: tiles of [128 n][32 k], whose
    // 128-byte rows take the 128-byte swizzle
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(s_km ? k : n), static_cast<cuuint64_t>(s_km ? n : k),
                                static_cast<cuuint64_t>(batches)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(pitch) * sizeof(float),
                                   static_cast<cuuint64_t>(batch_stride) * sizeof(float)};
    const cuuint32_t box[3] = {s_km ? cuuint32_t(BK) : static_cast<cuuint32_t>(nt), s_km ? cuuint32_t(128) : cuuint32_t(BK),
                               static_cast<cuuint32_t>(bpt)};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides,
                                       box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       s_km ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        fail(B200_INTERNAL_ERROR, "cuTensorMapEncodeTiled (streamed operand) failed with code " + std::to_string(rc));
    }
    return m;
}

template <int BNW>
void launch_stream(b200_ctx* ctx, bool three_pass, bool w_mn, bool s_km, const CUtensorMap& ms, const CUtensorMap& wh,
                   const CUtensorMap& wl, const StreamArgs& g, int grid) {
    using S = StreamSmem<BNW>;
#define B200_STREAM_CASE(T, W)                                                                             \
    if (three_pass == T && w_mn == W && s_km) {                                                            \
        auto kernel = gemm_stream_kernel<BNW, T, W, true>;                                                 \
        B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal)); \
        launch_kernel(ctx, kernel, grid, kStreamThreads, S::kTotal, ms, wh, wl, g);                        \
        return;                                                                                            \
    }                                                                                                      \
    if (three_pass == T && w_mn == W) {                                                                    \
        auto kernel = gemm_stream_kernel<BNW, T, W, false>;                                                \
        B200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal)); \
        launch_kernel(ctx, kernel, grid, kStreamThreads, S::kTotal, ms, wh, wl, g);                        \
        return;                                                                                            \
    }
    B200_STREAM_CASE(true, false)
    B200_STREAM_CASE(true, true)
    B200_STREAM_CASE(false, false)
    B200_STREAM_CASE(false, true)
#undef B200_STREAM_CASE
}

void gemm_stream(b200_ctx* ctx, const GemmProblem& p, bool three_pass, const StreamPlan& sp) {
    const int64_t batches = p.b0 * p.b1;
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    Operand ow = plan_operand(p.a, p.a_s[0], p.a_s[1], p.a_s[2], p.a_s[3], p.m, p.k, a_bcast, p);
    const int64_t k_blocks = align_up(p.k, BK) / BK;
    const int64_t tiles_m = ceil_div(p.m, sp.bnw);
    const int64_t tiles_n = sp.bpt > 1 ? 1 : ceil_div(p.n, 128);
    const int64_t batch_groups = ceil_div(batches, sp.bpt);
    const int64_t tiles = tiles_m * tiles_n * batch_groups;
    const int sms = ctx->prop.multiProcessorCount;
    int64_t splits = 1;
    if (tiles < sms && k_blocks >= 16 && tiles * 4 <= kStreamCounters) {
        splits = std::min<int64_t>(sms / tiles, k_blocks / 8);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 64));
    }
    const int64_t kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);
    const int64_t out_elems = batches * p.m * p.n;
    const size_t partial_bytes = splits > 1 ? static_cast<size_t>(align_up(out_elems * splits * 4, 1024)) : 0;

    // W's planes: from this span's cache, into it, or into the workspace
    const size_t planes = three_pass ? 2 : 1;
    bool hit = false;
    if (auto it = ctx->plane_cache.find(ow.key); it != ctx->plane_cache.end()) {
        ow.hi = it->second.hi;
        ow.lo = it->second.lo;
        ow.cached = hit = true;
        ++ctx->plane_hits;
    } else {
        auto uses = ctx->plane_uses.find(ow.key);
        const size_t bytes = planes * ow.plane_bytes;
        if (uses != ctx->plane_uses.end() && uses->second >= 2 &&
            ctx->plane_cache_bytes + bytes <= plane_cache_limit(ctx)) {
            char* block = static_cast<char*>(ctx->scratch.allocate(bytes));
            ow.hi = reinterpret_cast<float*>(block);
            ow.lo = three_pass ? reinterpret_cast<float*>(block + ow.plane_bytes) : nullptr;
            ctx->plane_cache[ow.key] = PlaneEntry{ow.hi, ow.lo, bytes, uses->second, ow.src_begin, ow.src_end};
            ctx->plane_cache_bytes += bytes;
            ow.cached = true;
        }
    }
    char* ws = static_cast<char*>(ctx->ensure_workspace(partial_bytes + 2048 + (ow.cached ? 0 : planes * ow.plane_bytes)));
    ws = reinterpret_cast<char*>(align_up(reinterpret_cast<int64_t>(ws), 1024));
    if (!ow.cached) {
        ow.hi = reinterpret_cast<float*>(ws);
        ow.lo = three_pass ? reinterpret_cast<float*>(ws + ow.plane_bytes) : nullptr;
        ws += planes * ow.plane_bytes;
    }
    float* partial = splits > 1 ? reinterpret_cast<float*>(ws) : nullptr;
    if (!hit) {
        ow.split.hi = ow.hi;
        ow.split.lo = ow.lo;
        launch_split(ctx, ow.split, "matmul.split_a");
        check_last_launch("matmul (operand split)");
    }

    const CUtensorMap ms = make_stream_map(p.b, p.n, p.k, sp.pitch, batches, sp.batch_stride, sp.nt, sp.bpt, sp.s_km);
    auto map_w = [&](float* plane) {
        return ow.mn ? make_map(plane, ow.nb * ow.rows_pad, ow.cols_pad, BK, true)
                     : make_map(plane, ow.nb * ow.rows_pad, ow.cols_pad, sp.bnw, false);
    };
    const CUtensorMap wh = map_w(ow.hi);
    const CUtensorMap wl = three_pass ? map_w(ow.lo) : wh;

    StreamArgs g{};
    g.out = splits > 1 ? partial : p.out;
    g.folded = p.out;
    g.m = p.m;
    g.n = p.n;
    g.batches = batches;
    g.w_batch_rows = a_bcast ? 0 : ow.rows_pad;
    g.k_blocks = k_blocks;
    g.kb_per_split = kb_per_split;
    g.splits = static_cast<int>(splits);
    g.split_stride = out_elems;
    g.tiles_m = tiles_m;
    g.tiles_n = tiles_n;
    g.nt = sp.nt;
    g.bpt = sp.bpt;
    g.batch_groups = batch_groups;
    g.status = ctx->d_status;
    g.counters = ctx->d_counters + kStreamCounterBase;
    const int grid = static_cast<int>(std::min<int64_t>(tiles * splits, sms));
    {
        ProfScope scope(ctx, three_pass ? "matmul.tcgen05_3xtf32_stream" : "matmul.tcgen05_tf32_stream");
        if (sp.bnw == 64) {
            launch_stream<64>(ctx, three_pass, ow.mn, sp.s_km, ms, wh, wl, g, grid);
        } else {
            launch_stream<128>(ctx, three_pass, ow.mn, sp.s_km, ms, wh, wl, g, grid);
        }
    }
    ctx->count_launch();
    check_last_launch("matmul (tcgen05, streamed operand)");
    release_use(ctx, ow);
}

}  // namespace

bool gemm_tc_eligible(const b200_ctx* ctx, const GemmProblem& p) {
    if (ctx->prop.major != 10 || encode_tiled() == nullptr) {
        return false;
    }
    const int64_t batches = p.b0 * p.b1;
    if (p.m < 32 || p.n < 16 || p.k < 16 || batches < 1) {  // K is zero-padded to the 32-wide K-block
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

bool gemm_tc_streams(const b200_ctx* ctx, const GemmProblem& p) { return plan_stream(ctx, p).ok; }

// Whether gemm_tc would read this product's operands directly (no planes), taken by itself: the
// same conditions as in gemm_tc below, with no other matmul of a span sharing the planes.
bool gemm_tc_reads_directly(const b200_ctx* ctx, const GemmProblem& p) {
    if (plan_stream(ctx, p).ok || ctx->gemm_operands == 0) return false;
    const int64_t batches = p.b0 * p.b1;
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    const bool b_bcast = (p.b_s[0] == 0 || p.b0 == 1) && (p.b_s[1] == 0 || p.b1 == 1);
    const Operand oa = plan_operand(p.a, p.a_s[0], p.a_s[1], p.a_s[2], p.a_s[3], p.m, p.k, a_bcast, p);
    const Operand ob = plan_operand(p.b, p.b_s[0], p.b_s[1], p.b_s[3], p.b_s[2], p.n, p.k, b_bcast, p);
    const bool want_dynamic = ctx->gemm_schedule == 1;
    return oa.dense && ob.dense && !want_dynamic && (ctx->gemm_operands == 1 || direct_pays(ctx, p, batches, oa, ob));
}

void gemm_tc_wait_probe(b200_ctx* ctx, uint64_t limit_ns) {
    wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, limit_ns);
    ctx->count_launch();
    check_last_launch("wait probe");
}

void gemm_tc(b200_ctx* ctx, const GemmProblem& p, bool three_pass) {
    if (const StreamPlan sp = plan_stream(ctx, p); sp.ok) {
        gemm_stream(ctx, p, three_pass, sp);
        return;
    }
    const int64_t batches = p.b0 * p.b1;
    const int64_t kp = align_up(p.k, BK);
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    const bool b_bcast = (p.b_s[0] == 0 || p.b0 == 1) && (p.b_s[1] == 0 || p.b1 == 1);

    // Tile width: 128x256 tiles are the most efficient per tile (measured 5.5 % better than two
    // 128x128 tiles), but the persistent grid runs whole waves of 148 tiles, so the narrower
    // tile wins whenever it wastes less of the last wave (M=2048, N=8192: 4 waves of 256-wide
    // tiles against 7 half-cost waves of 128-wide ones).
    int bn = 64;
    if (p.n > 64) bn = 128;
    if (p.n > 128 && p.m * p.n * batches >= int64_t(128) * 256 * sm_count()) {
        const int64_t tm = ceil_div(p.m, BM);
        const double cost256 = double(ceil_div(tm * ceil_div(p.n, 256) * batches, sm_count()));
        const double cost128 = double(ceil_div(tm * ceil_div(p.n, 128) * batches, sm_count())) * 0.5275;
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
    if (tiles < sm_count() && k_blocks >= 16) {
        // as many K-slices as keep every unit in ONE wave of the persistent grid: rounding up
        // instead (32 tiles x 5 slices = 160 units on 148 SMs) runs a second, nearly empty wave
        splits = std::min<int64_t>(sm_count() / tiles, k_blocks / 8);
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 64));
    }
    int64_t kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);

    const int64_t out_elems = batches * p.m * p.n;
    const size_t partial_bytes = splits > 1 ? static_cast<size_t>(align_up(out_elems * splits * 4, 1024)) : 0;
    Operand oa = plan_operand(p.a, p.a_s[0], p.a_s[1], p.a_s[2], p.a_s[3], p.m, p.k, a_bcast, p);
    Operand ob = plan_operand(p.b, p.b_s[0], p.b_s[1], p.b_s[3], p.b_s[2], p.n, p.k, b_bcast, p);
    const bool a_mn = oa.mn, b_mn = ob.mn;

    // ---- direct operands: no planes at all ----
    const bool want_dynamic = ctx->gemm_schedule == 1 || (ctx->gemm_schedule < 0 && ctx->in_grad_sync_span);
    if (ctx->gemm_operands != 0 && oa.dense && ob.dense && !want_dynamic &&
        (ctx->gemm_operands == 1 || direct_pays(ctx, p, batches, oa, ob))) {
        float* partial = nullptr;
        if (splits > 1) {
            char* ws = static_cast<char*>(ctx->ensure_workspace(partial_bytes + 2048));
            partial = reinterpret_cast<float*>(align_up(reinterpret_cast<int64_t>(ws), 1024));
        }
        DirectArgs da{};
        da.b1 = p.b1;
        da.a_bcast = a_bcast ? 1 : 0;
        da.b_bcast = b_bcast ? 1 : 0;
        // A: K-major = rows M with pitch a_s[2]; MN-major = rows K with pitch a_s[3]
        const CUtensorMap raw_a =
            a_mn ? make_raw_map(p.a, p.m, p.k, p.a_s[3], a_bcast ? 1 : p.b1, p.a_s[1], a_bcast ? 1 : p.b0, p.a_s[0], BK, true)
                 : make_raw_map(p.a, p.k, p.m, p.a_s[2], a_bcast ? 1 : p.b1, p.a_s[1], a_bcast ? 1 : p.b0, p.a_s[0], BM, false);
        const CUtensorMap raw_b =
            b_mn ? make_raw_map(p.b, p.n, p.k, p.b_s[2], b_bcast ? 1 : p.b1, p.b_s[1], b_bcast ? 1 : p.b0, p.b_s[0], BK, true)
                 : make_raw_map(p.b, p.k, p.n, p.b_s[3], b_bcast ? 1 : p.b1, p.b_s[1], b_bcast ? 1 : p.b0, p.b_s[0], bn, false);
        TcArgs g{};
        g.out = splits > 1 ? partial : p.out;
        g.m = p.m;
        g.n = p.n;
        g.batches = batches;
        g.k_blocks = k_blocks;
        g.kb_per_split = kb_per_split;
        g.splits = static_cast<int>(splits);
        g.split_stride = out_elems;
        g.tiles_m = tiles_m;
        g.tiles_n = tiles_n;
        g.group_m = ctx->gemm_group_m > 0 ? ctx->gemm_group_m : kGroupM;
        g.status = ctx->d_status;
        const int grid = static_cast<int>(std::min<int64_t>(tiles * splits, ctx->prop.multiProcessorCount));
        {
            ProfScope scope(ctx, three_pass ? "matmul.tcgen05_3xtf32_direct" : "matmul.tcgen05_tf32_direct");
            if (bn == 256) {
                launch_main<256, 2>(ctx, three_pass, a_mn, b_mn, raw_a, raw_a, raw_b, raw_b, g, grid, &da);
            } else if (bn == 128) {
                launch_main<128, 3>(ctx, three_pass, a_mn, b_mn, raw_a, raw_a, raw_b, raw_b, g, grid, &da);
            } else {
                launch_main<64, 4>(ctx, three_pass, a_mn, b_mn, raw_a, raw_a, raw_b, raw_b, g, grid, &da);
            }
        }
        ctx->count_launch();
        check_last_launch("matmul (tcgen05, direct operands)");
        if (splits > 1) {
            ProfScope scope(ctx, "matmul.fold");
            launch_kernel(ctx, fold_partials_kernel, grid_for(out_elems, 256), 256, 0, p.out, partial, out_elems,
                                                                                  static_cast<int>(splits));
            ctx->count_launch();
            check_last_launch("matmul (fold)");
        }
        return;
    }

    // ---- operand planes: from this span's cache, into it, or into the workspace ----
    const size_t planes = three_pass ? 2 : 1;
    auto from_cache = [&](Operand& o) {
        auto it = ctx->plane_cache.find(o.key);
        if (it == ctx->plane_cache.end()) return false;
        o.hi = it->second.hi;
        o.lo = it->second.lo;
        o.cached = true;
        ++ctx->plane_hits;
        return true;
    };
    auto into_cache = [&](Operand& o) {
        auto uses = ctx->plane_uses.find(o.key);
        const size_t bytes = planes * o.plane_bytes;
        if (uses == ctx->plane_uses.end() || uses->second < 2 ||
            ctx->plane_cache_bytes + bytes > plane_cache_limit(ctx)) {
            return false;
        }
        char* block = static_cast<char*>(ctx->scratch.allocate(bytes));
        o.hi = reinterpret_cast<float*>(block);
        o.lo = three_pass ? reinterpret_cast<float*>(block + o.plane_bytes) : nullptr;
        ctx->plane_cache[o.key] = PlaneEntry{o.hi, o.lo, bytes, uses->second, o.src_begin, o.src_end};
        ctx->plane_cache_bytes += bytes;
        o.cached = true;
        return true;
    };
    const bool a_hit = from_cache(oa);
    if (!a_hit) into_cache(oa);
    // (B may be the very plane A just put there: x times its own transpose)
    const bool b_hit = from_cache(ob);
    if (!b_hit) into_cache(ob);
    size_t ws_bytes = partial_bytes + 2048;
    if (!oa.cached) ws_bytes += planes * oa.plane_bytes;
    if (!ob.cached) ws_bytes += planes * ob.plane_bytes;
    char* ws = static_cast<char*>(ctx->ensure_workspace(ws_bytes));
    ws = reinterpret_cast<char*>(align_up(reinterpret_cast<int64_t>(ws), 1024));
    auto from_workspace = [&](Operand& o) {
        if (o.cached) return;
        o.hi = reinterpret_cast<float*>(ws);
        o.lo = three_pass ? reinterpret_cast<float*>(ws + o.plane_bytes) : nullptr;
        ws += planes * o.plane_bytes;
    };
    from_workspace(oa);
    from_workspace(ob);
    float* partial = splits > 1 ? reinterpret_cast<float*>(ws) : nullptr;

    if (!a_hit) {
        oa.split.hi = oa.hi;
        oa.split.lo = oa.lo;
        launch_split(ctx, oa.split, "matmul.split_a");
    }
    if (!b_hit) {
        ob.split.hi = ob.hi;
        ob.split.lo = ob.lo;
        launch_split(ctx, ob.split, "matmul.split_b");
    }
    if (!a_hit || !b_hit) {
        check_last_launch("matmul (operand split)");
    }

    // ---- main kernel ----
    // K-major plane: [batch][MN rows (padded)][Kp]; MN-major plane: [batch][Kp rows][MN padded]
    auto map_of = [&](float* plane, const Operand& o, int tile) {
        return o.mn ? make_map(plane, o.nb * o.rows_pad, o.cols_pad, BK, true)
                    : make_map(plane, o.nb * o.rows_pad, o.cols_pad, tile, false);
    };
    const CUtensorMap ah = map_of(oa.hi, oa, BM);
    const CUtensorMap al = three_pass ? map_of(oa.lo, oa, BM) : ah;
    const CUtensorMap bh = map_of(ob.hi, ob, bn);
    const CUtensorMap bl = three_pass ? map_of(ob.lo, ob, bn) : bh;

    TcArgs g{};
    g.out = splits > 1 ? partial : p.out;
    g.m = p.m;
    g.n = p.n;
    g.batches = batches;
    g.a_batch_rows = a_bcast ? 0 : oa.rows_pad;  // plane rows between consecutive batches
    g.b_batch_rows = b_bcast ? 0 : ob.rows_pad;
    g.k_blocks = k_blocks;
    g.kb_per_split = kb_per_split;
    g.splits = static_cast<int>(splits);
    g.split_stride = out_elems;
    g.tiles_m = tiles_m;
    g.tiles_n = tiles_n;
    g.group_m = ctx->gemm_group_m > 0 ? ctx->gemm_group_m : kGroupM;
    g.status = ctx->d_status;
    int sms = ctx->prop.multiProcessorCount;
    if (ctx->in_grad_sync_span && ctx->comm_pending) {
        sms = std::max(sms - ctx->comm_sms, sms / 2);  // leave room for the all-reduce kernels
    }
    const int grid = static_cast<int>(std::min<int64_t>(tiles * splits, sms));
    const bool dynamic = (ctx->gemm_schedule == 1 || (ctx->gemm_schedule < 0 && ctx->in_grad_sync_span)) &&
                         tiles * splits > grid && tiles * splits < (int64_t(1) << 30);
    if (dynamic) {
        g.sched = ctx->d_counters + 4096;  // past the reductions' arrival counters
        B200_CUDA_CHECK(cudaMemsetAsync(g.sched, 0, sizeof(unsigned int), ctx->stream));
    }
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
        launch_kernel(ctx, fold_partials_kernel, grid_for(out_elems, 256), 256, 0, p.out, partial, out_elems,
                                                                              static_cast<int>(splits));
        ctx->count_launch();
        check_last_launch("matmul (fold)");
    }
    // the stream is in order: a plane released here is only reused by later work
    release_use(ctx, oa);
    release_use(ctx, ob);
}

void gemm_tc_note_uses(b200_ctx* ctx, const GemmProblem& p) {
    const int64_t batches = p.b0 * p.b1;
    (void)batches;
    const bool a_bcast = (p.a_s[0] == 0 || p.b0 == 1) && (p.a_s[1] == 0 || p.b1 == 1);
    const bool b_bcast = (p.b_s[0] == 0 || p.b0 == 1) && (p.b_s[1] == 0 || p.b1 == 1);
    ++ctx->plane_uses[plan_operand(p.a, p.a_s[0], p.a_s[1], p.a_s[2], p.a_s[3], p.m, p.k, a_bcast, p).key];
    if (plan_stream(ctx, p).ok) {
        return;  // the right operand is streamed as it is: it gets no planes
    }
    ++ctx->plane_uses[plan_operand(p.b, p.b_s[0], p.b_s[1], p.b_s[3], p.b_s[2], p.n, p.k, b_bcast, p).key];
}

void gemm_tc_invalidate(b200_ctx* ctx, const void* begin, const void* end) {
    if (ctx->plane_cache.empty()) return;
    const char* lo = static_cast<const char*>(begin);
    const char* hi = static_cast<const char*>(end);
    for (auto it = ctx->plane_cache.begin(); it != ctx->plane_cache.end();) {
        if (lo < it->second.src_end && it->second.src_begin < hi) {
            ctx->scratch.release(it->second.hi);
            ctx->plane_cache_bytes -= it->second.bytes;
            it = ctx->plane_cache.erase(it);
        } else {
            ++it;
        }
    }
}

void gemm_tc_end_span(b200_ctx* ctx) {
    for (auto& kv : ctx->plane_cache) {
        ctx->scratch.release(kv.second.hi);
    }
    ctx->plane_cache.clear();
    ctx->plane_uses.clear();
    ctx->plane_cache_bytes = 0;
}

}  // namespace b200
