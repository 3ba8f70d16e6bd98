// Batched GEMM problem as vkML's matmul node presents it
// (src/backend/cpu/kernels_matmul.cpp:35-87): rank-4 operands
// a[B0,B1,M,K], b[B0,B1,K,N] with arbitrary element strides (stride 0 on a batch
// axis = broadcast, transposed views = swapped inner strides), dense output
// out[B0,B1,M,N].
#pragma once

#include "context.h"

namespace b200 {

struct GemmProblem {
    const float* a;
    const float* b;
    float* out;
    int64_t b0, b1, m, n, k;
    int64_t a_s[4];  // element strides of a over (b0, b1, m, k)
    int64_t b_s[4];  // element strides of b over (b0, b1, k, n)
};

// fp32 FMA on the CUDA cores; any strides, any size. gemm_simt.cu
void gemm_simt(b200_ctx* ctx, const GemmProblem& p);

// tcgen05 tensor-core path (3xTF32 or single-pass TF32). gemm_tc.cu
bool gemm_tc_eligible(const b200_ctx* ctx, const GemmProblem& p);
void gemm_tc(b200_ctx* ctx, const GemmProblem& p, bool three_pass);
// True when gemm_tc would serve `p` with the streamed-operand kernel (a small left operand, the
// right operand read once from HBM) rather than from operand planes.
bool gemm_tc_streams(const b200_ctx* ctx, const GemmProblem& p);
bool gemm_tc_reads_directly(const b200_ctx* ctx, const GemmProblem& p);  // (taken by itself: no shared planes)
// Diagnostic: one block waits `limit_ns` on a barrier nobody arrives on and gives up (gemm_tc.cu).
void gemm_tc_wait_probe(b200_ctx* ctx, uint64_t limit_ns);

// Reuse of split operand planes inside one compute span: count the operands of every
// tensor-core matmul before the span runs, drop planes whose source a node overwrites, and
// release what is left when the span ends.
void gemm_tc_note_uses(b200_ctx* ctx, const GemmProblem& p);
void gemm_tc_invalidate(b200_ctx* ctx, const void* begin, const void* end);
void gemm_tc_end_span(b200_ctx* ctx);

}  // namespace b200
