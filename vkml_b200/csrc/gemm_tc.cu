#include "gemm.h"
namespace b200 {
bool gemm_tc_eligible(const b200_ctx*, const GemmProblem&) { return false; }
void gemm_tc(b200_ctx*, const GemmProblem&, bool) { fail(B200_NOT_IMPLEMENTED, "tensor-core GEMM not built"); }
}
