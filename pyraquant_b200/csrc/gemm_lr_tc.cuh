// Launcher of the fused INT8 GEMM whose rank-32 term runs on the tcgen05 tensor cores (gemm_lr_tc.cu).
#pragma once

#include "gemm_common.cuh"

namespace pq {

// t [M,32] (row stride ldt) and lb_t [N,32] contiguous, both in the output dtype; tensor maps of the int8
// operands are passed in.  Returns a pq_status.
int launch_gemm_lr_tc(int bn, bool bf16, bool dbg, const CUtensorMap& tmA, const CUtensorMap& tmW0,
                      const CUtensorMap& tmW1, const void* t, int64_t ldt, const void* lb_t, int64_t M, int64_t N,
                      const GemmParams& p, int grid, cudaStream_t st);

}  // namespace pq
