// Launcher of the CTA-pair (tcgen05 cta_group::2) fused INT8 GEMM (gemm_2cta.cu).
#pragma once

#include "gemm_common.cuh"

namespace pq {

// One or two weight sets (rows [0, p.m_split) use w, the rest w1; w1 is ignored when p.m_split == M).  t / lb_t may both be NULL (no low-rank term); otherwise t [M,32] (row stride ldt) and
// lb_t [N,32] contiguous in the output dtype.  The tile schedule fields of `p` are filled in here.
int launch_gemm_pair(bool bf16, bool dbg, const void* xq, int64_t ldx, const void* w, const void* w1, int64_t ldw,
                     const void* t, int64_t ldt, const void* lb_t, int64_t M, int64_t N, int64_t K, const GemmParams& p,
                     cudaStream_t st);

}  // namespace pq
