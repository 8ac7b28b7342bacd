// Shared host/device helpers for libpq_b200: status plumbing, vector memory access and the
// sm_100a PTX wrappers (mbarrier, TMA, tcgen05) used by the GEMM kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pq_b200.h"

namespace pq {

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return PQ_ERR_CUDA;
}

#define PQ_CUDA_TRY(expr)                                  \
  do {                                                     \
    cudaError_t _e = (expr);                               \
    if (_e != cudaSuccess) return ::pq::cuda_fail(_e);     \
  } while (0)

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Number of SMs of the current device (cached per device id).
int sm_count();

// Option table shared by the .cu files (see pq_set_option).
struct Options {
  int quant_tpr = 0;       // quantisation kernel: threads per row override (0 = auto)
  int gemm_stages = 0;     // 0 = auto
  int gemm_block_n = 0;    // 0 = auto, else 128 or 256
  int gemm_pm = 0;         // tile schedule override: CTA grid rows (0 = auto)
  int gemm_pn = 0;         // tile schedule override: CTA grid columns (0 = auto)
  int gemm_max_ctas = 0;   // 0 = one per SM
  int gemm_debug_timing = 0;   // experiments: cycle counters into workspace + 256 (CTA-pair kernel)
  int gemm_epi_warps = 0;  // epilogue warps of the CTA-pair kernel: 0 automatic (16 up to K = 1536 without low-rank term, else 8), 8 or 16
  int gemm_tma_store = 1;  // sixteen-warp pair tiles store through shared memory + TMA (0: register stores)
  int gemm_pair = 1;       // CTA-pair (cta_group::2) kernel: 0 off, 1 when the problem is large enough, 2 whenever it applies
  int gemm_tail_pairs = 1; // CTA-pair kernel: SM pairs that the pm x pn grid leaves over take a tail region of the tiles (0: they idle)
  int gemm_panel_mb = 0;   // CTA-pair kernel, several column rounds: megabytes of activation rows per row panel (0 = one panel)
  int gemm_l2_hints = 0;   // CTA-pair kernel: bit 0 weights evict-last, bit 1 activations evict-first, bit 2 activations evict-last, bit 3 streaming output stores
  int g32_variant = 0;     // group-32 GEMM: bit 0 eight epilogue warps, bit 1 scalar fp32 operations, bit 3 data path only
};
Options& options();

// ---------------------------------------------------------------------------------------------
// device side: error word written by bounded waits
// ---------------------------------------------------------------------------------------------
// word = 0x10000 * role + 0x100 * barrier class + 1;  role 1 producer, 2 mma, 3 epilogue
__device__ __forceinline__ void report_timeout(int32_t* status, int role, int what) {
  if (status != nullptr) atomicCAS(status, 0, (role << 16) | (what << 8) | 1);
}

// ---------------------------------------------------------------------------------------------
// vector global memory access
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
// TMA tile store (shared memory -> global) and its bulk-group bookkeeping; all three by the one issuing thread
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_src))), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_u32(void* p, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))), "r"(v) : "memory");
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_v4_cs(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// shared memory / mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe of a phase (try_wait may suspend the thread for a while; this never does).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up after kWaitBudgetNs of wall time (checked every 256 polls) or
// kWaitMaxPolls polls, whichever comes first.  Returns false on give-up.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;   // 2 s
constexpr uint32_t kWaitMaxPolls = 1u << 30;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t i = 1; i < kWaitMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0) {
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitBudgetNs) return false;
    }
  }
  return false;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// TMA (no multicast anywhere)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 (tensor memory + MMA), single-CTA group
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// All MMAs issued so far by this thread arrive (once) on `bar` when they have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], int8 x int8 -> int32.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 128 bytes x rows with CU_TENSOR_MAP_SWIZZLE_128B writes):
// 8-row swizzle atoms are 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                             // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                     // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                             // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                             // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::i8: D int32, A and B signed int8, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t make_idesc_i8(int M, int N) {
  return (2u << 4)                       // D format: S32
         | (1u << 7)                     // A format: signed 8-bit
         | (1u << 10)                    // B format: signed 8-bit
         | (0u << 15) | (0u << 16)       // A, B K-major
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (static_cast<uint32_t>(M >> 4) << 24);
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives lane (row) base+i, v[j] = column j.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// 16 lanes x (8*4=32) columns of 32-bit in the mma.sync accumulator arrangement: with g = lane/4 and
// q = lane%4, v[4j+0], v[4j+1] = row base+g, columns 8j+2q, 8j+2q+1 and v[4j+2], v[4j+3] = row base+g+8.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// Same arrangement, 64 columns: v[4j..4j+3] belong to columns 8j..8j+7.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// legacy warp MMA used for the rank-32 low-rank term inside the GEMM epilogue
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

// ---------------------------------------------------------------------------------------------
// conversions that stay off the (slow) conversion pipe
// ---------------------------------------------------------------------------------------------
// Correctly rounded int32 -> fp32 (same result as cvt.rn.f32.s32) from integer/FMA-pipe operations only:
// v = hi * 2048 + lo with lo in [0, 2048) and |hi| <= 2^20; both halves convert exactly through the
// "add a large power of two" trick and one fused multiply-add rounds the sum once.
__device__ __forceinline__ float int_to_float_rn(int32_t v) {
  const float fh = __int_as_float(0x4B400000 + (v >> 11)) - 12582912.0f;             // exact: |hi| < 2^22
  const float fl = __int_as_float(0x4B000000 | (v & 0x7FF)) - 8388608.0f;            // exact: 0 <= lo < 2^23
  return fmaf(fh, 2048.0f, fl);
}

// Two at once on the packed fp32 pipe (identical results), with one operation less per value: the high part is placed
// at its final weight by the exponent of the constant (1.5 * 2^34 has a unit in the last place of 2^11, so adding
// v >> 11 to its bit pattern adds (v >> 11) * 2048 to its value), the low part keeps its 2^23 offset, and the first
// addition removes both offsets at once: d = (v >> 11) * 2048 - 2^23 exactly, d + (2^23 + lo) = v rounded once.
__device__ __forceinline__ float2 int2_to_float2_rn(int32_t a, int32_t b) {
  constexpr float kOffsets = 25778192384.0f;                                           // 1.5 * 2^34 + 2^23
  // (v >> 11) + constant as one multiply-high-add: it issues on the multiply pipe, which the epilogues leave idle,
  // instead of a shift and an addition on the integer pipe, which they saturate
  int32_t ha, hb;
  asm("mad.hi.s32 %0, %1, %2, %3;" : "=r"(ha) : "r"(a), "r"(1 << 21), "r"(0x50C00000));
  asm("mad.hi.s32 %0, %1, %2, %3;" : "=r"(hb) : "r"(b), "r"(1 << 21), "r"(0x50C00000));
  const float2 d = __fadd2_rn(make_float2(__int_as_float(ha), __int_as_float(hb)), make_float2(-kOffsets, -kOffsets));
  return __fadd2_rn(d, make_float2(__int_as_float(0x4B000000 | (a & 0x7FF)), __int_as_float(0x4B000000 | (b & 0x7FF))));
}

// ---------------------------------------------------------------------------------------------
// 16-bit float helpers
// ---------------------------------------------------------------------------------------------
template <typename T> struct Half2Of;
template <> struct Half2Of<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Half2Of<__half> { using type = __half2; };

__device__ __forceinline__ float lo_f32(uint32_t w, __nv_bfloat16) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f32(uint32_t w, __nv_bfloat16) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float lo_f32(uint32_t w, __half) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
}
__device__ __forceinline__ float hi_f32(uint32_t w, __half) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Packed 16-bit arithmetic on two values per register, round-to-nearest-even, never contracted into a fused
// multiply-add.  For operands that are themselves 16-bit values the result is bit-identical to the fp32 operation
// followed by one rounding (which is how the reference's 16-bit tensors compute): a product of two 8- or 11-bit
// significands is exact in fp32, and a sum of two such values is either exact in fp32 or dominated by the larger
// operand far beyond the rounding position.
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b, __nv_bfloat16) {
  uint32_t r; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b, __nv_bfloat16) {
  uint32_t r; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b, __half) {
  uint32_t r; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b, __half) {
  uint32_t r; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
}  // namespace pq
