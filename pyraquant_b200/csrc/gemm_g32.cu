// Group-32 W8A8 GEMM for sm_100a:
//   out[m,n] = sum_g s_a[m,g] * s_w[g,n] * (sum_{k in group g} xq[m,k] * w[n,k])  (+ bias[n])
// A group is 32 consecutive K = exactly one tcgen05.mma kind::i8 instruction, so every instruction starts a
// fresh int32 accumulator (exact per-group partial sum) in one of four tensor-memory slots (the four groups of
// a 128-byte stage are issued back to back and handed over with one barrier); the epilogue warps drain each slot
// and fold it into fp32 running sums in registers with one packed fused multiply-add per pair of
// outputs: sum = fma(float(partial), s_a * s_w, sum).
// The scale work (one multiply and one add per output element and group) is what bounds this kernel, not the
// tensor pipe.  Roles and barriers mirror the per-channel GEMM: warp 0 TMA producer (operand stages plus a ring
// of scale tiles), warp 1 MMA issuer, warps 2-9 epilogue.  Every wait is bounded.  No clusters, no multicast.
#include <type_traits>

#include "gemm_common.cuh"

namespace pq {
namespace {

constexpr int GBN = 128;                 // columns per tile = one tensor-memory slot
constexpr int kSlots = 4;
constexpr int kG32Stages = 4;
constexpr int kGroupsPerStage = BK / 32;  // 4
constexpr int kG32EpiWarps = 8;          // two per tensor-memory lane quarter (16 measured the same: not latency-bound)
constexpr int kColW = GBN / (kG32EpiWarps / 4);   // columns of the tile per epilogue warp (64)
constexpr int kNB = kColW / 8;           // 8-column blocks per warp
constexpr int kG32Threads = 64 + 32 * kG32EpiWarps;

// 16 lanes x (8 x NB) columns of tensor memory -> 4 x NB registers per thread
__device__ __forceinline__ void tmem_ld_cols(uint32_t addr, uint32_t (&v)[32]) { tmem_ld_16x256b_x8(addr, v); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t addr, uint32_t (&v)[16]) { tmem_ld_16x256b_x4(addr, v); }

struct G32Params {
  const float* bias;
  void* out;
  int32_t* status;
  int64_t ldo;
  int M, N, K;
  int sched_pm, sched_pn;
  int has_bias;
};

struct G32Smem {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = GBN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSaBytes = BM * kGroupsPerStage * 4;     // [128 rows][4 groups] fp32
  static constexpr int kSwBytes = kGroupsPerStage * GBN * 4;    // [4 groups][128 cols] fp32
  static constexpr int kScaleBytes = kSaBytes + kSwBytes;
  static constexpr int kScaleOff = kG32Stages * kStageBytes;
  static constexpr int kBarOff = kScaleOff + kG32Stages * kScaleBytes;
  static constexpr int kNumBars = 4 * kG32Stages + 2 * kSlots;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kDynamic = kMiscOff + 16 + 1024;
};

template <typename OutT>
__global__ void __launch_bounds__(kG32Threads, 1)
pq_int8_gemm_g32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                        const __grid_constant__ CUtensorMap tmSa, const __grid_constant__ CUtensorMap tmSw,
                        const G32Params p) {
  using L = G32Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kG32Stages;
  uint64_t* sfull_bar = empty_bar + kG32Stages;
  uint64_t* sempty_bar = sfull_bar + kG32Stages;
  uint64_t* slot_full = sempty_bar + kG32Stages;
  uint64_t* slot_empty = slot_full + kSlots;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int mt_total = (p.M + BM - 1) / BM;
  const int nt = (p.N + GBN - 1) / GBN;
  const int num_kb = p.K / BK;                      // host guarantees K % 128 == 0
  constexpr uint32_t kTmemCols = kSlots * GBN;      // 512

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmSa); tma_prefetch_desc(&tmSw);
    for (int s = 0; s < kG32Stages; ++s) {
      mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1);
      mbar_init(&sfull_bar[s], 1); mbar_init(&sempty_bar[s], kG32EpiWarps);
    }
    for (int s = 0; s < kSlots; ++s) { mbar_init(&slot_full[s], 1); mbar_init(&slot_empty[s], kG32EpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) { tmem_alloc(tmem_holder, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0; long long issued = 0; bool ok = true;
      TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance()) {
        const int row0 = w.mt * BM, n0 = w.ntile * GBN;
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag) ||
              !wait_or_abort(&sempty_bar[stage], phase ^ 1u, abort_flag)) {
            report_timeout(p.status, 1, 1); *abort_flag = 1; ok = false; break;
          }
          uint8_t* a_s = smem + stage * L::kStageBytes;
          uint8_t* sc_s = smem + L::kScaleOff + stage * L::kScaleBytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(a_s, &tmA, &full_bar[stage], kb * BK, row0);
          tma_load_2d(a_s + L::kABytes, &tmW, &full_bar[stage], kb * BK, n0);
          mbar_arrive_expect_tx(&sfull_bar[stage], L::kScaleBytes);
          tma_load_2d(sc_s, &tmSa, &sfull_bar[stage], kb * kGroupsPerStage, row0);           // [128 rows][4 groups]
          tma_load_2d(sc_s + L::kSaBytes, &tmSw, &sfull_bar[stage], n0, kb * kGroupsPerStage);  // [4 groups][128 cols]
          ++issued;
          if (++stage == kG32Stages) { stage = 0; phase ^= 1u; }
        }
      }
      const int pending = issued < kG32Stages ? static_cast<int>(issued) : kG32Stages;
      for (int i = 0; i < pending; ++i) {          // copies in flight must land before the CTA may exit
        if (--stage < 0) { stage = kG32Stages - 1; phase ^= 1u; }
        if (!wait_or_abort(&full_bar[stage], phase, abort_flag) || !wait_or_abort(&sfull_bar[stage], phase, abort_flag)) {
          for (int k = 0; k < 64; ++k) __nanosleep(1000);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer: one instruction per group
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8(BM, GBN);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      uint32_t gc = 0;                                // stages issued so far
      TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance()) {
#pragma unroll 1
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
            report_timeout(p.status, 2, 1); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + L::kABytes);
          // the four groups of a stage go to the four slots back to back; one "slots free" wait and one "slots
          // written" commit per stage (every barrier operation costs this thread a few hundred cycles)
          if (!wait_or_abort(&slot_empty[0], (gc & 1u) ^ 1u, abort_flag)) {
            report_timeout(p.status, 2, 2); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
#pragma unroll
          for (int g = 0; g < kGroupsPerStage; ++g)
            tc_mma_i8(tmem_base + g * GBN, a_desc + static_cast<uint64_t>(2 * g), b_desc + static_cast<uint64_t>(2 * g),
                      idesc, 0u);
          tc_commit(&slot_full[0]);
          ++gc;
          if (ok) tc_commit(&empty_bar[stage]);
          if (++stage == kG32Stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..)
    const int quarter = warp & 3;              // tensor-memory lanes [32*quarter, +32)
    const int colg = (warp - 2) >> 2;          // columns [kColW*colg, +kColW) of the tile
    auto ld_cols = [](uint32_t addr, uint32_t (&v)[4 * kNB]) { tmem_ld_cols(addr, v); };
    const int g4 = lane >> 2, q = lane & 3;
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_store = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool aborted = false;
    int stage = 0; uint32_t phase = 0;
    uint32_t gc = 0;
    TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
    for (; w.valid(); w.advance()) {
      const int row0 = w.mt * BM, n0 = w.ntile * GBN;
      // y[mb][nb][0] = (row g4, cols 2q, 2q+1), y[mb][nb][1] = (row g4 + 8, same cols) of n8 block nb, 16-row block mb
      float2 y[2][kNB][2];
#pragma unroll
      for (int mb = 0; mb < 2; ++mb)
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) { y[mb][nb][0] = make_float2(0.f, 0.f); y[mb][nb][1] = make_float2(0.f, 0.f); }

#pragma unroll 1
      for (int kb = 0; kb < num_kb; ++kb) {
        const float* sa_s = reinterpret_cast<const float*>(smem + L::kScaleOff + stage * L::kScaleBytes);
        const float* sw_s = sa_s + BM * kGroupsPerStage;
        if (!aborted) {
          const bool landed = wait_or_abort(&sfull_bar[stage], phase, abort_flag);
          if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 4); *abort_flag = 1; aborted = true; }
        }
        if (!aborted) {
          const bool landed = wait_or_abort(&slot_full[0], gc & 1u, abort_flag);
          if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true; }
        }
        ++gc;
        if (!aborted) tc_fence_after();
        uint32_t va[4 * kNB], vb[4 * kNB];
        if (!aborted) {
          const uint32_t t0_acc = tmem_base + colg * kColW;
          ld_cols(t0_acc + (static_cast<uint32_t>(quarter * 32) << 16), va);
        }
#pragma unroll 1
        for (int g = 0; g < kGroupsPerStage; ++g) {
          if (aborted) continue;
          const uint32_t t_acc = tmem_base + g * GBN + colg * kColW;
          const float2 kNegMagic2 = make_float2(-12582912.0f, -12582912.0f);
          // |partial| <= 32 * 127^2 < 2^22: adding the bit pattern of 1.5 * 2^23 converts exactly
          auto cvt2 = [&](uint32_t a, uint32_t b) {
            return __fadd2_rn(make_float2(__int_as_float(0x4B400000 + static_cast<int32_t>(a)),
                                          __int_as_float(0x4B400000 + static_cast<int32_t>(b))), kNegMagic2);
          };
          const float* swg = sw_s + g * GBN + colg * kColW + 2 * q;
          // row scales of this thread's four rows for this group (shared memory tile [128 rows][4 groups])
          const float* sag = sa_s + (quarter * 32 + g4) * kGroupsPerStage + g;
          tc_wait_ld();                                                       // rows 0..15 of group g are in va
          ld_cols(t_acc + (static_cast<uint32_t>(quarter * 32 + 16) << 16), vb);
          {
            const float saA = sag[0], saB = sag[8 * kGroupsPerStage];
#pragma unroll
            for (int nb = 0; nb < kNB; ++nb) {
              const float2 sw2 = *reinterpret_cast<const float2*>(swg + nb * 8);
              // same arithmetic as the CPU restatement: running sum = fma(partial, s_a * s_w, running sum)
              y[0][nb][0] = __ffma2_rn(cvt2(va[4 * nb + 0], va[4 * nb + 1]), __fmul2_rn(make_float2(saA, saA), sw2), y[0][nb][0]);
              y[0][nb][1] = __ffma2_rn(cvt2(va[4 * nb + 2], va[4 * nb + 3]), __fmul2_rn(make_float2(saB, saB), sw2), y[0][nb][1]);
            }
          }
          tc_wait_ld();                                                       // rows 16..31 of group g are in vb
          if (g + 1 < kGroupsPerStage) {
            ld_cols(t_acc + GBN + (static_cast<uint32_t>(quarter * 32) << 16), va);
          } else {
            tc_fence_before();                                                // all four slots are in registers:
            __syncwarp();                                                     // the MMA thread may refill them
            if (lane == 0) mbar_arrive(&slot_empty[0]);
          }
          {
            const float saA = sag[16 * kGroupsPerStage], saB = sag[24 * kGroupsPerStage];
#pragma unroll
            for (int nb = 0; nb < kNB; ++nb) {
              const float2 sw2 = *reinterpret_cast<const float2*>(swg + nb * 8);
              y[1][nb][0] = __ffma2_rn(cvt2(vb[4 * nb + 0], vb[4 * nb + 1]), __fmul2_rn(make_float2(saA, saA), sw2), y[1][nb][0]);
              y[1][nb][1] = __ffma2_rn(cvt2(vb[4 * nb + 2], vb[4 * nb + 3]), __fmul2_rn(make_float2(saB, saB), sw2), y[1][nb][1]);
            }
          }
        }
        // scales of this stage consumed
        __syncwarp();
        if (lane == 0) mbar_arrive(&sempty_bar[stage]);
        if (++stage == kG32Stages) { stage = 0; phase ^= 1u; }
      }
      if (aborted) continue;

      // ---- bias, rounding, store
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        const int rA = row0 + quarter * 32 + mb * 16 + g4;
        const int rB = rA + 8;
#pragma unroll
        for (int grp = 0; grp < kColW / 32; ++grp) {
          uint32_t wA[4], wB[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int nb = grp * 4 + j;
            const int col = n0 + colg * kColW + nb * 8 + 2 * q;
            float2 b2 = make_float2(0.f, 0.f);
            if (p.has_bias && col + 1 < p.N) b2 = *reinterpret_cast<const float2*>(p.bias + col);
            else if (p.has_bias && col < p.N) b2.x = p.bias[col];
            const float2 a = __fadd2_rn(y[mb][nb][0], b2), b = __fadd2_rn(y[mb][nb][1], b2);
            wA[j] = pack2(a.x, a.y, OutT{});
            wB[j] = pack2(b.x, b.y, OutT{});
          }
          const int col_grp = n0 + colg * kColW + grp * 32;
          if (vec_store && col_grp + 32 <= p.N) {
            quad_transpose(wA, q);
            quad_transpose(wB, q);
            if (rA < p.M) st_v4(out + static_cast<int64_t>(rA) * p.ldo + col_grp + q * 8, make_uint4(wA[0], wA[1], wA[2], wA[3]));
            if (rB < p.M) st_v4(out + static_cast<int64_t>(rB) * p.ldo + col_grp + q * 8, make_uint4(wB[0], wB[1], wB[2], wB[3]));
          } else {
            store_pairs_slow(p.out, p.ldo, rA, rB, col_grp + 2 * q, p.M, p.N, make_uint4(wA[0], wA[1], wA[2], wA[3]),
                             make_uint4(wB[0], wB[1], wB[2], wB[3]));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0) {
      for (int k = 0; k < 64; ++k) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename OutT>
int launch_g32(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSa, const CUtensorMap& tmSw,
               const G32Params& p, int grid, cudaStream_t st) {
  auto kern = pq_int8_gemm_g32_kernel<OutT>;
  PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G32Smem::kDynamic));
  kern<<<grid, kG32Threads, G32Smem::kDynamic, st>>>(tmA, tmW, tmSa, tmSw, p);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_int8_gemm_g32(const int8_t* xq, int64_t ldx, const float* s_a, const int8_t* w, int64_t ldw,
                                const float* s_w, const float* bias, void* out, int out_dtype, int64_t ldo, int64_t M,
                                int64_t N, int64_t K, void* workspace, size_t ws_bytes, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return PQ_ERR_SHAPE;
  if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return PQ_ERR_SHAPE;
  if (out_dtype != PQ_DTYPE_BF16 && out_dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (xq == nullptr || s_a == nullptr || w == nullptr || s_w == nullptr || out == nullptr) return PQ_ERR_NULL;
  if (ldx < K || ldw < K || ldo < N) return PQ_ERR_SHAPE;
  if (K % BK != 0) return PQ_ERR_UNSUPPORTED;            // whole 128-byte stages only (four groups per stage)
  if (ldx % 16 != 0 || ldw % 16 != 0 || N % 4 != 0) return PQ_ERR_ALIGN;
  if (!aligned_to(xq, 16) || !aligned_to(w, 16) || !aligned_to(s_a, 16) || !aligned_to(s_w, 16)) return PQ_ERR_ALIGN;
  if (ldo % 2 != 0 || !aligned_to(out, 4)) return PQ_ERR_ALIGN;
  if (bias != nullptr && !aligned_to(bias, 8)) return PQ_ERR_ALIGN;
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;

  const int64_t G = K / 32;
  CUtensorMap tmA, tmW, tmSa, tmSw;
  int rc = make_tile_map(&tmA, xq, M, K, ldx, BM);
  if (rc != PQ_OK) return rc;
  rc = make_tile_map(&tmW, w, N, K, ldw, GBN);
  if (rc != PQ_OK) return rc;
  rc = make_f32_map(&tmSa, s_a, M, G, G, kGroupsPerStage, BM);      // [M, G]: box 4 groups x 128 rows
  if (rc != PQ_OK) return rc;
  rc = make_f32_map(&tmSw, s_w, G, N, N, GBN, kGroupsPerStage);     // [G, N]: box 128 cols x 4 groups
  if (rc != PQ_OK) return rc;

  G32Params p;
  p.bias = bias; p.out = out; p.status = static_cast<int32_t*>(workspace); p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.has_bias = bias != nullptr ? 1 : 0;
  const int mt = static_cast<int>((M + BM - 1) / BM), ntl = static_cast<int>((N + GBN - 1) / GBN);
  const int max_ctas = options().gemm_max_ctas > 0 ? options().gemm_max_ctas : sm_count();
  choose_cta_grid(mt, ntl, max_ctas, &p.sched_pm, &p.sched_pn);
  const int grid = p.sched_pm * p.sched_pn;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == PQ_DTYPE_BF16) return launch_g32<__nv_bfloat16>(tmA, tmW, tmSa, tmSw, p, grid, st);
  return launch_g32<__half>(tmA, tmW, tmSa, tmSw, p, grid, st);
}
