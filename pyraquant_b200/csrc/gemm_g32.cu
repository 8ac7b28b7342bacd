// Group-32 W8A8 GEMM for sm_100a:
//   out[m,n] = sum_g s_a[m,g] * s_w[g,n] * (sum_{k in group g} xq[m,k] * w[n,k])  (+ bias[n])
// A group is 32 consecutive K = exactly one tcgen05.mma kind::i8 instruction, so every instruction produces the exact
// int32 partial sum of one group in one of four 128-column tensor-memory slots; the epilogue warps drain the slots and
// fold them into fp32 running sums in registers: sum = fma(float(partial), s_a * s_w, sum), ascending groups, the
// arithmetic of the CPU restatement (bit-equal outputs).
//
// Two things bound the kernel, and neither is the tensor pipe (under 10 % busy):
//  * every partial sum crosses from tensor memory to registers, 64 KB per 128 x 128 tile and group, at about 140 bytes
//    per clock and SM (measured with the arithmetic removed);
//  * a conversion, a product of the two scales and a fused multiply-add per output element and group.  The conversion
//    is the hardware one (cvt.rn.f32.s32): it issues on the integer pipe and leaves the fp32 pipe to the two packed
//    operations; converting with the add-a-magic-number trick puts three operations per element pair on the fp32 pipe
//    and runs 10 % slower.
// A thread owns four rows of an 8-column block pair (the tcgen05.ld 16x256b arrangement, two loads of 16 rows per group),
// so one 8-byte shared-memory load of column scales serves eight outputs.  Sixteen epilogue warps (32 columns each) hide
// the latency of the tensor-memory loads better than eight; within a slot pair the load of the next 16 rows is in flight
// while the current ones are folded.  Slots are handed over in pairs, so the MMA thread refills one pair while the
// warps work on the other.
// Probes of where the time goes (16384 x 1280 -> 10240, cycles per group and SM at 1.9 GHz): the full kernel 715; the
// same with the arithmetic removed 405; with the tensor-memory loads removed as well, i.e. only the slot hand-shakes
// between the MMA thread and the sixteen warps, 246 (a slot pair needs about 980 cycles from its release to being
// complete again, hidden as long as draining and folding the other pair takes longer); requesting all four chunks of a
// pair at once instead of one ahead does not speed up the loads (405 -> 400): the drain is a throughput limit of about
// 160-200 bytes per cycle, not a latency one.  Drain (about 320) and arithmetic (about 310: the conversion pipe takes
// 256 of them) add up instead of overlapping, whatever the warps' arrangement: requesting the next chunk only after
// the current one has been folded, i.e. with no overlap by construction, measures the same (415 against 406 TOPS).
// Tried and dropped: slots handed over one by one with the next chunk always requested across slot and stage boundaries
// (non-blocking probe of the next slot's barrier): 356 instead of 408 TOPS, spills at 96 registers;
// a row-per-thread arrangement (tcgen05.ld 32x32b: the row scale becomes a register, but the loads
// are no faster and the column scales need twice the shared-memory loads); accumulators pre-biased with 0x4B400000 so
// that the int32 result read as fp32 bits needs only a subtraction (the tcgen05.st that restores the bias costs more
// tensor-memory bandwidth than the integer additions it saves); keeping a load in flight across slot pairs, stages and
// tiles (more live registers than the 96 per thread that 18 warps leave).
// Roles: warp 0 TMA producer (operand stages plus a ring of scale tiles), warp 1 MMA issuer, warps 2.. epilogue.
// Every wait is bounded.  No clusters, no multicast.
#include <type_traits>

#include "gemm_common.cuh"

namespace pq {
namespace {

constexpr int GBN = 128;                 // columns per tile = one tensor-memory slot
constexpr int kSlots = 4;
constexpr int kSlotPairs = 2;
constexpr int kG32Stages = 4;
constexpr int kGroupsPerStage = BK / 32;  // 4
constexpr int g32_threads(int ew) { return 64 + 32 * ew; }

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
  static constexpr int kNumBars = 4 * kG32Stages + 2 * kSlotPairs;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kDynamic = kMiscOff + 16 + 1024;
};

// EW epilogue warps; ARITH = false replaces the scale arithmetic by a plain sum (measurement of the data path only, the
// output is then meaningless); PACKED = false uses scalar instead of packed fp32 operations.
template <typename OutT, int EW, bool ARITH, bool PACKED>
__global__ void __launch_bounds__(g32_threads(EW), 1)
pq_int8_gemm_g32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                        const __grid_constant__ CUtensorMap tmSa, const __grid_constant__ CUtensorMap tmSw,
                        const G32Params p) {
  using L = G32Smem;
  static_assert(EW == 8 || EW == 16, "eight or sixteen epilogue warps");
  constexpr int kColW = GBN / (EW / 4);       // columns of the tile per epilogue warp: 64 or 32
  constexpr int kNB = kColW / 8;              // 8-column blocks per warp: 8 or 4
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kG32Stages;
  uint64_t* sfull_bar = empty_bar + kG32Stages;
  uint64_t* sempty_bar = sfull_bar + kG32Stages;
  uint64_t* slot_full = sempty_bar + kG32Stages;      // [pair]
  uint64_t* slot_empty = slot_full + kSlotPairs;      // [pair]
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
      mbar_init(&sfull_bar[s], 1); mbar_init(&sempty_bar[s], EW);
    }
    for (int s = 0; s < kSlotPairs; ++s) { mbar_init(&slot_full[s], 1); mbar_init(&slot_empty[s], EW); }
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
      uint32_t uses = 0;                              // stages issued so far = uses of either slot pair
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
#pragma unroll
          for (int pr = 0; pr < kSlotPairs; ++pr) {
            // the epilogue's initial hand-over is completion 0 of slot_empty: use n of a pair waits for completion n
            if (!wait_or_abort(&slot_empty[pr], uses & 1u, abort_flag)) {
              report_timeout(p.status, 2, 2); *abort_flag = 1; ok = false; break;
            }
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int g = 2 * pr + j;
              tc_mma_i8(tmem_base + g * GBN, a_desc + static_cast<uint64_t>(2 * g), b_desc + static_cast<uint64_t>(2 * g),
                        idesc, 0u);
            }
            tc_commit(&slot_full[pr]);
          }
          if (!ok) break;
          ++uses;
          tc_commit(&empty_bar[stage]);
          if (++stage == kG32Stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..)
    // A stage is eight chunks: chunk k = rows [16 (k & 1), +16) of this warp's lane quarter, group k >> 1, slot pair
    // k >> 2.  Chunks alternate between two register buffers; inside a slot pair the load of chunk k + 1 is issued as
    // soon as chunk k has landed and stays in flight while chunk k is folded.  A slot pair is handed back to the MMA
    // thread as soon as its last chunk is in registers (before that chunk is folded).
    const int quarter = warp & 3;              // tensor-memory lanes [32*quarter, +32)
    const int colg = (warp - 2) >> 2;          // columns [kColW*colg, +kColW) of the tile
    const int g4 = lane >> 2, q = lane & 3;
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_store = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool aborted = false;
    int stage = 0; uint32_t phase = 0;
    uint32_t uses = 0;
    // lanes [32 quarter + 16 h, +16), this warp's columns, of slot g
    auto slot_addr = [&](int g, int h) {
      return tmem_base + static_cast<uint32_t>(g * GBN + colg * kColW) + (static_cast<uint32_t>(quarter * 32 + h * 16) << 16);
    };
    // the slots start out free
    if (lane == 0) { mbar_arrive(&slot_empty[0]); mbar_arrive(&slot_empty[1]); }

    TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
    for (; w.valid() && !aborted; w.advance()) {
      const int row0 = w.mt * BM, n0 = w.ntile * GBN;
      // y[h][nb][0] = (row 16 h + g4, cols 2q, 2q+1 of 8-column block nb), y[h][nb][1] = same columns, row + 8
      float2 y[2][kNB][2];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) { y[h][nb][0] = make_float2(0.f, 0.f); y[h][nb][1] = make_float2(0.f, 0.f); }

#pragma unroll 1
      for (int kb = 0; kb < num_kb && !aborted; ++kb) {
        const float* sa_s = reinterpret_cast<const float*>(smem + L::kScaleOff + stage * L::kScaleBytes);
        const float* sw_s = sa_s + BM * kGroupsPerStage;
        {
          const bool landed = wait_or_abort(&sfull_bar[stage], phase, abort_flag);
          if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 4); *abort_flag = 1; aborted = true; break; }
        }
        // row scales of this thread's four rows (g4 + 8 r) sit at sa_row[8 r * 4 + group]
        const float* sa_row = sa_s + (quarter * 32 + g4) * kGroupsPerStage;
        uint32_t va[4 * kNB], vb[4 * kNB];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int g = k >> 1, h = k & 1, pr = k >> 2;
          uint32_t (&v)[4 * kNB] = h == 0 ? va : vb;
          uint32_t (&vnext)[4 * kNB] = h == 0 ? vb : va;
          if ((k & 3) == 0) {                                        // first chunk of a pair: the MMAs have completed
            const bool landed = wait_or_abort(&slot_full[pr], uses & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true; break; }
            tc_fence_after();
            tmem_ld_cols(slot_addr(g, 0), v);
          }
          tc_wait_ld();                                              // chunk k is in v
          if ((k & 3) == 3) {                                        // the pair is in registers: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&slot_empty[pr]);
          } else {
            tmem_ld_cols(slot_addr((k + 1) >> 1, (k + 1) & 1), vnext);   // on its way while chunk k is folded
          }
          const float sa_lo = sa_row[(16 * h) * kGroupsPerStage + g], sa_hi = sa_row[(16 * h + 8) * kGroupsPerStage + g];
          const float* swp = sw_s + g * GBN + colg * kColW + 2 * q;
#pragma unroll
          for (int nb = 0; nb < kNB; ++nb) {
            // column scales: one 8-byte load per 8-column block serves the thread's two rows of this chunk
            const float2 sw2 = *reinterpret_cast<const float2*>(swp + nb * 8);
            const float2 pA = make_float2(__int2float_rn(static_cast<int32_t>(v[4 * nb + 0])), __int2float_rn(static_cast<int32_t>(v[4 * nb + 1])));
            const float2 pB = make_float2(__int2float_rn(static_cast<int32_t>(v[4 * nb + 2])), __int2float_rn(static_cast<int32_t>(v[4 * nb + 3])));
            if constexpr (!ARITH) {
              y[h][nb][0] = __fadd2_rn(make_float2(__uint_as_float(v[4 * nb + 0]), __uint_as_float(v[4 * nb + 1])), y[h][nb][0]);
              y[h][nb][1] = __fadd2_rn(make_float2(__uint_as_float(v[4 * nb + 2]), __uint_as_float(v[4 * nb + 3])), y[h][nb][1]);
            } else if constexpr (PACKED) {
              // same arithmetic as the CPU restatement: running sum = fma(partial, s_a * s_w, running sum)
              y[h][nb][0] = __ffma2_rn(pA, __fmul2_rn(make_float2(sa_lo, sa_lo), sw2), y[h][nb][0]);
              y[h][nb][1] = __ffma2_rn(pB, __fmul2_rn(make_float2(sa_hi, sa_hi), sw2), y[h][nb][1]);
            } else {
              y[h][nb][0].x = __fmaf_rn(pA.x, __fmul_rn(sa_lo, sw2.x), y[h][nb][0].x);
              y[h][nb][0].y = __fmaf_rn(pA.y, __fmul_rn(sa_lo, sw2.y), y[h][nb][0].y);
              y[h][nb][1].x = __fmaf_rn(pB.x, __fmul_rn(sa_hi, sw2.x), y[h][nb][1].x);
              y[h][nb][1].y = __fmaf_rn(pB.y, __fmul_rn(sa_hi, sw2.y), y[h][nb][1].y);
            }
          }
        }
        if (aborted) break;
        ++uses;
        // scales of this stage consumed
        __syncwarp();
        if (lane == 0) mbar_arrive(&sempty_bar[stage]);
        if (++stage == kG32Stages) { stage = 0; phase ^= 1u; }
      }
      if (aborted) break;

      // ---- bias, rounding, store
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int rA = row0 + quarter * 32 + h * 16 + g4;
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
            const float2 a = __fadd2_rn(y[h][nb][0], b2), b = __fadd2_rn(y[h][nb][1], b2);
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
    tc_wait_ld();                                  // nothing of this warp may be in flight when tensor memory is freed
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

template <typename OutT, int EW, bool ARITH, bool PACKED>
int launch_g32_variant(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSa, const CUtensorMap& tmSw,
                       const G32Params& p, int grid, cudaStream_t st) {
  auto kern = pq_int8_gemm_g32_kernel<OutT, EW, ARITH, PACKED>;
  PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G32Smem::kDynamic));
  kern<<<grid, g32_threads(EW), G32Smem::kDynamic, st>>>(tmA, tmW, tmSa, tmSw, p);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// Option "g32_variant": bit 0 = eight epilogue warps (default sixteen); bit 1 = scalar instead of packed fp32
// operations; bit 3 = data path only (no scale arithmetic: for measurements, output meaningless).
template <typename OutT, int EW>
int launch_g32_e(int v, const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSa, const CUtensorMap& tmSw,
                 const G32Params& p, int grid, cudaStream_t st) {
  if (v & 8) return launch_g32_variant<OutT, EW, false, true>(tmA, tmW, tmSa, tmSw, p, grid, st);
  if (v & 2) return launch_g32_variant<OutT, EW, true, false>(tmA, tmW, tmSa, tmSw, p, grid, st);
  return launch_g32_variant<OutT, EW, true, true>(tmA, tmW, tmSa, tmSw, p, grid, st);
}
template <typename OutT>
int launch_g32(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmSa, const CUtensorMap& tmSw,
               const G32Params& p, int grid, cudaStream_t st) {
  const int v = options().g32_variant;
  if (v & 1) return launch_g32_e<OutT, 8>(v, tmA, tmW, tmSa, tmSw, p, grid, st);
  return launch_g32_e<OutT, 16>(v, tmA, tmW, tmSa, tmSw, p, grid, st);
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
