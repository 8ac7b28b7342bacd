// Fused INT8 GEMM with the rank-32 low-rank term on the tcgen05 tensor cores.
//
//   out = float(xq @ w^T) * (s_row x s_col) + t @ lb + bias
//
// Same roles, operand ring, tile schedule and bounded waits as the kernel in gemm.cu; what differs is the
// epilogue.  Legacy warp-level mma.sync next to a saturated tcgen05 stream costs far more than its share of the
// arithmetic, so the low-rank product is issued as two tcgen05.mma kind::f16 instructions (128 x BN x 16 each)
// that accumulate IN PLACE onto the already scaled accumulator:
//   1. epilogue warps read the int32 accumulator, convert, multiply by s_row * s_col and write the fp32 value back
//      to the same tensor-memory columns (tcgen05.st), then signal the MMA thread;
//   2. the MMA thread, between two k-blocks of the next tile's main loop, issues D += t_tile * lbT_tile^T
//      (operands staged by TMA with the 64-byte swizzle: t tile 128 x 32 and lbT tile BN x 32, both K-major);
//   3. epilogue warps read the fp32 result, add the bias, round, transpose inside quads and store 16 bytes per thread.
// The operation order of the reference kernel (acc * scale, + low rank, + bias; deploy/int8_exec.py:303-309)
// is kept; the rank-32 dot product is summed by the tensor core in fp32.
#include <type_traits>

#include "gemm_common.cuh"
#include "gemm_lr_tc.cuh"

namespace pq {
namespace {

constexpr int kTRowBytes = kLR * 2;        // 64-byte rows of the t / lbT tiles (32 x 16-bit)

template <int BN, int STAGES>
struct LrSmem {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTOff = STAGES * kStageBytes;          // two t tiles (one per accumulator buffer)
  static constexpr int kTBytes = BM * kTRowBytes;
  static constexpr int kLbOff = kTOff + 2 * kTBytes;          // one lbT tile
  static constexpr int kLbBytes = BN * kTRowBytes;
  static constexpr int kScolOff = kLbOff + kLbBytes;
  static constexpr int kBiasOff = kScolOff + BN * 4;
  static constexpr int kBarOff = kBiasOff + BN * 4;
  // full[S], empty[S], tfull[2], tempty[2], t_full[2], lb_full[1], ylr_ready[2], lr_done[2]
  static constexpr int kNumBars = 2 * STAGES + 11;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal;                       // the base is declared 1024-byte aligned
  static_assert(kTotal <= 232448, "exceeds the 227 KB shared memory of one CTA");
};

// K-major operand tile with 64-byte rows and the 64-byte swizzle (TMA box of 64 bytes x rows with
// CU_TENSOR_MAP_SWIZZLE_64B): 8-row atoms are 512 bytes apart.
__device__ __forceinline__ uint64_t make_kmajor_sw64_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;                            // SWIZZLE_64B
  return d;
}

// Instruction descriptor, kind::f16: D fp32, A and B bf16 (or fp16), both K-major.
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Test hook: raw accumulators of one n8 block (rows rA / rB, columns col, col+1).
__device__ __noinline__ void dump_acc_lr(int32_t* dbg, int N, int rA, int rB, int col, int row_end, uint32_t v0, uint32_t v1,
                                         uint32_t v2, uint32_t v3) {
  if (rA < row_end && col < N) dbg[static_cast<int64_t>(rA) * N + col] = static_cast<int32_t>(v0);
  if (rA < row_end && col + 1 < N) dbg[static_cast<int64_t>(rA) * N + col + 1] = static_cast<int32_t>(v1);
  if (rB < row_end && col < N) dbg[static_cast<int64_t>(rB) * N + col] = static_cast<int32_t>(v2);
  if (rB < row_end && col + 1 < N) dbg[static_cast<int64_t>(rB) * N + col + 1] = static_cast<int32_t>(v3);
}

template <int BN, int STAGES, typename OutT, bool DBG>
__global__ void __launch_bounds__(kGemmThreads, 1)
pq_int8_gemm_fused_lr_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW0,
                             const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmT,
                             const __grid_constant__ CUtensorMap tmLbT, const GemmParams p) {
  using L = LrSmem<BN, STAGES>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* t_full = tempty_bar + 2;
  uint64_t* lb_full = t_full + 2;
  uint64_t* ylr_ready = lb_full + 1;
  uint64_t* lr_done = ylr_ready + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem) & 1023u) != 0) {           // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report_timeout(p.status, 7, 7);
    return;
  }

  const int mt0 = (p.m_split + BM - 1) / BM;
  const int mt_total = mt0 + (p.M - p.m_split + BM - 1) / BM;
  const int nt = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmW0); tma_prefetch_desc(&tmW1);
    tma_prefetch_desc(&tmT); tma_prefetch_desc(&tmLbT);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], kNumEpiWarps);
      mbar_init(&t_full[b], 1); mbar_init(&ylr_ready[b], kNumEpiWarps); mbar_init(&lr_done[b], 1);
    }
    mbar_init(lb_full, 1);
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
      int it = 0; int lb_col = -1;
      TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance(), ++it) {
        const TileCoord c = tile_coord(w, p, mt0, BN);
        const int buf = it & 1;
        if (w.ntile != lb_col) {
          // the single lbT tile may be replaced once every low-rank MMA that read it has completed, i.e. once the
          // epilogue of the previous tile has handed its accumulator back (phase (it-1)>>1 of that buffer)
          if (it > 0 && !wait_or_abort(&tempty_bar[(it - 1) & 1], static_cast<uint32_t>(((it - 1) >> 1) & 1), abort_flag)) {
            report_timeout(p.status, 1, 5); *abort_flag = 1; ok = false; break;
          }
          lb_col = w.ntile;
          mbar_arrive_expect_tx(lb_full, L::kLbBytes);
          tma_load_2d(smem + L::kLbOff, &tmLbT, lb_full, 0, c.n0);
        }
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            report_timeout(p.status, 1, 1); *abort_flag = 1; ok = false; break;
          }
          uint8_t* a_s = smem + stage * L::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(a_s, &tmA, &full_bar[stage], kb * BK, c.row0);
          if (c.set == 0) tma_load_2d(a_s + L::kABytes, &tmW0, &full_bar[stage], kb * BK, c.n0);
          else tma_load_2d(a_s + L::kABytes, &tmW1, &full_bar[stage], kb * BK, c.n0);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        // t tile of this row block: its shared-memory slot is free once the accumulator buffer of two tiles ago
        // has been released (the low-rank MMA that read the slot finished before that)
        if (!wait_or_abort(&tempty_bar[buf], (static_cast<uint32_t>(it >> 1) & 1u) ^ 1u, abort_flag)) {
          report_timeout(p.status, 1, 6); *abort_flag = 1; ok = false; break;
        }
        mbar_arrive_expect_tx(&t_full[buf], L::kTBytes);
        tma_load_2d(smem + L::kTOff + buf * L::kTBytes, &tmT, &t_full[buf], 0, c.row0);
      }
      const int pending = issued < STAGES ? static_cast<int>(issued) : STAGES;
      for (int i = 0; i < pending; ++i) {          // copies in flight must land before the CTA may exit
        if (--stage < 0) { stage = STAGES - 1; phase ^= 1u; }
        if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
          for (int k = 0; k < 64; ++k) __nanosleep(1000);
          break;
        }
      }
      // the t / lbT copies are consumed by low-rank MMAs that the epilogue waits for, so they have landed by the
      // time the CTA reaches its final barrier (or the abort path sleeps there)
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8(BM, BN);
      constexpr uint32_t idesc_lr = make_idesc_f16(BM, BN, std::is_same<OutT, __nv_bfloat16>::value);
      int stage = 0; uint32_t phase = 0; int it = 0; bool ok = true;
      int pending = -1;                 // tile whose scaled accumulator waits for its low-rank MMAs
      int lb_col = -1; uint32_t lb_count = 0; int pending_col = -1;
      // D(buffer of tile `pt`) += t_tile * lbT_tile^T as two K = 16 instructions
      auto issue_lowrank = [&](int pt, int pcol) -> bool {
        const int pb = pt & 1;
        const uint32_t par = static_cast<uint32_t>(pt >> 1) & 1u;
        if (!wait_or_abort(&ylr_ready[pb], par, abort_flag)) { report_timeout(p.status, 2, 3); return false; }
        if (!wait_or_abort(&t_full[pb], par, abort_flag)) { report_timeout(p.status, 2, 4); return false; }
        if (pcol != lb_col) {
          if (!wait_or_abort(lb_full, lb_count & 1u, abort_flag)) { report_timeout(p.status, 2, 5); return false; }
          lb_col = pcol; ++lb_count;
        }
        tc_fence_after();
        const uint64_t a_desc = make_kmajor_sw64_desc(smem_u32(smem + L::kTOff + pb * L::kTBytes));
        const uint64_t b_desc = make_kmajor_sw64_desc(smem_u32(smem + L::kLbOff));
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(pb * BN);
        tc_mma_f16(d_tmem, a_desc, b_desc, idesc_lr, 1u);
        tc_mma_f16(d_tmem, a_desc + 2, b_desc + 2, idesc_lr, 1u);      // next 16 K = +32 bytes
        tc_commit(&lr_done[pb]);
        return true;
      };
      TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance(), ++it) {
        const int buf = it & 1;
        const uint32_t use = static_cast<uint32_t>(it >> 1);
        if (!wait_or_abort(&tempty_bar[buf], (use & 1u) ^ 1u, abort_flag)) {
          report_timeout(p.status, 2, 2); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          // wait for the stage; while waiting, issue the low-rank MMAs of the previous tile as soon as its scaled
          // accumulator is back in tensor memory (the producer may itself be waiting for that tile to finish)
          {
            uint64_t t0 = 0; uint32_t polls = 0; bool got = false;
            while (true) {
              if (mbar_try_wait(&full_bar[stage], phase)) { got = true; break; }
              if (pending >= 0 && mbar_test_wait(&ylr_ready[pending & 1], static_cast<uint32_t>(pending >> 1) & 1u)) {
                if (!issue_lowrank(pending, pending_col)) break;
                pending = -1;
              }
              if ((++polls & 255u) == 0) {
                if (*abort_flag != 0) break;
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now; else if (now - t0 > kWaitBudgetNs) break;
              }
            }
            if (!got) { report_timeout(p.status, 2, 1); *abort_flag = 1; ok = false; break; }
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_i8(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
        if (pending >= 0) {             // keep the low-rank MMAs in tile order
          if (!issue_lowrank(pending, pending_col)) { *abort_flag = 1; ok = false; break; }
        }
        pending = it; pending_col = w.ntile;
      }
      if (ok && pending >= 0) {
        if (!issue_lowrank(pending, pending_col)) *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int etid = threadIdx.x - 64;
    const int g = lane >> 2, q = lane & 3;
    constexpr int HALF_N = BN / 2;
    constexpr int UNIT_N = 64;
    constexpr int kChunks = HALF_N / UNIT_N;
    OutT* out = static_cast<OutT*>(p.out);
    float* scol_s = reinterpret_cast<float*>(smem + L::kScolOff);
    float* bias_s = reinterpret_cast<float*>(smem + L::kBiasOff);
    const bool vec_store = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool aborted = false;
    int it = 0;
    int aux_n0 = -1, aux_set = -1;
    TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
#pragma unroll 1
    for (; w.valid(); w.advance(), ++it) {
      const TileCoord c = tile_coord(w, p, mt0, BN);
      const int buf = it & 1;
      const uint32_t par = static_cast<uint32_t>(it >> 1) & 1u;

      if (c.n0 != aux_n0 || c.set != aux_set) {      // column scales and bias of this column tile
        aux_n0 = c.n0; aux_set = c.set;
        epi_bar_sync();
        const float* scol = c.set == 0 ? p.s_col[0] : p.s_col[1];
#pragma unroll 1
        for (int i = etid; i < BN; i += kNumEpiWarps * 32) {
          const int col = c.n0 + i;
          scol_s[i] = col < p.N ? scol[col] : 0.0f;
          bias_s[i] = (p.has_bias && col < p.N) ? p.bias[col] : 0.0f;
        }
        epi_bar_sync();
      }
      float srow[2][2];
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        const int rA = c.row0 + quarter * 32 + mb * 16 + g;
        srow[mb][0] = rA < c.row_end ? p.s_row[rA] : 0.0f;
        srow[mb][1] = rA + 8 < c.row_end ? p.s_row[rA + 8] : 0.0f;
      }

      if (!aborted) {
        const bool landed = wait_or_abort(&tfull_bar[buf], par, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true; }
      }
      if (aborted) continue;
      tc_fence_after();

      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(buf * BN + half * HALF_N);
      auto unit_addr = [&](int ch, int mb) {
        return t_acc + (static_cast<uint32_t>(quarter * 32 + mb * 16) << 16) + static_cast<uint32_t>(ch * UNIT_N);
      };
      uint32_t va[32], vb[32];

      // ---- pass 1: int32 accumulator -> fp32 * (s_row * s_col), written back in place
      auto scale_unit = [&](uint32_t (&v)[32], int ch, int mb) {
        const int col_unit = half * HALF_N + ch * UNIT_N;
        const float srA = srow[mb][0], srB = srow[mb][1];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          const int cl = col_unit + nb * 8 + 2 * q;
          const float2 sc = *reinterpret_cast<const float2*>(scol_s + cl);
          if constexpr (DBG) {
            const int rA = c.row0 + quarter * 32 + mb * 16 + g;
            dump_acc_lr(p.dbg_acc, p.N, rA, rA + 8, c.n0 + cl, c.row_end, v[4 * nb + 0], v[4 * nb + 1], v[4 * nb + 2], v[4 * nb + 3]);
          }
          v[4 * nb + 0] = __float_as_uint(__fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 0])), __fmul_rn(srA, sc.x)));
          v[4 * nb + 1] = __float_as_uint(__fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 1])), __fmul_rn(srA, sc.y)));
          v[4 * nb + 2] = __float_as_uint(__fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 2])), __fmul_rn(srB, sc.x)));
          v[4 * nb + 3] = __float_as_uint(__fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 3])), __fmul_rn(srB, sc.y)));
        }
        tmem_st_16x256b_x8(unit_addr(ch, mb), v);
      };
      // a register block that a tcgen05.st still reads must not be reloaded: wait for the store first
      tmem_ld_16x256b_x8(unit_addr(0, 0), va);
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        tc_wait_ld();
        tc_wait_st();
        tmem_ld_16x256b_x8(unit_addr(ch, 1), vb);
        scale_unit(va, ch, 0);
        tc_wait_ld();
        tc_wait_st();
        if (ch + 1 < kChunks) tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
        scale_unit(vb, ch, 1);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ylr_ready[buf]);

      // ---- wait for the low-rank MMAs, then pass 2: + bias, round, store
      {
        const bool landed = wait_or_abort(&lr_done[buf], par, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 6); *abort_flag = 1; aborted = true; continue; }
      }
      tc_fence_after();
      auto store_unit = [&](const uint32_t (&v)[32], int ch, int mb) {
        const int col_unit = half * HALF_N + ch * UNIT_N;
        const int rA = c.row0 + quarter * 32 + mb * 16 + g;
        const int rB = rA + 8;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
          uint32_t wA[4], wB[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int nb = grp * 4 + j;
            const float2 bi = *reinterpret_cast<const float2*>(bias_s + col_unit + nb * 8 + 2 * q);
            wA[j] = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 0]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 1]), bi.y), OutT{});
            wB[j] = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 2]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 3]), bi.y), OutT{});
          }
          const int col_grp = c.n0 + col_unit + grp * 32;
          if (vec_store && col_grp + 32 <= p.N) {
            quad_transpose(wA, q);
            quad_transpose(wB, q);
            if (rA < c.row_end)
              st_v4(out + static_cast<int64_t>(rA) * p.ldo + col_grp + q * 8, make_uint4(wA[0], wA[1], wA[2], wA[3]));
            if (rB < c.row_end)
              st_v4(out + static_cast<int64_t>(rB) * p.ldo + col_grp + q * 8, make_uint4(wB[0], wB[1], wB[2], wB[3]));
          } else {
            store_pairs_slow(p.out, p.ldo, rA, rB, col_grp + 2 * q, c.row_end, p.N, make_uint4(wA[0], wA[1], wA[2], wA[3]),
                             make_uint4(wB[0], wB[1], wB[2], wB[3]));
          }
        }
      };
      tmem_ld_16x256b_x8(unit_addr(0, 0), va);
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        tc_wait_ld();
        tmem_ld_16x256b_x8(unit_addr(ch, 1), vb);
        store_unit(va, ch, 0);
        tc_wait_ld();
        if (ch + 1 < kChunks) tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
        store_unit(vb, ch, 1);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
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

template <int BN, int STAGES, typename OutT, bool DBG>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1, const CUtensorMap& tmT,
               const CUtensorMap& tmLbT, const GemmParams& p, int grid, cudaStream_t st) {
  using L = LrSmem<BN, STAGES>;
  auto kern = pq_int8_gemm_fused_lr_kernel<BN, STAGES, OutT, DBG>;
  static bool attr_set[64] = {false};
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  kern<<<grid, kGemmThreads, L::kDynamic, st>>>(tmA, tmW0, tmW1, tmT, tmLbT, p);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// 16-bit matrix [rows, 32] with row stride ld elements: box = 32 elements (64 bytes) x box_rows, 64-byte swizzle.
int make_lr_map(CUtensorMap* map, const void* base, int64_t rows, int64_t ld, int box_rows, bool bf16) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PQ_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(kLR), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kLR), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int>(r); return PQ_ERR_CUDA; }
  return PQ_OK;
}

}  // namespace

int launch_gemm_lr_tc(int bn, bool bf16, bool dbg, const CUtensorMap& tmA, const CUtensorMap& tmW0,
                      const CUtensorMap& tmW1, const void* t, int64_t ldt, const void* lb_t, int64_t M, int64_t N,
                      const GemmParams& p, int grid, cudaStream_t st) {
  CUtensorMap tmT, tmLbT;
  int rc = make_lr_map(&tmT, t, M, ldt, BM, bf16);
  if (rc != PQ_OK) return rc;
  rc = make_lr_map(&tmLbT, lb_t, N, kLR, bn, bf16);
  if (rc != PQ_OK) return rc;
  if (bn == 256) {
    if (bf16) return dbg ? launch_one<256, 4, __nv_bfloat16, true>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st)
                         : launch_one<256, 4, __nv_bfloat16, false>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st);
    return dbg ? launch_one<256, 4, __half, true>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st)
               : launch_one<256, 4, __half, false>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st);
  }
  if (bf16) return dbg ? launch_one<128, 6, __nv_bfloat16, true>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st)
                       : launch_one<128, 6, __nv_bfloat16, false>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st);
  return dbg ? launch_one<128, 6, __half, true>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st)
             : launch_one<128, 6, __half, false>(tmA, tmW0, tmW1, tmT, tmLbT, p, grid, st);
}

}  // namespace pq
