// Fused INT8 GEMM for sm_100a: out = float(xq @ w^T) * (s_row x s_col) (+ t @ lb) (+ bias).
//
// One persistent CTA per SM, 320 threads, three roles:
//   warp 0      TMA producer: streams 128 x 128-byte tiles of xq and BN x 128-byte tiles of w into a
//               ring of shared-memory stages (128-byte swizzle), one mbarrier pair per stage;
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::i8 (128 x BN x 32 per instruction) from the
//               staged tiles into an int32 accumulator in tensor memory; two accumulators alternate so
//               that the next tile's main loop overlaps the previous tile's epilogue;
//   warps 2-9   epilogue: read the accumulator back with tcgen05.ld.16x256b (which hands out the registers
//               in the mma.sync accumulator arrangement), apply the row/column scales, add the rank-32
//               low-rank term with warp-level bf16 mma.sync on the same fragments, add the bias, round to
//               the output type, transpose inside each quad with shuffles and store 16 bytes per thread.
//               Loads of the next 16x64 block are in flight while the current one is processed.
// Every wait on an mbarrier is bounded; a wait that gives up writes a code to the status word, raises
// a CTA-wide abort flag and the CTA drains and exits.  No cluster launch, no multicast.
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include "gemm_common.cuh"
#include "gemm_2cta.cuh"
#include "gemm_lr_tc.cuh"

namespace pq {
namespace {


template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kLbStride = (BN + 8) * 2;              // bytes per low-rank row in shared memory
  static constexpr int kLbBytes = kLR * kLbStride;
  static constexpr int kAuxOff = STAGES * kStageBytes;
  static constexpr int kScolOff = kAuxOff + kLbBytes;
  static constexpr int kBiasOff = kScolOff + BN * 4;
  static constexpr int kBarOff = kBiasOff + BN * 4;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;                // slack for manual 1024-byte alignment
};

// Test hook: raw accumulators of one n8 block (rows rA / rB, columns col, col+1).
__device__ __noinline__ void dump_acc(int32_t* dbg, int N, int rA, int rB, int col, int row_end, uint32_t v0, uint32_t v1,
                                      uint32_t v2, uint32_t v3) {
  if (rA < row_end && col < N) dbg[static_cast<int64_t>(rA) * N + col] = static_cast<int32_t>(v0);
  if (rA < row_end && col + 1 < N) dbg[static_cast<int64_t>(rA) * N + col + 1] = static_cast<int32_t>(v1);
  if (rB < row_end && col < N) dbg[static_cast<int64_t>(rB) * N + col] = static_cast<int32_t>(v2);
  if (rB < row_end && col + 1 < N) dbg[static_cast<int64_t>(rB) * N + col + 1] = static_cast<int32_t>(v3);
}

// HAS_LR: low-rank term present.  DBG: also dump the raw accumulators (tests only).
template <int BN, int STAGES, typename OutT, bool HAS_LR, bool DBG>
__global__ void __launch_bounds__(kGemmThreads, 1)
pq_int8_gemm_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW0,
                          const __grid_constant__ CUtensorMap tmW1, const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  using LrT = OutT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int mt0 = (p.m_split + BM - 1) / BM;
  const int mt_total = mt0 + (p.M - p.m_split + BM - 1) / BM;
  const int nt = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW0);
    tma_prefetch_desc(&tmW1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], kNumEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
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
        const TileCoord c = tile_coord(w, p, mt0, BN);
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
      }
      // Copies still in flight must land before the CTA may exit: wait (bounded) for the last stages issued.
      const int pending = issued < STAGES ? static_cast<int>(issued) : STAGES;
      for (int i = 0; i < pending; ++i) {
        if (--stage < 0) { stage = STAGES - 1; phase ^= 1u; }
        if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
          for (int k = 0; k < 64; ++k) __nanosleep(1000);   // abort raised elsewhere: short fixed delay instead
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8(BM, BN);
      int stage = 0; uint32_t phase = 0; int it = 0; bool ok = true;
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
          if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
            report_timeout(p.status, 2, 1); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K inside the 128-byte swizzle row: +32 bytes = +2 in the 16-byte address field
            tc_mma_i8(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);        // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&tfull_bar[buf]);    // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Warp w reads tensor-memory lanes [32*(w%4), +32) (hardware rule) and the column half (w-2)/4 of the tile.
    // The code is kept small on purpose (real loops, slow paths out of line): eight warps run it out of step
    // with each other and with the two main-loop warps, and an instruction footprint beyond the instruction
    // cache stalls them on instruction fetch while TMA traffic keeps the memory system busy.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int etid = threadIdx.x - 64;         // 0..255 among the epilogue threads
    const int g = lane >> 2, q = lane & 3;     // mma.sync fragment coordinates
    constexpr int HALF_N = BN / 2;             // columns per warp
    constexpr int UNIT_N = 64;                 // columns per tcgen05.ld (16 lanes x 64 columns = 32 registers)
    constexpr int kChunks = HALF_N / UNIT_N;   // column chunks per warp and tile
    constexpr bool kLrBf16 = std::is_same<LrT, __nv_bfloat16>::value;
    OutT* out = static_cast<OutT*>(p.out);
    const LrT* tptr = static_cast<const LrT*>(p.t);
    const LrT* lbptr = static_cast<const LrT*>(p.lb);
    uint8_t* lb_s = smem + L::kAuxOff;
    float* scol_s = reinterpret_cast<float*>(smem + L::kScolOff);
    float* bias_s = reinterpret_cast<float*>(smem + L::kBiasOff);
    const bool vec_store = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool aborted = false;
    int it = 0;
    int aux_n0 = -1, aux_set = -1;             // which column tile / weight set the shared-memory copies belong to

    // per-tile row data of this thread: low-rank A fragments (two 16-row blocks x two k-steps) and row scales;
    // the loads for the next tile are issued before the current tile is drained
    uint32_t af[2][2][4], af_nx[2][2][4];
    float srow[2][2], srow_nx[2][2];
    auto load_row_data = [&](const TileCoord& tc, uint32_t (&afr)[2][2][4], float (&sr)[2][2]) {
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        const int rA = tc.row0 + quarter * 32 + mb * 16 + g;
        const int rB = rA + 8;
        const bool okA = rA < tc.row_end, okB = rB < tc.row_end;
        sr[mb][0] = okA ? p.s_row[rA] : 0.0f;
        sr[mb][1] = okB ? p.s_row[rB] : 0.0f;
        if constexpr (HAS_LR) {
          const LrT* ta = tptr + static_cast<int64_t>(okA ? rA : 0) * p.ldt + 2 * q;
          const LrT* tb = tptr + static_cast<int64_t>(okB ? rB : 0) * p.ldt + 2 * q;
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            afr[mb][ks][0] = okA ? *reinterpret_cast<const uint32_t*>(ta + ks * 16) : 0u;
            afr[mb][ks][2] = okA ? *reinterpret_cast<const uint32_t*>(ta + ks * 16 + 8) : 0u;
            afr[mb][ks][1] = okB ? *reinterpret_cast<const uint32_t*>(tb + ks * 16) : 0u;
            afr[mb][ks][3] = okB ? *reinterpret_cast<const uint32_t*>(tb + ks * 16 + 8) : 0u;
          }
        }
      }
    };

    TileWalker w; w.init(p.sched_pm, p.sched_pn, mt_total, nt);
    TileCoord c = tile_coord(w, p, mt0, BN);
    if (w.valid()) load_row_data(c, af, srow);
#pragma unroll 1
    for (; w.valid(); ++it) {
      w.advance();
      const bool has_next = w.valid();
      const TileCoord c_nx = tile_coord(w, p, mt0, BN);
      const int buf = it & 1;
      const uint32_t use = static_cast<uint32_t>(it >> 1);

      // column scales, bias and the low-rank up-projection tile of this N range live in shared memory and are
      // reloaded only when the column tile (or the weight set) changes
      if (c.n0 != aux_n0 || c.set != aux_set) {
        aux_n0 = c.n0; aux_set = c.set;
        epi_bar_sync();                        // everyone is done reading the previous copies
        const float* scol = c.set == 0 ? p.s_col[0] : p.s_col[1];
#pragma unroll 1
        for (int i = etid; i < BN; i += kNumEpiWarps * 32) {
          const int col = c.n0 + i;
          scol_s[i] = col < p.N ? scol[col] : 0.0f;
          bias_s[i] = (p.has_bias && col < p.N) ? p.bias[col] : 0.0f;
        }
        if constexpr (HAS_LR) {
          constexpr int kChunksPerRow = BN / 8;
#pragma unroll 1
          for (int i = etid; i < kLR * kChunksPerRow; i += kNumEpiWarps * 32) {
            const int r = i / kChunksPerRow;
            const int ch = i - r * kChunksPerRow;
            const int col = c.n0 + ch * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (col < p.N) v = *reinterpret_cast<const uint4*>(lbptr + static_cast<int64_t>(r) * p.ldb + col);
            *reinterpret_cast<uint4*>(lb_s + r * L::kLbStride + ch * 16) = v;
          }
        }
        epi_bar_sync();
      }

      if (!aborted) {
        const bool landed = wait_or_abort(&tfull_bar[buf], use & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) {            // warp-uniform decision: tcgen05.ld below is warp-collective
          report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true;
        }
      }
      if (aborted) { c = c_nx; continue; }     // keep the loop shape (named barriers) but touch nothing
      tc_fence_after();

      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(buf * BN + half * HALF_N);
      // a unit is 16 rows (block mb) x 64 columns (chunk ch); the load of the next unit is issued before the
      // current one is processed, va holds the mb = 0 units and vb the mb = 1 units
      uint32_t va[32], vb[32];
      auto unit_addr = [&](int ch, int mb) {
        return t_acc + (static_cast<uint32_t>(quarter * 32 + mb * 16) << 16) + static_cast<uint32_t>(ch * UNIT_N);
      };
      auto process = [&](const uint32_t (&v)[32], int ch, int mb, const uint32_t (&afm)[2][4], float srA, float srB) {
        const int col_unit = half * HALF_N + ch * UNIT_N;                // first tile column of this unit
        const int rA = c.row0 + quarter * 32 + mb * 16 + g;
        const int rB = rA + 8;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {                              // 4 n8 blocks = 32 columns per group
          uint32_t wA[4], wB[4];
          // the group's legacy MMAs are issued back to back before any result is used: they queue behind the
          // tcgen05 stream on the tensor pipe, so their latency is long and has to be overlapped
          float lr[4][4];
          if constexpr (HAS_LR) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t bf[4];
              ldmatrix_x4_trans(bf, smem_u32(lb_s + lane * L::kLbStride + (col_unit + (grp * 4 + j) * 8) * 2));
              lr[j][0] = lr[j][1] = lr[j][2] = lr[j][3] = 0.0f;
              mma_m16n8k16<kLrBf16>(lr[j], afm[0], bf[0], bf[1]);
              mma_m16n8k16<kLrBf16>(lr[j], afm[1], bf[2], bf[3]);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int nb = grp * 4 + j;
            const int cl = col_unit + nb * 8 + 2 * q;                    // column inside the tile
            const float2 sc = *reinterpret_cast<const float2*>(scol_s + cl);
            const float2 bi = *reinterpret_cast<const float2*>(bias_s + cl);
            // same operation order as the reference kernel: acc * (s_row * s_col), + low rank, + bias
            float y0 = __fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 0])), __fmul_rn(srA, sc.x));
            float y1 = __fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 1])), __fmul_rn(srA, sc.y));
            float y2 = __fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 2])), __fmul_rn(srB, sc.x));
            float y3 = __fmul_rn(int_to_float_rn(static_cast<int32_t>(v[4 * nb + 3])), __fmul_rn(srB, sc.y));
            if constexpr (HAS_LR) {
              y0 = __fadd_rn(y0, lr[j][0]); y1 = __fadd_rn(y1, lr[j][1]); y2 = __fadd_rn(y2, lr[j][2]); y3 = __fadd_rn(y3, lr[j][3]);
            }
            y0 = __fadd_rn(y0, bi.x); y1 = __fadd_rn(y1, bi.y); y2 = __fadd_rn(y2, bi.x); y3 = __fadd_rn(y3, bi.y);
            wA[j] = pack2(y0, y1, OutT{});
            wB[j] = pack2(y2, y3, OutT{});
            if constexpr (DBG)
              dump_acc(p.dbg_acc, p.N, rA, rB, c.n0 + cl, c.row_end, v[4 * nb + 0], v[4 * nb + 1], v[4 * nb + 2], v[4 * nb + 3]);
          }
          const int col_grp = c.n0 + col_unit + grp * 32;                // first output column of the group
          if (vec_store && col_grp + 32 <= p.N) {
            // 4x4 transpose inside each quad: lane q ends up with all 8 columns of n8 block q -> one 16-byte store per row
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
      if (has_next) load_row_data(c_nx, af_nx, srow_nx);     // in flight while this tile is drained
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        tc_wait_ld();
        tmem_ld_16x256b_x8(unit_addr(ch, 1), vb);
        process(va, ch, 0, af[0], srow[0][0], srow[0][1]);
        tc_wait_ld();
        if (ch + 1 < kChunks) tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
        process(vb, ch, 1, af[1], srow[1][0], srow[1][1]);
      }
      // accumulator drained: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      c = c_nx;
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        srow[mb][0] = srow_nx[mb][0]; srow[mb][1] = srow_nx[mb][1];
        if constexpr (HAS_LR) {
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int e = 0; e < 4; ++e) af[mb][ks][e] = af_nx[mb][ks][e];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0) {
      for (int k = 0; k < 64; ++k) __nanosleep(1000);     // let MMAs that were already issued retire
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// tensor-pipe ceiling probe: MMAs on resident shared-memory tiles, no global traffic
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
pq_i8_mma_issue_loop_kernel(int iters, long long* cycles, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int kA = BM * BK, kB = 256 * BK;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + kA + kB);
  uint32_t* holder = reinterpret_cast<uint32_t*>(smem + kA + kB + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kA + kB + 24);
  // operands: all ones (iters >= 0), or pseudo-random bytes (iters < 0: data-dependent power of the tensor cores)
  const bool random_fill = iters < 0;
  if (random_fill) iters = -iters;
  for (int i = threadIdx.x; i < (kA + kB) / 16; i += blockDim.x) {
    uint4 v = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    if (random_fill) {
      uint32_t h = (static_cast<uint32_t>(i) * 4u + blockIdx.x * 7919u) * 2654435761u;
      v.x = h ^ (h >> 15); h = h * 2246822519u + 3266489917u;
      v.y = h ^ (h >> 13); h = h * 2246822519u + 3266489917u;
      v.z = h ^ (h >> 16); h = h * 2246822519u + 3266489917u;
      v.w = h ^ (h >> 14);
    }
    reinterpret_cast<uint4*>(smem)[i] = v;
  }
  if (threadIdx.x == 0) { mbar_init(bar, 1); *abort_flag = 0; fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(holder, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *holder;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_i8(BM, 256);
    const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(smem));
    const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(smem + kA));
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        tc_mma_i8(tmem_base, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                  (i > 0 || k > 0) ? 1u : 0u);
    }
    tc_commit(bar);
    if (!wait_or_abort(bar, 0u, abort_flag)) report_timeout(status, 4, 1);
    const long long t1 = clock64();
    cycles[blockIdx.x] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// Wait that nothing ends: one thread waits on a barrier no one arrives on, through the same bounded wait the GEMM
// roles use, with a budget of `budget_ns`; when the wait gives up it reports (role 5) and the kernel returns.
__global__ void pq_wait_probe_kernel(int32_t* status, unsigned long long budget_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_mbar_init(); }
  __syncthreads();
  if (threadIdx.x == 0 && !wait_or_abort(&bar, 0u, &abort_flag, budget_ns)) {
    report_timeout(status, 5, 1);
    abort_flag = 1;
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct WKey {
  const void* ptr; int64_t N, K, ld; int bn;
  bool operator==(const WKey& o) const { return ptr == o.ptr && N == o.N && K == o.K && ld == o.ld && bn == o.bn; }
};
struct WKeyHash {
  size_t operator()(const WKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= static_cast<size_t>(k.N) * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.K) * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    return h ^ static_cast<size_t>(k.ld * 31 + k.bn);
  }
};

// Weight tensor maps depend only on (address, shape, stride, box) and are reused across calls.
int weight_map(CUtensorMap* out, const void* w, int64_t N, int64_t K, int64_t ld, int bn) {
  static std::mutex mu;
  static std::unordered_map<WKey, CUtensorMap, WKeyHash> cache;
  WKey key{w, N, K, ld, bn};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return PQ_OK; }
  }
  int rc = make_tile_map(out, w, N, K, ld, bn);
  if (rc != PQ_OK) return rc;
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return PQ_OK;
}

template <int BN, int STAGES, typename OutT, bool HAS_LR, bool DBG>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1, const GemmParams& p,
                int grid, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = pq_int8_gemm_fused_kernel<BN, STAGES, OutT, HAS_LR, DBG>;
  static bool attr_set[64] = {false};     // per device; benign race: the attribute value never changes
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  kern<<<grid, kGemmThreads, L::kDynamic, st>>>(tmA, tmW0, tmW1, p);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

template <int BN, int STAGES, typename OutT>
int launch_by_flags(bool has_lr, bool dbg, const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1,
                    const GemmParams& p, int grid, cudaStream_t st) {
  if (dbg) {
    if (has_lr) return launch_gemm<BN, STAGES, OutT, true, true>(tmA, tmW0, tmW1, p, grid, st);
    return launch_gemm<BN, STAGES, OutT, false, true>(tmA, tmW0, tmW1, p, grid, st);
  }
  if (has_lr) return launch_gemm<BN, STAGES, OutT, true, false>(tmA, tmW0, tmW1, p, grid, st);
  return launch_gemm<BN, STAGES, OutT, false, false>(tmA, tmW0, tmW1, p, grid, st);
}

template <typename OutT>
int launch_by_shape(int bn, int stages, bool has_lr, bool dbg, const CUtensorMap& tmA, const CUtensorMap& tmW0,
                    const CUtensorMap& tmW1, const GemmParams& p, int grid, cudaStream_t st) {
  if (bn == 256) {
    if (stages == 3) return launch_by_flags<256, 3, OutT>(has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
    return launch_by_flags<256, 4, OutT>(has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
  }
  if (stages == 4) return launch_by_flags<128, 4, OutT>(has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
  return launch_by_flags<128, 6, OutT>(has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
}

int choose_block_n(int64_t M, int64_t N) {
  const int forced = options().gemm_block_n;
  if (forced == 128 || forced == 256) return forced;
  const double pad256 = static_cast<double>((N + 255) / 256 * 256) / static_cast<double>(N);
  const double pad128 = static_cast<double>((N + 127) / 128 * 128) / static_cast<double>(N);
  if (pad256 > pad128 * 1.04) return 128;
  // small problems: prefer the tile count that fills the SMs
  const int64_t tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
  if (tiles256 < sm_count()) return 128;
  return 256;
}

int gemm_common(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w0, const float* sc0,
                const int8_t* w1, const float* sc1, int64_t ldw, const float* bias, const void* t, int64_t ldt,
                const void* lb, int64_t ldb, const void* lb_t, int R, int lr_dtype, void* out, int out_dtype,
                int64_t ldo, int64_t m_split, int64_t M, int64_t N, int64_t K, void* workspace, size_t ws_bytes,
                int32_t* dbg_acc, void* stream, int epi_flags = 0, void* const* out_more = nullptr, int n_out_more = 0,
                const void* gate = nullptr, int64_t ld_gate = 0, int64_t gate_rows = 0) {
  if (M < 0 || N <= 0 || K <= 0 || m_split < 0 || m_split > M) return PQ_ERR_SHAPE;
  if (epi_flags & ~(PQ_EPI_ACCUMULATE | PQ_EPI_GELU_TANH | PQ_EPI_GATE)) return PQ_ERR_UNSUPPORTED;
  if (((epi_flags & PQ_EPI_GATE) != 0) != (gate != nullptr)) return PQ_ERR_NULL;
  if (gate != nullptr && (gate_rows < 0 || ld_gate < N || ld_gate % 8 != 0 || !aligned_to(gate, 16))) return PQ_ERR_ALIGN;
  if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return PQ_ERR_SHAPE;
  if (out_dtype != PQ_DTYPE_BF16 && out_dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (xq == nullptr || s_row == nullptr || w0 == nullptr || sc0 == nullptr || out == nullptr) return PQ_ERR_NULL;
  if (m_split < M && (w1 == nullptr || sc1 == nullptr)) return PQ_ERR_NULL;
  if (ldx < K || ldw < K || ldo < N) return PQ_ERR_SHAPE;
  if (K % 16 != 0 || ldx % 16 != 0 || ldw % 16 != 0) return PQ_ERR_ALIGN;
  if (!aligned_to(xq, 16) || !aligned_to(w0, 16) || (w1 != nullptr && !aligned_to(w1, 16))) return PQ_ERR_ALIGN;
  if (ldo % 2 != 0 || !aligned_to(out, 4)) return PQ_ERR_ALIGN;
  const bool has_lr = (t != nullptr) || (lb != nullptr);
  if (has_lr) {
    if (t == nullptr || lb == nullptr) return PQ_ERR_NULL;
    if (R != kLR) return PQ_ERR_UNSUPPORTED;
    if (lr_dtype != PQ_DTYPE_BF16 && lr_dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
    if (lr_dtype != out_dtype) return PQ_ERR_UNSUPPORTED;
    if (ldt < R || ldb < N) return PQ_ERR_SHAPE;
    if (ldt % 8 != 0 || ldb % 8 != 0 || N % 8 != 0 || !aligned_to(t, 16) || !aligned_to(lb, 16)) return PQ_ERR_ALIGN;
    if (lb_t != nullptr && !aligned_to(lb_t, 16)) return PQ_ERR_ALIGN;
  }
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;

  const int bn = choose_block_n(M, N);
  int stages = options().gemm_stages;
  if (bn == 256) { if (stages != 3) stages = 4; }
  else { if (stages != 4) stages = 6; }

  GemmParams p;
  p.s_row = s_row; p.s_col[0] = sc0; p.s_col[1] = (m_split < M) ? sc1 : sc0; p.bias = bias;
  p.t = t; p.lb = lb; p.out = out; p.dbg_acc = dbg_acc; p.status = static_cast<int32_t*>(workspace);
  p.ldt = ldt; p.ldb = ldb; p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.m_split = static_cast<int>(m_split);
  p.has_bias = bias != nullptr ? 1 : 0;
  p.epi_flags = epi_flags;
  p.timing = (options().gemm_debug_timing != 0 && workspace != nullptr && ws_bytes >= 256 + 4096 * 64)
                 ? reinterpret_cast<long long*>(static_cast<char*>(workspace) + 256) : nullptr;
  p.sched_pm = p.sched_pn = p.sched_m_steps = p.sched_n_rounds = 1;
  p.sched_panel = 0; p.l2_hints = 0; p.tma_store = 0; p.sched_cut = 0; p.sched_tail_per = 0; p.sched_tail_rb = 1;
  p.gate = gate; p.ld_gate = ld_gate; p.gate_rows = gate_rows;
  p.n_out_more = n_out_more;
  for (int d = 0; d < 7; ++d) p.out_more[d] = d < n_out_more ? out_more[d] : nullptr;

  // CTA-pair kernel: 256-column tiles, enough 256-row tiles to occupy the SM pairs, and the K-major low-rank
  // factor when there is a low-rank term
  {
    const int64_t pair_rows = (m_split + 255) / 256 + (M - m_split + 255) / 256;
    const bool pair_legal = (!has_lr || lb_t != nullptr);
    if (epi_flags != 0 || n_out_more > 0) {
      // the epilogue variants exist in the CTA-pair kernel's vector store path only
      if (!pair_legal || N % 32 != 0 || ldo % 8 != 0 || !aligned_to(out, 16)) return PQ_ERR_UNSUPPORTED;
      return launch_gemm_pair(out_dtype == PQ_DTYPE_BF16, dbg_acc != nullptr || p.timing != nullptr, xq, ldx, w0, w1, ldw, has_lr ? t : nullptr, ldt,
                              has_lr ? lb_t : nullptr, M, N, K, p, static_cast<cudaStream_t>(stream));
    }
    if (options().gemm_pair != 0 && bn == 256 && pair_legal &&
        pair_rows * ((N + 255) / 256) >= (options().gemm_pair == 2 ? 1 : sm_count() / 2)) {
      return launch_gemm_pair(out_dtype == PQ_DTYPE_BF16, dbg_acc != nullptr || p.timing != nullptr, xq, ldx, w0, w1, ldw, has_lr ? t : nullptr, ldt,
                              has_lr ? lb_t : nullptr, M, N, K, p, static_cast<cudaStream_t>(stream));
    }
  }

  CUtensorMap tmA, tmW0, tmW1;
  int rc = make_tile_map(&tmA, xq, M, K, ldx, BM);
  if (rc != PQ_OK) return rc;
  rc = weight_map(&tmW0, w0, N, K, ldw, bn);
  if (rc != PQ_OK) return rc;
  if (m_split < M) {
    rc = weight_map(&tmW1, w1, N, K, ldw, bn);
    if (rc != PQ_OK) return rc;
  } else {
    tmW1 = tmW0;
  }

  // CTA grid pm x pn over the tile matrix: fewest steps first, then the widest pn (fewer sweeps over the rows)
  const int mt = static_cast<int>((m_split + BM - 1) / BM + (M - m_split + BM - 1) / BM);
  const int ntl = static_cast<int>((N + bn - 1) / bn);
  int max_ctas = options().gemm_max_ctas > 0 ? options().gemm_max_ctas : sm_count();
  int best_pm = 1, best_pn = 1;
  choose_cta_grid(mt, ntl, max_ctas, &best_pm, &best_pn);
  p.sched_pm = best_pm; p.sched_pn = best_pn;
  p.sched_m_steps = (mt + best_pm - 1) / best_pm;
  p.sched_n_rounds = (ntl + best_pn - 1) / best_pn;
  const int grid = best_pm * best_pn;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool dbg = dbg_acc != nullptr;
  if (has_lr && lb_t != nullptr)      // rank-32 term on the tensor cores (needs the K-major copy of lb)
    return launch_gemm_lr_tc(bn, out_dtype == PQ_DTYPE_BF16, dbg, tmA, tmW0, tmW1, t, ldt, lb_t, M, N, p, grid, st);
  if (out_dtype == PQ_DTYPE_BF16)
    return launch_by_shape<__nv_bfloat16>(bn, stages, has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
  return launch_by_shape<__half>(bn, stages, has_lr, dbg, tmA, tmW0, tmW1, p, grid, st);
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_int8_gemm(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w, int64_t ldw,
                            const float* s_col, const float* bias, const void* t, int64_t ldt, const void* lb,
                            int64_t ldb, const void* lb_t, int R, int lr_dtype, void* out, int out_dtype, int64_t ldo,
                            int64_t M, int64_t N, int64_t K, void* workspace, size_t ws_bytes, int32_t* dbg_acc,
                            void* stream) {
  return gemm_common(xq, ldx, s_row, w, s_col, nullptr, nullptr, ldw, bias, t, ldt, lb, ldb, lb_t, R, lr_dtype, out,
                     out_dtype, ldo, M, M, N, K, workspace, ws_bytes, dbg_acc, stream);
}

extern "C" int pq_int8_gemm_ex(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w, int64_t ldw,
                               const float* s_col, const float* bias, const void* t, int64_t ldt, const void* lb,
                               int64_t ldb, const void* lb_t, int R, int lr_dtype, void* out, int out_dtype, int64_t ldo,
                               int64_t M, int64_t N, int64_t K, int epilogue, void* workspace, size_t ws_bytes,
                               void* stream) {
  return gemm_common(xq, ldx, s_row, w, s_col, nullptr, nullptr, ldw, bias, t, ldt, lb, ldb, lb_t, R, lr_dtype, out,
                     out_dtype, ldo, M, M, N, K, workspace, ws_bytes, nullptr, stream, epilogue);
}

extern "C" int pq_int8_gemm_gated(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w, int64_t ldw,
                                  const float* s_col, const float* bias, const void* t, int64_t ldt, const void* lb,
                                  int64_t ldb, const void* lb_t, int R, int lr_dtype, const void* gate, int64_t ld_gate,
                                  int64_t rows_per_sample, void* out, int out_dtype, int64_t ldo, int64_t M, int64_t N,
                                  int64_t K, int epilogue, void* workspace, size_t ws_bytes, void* stream) {
  if (gate == nullptr) return PQ_ERR_NULL;
  return gemm_common(xq, ldx, s_row, w, s_col, nullptr, nullptr, ldw, bias, t, ldt, lb, ldb, lb_t, R, lr_dtype, out,
                     out_dtype, ldo, M, M, N, K, workspace, ws_bytes, nullptr, stream, epilogue | PQ_EPI_GATE, nullptr, 0,
                     gate, ld_gate, rows_per_sample);
}

extern "C" int pq_int8_gemm_bcast(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w, int64_t ldw,
                                  const float* s_col, const float* bias, const void* t, int64_t ldt, const void* lb,
                                  int64_t ldb, const void* lb_t, int R, int lr_dtype, void* out, void* const* out_more,
                                  int n_out_more, int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                  int epilogue, void* workspace, size_t ws_bytes, void* stream) {
  if (n_out_more < 0 || n_out_more > PQ_MAX_OUT_MORE) return PQ_ERR_SHAPE;
  if (n_out_more > 0 && out_more == nullptr) return PQ_ERR_NULL;
  for (int d = 0; d < n_out_more; ++d) {
    if (out_more[d] == nullptr) return PQ_ERR_NULL;
    if (!aligned_to(out_more[d], 16)) return PQ_ERR_ALIGN;
  }
  return gemm_common(xq, ldx, s_row, w, s_col, nullptr, nullptr, ldw, bias, t, ldt, lb, ldb, lb_t, R, lr_dtype, out,
                     out_dtype, ldo, M, M, N, K, workspace, ws_bytes, nullptr, stream, epilogue, out_more, n_out_more);
}

extern "C" int pq_int8_gemm_grouped(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w_hi,
                                    const float* s_col_hi, const int8_t* w_lo, const float* s_col_lo, int64_t ldw,
                                    const float* bias, const void* t, int64_t ldt, const void* lb, int64_t ldb,
                                    const void* lb_t, int R, int lr_dtype, void* out, int out_dtype, int64_t ldo,
                                    int64_t M_hi, int64_t M, int64_t N, int64_t K, void* workspace, size_t ws_bytes,
                                    void* stream) {
  return gemm_common(xq, ldx, s_row, w_hi, s_col_hi, w_lo, s_col_lo, ldw, bias, t, ldt, lb, ldb, lb_t, R, lr_dtype, out,
                     out_dtype, ldo, M_hi, M, N, K, workspace, ws_bytes, nullptr, stream);
}

extern "C" int pq_wait_probe(void* workspace, size_t ws_bytes, int budget_us, void* stream) {
  if (workspace == nullptr) return PQ_ERR_NULL;
  if (ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;
  if (budget_us <= 0 || budget_us > 100000) return PQ_ERR_SHAPE;
  pq_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<int32_t*>(workspace), static_cast<unsigned long long>(budget_us) * 1000ull);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

extern "C" int pq_i8_mma_issue_loop(int ctas, int iters, long long* cycles, void* workspace, size_t ws_bytes,
                                    void* stream) {
  if (ctas <= 0 || iters == 0 || ctas > 4096 || iters > (1 << 24) || iters < -(1 << 24)) return PQ_ERR_SHAPE;
  if (cycles == nullptr) return PQ_ERR_NULL;
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;
  constexpr int kSmem = BM * BK + 256 * BK + 64 + 1024;
  PQ_CUDA_TRY(cudaFuncSetAttribute(pq_i8_mma_issue_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  pq_i8_mma_issue_loop_kernel<<<ctas, 128, kSmem, static_cast<cudaStream_t>(stream)>>>(
      iters, cycles, static_cast<int32_t*>(workspace));
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}
