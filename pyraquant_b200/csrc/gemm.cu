// Fused INT8 GEMM for sm_100a: out = float(xq @ w^T) * (s_row x s_col) (+ t @ lb) (+ bias).
//
// One persistent CTA per SM, 192 threads, three roles:
//   warp 0      TMA producer: streams 128 x 128-byte tiles of xq and BN x 128-byte tiles of w into a
//               ring of shared-memory stages (128-byte swizzle), one mbarrier pair per stage;
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::i8 (128 x BN x 32 per instruction) from the
//               staged tiles into an int32 accumulator in tensor memory; two accumulators alternate so
//               that the next tile's main loop overlaps the previous tile's epilogue;
//   warps 2-5   epilogue: read the accumulator back with tcgen05.ld, apply the row/column scales, add
//               the rank-32 low-rank term (warp-level bf16 mma.sync on fragments that tcgen05.ld
//               .16x256b delivers in the matching register arrangement) and the bias, round to the
//               output type and store.
// Every wait on an mbarrier is bounded; a wait that gives up writes a code to the status word, raises
// a CTA-wide abort flag and the CTA drains and exits.  No cluster launch, no multicast.
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace pq {
namespace {

constexpr int BM = 128;          // rows per tile = tensor-memory lanes
constexpr int BK = 128;          // K bytes per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;       // K per tcgen05.mma kind::i8
constexpr int kGemmThreads = 192;
constexpr int kNumEpiWarps = 4;
constexpr int kLR = 32;          // low-rank width handled in the epilogue

struct GemmParams {
  const float* s_row;
  const float* s_col[2];
  const float* bias;
  const void* t;        // [M, 32] low-rank activations
  const void* lb;       // [32, N] low-rank up-projection
  void* out;
  int32_t* dbg_acc;
  int32_t* status;
  int64_t ldt, ldb, ldo;
  int M, N, K;
  int m_split;          // rows [0, m_split) use weight set 0, rows [m_split, M) weight set 1
  int group_m;
  int has_lr;
  int has_bias;
};

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

struct TileCoord {
  int row0, row_end, n0, set;
};

// Tile order: groups of `group_m` row tiles; inside a group the row tile index runs fastest so that
// CTAs working at the same time share weight tiles and a small set of activation tiles in L2.
__device__ __forceinline__ TileCoord decode_tile(int tile, int mt0, int mt_total, int nt, const GemmParams& p, int BN) {
  const int per_group = p.group_m * nt;
  const int group = tile / per_group;
  const int first_m = group * p.group_m;
  const int gsize = min(mt_total - first_m, p.group_m);
  const int in_group = tile - group * per_group;
  const int mt = first_m + in_group % gsize;
  const int ntile = in_group / gsize;
  TileCoord c;
  if (mt < mt0) {
    c.set = 0; c.row0 = mt * BM; c.row_end = p.m_split;
  } else {
    c.set = 1; c.row0 = p.m_split + (mt - mt0) * BM; c.row_end = p.M;
  }
  c.n0 = ntile * BN;
  return c;
}

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t i = 1; i < kWaitMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0) {
      if (*abort_flag != 0) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitBudgetNs) return false;
    }
  }
  return false;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename OutT>
__device__ __forceinline__ void store_pair(OutT* out, int64_t ldo, int row, int col, int row_end, int N, float a, float b) {
  if (row >= row_end) return;
  OutT* p = out + static_cast<int64_t>(row) * ldo + col;
  if (col + 1 < N) {
    *reinterpret_cast<uint32_t*>(p) = pack2(a, b, OutT{});
  } else if (col < N) {
    if constexpr (std::is_same<OutT, __nv_bfloat16>::value) p[0] = __float2bfloat16_rn(a);
    else p[0] = __float2half_rn(a);
  }
}

template <int BN, int STAGES, typename OutT, typename LrT>
__global__ void __launch_bounds__(kGemmThreads, 1)
pq_int8_gemm_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW0,
                          const __grid_constant__ CUtensorMap tmW1, const GemmParams p, const int epilogue_mode) {
  using L = SmemLayout<BN, STAGES>;
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
  const int mt1 = (p.M - p.m_split + BM - 1) / BM;
  const int mt_total = mt0 + mt1;
  const int nt = (p.N + BN - 1) / BN;
  const int total_tiles = mt_total * nt;
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileCoord c = decode_tile(tile, mt0, mt_total, nt, p, BN);
        const CUtensorMap* tmW = c.set == 0 ? &tmW0 : &tmW1;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            report_timeout(p.status, 1, 1); *abort_flag = 1; ok = false; break;
          }
          uint8_t* a_s = smem + stage * L::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(a_s, &tmA, &full_bar[stage], kb * BK, c.row0);
          tma_load_2d(a_s + L::kABytes, tmW, &full_bar[stage], kb * BK, c.n0);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      // Copies still in flight must land before the CTA may exit: wait (bounded) for the last stages issued.
      const int pending = issued < STAGES ? static_cast<int>(issued) : STAGES;
      for (int i = 0; i < pending; ++i) {
        if (--stage < 0) { stage = STAGES - 1; phase ^= 1u; }
        if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
          // abort raised elsewhere or copy never landed: fall back to a short fixed delay
          for (int k = 0; k < 64; ++k) __nanosleep(1000);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8(BM, BN);
      int stage = 0; uint32_t phase = 0; int it = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t use = static_cast<uint32_t>(it >> 1);
        if (!wait_or_abort(&tempty_bar[buf], (use & 1u) ^ 1u, abort_flag)) {
          report_timeout(p.status, 2, 2); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
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
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;              // tensor-memory lanes [32*quarter, 32*quarter+32) belong to this warp
    const int etid = threadIdx.x - 64;         // 0..127 among the epilogue threads
    OutT* out = static_cast<OutT*>(p.out);
    const LrT* tptr = static_cast<const LrT*>(p.t);
    const LrT* lbptr = static_cast<const LrT*>(p.lb);
    uint8_t* lb_s = smem + L::kAuxOff;
    float* scol_s = reinterpret_cast<float*>(smem + L::kScolOff);
    float* bias_s = reinterpret_cast<float*>(smem + L::kBiasOff);
    bool aborted = false;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const TileCoord c = decode_tile(tile, mt0, mt_total, nt, p, BN);
      const int buf = it & 1;
      const uint32_t use = static_cast<uint32_t>(it >> 1);

      // column scales, bias and the low-rank up-projection tile of this N range go to shared memory
      epi_bar_sync();                          // everyone is done reading the previous tile's copies
      {
        const float* scol = p.s_col[c.set];
        for (int i = etid; i < BN; i += 128) {
          const int col = c.n0 + i;
          scol_s[i] = col < p.N ? scol[col] : 0.0f;
          bias_s[i] = (p.has_bias && col < p.N) ? p.bias[col] : 0.0f;
        }
        if (p.has_lr) {
          constexpr int kChunksPerRow = BN / 8;
          for (int i = etid; i < kLR * kChunksPerRow; i += 128) {
            const int r = i / kChunksPerRow;
            const int ch = i - r * kChunksPerRow;
            const int col = c.n0 + ch * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (col < p.N) v = *reinterpret_cast<const uint4*>(lbptr + static_cast<int64_t>(r) * p.ldb + col);
            *reinterpret_cast<uint4*>(lb_s + r * L::kLbStride + ch * 16) = v;
          }
        }
      }
      epi_bar_sync();

      if (!aborted) {
        const bool landed = wait_or_abort(&tfull_bar[buf], use & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) {            // warp-uniform decision: tcgen05.ld below is warp-collective
          report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true;
        }
      }
      if (aborted) continue;                   // keep the loop shape (named barriers) but touch nothing
      tc_fence_after();

      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(buf * BN);
      if (epilogue_mode == 0) {
        // ---- one accumulator row per thread; low-rank term by scalar FMA (reference implementation of the epilogue)
        const int row = c.row0 + quarter * 32 + lane;
        const bool row_ok = row < c.row_end;
        const float sr = row_ok ? p.s_row[row] : 0.0f;
        float tv[kLR];
        if (p.has_lr) {
#pragma unroll
          for (int r = 0; r < kLR; ++r)
            tv[r] = row_ok ? static_cast<float>(tptr[static_cast<int64_t>(row) * p.ldt + r]) : 0.0f;
        }
        for (int cc = 0; cc < BN / 32; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_acc + (static_cast<uint32_t>(quarter * 32) << 16) + cc * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int cl = cc * 32 + j;
            float y0 = static_cast<float>(static_cast<int32_t>(v[j])) * (sr * scol_s[cl]);
            float y1 = static_cast<float>(static_cast<int32_t>(v[j + 1])) * (sr * scol_s[cl + 1]);
            if (p.has_lr) {
              float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
              for (int r = 0; r < kLR; ++r) {
                const LrT* lrow = reinterpret_cast<const LrT*>(lb_s + r * L::kLbStride);
                l0 = fmaf(tv[r], static_cast<float>(lrow[cl]), l0);
                l1 = fmaf(tv[r], static_cast<float>(lrow[cl + 1]), l1);
              }
              y0 += l0; y1 += l1;
            }
            y0 += bias_s[cl]; y1 += bias_s[cl + 1];
            store_pair<OutT>(out, p.ldo, row, c.n0 + cl, c.row_end, p.N, y0, y1);
            if (p.dbg_acc != nullptr && row_ok) {
              if (c.n0 + cl < p.N) p.dbg_acc[static_cast<int64_t>(row) * p.N + c.n0 + cl] = static_cast<int32_t>(v[j]);
              if (c.n0 + cl + 1 < p.N) p.dbg_acc[static_cast<int64_t>(row) * p.N + c.n0 + cl + 1] = static_cast<int32_t>(v[j + 1]);
            }
          }
        }
      } else {
        // ---- fragment epilogue: tcgen05.ld.16x256b hands out the accumulator in the mma.sync C arrangement
        const int g = lane >> 2, q = lane & 3;
#pragma unroll 1
        for (int mb = 0; mb < 2; ++mb) {
          const int rA = c.row0 + quarter * 32 + mb * 16 + g;
          const int rB = rA + 8;
          const bool okA = rA < c.row_end, okB = rB < c.row_end;
          const float srA = okA ? p.s_row[rA] : 0.0f;
          const float srB = okB ? p.s_row[rB] : 0.0f;
          uint32_t af[2][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
          if (p.has_lr) {
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const int k0 = ks * 16 + 2 * q;
              if (okA) {
                af[ks][0] = *reinterpret_cast<const uint32_t*>(tptr + static_cast<int64_t>(rA) * p.ldt + k0);
                af[ks][2] = *reinterpret_cast<const uint32_t*>(tptr + static_cast<int64_t>(rA) * p.ldt + k0 + 8);
              }
              if (okB) {
                af[ks][1] = *reinterpret_cast<const uint32_t*>(tptr + static_cast<int64_t>(rB) * p.ldt + k0);
                af[ks][3] = *reinterpret_cast<const uint32_t*>(tptr + static_cast<int64_t>(rB) * p.ldt + k0 + 8);
              }
            }
          }
          const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32 + mb * 16) << 16;
#pragma unroll 2
          for (int cc = 0; cc < BN / 32; ++cc) {
            uint32_t v[16];
            tmem_ld_16x256b_x4(t_acc + lane_addr + cc * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int cl = cc * 32 + j * 8 + 2 * q;      // column inside the tile
              float lr[4] = {0.0f, 0.0f, 0.0f, 0.0f};
              if (p.has_lr) {
                uint32_t bf[4];
                ldmatrix_x4_trans(bf, smem_u32(lb_s + lane * L::kLbStride + (cc * 32 + j * 8) * 2));
                mma_m16n8k16<std::is_same<LrT, __nv_bfloat16>::value>(lr, af[0], bf[0], bf[1]);
                mma_m16n8k16<std::is_same<LrT, __nv_bfloat16>::value>(lr, af[1], bf[2], bf[3]);
              }
              const float2 sc = *reinterpret_cast<const float2*>(scol_s + cl);
              const float2 bi = *reinterpret_cast<const float2*>(bias_s + cl);
              float y0 = static_cast<float>(static_cast<int32_t>(v[4 * j + 0])) * (srA * sc.x);
              float y1 = static_cast<float>(static_cast<int32_t>(v[4 * j + 1])) * (srA * sc.y);
              float y2 = static_cast<float>(static_cast<int32_t>(v[4 * j + 2])) * (srB * sc.x);
              float y3 = static_cast<float>(static_cast<int32_t>(v[4 * j + 3])) * (srB * sc.y);
              y0 += lr[0]; y1 += lr[1]; y2 += lr[2]; y3 += lr[3];
              y0 += bi.x; y1 += bi.y; y2 += bi.x; y3 += bi.y;
              const int col = c.n0 + cl;
              store_pair<OutT>(out, p.ldo, rA, col, c.row_end, p.N, y0, y1);
              store_pair<OutT>(out, p.ldo, rB, col, c.row_end, p.N, y2, y3);
              if (p.dbg_acc != nullptr) {
                if (okA && col < p.N) p.dbg_acc[static_cast<int64_t>(rA) * p.N + col] = static_cast<int32_t>(v[4 * j + 0]);
                if (okA && col + 1 < p.N) p.dbg_acc[static_cast<int64_t>(rA) * p.N + col + 1] = static_cast<int32_t>(v[4 * j + 1]);
                if (okB && col < p.N) p.dbg_acc[static_cast<int64_t>(rB) * p.N + col] = static_cast<int32_t>(v[4 * j + 2]);
                if (okB && col + 1 < p.N) p.dbg_acc[static_cast<int64_t>(rB) * p.N + col + 1] = static_cast<int32_t>(v[4 * j + 3]);
              }
            }
          }
        }
      }
      // accumulator drained: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
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
  for (int i = threadIdx.x; i < (kA + kB) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
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

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// int8 matrix [rows, K] with row stride ld bytes; box = 128 bytes x box_rows, 128-byte swizzle, zero fill.
int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PQ_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int>(r); return PQ_ERR_CUDA; }
  return PQ_OK;
}

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

template <int BN, int STAGES, typename OutT, typename LrT>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1, const GemmParams& p,
                int epilogue_mode, int grid, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = pq_int8_gemm_fused_kernel<BN, STAGES, OutT, LrT>;
  static bool attr_set[64] = {false};     // per device; benign race: the attribute value never changes
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  kern<<<grid, kGemmThreads, L::kDynamic, st>>>(tmA, tmW0, tmW1, p, epilogue_mode);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

template <typename OutT, typename LrT>
int launch_by_shape(int bn, int stages, const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1,
                    const GemmParams& p, int epilogue_mode, int grid, cudaStream_t st) {
  if (bn == 256) {
    if (stages == 2) return launch_gemm<256, 2, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
    if (stages == 3) return launch_gemm<256, 3, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
    return launch_gemm<256, 4, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
  }
  if (stages == 2) return launch_gemm<128, 2, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
  if (stages == 4) return launch_gemm<128, 4, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
  return launch_gemm<128, 6, OutT, LrT>(tmA, tmW0, tmW1, p, epilogue_mode, grid, st);
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
                const void* lb, int64_t ldb, int R, int lr_dtype, void* out, int out_dtype, int64_t ldo,
                int64_t m_split, int64_t M, int64_t N, int64_t K, void* workspace, size_t ws_bytes,
                int32_t* dbg_acc, void* stream) {
  if (M < 0 || N <= 0 || K <= 0 || m_split < 0 || m_split > M) return PQ_ERR_SHAPE;
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
  }
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;

  const int bn = choose_block_n(M, N);
  int stages = options().gemm_stages;
  if (bn == 256) { if (stages != 2 && stages != 3) stages = 4; }
  else { if (stages != 2 && stages != 4) stages = 6; }

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

  GemmParams p;
  p.s_row = s_row; p.s_col[0] = sc0; p.s_col[1] = (m_split < M) ? sc1 : sc0; p.bias = bias;
  p.t = t; p.lb = lb; p.out = out; p.dbg_acc = dbg_acc; p.status = static_cast<int32_t*>(workspace);
  p.ldt = ldt; p.ldb = ldb; p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.m_split = static_cast<int>(m_split);
  int gm = options().gemm_group_m; if (gm < 1) gm = 1;
  p.group_m = gm;
  p.has_lr = has_lr ? 1 : 0;
  p.has_bias = bias != nullptr ? 1 : 0;

  const int64_t mt = (m_split + BM - 1) / BM + (M - m_split + BM - 1) / BM;
  const int64_t tiles = mt * ((N + bn - 1) / bn);
  int max_ctas = options().gemm_max_ctas > 0 ? options().gemm_max_ctas : sm_count();
  const int grid = static_cast<int>(tiles < max_ctas ? tiles : max_ctas);
  const int epi = options().gemm_epilogue;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == PQ_DTYPE_BF16)
    return launch_by_shape<__nv_bfloat16, __nv_bfloat16>(bn, stages, tmA, tmW0, tmW1, p, epi, grid, st);
  return launch_by_shape<__half, __half>(bn, stages, tmA, tmW0, tmW1, p, epi, grid, st);
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_int8_gemm(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w, int64_t ldw,
                            const float* s_col, const float* bias, const void* t, int64_t ldt, const void* lb,
                            int64_t ldb, int R, int lr_dtype, void* out, int out_dtype, int64_t ldo, int64_t M,
                            int64_t N, int64_t K, void* workspace, size_t ws_bytes, int32_t* dbg_acc, void* stream) {
  return gemm_common(xq, ldx, s_row, w, s_col, nullptr, nullptr, ldw, bias, t, ldt, lb, ldb, R, lr_dtype, out,
                     out_dtype, ldo, M, M, N, K, workspace, ws_bytes, dbg_acc, stream);
}

extern "C" int pq_int8_gemm_grouped(const int8_t* xq, int64_t ldx, const float* s_row, const int8_t* w_hi,
                                    const float* s_col_hi, const int8_t* w_lo, const float* s_col_lo, int64_t ldw,
                                    const float* bias, const void* t, int64_t ldt, const void* lb, int64_t ldb,
                                    int R, int lr_dtype, void* out, int out_dtype, int64_t ldo, int64_t M_hi,
                                    int64_t M, int64_t N, int64_t K, void* workspace, size_t ws_bytes, void* stream) {
  return gemm_common(xq, ldx, s_row, w_hi, s_col_hi, w_lo, s_col_lo, ldw, bias, t, ldt, lb, ldb, R, lr_dtype, out,
                     out_dtype, ldo, M_hi, M, N, K, workspace, ws_bytes, nullptr, stream);
}

extern "C" int pq_i8_mma_issue_loop(int ctas, int iters, long long* cycles, void* workspace, size_t ws_bytes,
                                    void* stream) {
  if (ctas <= 0 || iters <= 0 || ctas > 4096 || iters > (1 << 24)) return PQ_ERR_SHAPE;
  if (cycles == nullptr) return PQ_ERR_NULL;
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;
  constexpr int kSmem = BM * BK + 256 * BK + 64 + 1024;
  PQ_CUDA_TRY(cudaFuncSetAttribute(pq_i8_mma_issue_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  pq_i8_mma_issue_loop_kernel<<<ctas, 128, kSmem, static_cast<cudaStream_t>(stream)>>>(
      iters, cycles, static_cast<int32_t*>(workspace));
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}
