// Fused INT8 GEMM on CTA pairs (tcgen05 cta_group::2): out = float(xq @ w^T) * (s_row x s_col) (+ t @ lb) (+ bias).
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile: CTA r owns rows [128 r, 128 r + 128) of
// the tile and keeps them in its own tensor memory; each CTA stages its own 128 x 128-byte activation tile and only
// HALF of the weight tile (rows [128 r, +128) of the 256) per stage, and one thread of CTA 0 issues every
// tcgen05.mma.cta_group::2 (256 x 256 x 32) for the pair.  Compared with the single-CTA kernel this halves the
// weight bytes each SM pulls from L2 and writes into shared memory, which is what bounds that kernel, and leaves
// room for a six-stage ring.  No TMA multicast is used: every CTA loads its own bytes.
//
// Synchronisation.  "full" barriers live in CTA 0 and count the bytes of both CTAs' copies (CTA 1's TMA instructions
// name CTA 0's barrier).  Everything the MMA thread publishes ("stage free", "accumulator complete", "low-rank MMAs
// done") is committed twice, once to each CTA's copy of the barrier.  What the MMA thread waits for from the
// epilogues ("accumulator drained", "scaled accumulator written back") is one barrier in CTA 0 with 16 arrivals, the
// eight epilogue warps of CTA 1 arriving remotely.  Every wait is bounded; a wait that gives up records a code in the
// status word, raises its CTA's abort flag and lets the CTA drain; the peer then runs into its own limits.  Both
// CTAs meet at a cluster barrier before they exit so that neither leaves while its peer may still signal it.
#include <type_traits>

#include "gemm_2cta.cuh"
#include "gemm_common.cuh"

namespace pq {
namespace {

constexpr int PBN = 256;                   // tile columns
constexpr int PSTAGES = 6;
constexpr int kHalfB = PBN / 2;            // weight rows staged per CTA
constexpr int kRowBytesLr = kLR * 2;       // 64-byte rows of the t / lbT tiles
constexpr int kLrChunks = 2;               // the low-rank term is added in column chunks of PBN / kLrChunks
constexpr int kLrChunkN = PBN / kLrChunks; // 128 columns: one kind::f16 MMA pair per chunk
constexpr int kLbChunkRows = kLrChunkN / 2;   // lbT rows each CTA stages per chunk
// Warps of a CTA: 0 TMA producer, 1 MMA issuer, 2 .. 2 + EW - 1 epilogue, 2 + EW issuer of the low-rank MMAs (leader
// CTA).  EW = 8 when the main loop of a tile outlasts its epilogue (long K); EW = 16 for short K without a low-rank
// term, where the epilogue is the critical path: each warp then owns 16 rows x 128 columns instead of 32 x 128.
constexpr int pair_threads(int ew) { return (3 + ew) * 32; }
constexpr int kShortK = 1536;              // up to this K (and without a low-rank term) the sixteen-warp epilogue is used

struct PairSmem {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = kHalfB * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;            // per CTA
  static constexpr int kTOff = PSTAGES * kStageBytes;
  static constexpr int kTBytes = BM * kRowBytesLr;                 // per CTA: its 128 rows of t
  static constexpr int kLbOff = kTOff + 2 * kTBytes;
  static constexpr int kLbBytes = kHalfB * kRowBytesLr;            // per CTA: its 128 rows of lbT
  static constexpr int kScolOff = kLbOff + 2 * kLbBytes;            // two lbT buffers: consecutive column tiles alternate
  static constexpr int kBiasOff = kScolOff + PBN * 4;
  static constexpr int kBarOff = kBiasOff + PBN * 4;
  // full[S], empty[S], tfull[2], tempty[2], t_full[2], lb_full[2], ylr_ready[2][chunks], lr_done[2][chunks]
  static constexpr int kNumBars = 2 * PSTAGES + 8 + 4 * kLrChunks;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16 + 64;      // + time stamps of the cycle-counter experiments
  static_assert(kTotal <= 232448, "exceeds the 227 KB shared memory of one CTA");
};

// ---------------------------------------------------------------------------------------------
// cluster / pair primitives
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `smem_addr` (an address of the executing CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrival on a barrier of either CTA of the pair.  What the arrival publishes lives in tensor memory or registers and
// is ordered by tcgen05.wait / tcgen05.fence, so the default (CTA-scope release) form is used: a cluster-scope
// release would make the warp wait for its outstanding global stores to be acknowledged first.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted by a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// the same with an L2 eviction-priority policy (createpolicy) attached to the copy
__device__ __forceinline__ void tma_load_2d_pair_hint(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// completion of all MMAs issued so far -> one arrival on the barrier at `cluster_addr` (any CTA of the pair)
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ uint64_t kmajor_sw64_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;
  return d;
}
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&v)[32]) {
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
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __noinline__ void dump_acc_pair(int32_t* dbg, int N, int rA, int rB, int col, int row_end, uint32_t v0, uint32_t v1,
                                           uint32_t v2, uint32_t v3) {
  if (rA < row_end && col < N) dbg[static_cast<int64_t>(rA) * N + col] = static_cast<int32_t>(v0);
  if (rA < row_end && col + 1 < N) dbg[static_cast<int64_t>(rA) * N + col + 1] = static_cast<int32_t>(v1);
  if (rB < row_end && col < N) dbg[static_cast<int64_t>(rB) * N + col] = static_cast<int32_t>(v2);
  if (rB < row_end && col + 1 < N) dbg[static_cast<int64_t>(rB) * N + col + 1] = static_cast<int32_t>(v3);
}

// Walker over pair tiles.  The first pm x pn pairs form a grid laid over (row tile, column tile).  Order of the tiles a
// grid pair visits: the row steps are cut into panels of `panel` steps; inside a panel the pair runs down its column
// (all row steps of the panel) before it moves pn column tiles to the right, and only after the last column round does
// it enter the next panel.  A panel that covers all row steps is the plain column-round-major order.  With several
// column rounds a short panel keeps the panel's activation rows in L2 across the rounds instead of streaming all M rows
// once per round.
// Pairs beyond the grid (the SM pairs a pm x pn rectangle leaves over: 2 of 74 with the 6 x 12 grid of the FLUX layers)
// take a tail region off the grid's hands: the row tiles from `cut` on in the last column round, in small row blocks, a
// contiguous share of `tail_per` tiles each; the grid pairs stop at `cut` in that round.  The host picks `cut` so that
// grid pairs and tail pairs finish together.
struct PairWalker {
  int mt, ntile, bn, pm, pn, mt_total, nt, panel0, panel_span;
  int col0, cut;       // first column tile of the last column round; row limit of the grid pairs there
  int tail_left;       // tiles left for a tail pair; -1 for a grid pair
  int t_rb0, t_hb, t_rb;   // tail pair: first row tile and height of its current row block, rows per block
  __device__ __forceinline__ void init(int pair, const GemmParams& p, int mt_total_, int nt_) {
    pm = p.sched_pm; pn = p.sched_pn; mt_total = mt_total_; nt = nt_;
    col0 = ((nt + pn - 1) / pn - 1) * pn;
    cut = p.sched_tail_per > 0 ? p.sched_cut : mt_total;
    panel_span = (p.sched_panel > 0 && p.sched_panel < (1 << 20)) ? p.sched_panel * pm : (1 << 30);
    t_rb0 = 0; t_hb = 1; t_rb = p.sched_tail_rb > 0 ? p.sched_tail_rb : 1;
    if (pair < pm * pn) {
      const int bm = pair / pn; bn = pair - bm * pn;
      panel0 = bm; mt = bm; ntile = bn; tail_left = -1;
    } else {
      // The tail region in blocks of t_rb row tiles, block after block; inside a block column after column, the rows of
      // the block innermost: a block's activation rows are used again after t_rb tiles (they stay in L2) and the column
      // changes every t_rb tiles.
      const int wl = nt - col0;
      const int total = (mt_total - cut) * wl;
      const int j = (pair - pm * pn) * p.sched_tail_per;
      const int j_end = j + p.sched_tail_per < total ? j + p.sched_tail_per : total;
      tail_left = j_end > j ? j_end - j : 0;
      bn = 0; panel0 = 0;
      if (tail_left > 0) {
        const int b = j / (t_rb * wl), rem = j - b * (t_rb * wl);
        t_rb0 = cut + b * t_rb;
        t_hb = mt_total - t_rb0 < t_rb ? mt_total - t_rb0 : t_rb;
        ntile = col0 + rem / t_hb; mt = t_rb0 + rem % t_hb;
      } else { ntile = nt; mt = mt_total; }
    }
  }
  __device__ __forceinline__ int row_limit() const { return ntile >= col0 ? cut : mt_total; }
  __device__ __forceinline__ bool valid() const { return tail_left >= 0 ? tail_left > 0 : (ntile < nt && mt < row_limit()); }
  __device__ __forceinline__ void advance() {
    if (tail_left >= 0) {
      --tail_left;
      if (++mt >= t_rb0 + t_hb) {
        mt = t_rb0;
        if (++ntile >= nt) {
          ntile = col0; t_rb0 += t_rb; mt = t_rb0;
          t_hb = mt_total - t_rb0 < t_rb ? mt_total - t_rb0 : t_rb;
        }
      }
      return;
    }
    mt += pm;
    if (mt >= row_limit() || mt - panel0 >= panel_span) {
      ntile += pn; mt = panel0;
      if (ntile >= nt && panel_span < (1 << 30) && panel0 + panel_span < mt_total) { ntile = bn; panel0 += panel_span; mt = panel0; }
    }
  }
};

// Rows of a pair tile.  Row tiles [0, mt0) cover rows [0, m_split) with weight set 0, the rest cover [m_split, M) with
// weight set 1; a tile never straddles the split (its tail rows are masked at row_end).
struct PairCoord { int row0, row_end, set; };
__device__ __forceinline__ PairCoord pair_coord(int mt, int mt0, const GemmParams& p, uint32_t rank) {
  PairCoord c;
  if (mt < mt0) { c.set = 0; c.row0 = mt * 2 * BM; c.row_end = p.m_split; }
  else { c.set = 1; c.row0 = p.m_split + (mt - mt0) * 2 * BM; c.row_end = p.M; }
  c.row0 += static_cast<int>(rank) * BM;
  return c;
}

template <int EW>
__device__ __forceinline__ void pair_epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EW * 32) : "memory"); }

template <typename OutT, bool HAS_LR, bool DBG, int EW>
__global__ void __launch_bounds__(pair_threads(EW), 1)
pq_int8_gemm_fused_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                               const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmT, const __grid_constant__ CUtensorMap tmLbT,
                               const __grid_constant__ CUtensorMap tmOut, const GemmParams p) {
  using L = PairSmem;
  static_assert(EW == 8 || EW == 16, "eight or sixteen epilogue warps");
  constexpr int kLrWarp = 2 + EW;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + PSTAGES;
  uint64_t* tfull_bar = empty_bar + PSTAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* t_full = tempty_bar + 2;
  uint64_t* lb_full = t_full + 2;
  uint64_t* ylr_ready = lb_full + 2;
  uint64_t* lr_done = ylr_ready + 2 * kLrChunks;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  volatile long long* stamp = reinterpret_cast<volatile long long*>(smem + L::kMiscOff + 16);   // [0..3] arrive, [4..7] issue

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = leader (issues the MMAs), 1 = peer
  const bool aligned_ok = (smem_u32(smem) & 1023u) == 0;

  const int mt0 = (p.m_split + 2 * BM - 1) / (2 * BM);   // pair tiles of 256 rows: first tier, then second tier
  const int mt_total = mt0 + (p.M - p.m_split + 2 * BM - 1) / (2 * BM);
  const int nt = (p.N + PBN - 1) / PBN;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t kTmemCols = 2 * PBN;
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  // cycle-counter experiments exist in the DBG instantiation only: in the production kernel `timing` is a
  // compile-time null pointer and every branch on it is removed.  Wall-clock trace of the first pair, 24 slots per tile.
  long long* const timing = DBG ? p.timing : nullptr;
  long long* trace = (timing != nullptr && pair == 0) ? timing + 8192 : nullptr;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmW1);
    if (HAS_LR) { tma_prefetch_desc(&tmT); tma_prefetch_desc(&tmLbT); }
    for (int s = 0; s < PSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 2 * EW);
      mbar_init(&t_full[b], 1);
      for (int c = 0; c < kLrChunks; ++c) {
        mbar_init(&ylr_ready[b * kLrChunks + c], 2 * EW); mbar_init(&lr_done[b * kLrChunks + c], 1);
      }
    }
    mbar_init(&lb_full[0], 1); mbar_init(&lb_full[1], 1);
    *abort_flag = aligned_ok ? 0 : 1;
    if (!aligned_ok) report_timeout(p.status, 7, 7);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_holder, kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const bool run = aligned_ok;

  // barrier addresses in the leader CTA (for remote arrivals / byte counts) and in the peer (for the second commit)
  auto leader_addr = [&](const uint64_t* bar) { return map_to_cta(smem_u32(bar), 0u); };
  auto peer_addr = [&](const uint64_t* bar) { return map_to_cta(smem_u32(bar), 1u); };

  if (run && warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0; long long issued = 0; bool ok = true;
      int it = 0; int lb_col = -1; uint32_t lb_count = 0;
      // L2 priorities of the operand streams (l2_hints bit 0: weights evict-last; bit 1: activations evict-first; bit 2:
      // activations evict-last)
      const uint64_t pol_w = l2_policy_evict_last();
      const uint64_t pol_a = (p.l2_hints & 4) ? l2_policy_evict_last() : l2_policy_evict_first();
      PairWalker w; w.init(pair, p, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance(), ++it) {
        const PairCoord c = pair_coord(w.mt, mt0, p, rank);
        const int row0 = c.row0;                                            // this CTA's 128 rows
        const int n0 = w.ntile * PBN;
        const int nhalf0 = n0 + static_cast<int>(rank) * kHalfB;            // this CTA's half of the weight tile
        const int buf = it & 1;
        if (HAS_LR && w.ntile != lb_col) {
          // consecutive column tiles alternate between two lbT buffers; the buffer about to be overwritten was last
          // read by low-rank MMAs of a tile at least two back in this CTA's sequence
          if (it >= 2 && !wait_or_abort(&lr_done[buf * kLrChunks + kLrChunks - 1], static_cast<uint32_t>(((it - 2) >> 1) & 1), abort_flag)) {
            report_timeout(p.status, 1, 5); *abort_flag = 1; ok = false; break;
          }
          lb_col = w.ntile;
          const int lbuf = static_cast<int>(lb_count & 1u);
          if (rank == 0) mbar_arrive_expect_tx(&lb_full[lbuf], 2 * L::kLbBytes);
          // chunk c of the low-rank MMAs covers columns [n0 + c * kLrChunkN, + kLrChunkN): this CTA supplies its half
#pragma unroll
          for (int c = 0; c < kLrChunks; ++c)
            tma_load_2d_pair(smem + L::kLbOff + lbuf * L::kLbBytes + c * kLbChunkRows * kRowBytesLr, &tmLbT,
                             leader_addr(&lb_full[lbuf]), 0, n0 + c * kLrChunkN + static_cast<int>(rank) * kLbChunkRows);
          ++lb_count;
        }
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            report_timeout(p.status, 1, 1); *abort_flag = 1; ok = false; break;
          }
          uint8_t* a_s = smem + stage * L::kStageBytes;
          const uint32_t fb = leader_addr(&full_bar[stage]);
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          if (p.l2_hints & 6) tma_load_2d_pair_hint(a_s, &tmA, fb, kb * BK, row0, pol_a);
          else tma_load_2d_pair(a_s, &tmA, fb, kb * BK, row0);
          const CUtensorMap* wm = c.set == 0 ? &tmW : &tmW1;
          if (p.l2_hints & 1) tma_load_2d_pair_hint(a_s + L::kABytes, wm, fb, kb * BK, nhalf0, pol_w);
          else tma_load_2d_pair(a_s + L::kABytes, wm, fb, kb * BK, nhalf0);
          ++issued;
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (HAS_LR) {
          // this CTA's rows of t: the slot is free once the low-rank MMAs of two tiles ago have completed
          if (it >= 2 && !wait_or_abort(&lr_done[buf * kLrChunks + kLrChunks - 1], static_cast<uint32_t>(((it - 2) >> 1) & 1), abort_flag)) {
            report_timeout(p.status, 1, 6); *abort_flag = 1; ok = false; break;
          }
          if (rank == 0) mbar_arrive_expect_tx(&t_full[buf], 2 * L::kTBytes);
          tma_load_2d_pair(smem + L::kTOff + buf * L::kTBytes, &tmT, leader_addr(&t_full[buf]), 0, row0);
        }
      }
      // copies in flight must land before the CTA may exit: the last stages issued are consumed by MMAs whose
      // completion is committed to this CTA's empty barriers
      const int pending = issued < PSTAGES ? static_cast<int>(issued) : PSTAGES;
      for (int i = 0; i < pending; ++i) {
        if (--stage < 0) { stage = PSTAGES - 1; phase ^= 1u; }
        if (!wait_or_abort(&empty_bar[stage], phase, abort_flag)) {
          for (int k = 0; k < 64; ++k) __nanosleep(1000);
          break;
        }
      }
    }
  } else if (run && warp == 1 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    // The loop is kept minimal on purpose: one barrier probe, four MMAs and two commits per k-block.  A probe of a
    // shared-memory barrier takes a few hundred cycles while the tensor cores and the TMA unit saturate shared
    // memory, so every extra probe per k-block (a run-ahead limit, a look at the low-rank barriers) made this thread
    // the bottleneck; the low-rank MMAs therefore have an issuing thread of their own (warp kLrWarp).
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8(2 * BM, PBN);
      int stage = 0; uint32_t phase = 0; int it = 0; bool ok = true;
      long long tm_tempty = 0, tm_full = 0;
      auto commit_both = [&](uint64_t* bar) { tc_commit_pair(smem_u32(bar)); tc_commit_pair(peer_addr(bar)); };
      PairWalker w; w.init(pair, p, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance(), ++it) {
        const int buf = it & 1;
        const uint32_t use = static_cast<uint32_t>(it >> 1);
        const long long c0 = timing ? clock64() : 0;
        if (!wait_or_abort(&tempty_bar[buf], (use & 1u) ^ 1u, abort_flag)) {
          report_timeout(p.status, 2, 2); *abort_flag = 1; ok = false; break;
        }
        if (timing) tm_tempty += clock64() - c0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * PBN);
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long c1 = timing ? clock64() : 0;
          if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
            report_timeout(p.status, 2, 1); *abort_flag = 1; ok = false; break;
          }
          if (timing) tm_full += clock64() - c1;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_i8_pair(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                           (kb > 0 || k > 0) ? 1u : 0u);
          commit_both(&empty_bar[stage]);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        commit_both(&tfull_bar[buf]);
        if (trace && it < 1000) trace[it * 24 + 18] = static_cast<long long>(global_timer_ns());
      }
      if (timing) { timing[blockIdx.x * 16 + 0] = tm_tempty; timing[blockIdx.x * 16 + 1] = tm_full; }
    }
  } else if (HAS_LR && run && warp == kLrWarp && rank == 0) {
    // ------------------------------------------------------------------ low-rank MMA issuer (leader CTA only)
    // Per tile and column chunk: wait until all sixteen epilogue warps of the pair have written the scaled chunk back
    // to tensor memory, add t @ lbT on top with two kind::f16 MMAs (K = 16 each), publish "chunk complete" to both CTAs.
    if (elect_one()) {
      constexpr uint32_t idesc_lr = idesc_f16(2 * BM, kLrChunkN, std::is_same<OutT, __nv_bfloat16>::value);
      int it = 0, lb_col = -1; uint32_t lb_count = 0; bool ok = true;
      long long tm_det[2] = {0, 0};
      auto commit_both = [&](uint64_t* bar) { tc_commit_pair(smem_u32(bar)); tc_commit_pair(peer_addr(bar)); };
      PairWalker w; w.init(pair, p, mt_total, nt);
#pragma unroll 1
      for (; w.valid() && ok; w.advance(), ++it) {
        const int pb = it & 1;
        const uint32_t par = static_cast<uint32_t>(it >> 1) & 1u;
#pragma unroll 1
        for (int chunk = 0; chunk < kLrChunks; ++chunk) {
          if (!wait_or_abort(&ylr_ready[pb * kLrChunks + chunk], par, abort_flag)) { report_timeout(p.status, 4, 3); ok = false; break; }
          if (trace && it < 1000 && chunk == 0) trace[it * 24 + 16] = static_cast<long long>(global_timer_ns());
          if (chunk == 0) {
            if (!wait_or_abort(&t_full[pb], par, abort_flag)) { report_timeout(p.status, 4, 4); ok = false; break; }
            if (w.ntile != lb_col) {          // first tile of a column: its lbT buffer is (column ordinal) & 1
              if (!wait_or_abort(&lb_full[lb_count & 1u], (lb_count >> 1) & 1u, abort_flag)) { report_timeout(p.status, 4, 5); ok = false; break; }
              lb_col = w.ntile; ++lb_count;
            }
          }
          tc_fence_after();
          if (trace && it < 1000 && chunk == 0) trace[it * 24 + 17] = static_cast<long long>(global_timer_ns());
          const uint64_t a_desc = kmajor_sw64_desc(smem_u32(smem + L::kTOff + pb * L::kTBytes));
          const uint64_t b_desc = kmajor_sw64_desc(smem_u32(smem + L::kLbOff + static_cast<int>((lb_count - 1u) & 1u) * L::kLbBytes +
                                                            chunk * kLbChunkRows * kRowBytesLr));
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(pb * PBN + chunk * kLrChunkN);
          tc_mma_f16_pair(d_tmem, a_desc, b_desc, idesc_lr, 1u);
          tc_mma_f16_pair(d_tmem, a_desc + 2, b_desc + 2, idesc_lr, 1u);
          commit_both(&lr_done[pb * kLrChunks + chunk]);
          if (timing) { const long long now = clock64(); tm_det[chunk] += now - stamp[pb * kLrChunks + chunk]; stamp[4 + pb * kLrChunks + chunk] = now; }
        }
      }
      if (!ok) *abort_flag = 1;
      if (timing) { timing[blockIdx.x * 16 + 8] = tm_det[0]; timing[blockIdx.x * 16 + 9] = tm_det[1]; }
    }
  } else if (run && warp >= 2 && warp < 2 + EW) {
    // ------------------------------------------------------------------ epilogue (warps 2 .. 2 + EW - 1 of both CTAs)
    const int quarter = warp & 3;
    const int half = ((warp - 2) >> 2) & 1;
    // sixteen warps: warps 2..9 take the first 16 rows of each 32-row lane quarter, warps 10..17 the other 16
    constexpr int MBN = EW == 16 ? 1 : 2;                // 16-row blocks per warp
    const int mb_base = EW == 16 ? ((warp - 2) >> 3) : 0;
    const int etid = threadIdx.x - 64;
    const int g = lane >> 2, q = lane & 3;
    constexpr int UNIT_N = 64;
    static_assert(kLrChunkN == 2 * UNIT_N, "two column halves of 64 per chunk");
    OutT* out = static_cast<OutT*>(p.out);
    float* scol_s = reinterpret_cast<float*>(smem + L::kScolOff);
    float* bias_s = reinterpret_cast<float*>(smem + L::kBiasOff);
    const bool vec_store = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool aborted = false;
    int it = 0;
    int aux_n0 = -1, aux_set = -1;
    long long te_tfull = 0, te_p1 = 0, te_lr = 0, te_p2 = 0, te_aux = 0, te_exec[2] = {0, 0};
    float srow_next[2][2];
    auto load_srow = [&](const PairCoord& pc, float (&dst)[2][2]) {
#pragma unroll
      for (int mb = 0; mb < MBN; ++mb) {
        const int rA = pc.row0 + quarter * 32 + (mb_base + mb) * 16 + g;
        dst[mb][0] = rA < pc.row_end ? p.s_row[rA] : 0.0f;
        dst[mb][1] = rA + 8 < pc.row_end ? p.s_row[rA + 8] : 0.0f;
      }
    };
    PairWalker w; w.init(pair, p, mt_total, nt);
#pragma unroll 1
    for (; w.valid(); w.advance(), ++it) {
      const PairCoord c = pair_coord(w.mt, mt0, p, rank);
      const int row0 = c.row0;
      const int n0 = w.ntile * PBN;
      const int row_end = c.row_end;
      const int buf = it & 1;
      const uint32_t par = static_cast<uint32_t>(it >> 1) & 1u;

      const long long e0 = timing ? clock64() : 0;
      if (n0 != aux_n0 || c.set != aux_set) {
        aux_n0 = n0; aux_set = c.set;
        const float* scol_g = p.s_col[0];
        if (c.set != 0) scol_g = p.s_col[1];
        pair_epi_bar_sync<EW>();
#pragma unroll 1
        for (int i = etid; i < PBN; i += EW * 32) {
          const int col = n0 + i;
          scol_s[i] = col < p.N ? scol_g[col] : 0.0f;
          bias_s[i] = (p.has_bias && col < p.N) ? p.bias[col] : 0.0f;
        }
        pair_epi_bar_sync<EW>();
      }
      // row scales of this tile: fetched while the previous tile was being stored (first tile: here)
      float srow[2][2];
      if (it == 0) load_srow(c, srow_next);
#pragma unroll
      for (int mb = 0; mb < MBN; ++mb) { srow[mb][0] = srow_next[mb][0]; srow[mb][1] = srow_next[mb][1]; }

      const long long e1 = timing ? clock64() : 0;
      if (!aborted) {
        const bool landed = wait_or_abort(&tfull_bar[buf], par, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 3); *abort_flag = 1; aborted = true; }
      }
      if (aborted) continue;
      tc_fence_after();
      if (trace && it < 1000 && warp == 2 && lane == 0) trace[it * 24 + 20 + rank] = static_cast<long long>(global_timer_ns());
      const long long e2 = timing ? clock64() : 0;
      long long e3 = e2, e4 = e2;
      {
        PairWalker wn = w; wn.advance();
        if (wn.valid()) load_srow(pair_coord(wn.mt, mt0, p, rank), srow_next);
      }

      // Column assignment: chunk ch of the tile is columns [ch * 128, +128); the warps of half 0 take its first 64
      // columns, those of half 1 the other 64, so that one low-rank MMA pair per chunk serves all sixteen warps.
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(buf * PBN + half * UNIT_N);
      auto unit_addr = [&](int ch, int mb) {
        return t_acc + (static_cast<uint32_t>(quarter * 32 + (mb_base + mb) * 16) << 16) + static_cast<uint32_t>(ch * kLrChunkN);
      };
      uint32_t va[32], vb[32];

      // scale one 16 x 64 block: int32 -> fp32 * (s_row * s_col), in place in the registers
      auto scale_unit = [&](uint32_t (&v)[32], int ch, int mb) {
        const int col_unit = ch * kLrChunkN + half * UNIT_N;
        const float2 srA = make_float2(srow[mb][0], srow[mb][0]), srB = make_float2(srow[mb][1], srow[mb][1]);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          const int cl = col_unit + nb * 8 + 2 * q;
          const float2 sc = *reinterpret_cast<const float2*>(scol_s + cl);
          if constexpr (DBG) {
            const int rA = row0 + quarter * 32 + (mb_base + mb) * 16 + g;
            if (p.dbg_acc != nullptr) dump_acc_pair(p.dbg_acc, p.N, rA, rA + 8, n0 + cl, row_end, v[4 * nb + 0], v[4 * nb + 1], v[4 * nb + 2], v[4 * nb + 3]);
          }
          const float2 yA = __fmul2_rn(int2_to_float2_rn(static_cast<int32_t>(v[4 * nb + 0]), static_cast<int32_t>(v[4 * nb + 1])),
                                       __fmul2_rn(srA, sc));
          const float2 yB = __fmul2_rn(int2_to_float2_rn(static_cast<int32_t>(v[4 * nb + 2]), static_cast<int32_t>(v[4 * nb + 3])),
                                       __fmul2_rn(srB, sc));
          v[4 * nb + 0] = __float_as_uint(yA.x); v[4 * nb + 1] = __float_as_uint(yA.y);
          v[4 * nb + 2] = __float_as_uint(yB.x); v[4 * nb + 3] = __float_as_uint(yB.y);
        }
      };
      // + bias, round, transpose inside quads, store one 16 x 64 block of fp32 values
      auto store_unit = [&](const uint32_t (&v)[32], int ch, int mb) {
        const int col_unit = ch * kLrChunkN + half * UNIT_N;
        const int rA = row0 + quarter * 32 + (mb_base + mb) * 16 + g;
        const int rB = rA + 8;
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
          uint32_t wA[4], wB[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int nb = grp * 4 + j;
            const float2 bi = *reinterpret_cast<const float2*>(bias_s + col_unit + nb * 8 + 2 * q);
            if constexpr (HAS_LR) {
              const float2 yA = __fadd2_rn(make_float2(__uint_as_float(v[4 * nb + 0]), __uint_as_float(v[4 * nb + 1])), bi);
              const float2 yB = __fadd2_rn(make_float2(__uint_as_float(v[4 * nb + 2]), __uint_as_float(v[4 * nb + 3])), bi);
              wA[j] = pack2(yA.x, yA.y, OutT{});
              wB[j] = pack2(yB.x, yB.y, OutT{});
            } else {
              // scalar additions: right behind the packed multiplication of scale_unit a packed addition gets
              // contracted into a fused multiply-add, which would round differently from product-then-sum
              wA[j] = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 0]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 1]), bi.y), OutT{});
              wB[j] = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 2]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 3]), bi.y), OutT{});
            }
          }
          const int col_grp = n0 + col_unit + grp * 32;
          if (p.epi_flags & PQ_EPI_GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 4; ++j) { wA[j] = gelu_word<OutT>(wA[j]); wB[j] = gelu_word<OutT>(wB[j]); }
          }
          if (vec_store && col_grp + 32 <= p.N) {
            quad_transpose(wA, q);
            quad_transpose(wB, q);
            OutT* pA = out + static_cast<int64_t>(rA) * p.ldo + col_grp + q * 8;
            OutT* pB = out + static_cast<int64_t>(rB) * p.ldo + col_grp + q * 8;
            if (p.epi_flags & PQ_EPI_GATE) {
              // y * gate[sample, column] in the output type (the rounded Linear output times the block's gate vector, as
              // the reference's 16-bit tensors compute it), then the residual sum below; the eight columns of this lane
              // are one 16-byte load of the gate row
              const OutT* gbase = static_cast<const OutT*>(p.gate) + col_grp + q * 8;
              int64_t sA = 0, sB = 0;
              if (p.gate_rows > 0) { sA = rA / p.gate_rows; sB = rB / p.gate_rows; }
              if (rA < row_end) {
                const uint4 gv = ld_v4(gbase + sA * p.ld_gate);
                wA[0] = mul2(wA[0], gv.x, OutT{}); wA[1] = mul2(wA[1], gv.y, OutT{});
                wA[2] = mul2(wA[2], gv.z, OutT{}); wA[3] = mul2(wA[3], gv.w, OutT{});
              }
              if (rB < row_end) {
                const uint4 gv = ld_v4(gbase + sB * p.ld_gate);
                wB[0] = mul2(wB[0], gv.x, OutT{}); wB[1] = mul2(wB[1], gv.y, OutT{});
                wB[2] = mul2(wB[2], gv.z, OutT{}); wB[3] = mul2(wB[3], gv.w, OutT{});
              }
            }
            if (p.epi_flags & PQ_EPI_ACCUMULATE) {          // out += y: the sum of two rounded tensors, rounded once
              const bool clip = (p.epi_flags & PQ_EPI_GATE) != 0;      // the block tail clips fp16 sums (no-op for bf16)
              if (rA < row_end) {
                const uint4 o = ld_v4(pA);
                if (clip) {
                  wA[0] = add_word_clipped<OutT>(wA[0], o.x); wA[1] = add_word_clipped<OutT>(wA[1], o.y);
                  wA[2] = add_word_clipped<OutT>(wA[2], o.z); wA[3] = add_word_clipped<OutT>(wA[3], o.w);
                } else {
                  wA[0] = add_word<OutT>(wA[0], o.x); wA[1] = add_word<OutT>(wA[1], o.y);
                  wA[2] = add_word<OutT>(wA[2], o.z); wA[3] = add_word<OutT>(wA[3], o.w);
                }
              }
              if (rB < row_end) {
                const uint4 o = ld_v4(pB);
                if (clip) {
                  wB[0] = add_word_clipped<OutT>(wB[0], o.x); wB[1] = add_word_clipped<OutT>(wB[1], o.y);
                  wB[2] = add_word_clipped<OutT>(wB[2], o.z); wB[3] = add_word_clipped<OutT>(wB[3], o.w);
                } else {
                  wB[0] = add_word<OutT>(wB[0], o.x); wB[1] = add_word<OutT>(wB[1], o.y);
                  wB[2] = add_word<OutT>(wB[2], o.z); wB[3] = add_word<OutT>(wB[3], o.w);
                }
              }
            }
            if (p.n_out_more > 0) {
              // the same words go to the further output buffers (other GPUs' memory mapped into this process: the
              // all-gather of a row-sharded layer happens here, tile by tile, while the main loop keeps running)
              const int64_t offA = static_cast<int64_t>(rA) * p.ldo + col_grp + q * 8;
              const int64_t offB = static_cast<int64_t>(rB) * p.ldo + col_grp + q * 8;
#pragma unroll 1
              for (int d = 0; d < p.n_out_more; ++d) {
                OutT* o = static_cast<OutT*>(p.out_more[d]);
                if (rA < row_end) st_v4(o + offA, make_uint4(wA[0], wA[1], wA[2], wA[3]));
                if (rB < row_end) st_v4(o + offB, make_uint4(wB[0], wB[1], wB[2], wB[3]));
              }
            }
            if (p.l2_hints & 8) {                          // outputs are not read again by this kernel: evict first
              if (rA < row_end) st_v4_cs(pA, make_uint4(wA[0], wA[1], wA[2], wA[3]));
              if (rB < row_end) st_v4_cs(pB, make_uint4(wB[0], wB[1], wB[2], wB[3]));
            } else {
              if (rA < row_end) st_v4(pA, make_uint4(wA[0], wA[1], wA[2], wA[3]));
              if (rB < row_end) st_v4(pB, make_uint4(wB[0], wB[1], wB[2], wB[3]));
            }
          } else {
            store_pairs_slow(p.out, p.ldo, rA, rB, col_grp + 2 * q, row_end, p.N, make_uint4(wA[0], wA[1], wA[2], wA[3]),
                             make_uint4(wB[0], wB[1], wB[2], wB[3]));
          }
        }
      };

      // Sixteen-warp tiles without low-rank term are bound by the integer pipe and the global-store path: the rounded
      // 16 x 64 block goes to shared memory in the 128-byte-swizzled layout (conflict-free: the eight rows of a store
      // land in eight different 16-byte columns) and one TMA store writes it; no in-quad transposes, no row
      // predicates (TMA clips at M and N).  The staging buffers are the t / lbT tiles this variant does not use.
      auto stage_unit = [&](const uint32_t (&v)[32], int ch) {
        const int col_unit = ch * kLrChunkN + half * UNIT_N;
        uint8_t* sbuf = smem + L::kTOff + (warp - 2) * 2048;
        if (lane == 0) bulk_wait_group_read0();            // the previous store of this warp has read the buffer
        __syncwarp();
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          const float2 bi = *reinterpret_cast<const float2*>(bias_s + col_unit + nb * 8 + 2 * q);
          uint32_t wA = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 0]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 1]), bi.y), OutT{});
          uint32_t wB = pack2(__fadd_rn(__uint_as_float(v[4 * nb + 2]), bi.x), __fadd_rn(__uint_as_float(v[4 * nb + 3]), bi.y), OutT{});
          if (p.epi_flags & PQ_EPI_GELU_TANH) { wA = gelu_word<OutT>(wA); wB = gelu_word<OutT>(wB); }
          uint8_t* dst = sbuf + g * 128 + ((nb ^ g) << 4) + q * 4;
          st_shared_u32(dst, wA);
          st_shared_u32(dst + 8 * 128, wB);                // row g + 8: same swizzle phase
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int r_first = row0 + quarter * 32 + mb_base * 16;
        if (lane == 0 && r_first < row_end && n0 + col_unit < p.N) {
          tma_store_2d(&tmOut, sbuf, n0 + col_unit, r_first);
          bulk_commit_group();
        }
      };

      long long lr_wait = 0;
      if constexpr (HAS_LR) {
        // pass 1, chunk by chunk: scaled accumulator back to tensor memory; the MMA thread adds t @ lb on top of a
        // chunk as soon as all sixteen warps have written it, while the warps scale the next chunk
        tmem_ld_16x256b_x8(unit_addr(0, 0), va);
#pragma unroll 1
        for (int ch = 0; ch < kLrChunks; ++ch) {
          tc_wait_ld();
          if constexpr (EW == 16) {                       // one 16-row block per warp and chunk; the other warps overlap
            scale_unit(va, ch, 0);
            tmem_st_x8(unit_addr(ch, 0), va);
            wait_st();
            if (ch + 1 < kLrChunks) tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
          } else {
            tmem_ld_16x256b_x8(unit_addr(ch, 1), vb);
            scale_unit(va, ch, 0);
            tmem_st_x8(unit_addr(ch, 0), va);
            tc_wait_ld();
            scale_unit(vb, ch, 1);
            tmem_st_x8(unit_addr(ch, 1), vb);
            wait_st();
            if (ch + 1 < kLrChunks) tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
          }
          tc_fence_before();
          __syncwarp();
          if (timing && warp == 2 && lane == 0) stamp[buf * kLrChunks + ch] = clock64();
          if (trace && it < 1000 && ch == 0 && lane == 0 && warp < 10) trace[it * 24 + rank * 8 + (warp - 2)] = static_cast<long long>(global_timer_ns());
          if (lane == 0) mbar_arrive_cluster(leader_addr(&ylr_ready[buf * kLrChunks + ch]));
        }
        if (timing) e3 = clock64();
      }
      // final pass: (scale when there is no low-rank term,) + bias, round, store
      auto chunk_ready = [&](int ch) -> bool {     // low-rank term of chunk ch has landed in tensor memory
        if constexpr (HAS_LR) {
          const long long c0 = timing ? clock64() : 0;
          const bool landed = wait_or_abort(&lr_done[buf * kLrChunks + ch], par, abort_flag);
          if (!__all_sync(0xffffffffu, landed)) { report_timeout(p.status, 3, 6); *abort_flag = 1; return false; }
          tc_fence_after();
          if (trace && it < 1000 && ch == 0 && warp == 2 && lane == 0) trace[it * 24 + (rank ? 22 : 19)] = static_cast<long long>(global_timer_ns());
          if (timing) { const long long now = clock64(); lr_wait += now - c0; te_exec[ch] += now - stamp[4 + buf * kLrChunks + ch]; }
        }
        return true;
      };
      if (!chunk_ready(0)) { aborted = true; continue; }
      tmem_ld_16x256b_x8(unit_addr(0, 0), va);
#pragma unroll 1
      for (int ch = 0; ch < kLrChunks; ++ch) {
        tc_wait_ld();
        if constexpr (EW == 16) {                         // one 16-row block per warp and chunk; the other warps overlap
          if constexpr (!HAS_LR) scale_unit(va, ch, 0);
          bool staged = false;
          if constexpr (!HAS_LR) {
            if (p.tma_store) { stage_unit(va, ch); staged = true; }
          }
          if (!staged) store_unit(va, ch, 0);
          if (ch + 1 < kLrChunks) {
            if (!chunk_ready(ch + 1)) { aborted = true; break; }
            tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
          }
        } else {
          tmem_ld_16x256b_x8(unit_addr(ch, 1), vb);
          if constexpr (!HAS_LR) scale_unit(va, ch, 0);
          store_unit(va, ch, 0);
          tc_wait_ld();
          if (ch + 1 < kLrChunks) {
            if (!chunk_ready(ch + 1)) { aborted = true; break; }
            tmem_ld_16x256b_x8(unit_addr(ch + 1, 0), va);
          }
          if constexpr (!HAS_LR) scale_unit(vb, ch, 1);
          store_unit(vb, ch, 1);
        }
      }
      if (aborted) continue;
      e4 = e3 + lr_wait;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_addr(&tempty_bar[buf]));
      if (timing) { te_aux += e1 - e0; te_tfull += e2 - e1; te_p1 += e3 - e2; te_lr += e4 - e3; te_p2 += clock64() - e4; }
    }
    if (EW == 16 && !HAS_LR && p.tma_store && lane == 0) bulk_wait_group0();   // stores done before shared memory goes
    if (timing && warp == 2 && lane == 0) {
      timing[blockIdx.x * 16 + 2] = te_aux; timing[blockIdx.x * 16 + 3] = te_tfull; timing[blockIdx.x * 16 + 4] = te_p1;
      timing[blockIdx.x * 16 + 5] = te_lr; timing[blockIdx.x * 16 + 6] = te_p2; timing[blockIdx.x * 16 + 7] = it;
      timing[blockIdx.x * 16 + 10] = te_exec[0]; timing[blockIdx.x * 16 + 11] = te_exec[1];
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // neither CTA leaves (or frees tensor memory) while its peer may still signal it
  if (warp == 1) {
    if (*abort_flag != 0) {
      for (int k = 0; k < 64; ++k) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// Output [M, N] of 16-bit elements, row stride ldo: boxes of 64 columns x 16 rows, 128-byte swizzle (TMA store).
int make_out_map16(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ldo, bool bf16) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PQ_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldo) * 2};
  cuuint32_t box[2] = {64, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int>(r); return PQ_ERR_CUDA; }
  return PQ_OK;
}

template <typename OutT, bool HAS_LR, bool DBG, int EW>
int launch_pair_ew(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmW1, const CUtensorMap& tmT,
                const CUtensorMap& tmLbT, GemmParams p, int mt_pairs, int ntl, cudaStream_t st) {
  // sixteen-warp tiles of a plain single-tier call store through shared memory + TMA when the output allows it
  CUtensorMap tmOut = tmA;
  p.tma_store = 0;
  if (EW == 16 && !HAS_LR && p.m_split == p.M && !(p.epi_flags & (PQ_EPI_ACCUMULATE | PQ_EPI_GATE)) && p.n_out_more == 0 && options().gemm_tma_store != 0 &&
      p.ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
    const int rc = make_out_map16(&tmOut, p.out, p.M, p.N, p.ldo, std::is_same<OutT, __nv_bfloat16>::value);
    if (rc != PQ_OK) return rc;
    p.tma_store = 1;
  }
  auto kern = pq_int8_gemm_fused_pair_kernel<OutT, HAS_LR, DBG, EW>;
  static int max_pairs[64] = {0};
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PQ_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(pair_threads(EW), 1, 1);
  cfg.dynamicSmemBytes = PairSmem::kTotal;
  cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kTotal));
    cfg.gridDim = dim3(2 * sm_count(), 1, 1);
    int n = 0;
    PQ_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return PQ_ERR_UNSUPPORTED;
    max_pairs[dev] = n;
  }
  int pairs_cap = max_pairs[dev];
  if (options().gemm_max_ctas > 0 && options().gemm_max_ctas / 2 < pairs_cap) pairs_cap = options().gemm_max_ctas / 2;
  if (pairs_cap < 1) pairs_cap = 1;
  choose_cta_grid(mt_pairs, ntl, pairs_cap, &p.sched_pm, &p.sched_pn);
  // Row panels.  With several column rounds, the activation rows of a panel (panel steps x pm pair tiles x 256 rows x
  // K bytes) are meant to stay in L2 from one round to the next: the panel is sized to gemm_panel_mb megabytes.
  p.sched_panel = 0;
  const int rounds = (ntl + p.sched_pn - 1) / p.sched_pn;
  if (rounds > 1 && options().gemm_panel_mb > 0) {
    const double step_bytes = static_cast<double>(p.sched_pm) * 2 * BM * p.K;
    int steps = static_cast<int>(options().gemm_panel_mb * 1048576.0 / step_bytes);
    if (steps < 1) steps = 1;
    if (steps < (mt_pairs + p.sched_pm - 1) / p.sched_pm) p.sched_panel = steps;
  }
  p.l2_hints = options().gemm_l2_hints;
  // Tail pairs.  The pm x pn grid leaves pairs_cap - pm * pn SM pairs idle; they take the row tiles from `cut` on of the
  // last column round, and `cut` (a multiple of pm) is chosen for the fewest steps of the slower of the two groups.
  p.sched_cut = mt_pairs; p.sched_tail_per = 0;
  // rows per block of the tail order: the whole region as one block, i.e. column after column (blocks of 1, 2 or 4 row
  // tiles measured the same time)
  p.sched_tail_rb = mt_pairs;
  int extra = pairs_cap - p.sched_pm * p.sched_pn;
  if (extra > 0 && p.sched_panel == 0 && options().gemm_tail_pairs != 0) {
    const int row_steps = (mt_pairs + p.sched_pm - 1) / p.sched_pm;
    const int col0 = (rounds - 1) * p.sched_pn, wl = ntl - col0;
    long long best = static_cast<long long>(row_steps) * rounds;
    for (int k = 0; k < row_steps; ++k) {               // the grid keeps k row steps of the last round
      const int cut = k * p.sched_pm;
      const long long tail = static_cast<long long>(mt_pairs - cut) * wl;
      const long long per = (tail + extra - 1) / extra;
      const long long grid_steps = static_cast<long long>(row_steps) * (rounds - 1) + k;
      const long long steps = grid_steps > per ? grid_steps : per;
      if (steps < best && per <= 0x7fffffffLL) { best = steps; p.sched_cut = cut; p.sched_tail_per = static_cast<int>(per); }
    }
  }
  if (p.sched_tail_per == 0) extra = 0;
  cfg.gridDim = dim3(2 * (p.sched_pm * p.sched_pn + extra), 1, 1);
  PQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmA, tmW, tmW1, tmT, tmLbT, tmOut, p));
  return PQ_OK;
}

// Sixteen epilogue warps when the K loop of a tile is shorter than its epilogue and there is no low-rank term (measured:
// 5-12 % faster there, slower with the two-pass low-rank epilogue); option gemm_epi_warps overrides (0 = this rule).
template <typename OutT, bool HAS_LR, bool DBG>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmW1, const CUtensorMap& tmT,
                const CUtensorMap& tmLbT, GemmParams p, int mt_pairs, int ntl, cudaStream_t st) {
  const int want = options().gemm_epi_warps;
  const bool wide = want == 16 || (want != 8 && !HAS_LR && p.K <= kShortK);
  if (wide) return launch_pair_ew<OutT, HAS_LR, DBG, 16>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
  return launch_pair_ew<OutT, HAS_LR, DBG, 8>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
}

int make_lr_map64(CUtensorMap* map, const void* base, int64_t rows, int64_t ld, int box_rows, bool bf16) {
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

int launch_gemm_pair(bool bf16, bool dbg, const void* xq, int64_t ldx, const void* w, const void* w1, int64_t ldw,
                     const void* t, int64_t ldt, const void* lb_t, int64_t M, int64_t N, int64_t K, const GemmParams& p,
                     cudaStream_t st) {
  CUtensorMap tmA, tmW, tmW1, tmT, tmLbT;
  int rc = make_tile_map(&tmA, xq, M, K, ldx, BM);
  if (rc != PQ_OK) return rc;
  rc = make_tile_map(&tmW, w, N, K, ldw, kHalfB);
  if (rc != PQ_OK) return rc;
  if (p.m_split < p.M) {
    rc = make_tile_map(&tmW1, w1, N, K, ldw, kHalfB);
    if (rc != PQ_OK) return rc;
  } else {
    tmW1 = tmW;
  }
  const bool has_lr = t != nullptr;
  if (has_lr) {
    rc = make_lr_map64(&tmT, t, M, ldt, BM, bf16);
    if (rc != PQ_OK) return rc;
    rc = make_lr_map64(&tmLbT, lb_t, N, kLR, kLbChunkRows, bf16);
    if (rc != PQ_OK) return rc;
  } else {
    tmT = tmA; tmLbT = tmA;
  }
  const int mt_pairs = (p.m_split + 2 * BM - 1) / (2 * BM) + (p.M - p.m_split + 2 * BM - 1) / (2 * BM);
  const int ntl = static_cast<int>((N + PBN - 1) / PBN);
  if (bf16) {
    if (has_lr) return dbg ? launch_pair<__nv_bfloat16, true, true>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st)
                           : launch_pair<__nv_bfloat16, true, false>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
    return dbg ? launch_pair<__nv_bfloat16, false, true>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st)
               : launch_pair<__nv_bfloat16, false, false>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
  }
  if (has_lr) return dbg ? launch_pair<__half, true, true>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st)
                         : launch_pair<__half, true, false>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
  return dbg ? launch_pair<__half, false, true>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st)
             : launch_pair<__half, false, false>(tmA, tmW, tmW1, tmT, tmLbT, p, mt_pairs, ntl, st);
}

}  // namespace pq
