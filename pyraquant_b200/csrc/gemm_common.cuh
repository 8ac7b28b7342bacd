// Pieces shared by the tcgen05 GEMM kernels (per-channel and group-32): tile constants, bounded mbarrier
// waits, the in-quad transpose used for 16-byte output stores, the out-of-line ragged store and the host-side
// TMA tensor-map encoder.
#pragma once

#include "common.cuh"

namespace pq {

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
  int sched_pm, sched_pn;   // the CTAs form a sched_pm x sched_pn grid over (row tile, column tile)
  int sched_m_steps;        // ceil(row tiles / sched_pm)
  int sched_n_rounds;       // ceil(column tiles / sched_pn)
  int has_bias;
  int epi_flags;            // PQ_EPI_* bits (CTA-pair kernel only)
  int sched_panel;          // CTA-pair kernel: row steps per panel (0 = all rows in one panel)
  int sched_cut;            // CTA-pair kernel: in the last column round the pair grid takes row tiles below this one only ...
  int sched_tail_per;       // ... and the pairs beyond the grid take the rest, this many tiles each (0: no such pairs),
  int sched_tail_rb;        // in blocks of this many row tiles
  int l2_hints;             // CTA-pair kernel: Options::gemm_l2_hints
  int tma_store;            // CTA-pair kernel, sixteen epilogue warps: output tiles leave through shared memory + TMA
  const void* gate;         // CTA-pair kernel, PQ_EPI_GATE: [samples, N] factors in the output type (row stride ld_gate)
  int64_t ld_gate;
  int64_t gate_rows;        // rows per sample (0: one sample)
  void* out_more[7];        // CTA-pair kernel: further buffers (same shape and row stride as out) that receive every output store
  int n_out_more;
  long long* timing;        // experiments: per-CTA cycle counters [grid][8] (NULL in normal use)
};

// out = act(y) or out += y variants of the epilogue, on values already rounded to the output type (what separate
// elementwise kernels after the Linear would see).
__device__ __forceinline__ float gelu_tanh_f32(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), tanh by the hardware approximation (relative error ~2^-11)
  const float inner = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
  return 0.5f * x * (1.0f + th);
}
template <typename OutT>
__device__ __forceinline__ uint32_t gelu_word(uint32_t w) {
  return pack2(gelu_tanh_f32(lo_f32(w, OutT{})), gelu_tanh_f32(hi_f32(w, OutT{})), OutT{});
}
// The FLUX blocks clip fp16 hidden states to the finite range after the residual sum (flux/transformer_flux.py:148-149);
// clamping the fp32 sum before the rounding gives the same value (a sum beyond 65520 would round to infinity and be clipped
// to 65504, anything up to 65520 rounds to at most 65504 by itself).
__device__ __forceinline__ float clip_like_block(float v, __half) { return fminf(fmaxf(v, -65504.0f), 65504.0f); }
__device__ __forceinline__ float clip_like_block(float v, __nv_bfloat16) { return v; }
template <typename OutT>
__device__ __forceinline__ uint32_t add_word_clipped(uint32_t w, uint32_t prev) {
  return pack2(clip_like_block(lo_f32(w, OutT{}) + lo_f32(prev, OutT{}), OutT{}),
               clip_like_block(hi_f32(w, OutT{}) + hi_f32(prev, OutT{}), OutT{}), OutT{});
}
template <typename OutT>
__device__ __forceinline__ uint32_t add_word(uint32_t w, uint32_t prev) {
  return pack2(lo_f32(w, OutT{}) + lo_f32(prev, OutT{}), hi_f32(w, OutT{}) + hi_f32(prev, OutT{}), OutT{});
}

struct TileCoord {
  int row0, row_end, n0, set;
};

namespace {

constexpr int BM = 128;          // rows per tile = tensor-memory lanes
constexpr int BK = 128;          // K bytes per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;       // K per tcgen05.mma kind::i8

constexpr int kNumEpiWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kNumEpiWarps;
constexpr int kLR = 32;          // low-rank width handled in the epilogue

// Bounded wait on an mbarrier phase.  The first probe is inline; the polling loop (wall-clock budget, abort
// flag) lives out of line to keep the role loops small.
__device__ __noinline__ bool wait_or_abort_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                uint64_t budget_ns = kWaitBudgetNs) {
  uint64_t t0 = 0;
  for (uint32_t i = 1; i < kWaitMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0) {
      if (*abort_flag != 0) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
  return false;
}
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              uint64_t budget_ns = kWaitBudgetNs) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_or_abort_slow(bar, parity, abort_flag, budget_ns);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// In-quad 4x4 transpose: on entry lane q of a quad holds w[j] = word (source lane q, block j); on exit it
// holds w[k] = word (source lane k, block q).
__device__ __forceinline__ void quad_transpose(uint32_t (&w)[4], int q) {
  const bool hi = (q & 2) != 0;
  uint32_t s0 = hi ? w[0] : w[2], s1 = hi ? w[1] : w[3];
  uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2), r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
  uint32_t v0 = hi ? r0 : w[0], v1 = hi ? r1 : w[1], v2 = hi ? w[2] : r0, v3 = hi ? w[3] : r1;
  const bool odd = (q & 1) != 0;
  s0 = odd ? v0 : v1; s1 = odd ? v2 : v3;
  r0 = __shfl_xor_sync(0xffffffffu, s0, 1); r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
  w[0] = odd ? r0 : v0; w[1] = odd ? v1 : r0; w[2] = odd ? r1 : v2; w[3] = odd ? v3 : r1;
}

// Ragged / unaligned outputs: one packed pair (columns col, col+1 of one row) at a time.  Kept out of line so
// that the common path stays small.
__device__ __noinline__ void store_pairs_slow(void* out, int64_t ldo, int rA, int rB, int col0, int row_end, int N,
                                              uint4 a, uint4 b) {
  const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
  unsigned short* o = static_cast<unsigned short*>(out);
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    const int col = col0 + j * 8;
#pragma unroll 1
    for (int r = 0; r < 2; ++r) {
      const int row = r == 0 ? rA : rB;
      const uint32_t w = r == 0 ? wa[j] : wb[j];
      if (row >= row_end) continue;
      unsigned short* p = o + static_cast<int64_t>(row) * ldo + col;
      if (col < N) p[0] = static_cast<unsigned short>(w & 0xFFFFu);
      if (col + 1 < N) p[1] = static_cast<unsigned short>(w >> 16);
    }
  }
}

// Tile schedule.  CTA b sits at (bm, bn) = (b / pn, b % pn) of a pm x pn grid laid over the tile matrix and
// walks it with strides (pm, pn): all row tiles of one column tile first, then the next column tile.  At any
// moment the CTAs touch pn weight tiles (each shared by pm CTAs, unchanged from step to step, so they stay in
// L2) and pm activation tiles (each shared by pn CTAs); a CTA's column tile changes only once per sweep over
// the rows, so per-column epilogue data is loaded rarely.  Every role of a CTA walks the same sequence with
// its own walker; there are no divisions in the loop.
struct TileWalker {
  int mt, ntile;        // current row tile / column tile
  int bm, pm, pn, mt_total, nt;
  __device__ __forceinline__ void init(int pm_, int pn_, int mt_total_, int nt_) {
    pm = pm_; pn = pn_; mt_total = mt_total_; nt = nt_;
    bm = static_cast<int>(blockIdx.x) / pn;
    mt = bm; ntile = static_cast<int>(blockIdx.x) - bm * pn;
  }
  __device__ __forceinline__ bool valid() const { return ntile < nt && mt < mt_total; }
  __device__ __forceinline__ void advance() {       // to the next tile of this CTA (or past the end)
    mt += pm;
    if (mt >= mt_total) { mt = bm; ntile += pn; }
  }
};

// Row range, column start and weight set of the walker's current tile.
__device__ __forceinline__ TileCoord tile_coord(const TileWalker& w, const GemmParams& p, int mt0, int BN) {
  TileCoord c;
  if (w.mt < mt0) { c.set = 0; c.row0 = w.mt * BM; c.row_end = p.m_split; }
  else { c.set = 1; c.row0 = p.m_split + (w.mt - mt0) * BM; c.row_end = p.M; }
  c.n0 = w.ntile * BN;
  return c;
}

// Host: CTA grid pm x pn (pm * pn <= max_ctas) with the fewest steps ceil(mt/pm) * ceil(nt/pn) plus a small charge
// per column change; ties go to the widest pn (fewer sweeps over the rows).  Option overrides gemm_pn / gemm_pm win when they fit.
inline void choose_cta_grid(int mt, int ntl, int max_ctas, int* pm_out, int* pn_out) {
  int best_pm = 1, best_pn = 1;
  long long best_steps = -1;
  for (int pn = 1; pn <= ntl && pn <= max_ctas; ++pn) {
    int pm = max_ctas / pn;
    if (pm > mt) pm = mt;
    if (pm < 1) continue;
    // cost in quarter tiles: every step is one tile, every change of column tile costs about a quarter of one
    const long long rounds = (ntl + pn - 1) / pn;
    const long long steps = 4 * static_cast<long long>((mt + pm - 1) / pm) * rounds + rounds;
    if (best_steps < 0 || steps < best_steps || (steps == best_steps && pn > best_pn)) {
      best_steps = steps; best_pm = pm; best_pn = pn;
    }
  }
  if (options().gemm_pn > 0 && options().gemm_pn <= ntl && options().gemm_pn <= max_ctas) {
    best_pn = options().gemm_pn;
    best_pm = max_ctas / best_pn; if (best_pm > mt) best_pm = mt;
    if (options().gemm_pm > 0 && options().gemm_pm <= best_pm) best_pm = options().gemm_pm;
  }
  *pm_out = best_pm; *pn_out = best_pn;
}

// ---------------------------------------------------------------------------------------------
// host side: TMA tensor maps
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
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
inline int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
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


// fp32 matrix [rows, cols] with row stride ld elements; box = box_cols x box_rows, no swizzle, zero fill.
inline int make_f32_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols,
                        int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PQ_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int>(r); return PQ_ERR_CUDA; }
  return PQ_OK;
}

}  // namespace
}  // namespace pq
