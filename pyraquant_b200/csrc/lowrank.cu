// Low-rank down-projection t = x @ A for the rank-32 branch (deploy/int8_exec.py:390), as a streaming tcgen05 kernel:
//   t[m, 0:32] = round_to_dtype( sum_k x[m,k] * A[k, 0:32] )   with fp32 accumulation in tensor memory.
// The product is a skinny GEMM that reads all of x once and is bound by HBM.  A CTA owns 64-row tiles of x (small
// tiles: 1032 of them at M = 66048 spread evenly over the SMs), streams them through a six-stage TMA ring
// (two boxes of {x tile 64 x 64 elements, A^T tile 32 x 64 elements} per stage, 128-byte swizzle), one thread issues
// tcgen05.mma.kind::f16 64 x 32 x 16 (eight per stage) into one of two 32-column accumulators, and four epilogue warps
// round and store finished tiles while the next tile streams.  A is passed transposed ([32, K], K-contiguous) so
// that both operands are K-major.  Every wait is bounded (status word, abort flag) like in the GEMM kernels.
#include <type_traits>

#include "gemm_common.cuh"

namespace pq {
namespace {

constexpr int LM = 64;                 // rows of x per tile (tcgen05 M = 64)
constexpr int LKE = 64;                // elements of K per TMA box (128 bytes of a 16-bit type: one swizzle row)
constexpr int LBOX = 2;                // boxes per operand and stage: fewer barrier operations per byte for the two
                                       // single threads that drive the ring (they are latency-bound at low SM clocks)
constexpr int kLowMaxCols = 128;       // up to four rank-32 branches side by side (layers that share their input)
constexpr int kLowThreads = 64 + 4 * 32;

template <int NC>                      // NC output columns: 32, 64, 96 or 128
struct LowSmem {
  static constexpr int kStages = NC <= 32 ? 6 : (NC <= 64 ? 5 : 4);
  static constexpr int kXBytes = LM * LKE * 2;       // 8 KB per box
  static constexpr int kABytes = NC * LKE * 2;       // 4 .. 16 KB per box
  static constexpr int kStageBytes = LBOX * (kXBytes + kABytes);
  static constexpr int kBarOff = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 4;   // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int kTmemCols = NC <= 32 ? 64 : (NC <= 64 ? 128 : 256);   // two accumulators, a power of two
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kDynamic = kMiscOff + 16 + 1024;
};

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__host__ __device__ constexpr uint32_t idesc_f16_f32acc(int M, int N, bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

template <typename T, int NC>
__global__ void __launch_bounds__(kLowThreads, 1)
pq_lowrank_down_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmX1,
                       const __grid_constant__ CUtensorMap tmA, T* __restrict__ t,
                       int64_t ldt, int M, int K, int k0, int32_t* status) {
  using L = LowSmem<NC>;
  constexpr int LSTAGES = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + LSTAGES;
  uint64_t* tfull_bar = empty_bar + LSTAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles = (M + LM - 1) / LM;
  const int num_kb = (K + LBOX * LKE - 1) / (LBOX * LKE);
  constexpr uint32_t kTmemCols = L::kTmemCols;       // two accumulators of NC columns

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmX); tma_prefetch_desc(&tmX1); tma_prefetch_desc(&tmA);
    for (int s = 0; s < LSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
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
#pragma unroll 1
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int row0 = tile * LM;
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            report_timeout(status, 1, 1); *abort_flag = 1; ok = false; break;
          }
          uint8_t* xs = smem + stage * L::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
#pragma unroll
          for (int b = 0; b < LBOX; ++b) {             // boxes past the end of K are zero-filled by TMA
            // x may be the concatenation of two tensors along K: columns from k0 on come from the second one
            const int col = (kb * LBOX + b) * LKE;
            if (col < k0) tma_load_2d(xs + b * (L::kXBytes + L::kABytes), &tmX, &full_bar[stage], col, row0);
            else tma_load_2d(xs + b * (L::kXBytes + L::kABytes), &tmX1, &full_bar[stage], col - k0, row0);
            tma_load_2d(xs + b * (L::kXBytes + L::kABytes) + L::kXBytes, &tmA, &full_bar[stage], (kb * LBOX + b) * LKE, 0);
          }
          ++issued;
          if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      const int pending = issued < LSTAGES ? static_cast<int>(issued) : LSTAGES;
      for (int i = 0; i < pending; ++i) {            // copies in flight must land before the CTA may exit
        if (--stage < 0) { stage = LSTAGES - 1; phase ^= 1u; }
        if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
          for (int k = 0; k < 64; ++k) __nanosleep(1000);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_f16_f32acc(LM, NC, std::is_same<T, __nv_bfloat16>::value);
      int stage = 0; uint32_t phase = 0; int it = 0; bool ok = true;
#pragma unroll 1
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!wait_or_abort(&tempty_bar[buf], (static_cast<uint32_t>(it >> 1) & 1u) ^ 1u, abort_flag)) {
          report_timeout(status, 2, 2); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * NC);
#pragma unroll 1
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&full_bar[stage], phase, abort_flag)) {
            report_timeout(status, 2, 1); *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
#pragma unroll
          for (int b = 0; b < LBOX; ++b) {
            const uint32_t x_addr = smem_u32(smem + stage * L::kStageBytes + b * (L::kXBytes + L::kABytes));
            const uint64_t a_desc = make_kmajor_sw128_desc(x_addr);
            const uint64_t b_desc = make_kmajor_sw128_desc(x_addr + L::kXBytes);
#pragma unroll
            for (int k = 0; k < LKE / 16; ++k)
              tc_mma_f16(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                         (kb > 0 || b > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    // A 64-row accumulator keeps rows 16 q .. 16 q + 15 in the first sixteen lanes of lane quarter q.
    const int quarter = warp & 3;
    bool aborted = false;
    int it = 0;
#pragma unroll 1
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      if (!aborted) {
        const bool landed = wait_or_abort(&tfull_bar[buf], static_cast<uint32_t>(it >> 1) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) { report_timeout(status, 3, 3); *abort_flag = 1; aborted = true; }
      }
      if (aborted) continue;
      tc_fence_after();
      const int row = tile * LM + quarter * 16 + lane;
#pragma unroll
      for (int cg = 0; cg < NC / 32; ++cg) {           // 32 columns at a time
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + static_cast<uint32_t>(buf * NC + cg * 32) + (static_cast<uint32_t>(quarter * 32) << 16), v);
        tc_wait_ld();
        if (cg == NC / 32 - 1) {                       // the accumulator is in registers: the MMA thread may reuse it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        }
        if (lane < 16 && row < M) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) w[j] = pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), T{});
          T* dst = t + static_cast<int64_t>(row) * ldt + cg * 32;
#pragma unroll
          for (int j = 0; j < 4; ++j) st_v4(dst + 8 * j, make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
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

// 16-bit matrix [rows, K] with row stride ld elements; box = 64 elements (128 bytes) x box_rows, 128-byte swizzle.
int make_map16(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows, bool bf16) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return PQ_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(LKE), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int>(r); return PQ_ERR_CUDA; }
  return PQ_OK;
}

template <typename T, int NC>
int launch_low(const CUtensorMap& tmX, const CUtensorMap& tmX1, int k0, const CUtensorMap& tmA, void* t, int64_t ldt, int64_t M,
               int64_t K, int32_t* status, cudaStream_t st) {
  auto kern = pq_lowrank_down_kernel<T, NC>;
  using LS = LowSmem<NC>;
  static bool attr_set[64] = {false};
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PQ_ERR_UNSUPPORTED;
  if (!attr_set[dev]) {
    PQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LS::kDynamic));
    attr_set[dev] = true;
  }
  const int64_t tiles = (M + LM - 1) / LM;
  int64_t grid = sm_count();
  if (grid > tiles) grid = tiles;
  kern<<<static_cast<unsigned>(grid), kLowThreads, LS::kDynamic, st>>>(tmX, tmX1, tmA, static_cast<T*>(t), ldt,
                                                                           static_cast<int>(M), static_cast<int>(K), k0, status);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

template <typename T>
int launch_low_cols(int R, const CUtensorMap& tmX, const CUtensorMap& tmX1, int k0, const CUtensorMap& tmA, void* t, int64_t ldt,
                    int64_t M, int64_t K, int32_t* status, cudaStream_t st) {
  switch (R) {
    case 32: return launch_low<T, 32>(tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
    case 64: return launch_low<T, 64>(tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
    case 96: return launch_low<T, 96>(tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
    case 128: return launch_low<T, 128>(tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
    default: return PQ_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace pq

using namespace pq;

namespace {
int lowrank_down_impl(const void* x, int64_t K0, int64_t ldx, const void* x1, int64_t K1, int64_t ldx1, int dtype,
                      const void* a_t, int64_t lda, int R, void* t, int64_t ldt, int64_t M, void* workspace, size_t ws_bytes,
                      void* stream) {
  const int64_t K = K0 + K1;
  if (M < 0 || K0 <= 0 || K1 < 0 || M > 0x7fffff00LL || K > 0x7fffff00LL || ldx < K0 || lda < K || R <= 0 || ldt < R) return PQ_ERR_SHAPE;
  if (x1 != nullptr && ldx1 < K1) return PQ_ERR_SHAPE;
  if (R % 32 != 0 || R > kLowMaxCols) return PQ_ERR_UNSUPPORTED;
  if (dtype != PQ_DTYPE_BF16 && dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (x == nullptr || a_t == nullptr || t == nullptr || (K1 > 0 && x1 == nullptr)) return PQ_ERR_NULL;
  if (K0 % 8 != 0 || ldx % 8 != 0 || lda % 8 != 0 || ldt % 8 != 0 || !aligned_to(x, 16) || !aligned_to(a_t, 16) ||
      !aligned_to(t, 16))
    return PQ_ERR_ALIGN;
  if (K1 > 0 && (K1 % 8 != 0 || ldx1 % 8 != 0 || !aligned_to(x1, 16))) return PQ_ERR_ALIGN;
  if (K1 > 0 && K0 % LKE != 0) return PQ_ERR_UNSUPPORTED;       // the seam has to fall between two 64-element boxes
  if (workspace != nullptr && ws_bytes < PQ_GEMM_WORKSPACE_BYTES) return PQ_ERR_WORKSPACE;
  const bool bf16 = dtype == PQ_DTYPE_BF16;
  CUtensorMap tmX, tmX1, tmA;
  int rc = make_map16(&tmX, x, M, K0, ldx, LM, bf16);
  if (rc != PQ_OK) return rc;
  if (K1 > 0) {
    rc = make_map16(&tmX1, x1, M, K1, ldx1, LM, bf16);
    if (rc != PQ_OK) return rc;
  } else {
    tmX1 = tmX;
  }
  rc = make_map16(&tmA, a_t, R, K, lda, R, bf16);
  if (rc != PQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* status = static_cast<int32_t*>(workspace);
  const int k0 = static_cast<int>(K1 > 0 ? K0 : K + LKE * LBOX);        // one source: every box comes from it
  if (bf16) return launch_low_cols<__nv_bfloat16>(R, tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
  return launch_low_cols<__half>(R, tmX, tmX1, k0, tmA, t, ldt, M, K, status, st);
}
}  // namespace

extern "C" int pq_lowrank_down(const void* x, int dtype, int64_t ldx, const void* a_t, int64_t lda, int R, void* t,
                               int64_t ldt, int64_t M, int64_t K, void* workspace, size_t ws_bytes, void* stream) {
  return lowrank_down_impl(x, K, ldx, nullptr, 0, 0, dtype, a_t, lda, R, t, ldt, M, workspace, ws_bytes, stream);
}

extern "C" int pq_lowrank_down_cat(const void* x0, int64_t K0, int64_t ldx0, const void* x1, int64_t K1, int64_t ldx1,
                                   int dtype, const void* a_t, int64_t lda, int R, void* t, int64_t ldt, int64_t M,
                                   void* workspace, size_t ws_bytes, void* stream) {
  if (x1 == nullptr || K1 <= 0) return x1 == nullptr ? PQ_ERR_NULL : PQ_ERR_SHAPE;
  return lowrank_down_impl(x0, K0, ldx0, x1, K1, ldx1, dtype, a_t, lda, R, t, ldt, M, workspace, ws_bytes, stream);
}
