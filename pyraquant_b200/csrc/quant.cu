// Memory-bound kernels of the hot path: per-token INT8 quantisation (plain, gathered, group-32) and
// the plain row gather.  One HBM pass: each thread keeps its 16-byte chunks of the row in registers
// between the absmax reduction and the quantisation, loads are 128-bit and coalesced, the per-token
// absmax is a warp-shuffle reduction (plus one shared-memory hop when a row spans several warps).
//
// Arithmetic contract (bit-exact with torch on CPU; deploy/int8_exec.py:508-509 and :83-101):
//   scale = max(absmax, 1e-8) / 127        IEEE fp32 division
//   q     = round_half_even(x / scale)     IEEE fp32 division, clamp to [-127, 127]
// The division per element is replaced by two fused multiply-adds that bracket the quotient; only chunks in
// which a bracket straddles a rounding boundary take the IEEE division (see quant_chunk).
#include "common.cuh"
#include "quant_common.cuh"

namespace pq {
namespace {

constexpr int kThreads = 256;

// TPR threads cooperate on one row, each holding CPT chunks of 8 elements (chunk c of the row is owned
// by thread c % TPR).  GROUP32: one scale per 32 elements (4 neighbouring threads) instead of per row.
template <typename T, int TPR, int CPT, bool GATHER, bool GROUP32>
__global__ void __launch_bounds__(kThreads)
pq_quant_rows_kernel(const T* __restrict__ x, int64_t ldx, const int32_t* __restrict__ row_idx, int64_t src_rows,
                     int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K,
                     const T* __restrict__ x1, int64_t ldx1, int nchunk0) {
  constexpr int RPB = kThreads / TPR;                  // rows per block
  constexpr int WPR = (TPR + 31) / 32;                 // warps per row
  __shared__ float s_part[kThreads / 32];
  const int tid = threadIdx.x;
  const int r_in_blk = tid / TPR;
  const int lane_in_row = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPB + r_in_blk;
  const bool row_ok = row < M;
  const int nchunk = K >> 3;

  int64_t src = row;
  if (GATHER && row_ok) src = row_idx[row];
  const bool have_src = row_ok && src >= 0 && (!GATHER || src < src_rows);   // out-of-range indices read nothing
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (have_src ? src : 0) * ldx);
  // second source: the row continues in another tensor from chunk nchunk0 on (the row is the concatenation of the
  // two along K; nchunk0 == nchunk when there is no second source)
  const uint4* xrow1 = x1 != nullptr ? reinterpret_cast<const uint4*>(x1 + (have_src ? src : 0) * ldx1) - nchunk0 : xrow;

  uint4 v[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const int c = lane_in_row + j * TPR;
    if (have_src && c < nchunk) v[j] = ld_stream_v4((c < nchunk0 ? xrow : xrow1) + c);
    else v[j] = make_uint4(0u, 0u, 0u, 0u);
  }

  if constexpr (!GROUP32) {
    uint32_t acc = 0u;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      acc = absmax_chunk<T>(acc, v[j]);
    }
    float amax = amax_of_packed<T>(acc);
    constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if constexpr (WPR > 1) {
      const int warp = tid >> 5;
      if ((tid & 31) == 0) s_part[warp] = amax;
      __syncthreads();
      const int w0 = r_in_blk * WPR;
      amax = s_part[w0];
#pragma unroll
      for (int w = 1; w < WPR; ++w) amax = fmaxf(amax, s_part[w0 + w]);
    }
    const QuantScale qs = make_quant_scale(amax);
    if (row_ok) {
      if (lane_in_row == 0) s[row] = qs.scale;
      int8_t* qrow = q + row * static_cast<int64_t>(K);
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        const int c = lane_in_row + j * TPR;
        if (c < nchunk) {
          uint32_t lo, hi;
          quant_chunk<T>(v[j], qs, lo, hi);
          st_v2(qrow + (static_cast<int64_t>(c) << 3), lo, hi);
        }
      }
    }
  } else {
    // group of 32 elements = chunks 4i..4i+3 = four neighbouring threads of the row (TPR % 4 == 0)
    const int ngroup = K >> 5;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      uint32_t acc = 0u;
      acc = absmax_chunk<T>(acc, v[j]);
      float amax = amax_of_packed<T>(acc);
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const QuantScale qs = make_quant_scale(amax);
      const int c = lane_in_row + j * TPR;
      if (row_ok && c < nchunk) {
        if ((c & 3) == 0) s[row * static_cast<int64_t>(ngroup) + (c >> 2)] = qs.scale;
        uint32_t lo, hi;
        quant_chunk<T>(v[j], qs, lo, hi);
        st_v2(q + row * static_cast<int64_t>(K) + (static_cast<int64_t>(c) << 3), lo, hi);
      }
    }
  }
}

// Rows too long for the register-resident kernel: one block per row, two sweeps (the second one is
// served by L2 for any row that fits there).
template <typename T, bool GATHER>
__global__ void __launch_bounds__(kThreads)
pq_quant_rows_kernel_long(const T* __restrict__ x, int64_t ldx, const int32_t* __restrict__ row_idx, int64_t src_rows,
                          int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K) {
  __shared__ float s_part[kThreads / 32];
  const int64_t row = blockIdx.x;
  int64_t src = row;
  if (GATHER) src = row_idx[row];
  const bool have_src = src >= 0 && (!GATHER || src < src_rows);
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (have_src ? src : 0) * ldx);
  const int nchunk = K >> 3;
  uint32_t acc = 0u;
  if (have_src) {
    for (int c = threadIdx.x; c < nchunk; c += kThreads) {
      uint4 v = xrow[c];
      acc = absmax_chunk<T>(acc, v);
    }
  }
  float amax = amax_of_packed<T>(acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_part[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, s_part[w]);
  const QuantScale qs = make_quant_scale(amax);
  if (threadIdx.x == 0) s[row] = qs.scale;
  int8_t* qrow = q + row * static_cast<int64_t>(K);
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    uint4 v = have_src ? xrow[c] : make_uint4(0u, 0u, 0u, 0u);
    uint32_t lo, hi;
    quant_chunk<T>(v, qs, lo, hi);
    st_v2(qrow + (static_cast<int64_t>(c) << 3), lo, hi);
  }
}

// Plain gather: out[m,:] = canvas[row_idx[m],:] (zeros for negative indices), 16-byte chunks.
__global__ void __launch_bounds__(kThreads)
pq_gather_rows_kernel(const uint4* __restrict__ x, int64_t ld16, const int32_t* __restrict__ row_idx, int64_t src_rows,
                      uint4* __restrict__ out, int64_t ldo16, int64_t M, int nchunk) {
  const int64_t total = M * static_cast<int64_t>(nchunk);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t m = i / nchunk;
    const int c = static_cast<int>(i - m * nchunk);
    const int64_t src = row_idx[m];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (src >= 0 && src < src_rows) v = ld_stream_v4(x + src * ld16 + c);
    st_v4(out + m * ldo16 + c, v);
  }
}


// int32 accumulators -> scaled 16-bit output, one read and one write per element.
template <typename OutT>
__global__ void __launch_bounds__(kThreads)
pq_dequant_epilogue_kernel(const int32_t* __restrict__ acc, const float* __restrict__ s_row,
                           const float* __restrict__ s_col, const float* __restrict__ bias, OutT* __restrict__ out,
                           int64_t M, int64_t N) {
  const int64_t total = M * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t m = i / N;
    const int64_t n = i - m * N;
    float yv = __fmul_rn(int_to_float_rn(acc[i]), __fmul_rn(s_row[m], s_col[n]));
    if (bias != nullptr) yv = __fadd_rn(yv, bias[n]);
    if constexpr (sizeof(OutT) == 2 && __is_same(OutT, __nv_bfloat16)) out[i] = __float2bfloat16_rn(yv);
    else out[i] = __float2half_rn(yv);
  }
}

// Second source of a row that is the concatenation of two tensors along K (x1 == nullptr: none).
struct SecondSrc { const void* x1 = nullptr; int64_t ldx1 = 0; int k0 = 0; };

template <typename T, bool GATHER, bool GROUP32, int TPR, int CPT>
int launch_one(const void* x, int64_t ldx, const int32_t* row_idx, int64_t src_rows, int8_t* q, float* s, int64_t M,
               int K, cudaStream_t st, const SecondSrc& s2 = SecondSrc()) {
  constexpr int RPB = kThreads / TPR;
  const int64_t blocks = (M + RPB - 1) / RPB;
  if (blocks > 0x7fffffffLL) return PQ_ERR_SHAPE;
  pq_quant_rows_kernel<T, TPR, CPT, GATHER, GROUP32>
      <<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(static_cast<const T*>(x), ldx, row_idx, src_rows, q, s, M, K,
                                                           static_cast<const T*>(s2.x1), s2.ldx1,
                                                           s2.x1 != nullptr ? (s2.k0 >> 3) : (K >> 3));
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

template <typename T, bool GATHER, bool GROUP32>
int dispatch(const void* x, int64_t ldx, const int32_t* row_idx, int64_t src_rows, int8_t* q, float* s, int64_t M,
             int K, cudaStream_t st, const SecondSrc& s2 = SecondSrc()) {
  const int nchunk = K >> 3;
  // team size (threads per row) and chunks per thread: the row must fit the team's registers
  const int force = options().quant_tpr;
  if (force == 16 && nchunk <= 16 * 5) return launch_one<T, GATHER, GROUP32, 16, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 16 && nchunk <= 16 * 10) return launch_one<T, GATHER, GROUP32, 16, 10>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 32 && nchunk <= 32 * 8) return launch_one<T, GATHER, GROUP32, 32, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 32 && nchunk <= 32 * 12) return launch_one<T, GATHER, GROUP32, 32, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 64 && nchunk <= 64 * 8) return launch_one<T, GATHER, GROUP32, 64, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 64 && nchunk <= 64 * 12) return launch_one<T, GATHER, GROUP32, 64, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 128 && nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (force == 256 && nchunk <= 256 * 8) return launch_one<T, GATHER, GROUP32, 256, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  // short rows: half a warp per row, so that a warp amortises its per-row work over two rows (measured: K = 640
  // 28 -> 21 us at 65536 rows; K = 1280 48 -> 44 us without group scales, no gain with them)
  if (nchunk <= 16 * 5) return launch_one<T, GATHER, GROUP32, 16, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if constexpr (!GROUP32) {
    if (nchunk <= 16 * 10) return launch_one<T, GATHER, GROUP32, 16, 10>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  }
  if (nchunk <= 32 * 4) return launch_one<T, GATHER, GROUP32, 32, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if constexpr (!GROUP32) {
    // per-row scales: a single warp per row up to 3072 elements (no shared-memory hop, the per-row work is spread over
    // up to 96 elements per thread: a quarter fewer instructions than four warps per row), measured best per rung
    if (nchunk <= 32 * 8) return launch_one<T, GATHER, GROUP32, 32, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
    if (nchunk <= 32 * 12) return launch_one<T, GATHER, GROUP32, 32, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
    if (nchunk <= 64 * 8) return launch_one<T, GATHER, GROUP32, 64, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
    if (nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
    if (nchunk <= 64 * 12) return launch_one<T, GATHER, GROUP32, 64, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  }
  if (nchunk <= 64 * 4) return launch_one<T, GATHER, GROUP32, 64, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (nchunk <= 128 * 3) return launch_one<T, GATHER, GROUP32, 128, 3>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (nchunk <= 256 * 4) return launch_one<T, GATHER, GROUP32, 256, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (nchunk <= 256 * 6) return launch_one<T, GATHER, GROUP32, 256, 6>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if (nchunk <= 256 * 8) return launch_one<T, GATHER, GROUP32, 256, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st, s2);
  if constexpr (GROUP32) {
    return PQ_ERR_UNSUPPORTED;   // K > 16384 with group scales: not a shape of the path
  } else {
    if (M > 0x7fffffffLL) return PQ_ERR_SHAPE;
    if (s2.x1 != nullptr) return PQ_ERR_UNSUPPORTED;         // two sources: rows up to 16384 elements
    pq_quant_rows_kernel_long<T, GATHER>
        <<<static_cast<unsigned>(M), kThreads, 0, st>>>(static_cast<const T*>(x), ldx, row_idx, src_rows, q, s, M, K);
    PQ_CUDA_TRY(cudaGetLastError());
    return PQ_OK;
  }
}

int check_common(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const void* q, const void* s,
                 int kmult) {
  if (M < 0 || K <= 0 || K > 0x7fffffffLL || ldx < K) return PQ_ERR_SHAPE;
  if (dtype != PQ_DTYPE_BF16 && dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (x == nullptr || q == nullptr || s == nullptr) return PQ_ERR_NULL;
  if (K % kmult != 0 || ldx % 8 != 0) return PQ_ERR_ALIGN;
  if (!aligned_to(x, 16) || !aligned_to(q, 8) || !aligned_to(s, 4)) return PQ_ERR_ALIGN;
  return PQ_OK;
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_quant_rows(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int8_t* q, float* s,
                             void* stream) {
  int rc = check_common(x, dtype, M, K, ldx, q, s, 8);
  if (rc != PQ_OK || M == 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16)
    return dispatch<__nv_bfloat16, false, false>(x, ldx, nullptr, M, q, s, M, static_cast<int>(K), st);
  return dispatch<__half, false, false>(x, ldx, nullptr, M, q, s, M, static_cast<int>(K), st);
}

extern "C" int pq_quant_rows_cat(const void* x0, int64_t K0, int64_t ldx0, const void* x1, int64_t K1, int64_t ldx1,
                                 int dtype, int64_t M, int8_t* q, float* s, void* stream) {
  if (K0 <= 0 || K1 <= 0 || ldx1 < K1) return PQ_ERR_SHAPE;
  int rc = check_common(x0, dtype, M, K0, ldx0, q, s, 8);
  if (rc != PQ_OK || M == 0) return rc;
  if (x1 == nullptr) return PQ_ERR_NULL;
  if (K1 % 8 != 0 || ldx1 % 8 != 0 || !aligned_to(x1, 16)) return PQ_ERR_ALIGN;
  if (K0 + K1 > 16384) return PQ_ERR_UNSUPPORTED;
  SecondSrc s2; s2.x1 = x1; s2.ldx1 = ldx1; s2.k0 = static_cast<int>(K0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16)
    return dispatch<__nv_bfloat16, false, false>(x0, ldx0, nullptr, M, q, s, M, static_cast<int>(K0 + K1), st, s2);
  return dispatch<__half, false, false>(x0, ldx0, nullptr, M, q, s, M, static_cast<int>(K0 + K1), st, s2);
}

extern "C" int pq_gather_quant_rows(const void* canvas, int dtype, int64_t rows, int64_t K, int64_t ld,
                                    const int32_t* row_idx, int64_t M, int8_t* q, float* s, void* stream) {
  if (rows < 0) return PQ_ERR_SHAPE;
  int rc = check_common(canvas, dtype, M, K, ld, q, s, 8);
  if (rc != PQ_OK || M == 0) return rc;
  if (row_idx == nullptr) return PQ_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16)
    return dispatch<__nv_bfloat16, true, false>(canvas, ld, row_idx, rows, q, s, M, static_cast<int>(K), st);
  return dispatch<__half, true, false>(canvas, ld, row_idx, rows, q, s, M, static_cast<int>(K), st);
}

extern "C" int pq_quant_rows_g32(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int8_t* q, float* s,
                                 void* stream) {
  int rc = check_common(x, dtype, M, K, ldx, q, s, 32);
  if (rc != PQ_OK || M == 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16)
    return dispatch<__nv_bfloat16, false, true>(x, ldx, nullptr, M, q, s, M, static_cast<int>(K), st);
  return dispatch<__half, false, true>(x, ldx, nullptr, M, q, s, M, static_cast<int>(K), st);
}

extern "C" int pq_gather_rows(const void* canvas, int dtype, int64_t rows, int64_t K, int64_t ld,
                              const int32_t* row_idx, int64_t M, void* out, int64_t ldo, void* stream) {
  if (M < 0 || rows < 0 || K <= 0 || K > 0x7fffffffLL || ld < K || ldo < K) return PQ_ERR_SHAPE;
  if (dtype != PQ_DTYPE_BF16 && dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (canvas == nullptr || row_idx == nullptr || out == nullptr) return PQ_ERR_NULL;
  if (K % 8 != 0 || ld % 8 != 0 || ldo % 8 != 0 || !aligned_to(canvas, 16) || !aligned_to(out, 16))
    return PQ_ERR_ALIGN;
  const int nchunk = static_cast<int>(K >> 3);
  const int64_t total = M * nchunk;
  int64_t blocks = (total + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  pq_gather_rows_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(canvas), ld >> 3, row_idx, rows, static_cast<uint4*>(out), ldo >> 3, M, nchunk);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

extern "C" int pq_dequant_epilogue(const int32_t* acc, const float* s_row, const float* s_col, const float* bias,
                                   void* out, int out_dtype, int64_t M, int64_t N, void* stream) {
  if (M < 0 || N <= 0) return PQ_ERR_SHAPE;
  if (out_dtype != PQ_DTYPE_BF16 && out_dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (acc == nullptr || s_row == nullptr || s_col == nullptr || out == nullptr) return PQ_ERR_NULL;
  const int64_t total = M * N;
  int64_t blocks = (total + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == PQ_DTYPE_BF16)
    pq_dequant_epilogue_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        acc, s_row, s_col, bias, static_cast<__nv_bfloat16*>(out), M, N);
  else
    pq_dequant_epilogue_kernel<__half><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        acc, s_row, s_col, bias, static_cast<__half*>(out), M, N);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}
