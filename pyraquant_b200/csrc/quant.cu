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

namespace pq {
namespace {

constexpr int kThreads = 256;

// Running maximum of |x| over packed 16-bit floats, kept as two packed magnitudes.  Clearing the sign bits leaves
// non-negative bf16 / fp16 bit patterns, whose order as unsigned 16-bit integers is their order as numbers, so the
// maximum is an integer one: two masked words and the running value per three-input halfword maximum.  (The
// floating-point packed abs / max instructions of these types issue on the slow special-function pipe.)
template <typename T>
__device__ __forceinline__ uint32_t absmax_chunk(uint32_t acc, const uint4& v) {
  constexpr uint32_t kMag = 0x7FFF7FFFu;
  acc = __vimax3_u16x2(acc, v.x & kMag, v.y & kMag);
  acc = __vimax3_u16x2(acc, v.z & kMag, v.w & kMag);
  return acc;
}

// Quantisation of one 16-byte chunk (8 elements) to 8 int8 codes (two 32-bit words).
//
// Exact contract: code = round_half_even(fl(x / scale)) with the IEEE quotient.  Fast path without a division:
// with inv = fl(1/scale), both x * inv * (1 - 2^-21) and x * inv * (1 + 2^-21) are rounded to the nearest integer by
// a fused multiply-add with 1.5 * 2^23 (one rounding, integer left in the low mantissa bits).  The IEEE quotient
// lies between the two products: it, inv and the two scaled reciprocals each carry a relative rounding error of at
// most 2^-24, so a margin of 1.5 * 2^-23 would do and 2^-21 is 2.7 times that.  Rounding is monotonic, so whenever
// both products give the same integer it is the exact answer.  If any of the 8 elements disagrees (a quotient
// within ~2^-20 relative of a rounding boundary) the chunk is redone with real divisions; the margin is kept
// small because one such element sends its whole warp through the slow path.  Codes never leave [-127, 127] because |x| <= absmax.  No conversion instructions are used: those run
// on a slow pipe and made the first version of this kernel issue-bound.
struct QuantScale {
  float scale;       // absmax / 127 (or the 1e-8 floor / 127)
  float2 inv_lo;     // (1/scale) * (1 - 2^-21), twice
  float2 inv_hi;     // (1/scale) * (1 + 2^-21), twice
};
__device__ __forceinline__ QuantScale make_quant_scale(float amax) {
  QuantScale qs;
  // absmax / 127, correctly rounded, without the generic division routine: quotient estimate with the rounded
  // reciprocal, exact residual, one correction.  absmax is a bf16 or fp16 value (or the 1e-8 floor): the sequence
  // was checked against the IEEE quotient for every such value on the host and is checked again for all of them
  // on the device by the tests.
  const float a = fmaxf(amax, 1e-8f);
  const float r127 = 0.007874015718698502f;           // RN(1/127)
  const float q0 = __fmul_rn(a, r127);
  const float rem = __fmaf_rn(-q0, 127.0f, a);
  qs.scale = __fmaf_rn(rem, r127, q0);
  const float inv = __frcp_rn(qs.scale);               // correctly rounded reciprocal = IEEE 1 / scale
  const float lo = inv * (1.0f - 4.76837158203125e-7f), hi = inv * (1.0f + 4.76837158203125e-7f);   // 1 -+ 2^-21
  qs.inv_lo = make_float2(lo, lo);
  qs.inv_hi = make_float2(hi, hi);
  return qs;
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  T tag{};
  return make_float2(lo_f32(w, tag), hi_f32(w, tag));
}

// The rare exact path: real divisions, in line (a call in the hot loop costs more in register shuffling around
// it than these instructions cost in size; an array argument even put a stack frame and its stores on the hot path).
template <typename T>
__device__ __forceinline__ void quant_chunk_exact(const uint4& v, float scale, uint32_t& lo, uint32_t& hi) {
  const float kMagic = 12582912.0f;
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t c[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<T>(w[i]);
    c[2 * i] = __float_as_uint(__fdiv_rn(f.x, scale) + kMagic);
    c[2 * i + 1] = __float_as_uint(__fdiv_rn(f.y, scale) + kMagic);
  }
  lo = __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
  hi = __byte_perm(__byte_perm(c[4], c[5], 0x0040), __byte_perm(c[6], c[7], 0x0040), 0x5410);
}

template <typename T>
__device__ __forceinline__ void quant_chunk(const uint4& v, const QuantScale& qs, uint32_t& lo, uint32_t& hi) {
  const float2 kMagic2 = make_float2(12582912.0f, 12582912.0f);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t m[8];
  // Disagreement test on the fp32 pipe (the integer pipe, half as wide, is the busiest one in this kernel): a - b
  // is a small exact integer, the squares are summed exactly, and the sum is zero only if every pair agrees.
  float2 dsq = make_float2(0.0f, 0.0f);
  const float2 kMinusOne2 = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<T>(w[i]);
    const float2 a = __ffma2_rn(f, qs.inv_lo, kMagic2);
    const float2 b = __ffma2_rn(f, qs.inv_hi, kMagic2);
    m[2 * i] = __float_as_uint(a.x); m[2 * i + 1] = __float_as_uint(a.y);
    const float2 d = __ffma2_rn(b, kMinusOne2, a);
    dsq = __ffma2_rn(d, d, dsq);
  }
  const bool differ = (dsq.x + dsq.y) != 0.0f;
  // low bytes of the eight integers -> two words
  lo = __byte_perm(__byte_perm(m[0], m[1], 0x0040), __byte_perm(m[2], m[3], 0x0040), 0x5410);
  hi = __byte_perm(__byte_perm(m[4], m[5], 0x0040), __byte_perm(m[6], m[7], 0x0040), 0x5410);
  if (differ) quant_chunk_exact<T>(v, qs.scale, lo, hi);
}

template <typename T>
__device__ __forceinline__ float amax_of_packed(uint32_t acc) {
  T tag{};
  return fmaxf(lo_f32(acc, tag), hi_f32(acc, tag));
}

// TPR threads cooperate on one row, each holding CPT chunks of 8 elements (chunk c of the row is owned
// by thread c % TPR).  GROUP32: one scale per 32 elements (4 neighbouring threads) instead of per row.
template <typename T, int TPR, int CPT, bool GATHER, bool GROUP32>
__global__ void __launch_bounds__(kThreads)
pq_quant_rows_kernel(const T* __restrict__ x, int64_t ldx, const int32_t* __restrict__ row_idx, int64_t src_rows,
                     int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K) {
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

  uint4 v[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const int c = lane_in_row + j * TPR;
    if (have_src && c < nchunk) v[j] = ld_stream_v4(xrow + c);
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

template <typename T, bool GATHER, bool GROUP32, int TPR, int CPT>
int launch_one(const void* x, int64_t ldx, const int32_t* row_idx, int64_t src_rows, int8_t* q, float* s, int64_t M,
               int K, cudaStream_t st) {
  constexpr int RPB = kThreads / TPR;
  const int64_t blocks = (M + RPB - 1) / RPB;
  if (blocks > 0x7fffffffLL) return PQ_ERR_SHAPE;
  pq_quant_rows_kernel<T, TPR, CPT, GATHER, GROUP32>
      <<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(static_cast<const T*>(x), ldx, row_idx, src_rows, q, s, M, K);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

template <typename T, bool GATHER, bool GROUP32>
int dispatch(const void* x, int64_t ldx, const int32_t* row_idx, int64_t src_rows, int8_t* q, float* s, int64_t M,
             int K, cudaStream_t st) {
  const int nchunk = K >> 3;
  // team size (threads per row) and chunks per thread: the row must fit the team's registers
  const int force = options().quant_tpr;
  if (force == 16 && nchunk <= 16 * 5) return launch_one<T, GATHER, GROUP32, 16, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 16 && nchunk <= 16 * 10) return launch_one<T, GATHER, GROUP32, 16, 10>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 32 && nchunk <= 32 * 8) return launch_one<T, GATHER, GROUP32, 32, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 32 && nchunk <= 32 * 12) return launch_one<T, GATHER, GROUP32, 32, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 64 && nchunk <= 64 * 8) return launch_one<T, GATHER, GROUP32, 64, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 64 && nchunk <= 64 * 12) return launch_one<T, GATHER, GROUP32, 64, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 128 && nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (force == 256 && nchunk <= 256 * 8) return launch_one<T, GATHER, GROUP32, 256, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  // short rows: half a warp per row, so that a warp amortises its per-row work over two rows (measured: K = 640
  // 28 -> 21 us at 65536 rows; K = 1280 48 -> 44 us without group scales, no gain with them)
  if (nchunk <= 16 * 5) return launch_one<T, GATHER, GROUP32, 16, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if constexpr (!GROUP32) {
    if (nchunk <= 16 * 10) return launch_one<T, GATHER, GROUP32, 16, 10>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  }
  if (nchunk <= 32 * 4) return launch_one<T, GATHER, GROUP32, 32, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if constexpr (!GROUP32) {
    // per-row scales: a single warp per row up to 3072 elements (no shared-memory hop, the per-row work is spread over
    // up to 96 elements per thread: a quarter fewer instructions than four warps per row), measured best per rung
    if (nchunk <= 32 * 8) return launch_one<T, GATHER, GROUP32, 32, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
    if (nchunk <= 32 * 12) return launch_one<T, GATHER, GROUP32, 32, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st);
    if (nchunk <= 64 * 8) return launch_one<T, GATHER, GROUP32, 64, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
    if (nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st);
    if (nchunk <= 64 * 12) return launch_one<T, GATHER, GROUP32, 64, 12>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  }
  if (nchunk <= 64 * 4) return launch_one<T, GATHER, GROUP32, 64, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (nchunk <= 128 * 3) return launch_one<T, GATHER, GROUP32, 128, 3>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (nchunk <= 128 * 5) return launch_one<T, GATHER, GROUP32, 128, 5>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (nchunk <= 256 * 4) return launch_one<T, GATHER, GROUP32, 256, 4>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (nchunk <= 256 * 6) return launch_one<T, GATHER, GROUP32, 256, 6>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if (nchunk <= 256 * 8) return launch_one<T, GATHER, GROUP32, 256, 8>(x, ldx, row_idx, src_rows, q, s, M, K, st);
  if constexpr (GROUP32) {
    return PQ_ERR_UNSUPPORTED;   // K > 16384 with group scales: not a shape of the path
  } else {
    if (M > 0x7fffffffLL) return PQ_ERR_SHAPE;
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
