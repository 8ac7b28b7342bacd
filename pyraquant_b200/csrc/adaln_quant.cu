// adaLN prologue fused into the per-token quantisation: for every row
//   y = LayerNorm(x) (no affine parameters)      z = y * (1 + scale) + shift      (q, s) = quantise(z)
// in one pass over x (flux/transformer_flux.py:195 `norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)`
// and :236-239 `norm2(h) * (1 + scale_mlp[:, None]) + shift_mlp[:, None]` feeding the feed-forward's first Linear).
// The reference runs four memory-bound kernels here (LayerNorm, multiply, add, then the Linear's quantisation):
// 15 bytes of traffic per element; this kernel reads 2, writes the int8 code and, only when asked for (the
// low-rank down-projection and the attention branch read the modulated activations), the 16-bit z: 3 or 5 bytes.
//
// Arithmetic follows the 16-bit tensor sequence of the reference step by step: mean and variance in fp32 over the
// row; y = round16((x - mean) * rstd); g = round16(1 + scale); z = round16(round16(y * g) + shift).  The row statistics
// are summed in another order than torch's LayerNorm kernel sums them, so y can differ from torch's by one unit in the
// last place where (x - mean) * rstd falls within ~1e-7 (relative) of a rounding boundary; everything after y, and the
// quantisation of z, is exact.
#include <type_traits>

#include "common.cuh"
#include "quant_common.cuh"

namespace pq {
namespace {

constexpr int kThreads = 256;

// Makes the compiler forget what it derived from a chunk: the three passes over the row each unpack it again (two
// instructions per pair) instead of keeping 96 unpacked floats alive next to the 48 packed registers.
__device__ __forceinline__ void forget(uint4& v) { asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)); }

// Sum over the TPR threads of a row team: shuffles inside the warp, one shared-memory hop when the team spans warps.
template <int TPR>
__device__ __forceinline__ float team_sum(float v, float* part, int tid, int r_in_blk) {
  constexpr int W = TPR < 32 ? TPR : 32;
  constexpr int WPR = (TPR + 31) / 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (WPR > 1) {
    if ((tid & 31) == 0) part[tid >> 5] = v;
    __syncthreads();
    const int w0 = r_in_blk * WPR;
    v = part[w0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) v += part[w0 + w];
  }
  return v;
}

template <typename T, int TPR, int CPT, bool WRITE_X>
__global__ void __launch_bounds__(kThreads, 3)
pq_adaln_quant_rows_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ scale, const T* __restrict__ shift,
                           int64_t ld_mod, int64_t rows_per_sample, float eps, T* __restrict__ xm, int64_t ldxm,
                           int8_t* __restrict__ q, float* __restrict__ s, int64_t M, int K) {
  constexpr int RPB = kThreads / TPR;                  // rows per block
  constexpr int WPR = (TPR + 31) / 32;                 // warps per row
  __shared__ float part_sum[kThreads / 32], part_var[kThreads / 32], part_max[kThreads / 32];
  T tag{};
  const int tid = threadIdx.x;
  const int r_in_blk = tid / TPR;
  const int lane_in_row = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPB + r_in_blk;
  const bool row_ok = row < M;
  const int nchunk = K >> 3;
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (row_ok ? row : 0) * ldx);

  uint4 v[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const int c = lane_in_row + j * TPR;
    if (row_ok && c < nchunk) v[j] = ld_stream_v4(xrow + c);
    else v[j] = make_uint4(0u, 0u, 0u, 0u);
  }

  // row statistics in fp32 (two passes over the registers: mean, then the centred sum of squares)
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) sum += lo_f32(w[i], tag) + hi_f32(w[i], tag);
  }
  const float mean = team_sum<TPR>(sum, part_sum, tid, r_in_blk) / static_cast<float>(K);
#pragma unroll
  for (int j = 0; j < CPT; ++j) forget(v[j]);
  float ssq = 0.0f;
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    if (lane_in_row + j * TPR < nchunk) {
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = lo_f32(w[i], tag) - mean, b = hi_f32(w[i], tag) - mean;
        ssq = fmaf(a, a, ssq); ssq = fmaf(b, b, ssq);
      }
    }
  }
  const float var = team_sum<TPR>(ssq, part_var, tid, r_in_blk) / static_cast<float>(K);
  const float rstd = rsqrtf(var + eps);
#pragma unroll
  for (int j = 0; j < CPT; ++j) forget(v[j]);

  // modulation vectors of the row's sample
  const int64_t sample = rows_per_sample > 0 ? (row_ok ? row : 0) / rows_per_sample : 0;
  const uint4* sc_row = reinterpret_cast<const uint4*>(scale + sample * ld_mod);
  const uint4* sh_row = reinterpret_cast<const uint4*>(shift + sample * ld_mod);
  const uint32_t one2 = pack2(1.0f, 1.0f, tag);
  uint32_t acc = 0u;
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const int c = lane_in_row + j * TPR;
    if (c < nchunk) {
      const uint4 sc = ld_v4(sc_row + c), sh = ld_v4(sh_row + c);
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
      uint32_t z[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t y = pack2(__fmul_rn(__fsub_rn(lo_f32(w[i], tag), mean), rstd),
                                 __fmul_rn(__fsub_rn(hi_f32(w[i], tag), mean), rstd), tag);
        z[i] = add2(mul2(y, add2(one2, scw[i], tag), tag), shw[i], tag);
      }
      v[j] = make_uint4(z[0], z[1], z[2], z[3]);
      if (WRITE_X && row_ok) st_v4(reinterpret_cast<uint4*>(xm + row * ldxm) + c, v[j]);
      acc = absmax_chunk<T>(acc, v[j]);
    }
  }

  // per-token quantisation of z, as pq_quant_rows does it
  float amax = amax_of_packed<T>(acc);
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if constexpr (WPR > 1) {
    if ((tid & 31) == 0) part_max[tid >> 5] = amax;
    __syncthreads();
    const int w0 = r_in_blk * WPR;
    amax = part_max[w0];
#pragma unroll
    for (int w = 1; w < WPR; ++w) amax = fmaxf(amax, part_max[w0 + w]);
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
}

struct AdaArgs {
  const void* x; int64_t ldx; const void* scale; const void* shift; int64_t ld_mod, rows_per_sample; float eps;
  void* xm; int64_t ldxm; int8_t* q; float* s; int64_t M; int K;
};

template <typename T, int TPR, int CPT>
int launch_one(const AdaArgs& a, cudaStream_t st) {
  constexpr int RPB = kThreads / TPR;
  const int64_t blocks = (a.M + RPB - 1) / RPB;
  if (blocks > 0x7fffffffLL) return PQ_ERR_SHAPE;
  if (a.xm != nullptr)
    pq_adaln_quant_rows_kernel<T, TPR, CPT, true><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        static_cast<const T*>(a.x), a.ldx, static_cast<const T*>(a.scale), static_cast<const T*>(a.shift), a.ld_mod,
        a.rows_per_sample, a.eps, static_cast<T*>(a.xm), a.ldxm, a.q, a.s, a.M, a.K);
  else
    pq_adaln_quant_rows_kernel<T, TPR, CPT, false><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        static_cast<const T*>(a.x), a.ldx, static_cast<const T*>(a.scale), static_cast<const T*>(a.shift), a.ld_mod,
        a.rows_per_sample, a.eps, nullptr, 0, a.q, a.s, a.M, a.K);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}

// team size and chunks per thread: the rungs of the plain quantisation kernel that keep a row in the team's registers
template <typename T>
int dispatch(const AdaArgs& a, cudaStream_t st) {
  const int nchunk = a.K >> 3;
  if (nchunk <= 16 * 5) return launch_one<T, 16, 5>(a, st);
  if (nchunk <= 32 * 4) return launch_one<T, 32, 4>(a, st);
  if (nchunk <= 32 * 8) return launch_one<T, 32, 8>(a, st);
  if (nchunk <= 32 * 12) return launch_one<T, 32, 12>(a, st);
  if (nchunk <= 64 * 8) return launch_one<T, 64, 8>(a, st);
  if (nchunk <= 64 * 12) return launch_one<T, 64, 12>(a, st);
  if (nchunk <= 256 * 4) return launch_one<T, 256, 4>(a, st);
  if (nchunk <= 256 * 8) return launch_one<T, 256, 8>(a, st);
  return PQ_ERR_UNSUPPORTED;               // rows beyond 16384 elements: not a shape of the path
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_adaln_quant_rows(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const void* scale,
                                   const void* shift, int64_t ld_mod, int64_t rows_per_sample, float eps,
                                   void* x_mod, int64_t ldxm, int8_t* q, float* s, void* stream) {
  if (M < 0 || K <= 0 || K > 0x7fffffffLL || ldx < K || rows_per_sample < 0 || !(eps >= 0.0f)) return PQ_ERR_SHAPE;
  if (x_mod != nullptr && ldxm < K) return PQ_ERR_SHAPE;
  if (dtype != PQ_DTYPE_BF16 && dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (M == 0) return PQ_OK;
  if (x == nullptr || scale == nullptr || shift == nullptr || q == nullptr || s == nullptr) return PQ_ERR_NULL;
  if (K % 8 != 0 || ldx % 8 != 0 || (rows_per_sample > 0 && ld_mod % 8 != 0) || (x_mod != nullptr && ldxm % 8 != 0)) return PQ_ERR_ALIGN;
  if (!aligned_to(x, 16) || !aligned_to(scale, 16) || !aligned_to(shift, 16) || !aligned_to(q, 8) || !aligned_to(s, 4) ||
      (x_mod != nullptr && !aligned_to(x_mod, 16)))
    return PQ_ERR_ALIGN;
  const AdaArgs a{x, ldx, scale, shift, ld_mod, rows_per_sample, eps, x_mod, ldxm, q, s, M, static_cast<int>(K)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16) return dispatch<__nv_bfloat16>(a, st);
  return dispatch<__half>(a, st);
}
