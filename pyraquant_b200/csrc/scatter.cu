// Feathered scatter of routed rows over the cached canvas (pull form of fuse_patch_predictions,
// flux/routing.py:328-379).  One thread owns one 16-byte chunk (8 channels) of one active canvas
// token and walks that token's contributor list in order, reproducing the reference's arithmetic
// step by step: every intermediate is rounded to the canvas dtype exactly where the reference's
// bf16/fp16 tensors round (fp32 operation followed by one rounding equals the 16-bit operation).
#include "common.cuh"

namespace pq {
namespace {

constexpr int kThreads = 128;             // 128 measured best (one thread per chunk with up to 512 threads: -12 %)

// Two fp32 values rounded to the canvas type and widened again: one packed conversion and two bit operations
// (the scalar round trips issue on the conversion pipe, and there are ~40 of them per chunk).
template <typename T>
__device__ __forceinline__ void rnd2(float& a, float& b) {
  T tag{};
  const uint32_t w = pack2(a, b, tag);
  a = lo_f32(w, tag); b = hi_f32(w, tag);
}
template <typename T>
__device__ __forceinline__ float rnd1(float v) {
  float z = 0.0f;
  rnd2<T>(v, z);
  return v;
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  T tag{};
  f[0] = lo_f32(v.x, tag); f[1] = hi_f32(v.x, tag); f[2] = lo_f32(v.y, tag); f[3] = hi_f32(v.y, tag);
  f[4] = lo_f32(v.z, tag); f[5] = hi_f32(v.z, tag); f[6] = lo_f32(v.w, tag); f[7] = hi_f32(v.w, tag);
}

// One block walks whole tokens (grid-stride over the touched tokens): the token's index data is read once per
// block and is uniform across it; threads stride over the token's 16-byte chunks.
template <typename T>
__global__ void __launch_bounds__(kThreads)
pq_scatter_rows_kernel(const T* __restrict__ y, int64_t ldy, int64_t M_act, const int32_t* __restrict__ tokens,
                       const int32_t* __restrict__ ptr, const int32_t* __restrict__ src,
                       const float* __restrict__ beta, int64_t n_tokens, T* __restrict__ canvas, int64_t ldc,
                       int64_t rows, int nchunk) {
  for (int64_t tk = blockIdx.x; tk < n_tokens; tk += gridDim.x) {
    const int64_t tok = tokens[tk];
    if (tok < 0 || tok >= rows) continue;
    const int e0 = ptr[tk], e1 = ptr[tk + 1];
    // blend weights of the token: the same for every chunk, rounded exactly where the reference rounds
    float bsum = 0.0f;
    for (int e = e0; e < e1; ++e) {
      const int64_t r = src[e];
      if (r < 0 || r >= M_act) continue;
      bsum = rnd1<T>(bsum + beta[e]);
    }
    const float bm = fminf(fmaxf(bsum, 0.0f), 1.0f);
    const float denom = rnd1<T>(fmaxf(bsum, 1e-8f));
    const float one_minus = rnd1<T>(1.0f - bm);
    // a power-of-two denominator (one or two full-weight contributors: the usual case) divides exactly by
    // multiplication with its reciprocal; anything else takes the IEEE division
    const bool pow2 = (__float_as_uint(denom) & 0x007FFFFFu) == 0u;
    const float rden = pow2 ? __frcp_rn(denom) : 0.0f;
    uint4* crow = reinterpret_cast<uint4*>(canvas + tok * ldc);
    for (int c = threadIdx.x; c < nchunk; c += kThreads) {
      float local[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int e = e0; e < e1; ++e) {
        const int64_t r = src[e];
        const float b = beta[e];
        if (r < 0 || r >= M_act) continue;
        const uint4 v = ld_stream_v4(reinterpret_cast<const uint4*>(y + r * ldy) + c);
        float f[8];
        unpack8<T>(v, f);
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
          float p0 = b * f[k], p1 = b * f[k + 1];
          rnd2<T>(p0, p1);
          local[k] += p0; local[k + 1] += p1;
          rnd2<T>(local[k], local[k + 1]);
        }
      }
      const uint4 bgv = crow[c];
      float bg[8], res[8];
      unpack8<T>(bgv, bg);
#pragma unroll
      for (int k = 0; k < 8; k += 2) {
        float c0 = 0.0f, c1 = 0.0f;
        if (bsum > 0.0f) {
          if (pow2) { c0 = local[k] * rden; c1 = local[k + 1] * rden; }
          else { c0 = __fdiv_rn(local[k], denom); c1 = __fdiv_rn(local[k + 1], denom); }
          rnd2<T>(c0, c1);
        }
        float t0 = one_minus * bg[k], t1 = one_minus * bg[k + 1];
        rnd2<T>(t0, t1);
        float u0 = bm * c0, u1 = bm * c1;
        rnd2<T>(u0, u1);
        res[k] = t0 + u0; res[k + 1] = t1 + u1;                  // final rounding happens in pack2
      }
      uint4 o;
      T tag{};
      o.x = pack2(res[0], res[1], tag); o.y = pack2(res[2], res[3], tag);
      o.z = pack2(res[4], res[5], tag); o.w = pack2(res[6], res[7], tag);
      st_v4(crow + c, o);
    }
  }
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_scatter_rows(const void* y, int64_t ldy, int64_t M_act, const int32_t* tokens, const int32_t* ptr,
                               const int32_t* src, const float* beta, int64_t n_tokens, void* canvas, int64_t ldc,
                               int64_t rows, int64_t C, int dtype, void* stream) {
  if (M_act < 0 || n_tokens < 0 || rows < 0 || C <= 0 || C > 0x7fffffffLL || ldy < C || ldc < C) return PQ_ERR_SHAPE;
  if (dtype != PQ_DTYPE_BF16 && dtype != PQ_DTYPE_FP16) return PQ_ERR_DTYPE;
  if (n_tokens == 0) return PQ_OK;
  if (y == nullptr || tokens == nullptr || ptr == nullptr || src == nullptr || beta == nullptr || canvas == nullptr)
    return PQ_ERR_NULL;
  if (C % 8 != 0 || ldy % 8 != 0 || ldc % 8 != 0 || !aligned_to(y, 16) || !aligned_to(canvas, 16)) return PQ_ERR_ALIGN;
  const int nchunk = static_cast<int>(C >> 3);
  int64_t blocks = n_tokens;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 64;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16) {
    pq_scatter_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(y), ldy, M_act, tokens, ptr, src, beta, n_tokens,
        static_cast<__nv_bfloat16*>(canvas), ldc, rows, nchunk);
  } else {
    pq_scatter_rows_kernel<__half><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        static_cast<const __half*>(y), ldy, M_act, tokens, ptr, src, beta, n_tokens, static_cast<__half*>(canvas),
        ldc, rows, nchunk);
  }
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}
