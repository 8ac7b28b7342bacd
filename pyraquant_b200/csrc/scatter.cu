// Feathered scatter of routed rows over the cached canvas (pull form of fuse_patch_predictions,
// flux/routing.py:328-379).  One warp owns one active canvas token; a lane owns 16-byte chunks (8 channels) of it
// and walks the token's contributor list in order, reproducing the reference's arithmetic step by step: every
// intermediate is rounded to the canvas dtype exactly where the reference's bf16/fp16 tensors round (an fp32
// operation followed by one rounding equals the 16-bit operation).
#include <type_traits>

#include "common.cuh"

namespace pq {
namespace {

constexpr int kWarps = 4;                 // warps per block; a warp works on one item (token or part of one) at a time
constexpr int kThreads = kWarps * 32;
constexpr int kBatch = 4;                 // 16-byte chunks per lane whose loads are issued together
constexpr int kCopyBatch = 12;            // the same for tokens that only copy a routed row

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

// Two packed 16-bit floats (bf16 or fp16: sign in bit 15 of each half): -0 becomes +0, everything else is kept.
// (magnitude + 0x7FFF) carries into bit 15 exactly when the magnitude is non-zero, and never beyond its half.
__device__ __forceinline__ uint32_t plus_zero(uint32_t w) {
  const uint32_t nz = (w & 0x7FFF7FFFu) + 0x7FFF7FFFu;
  return w & (nz | 0x7FFF7FFFu);
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  T tag{};
  f[0] = lo_f32(v.x, tag); f[1] = hi_f32(v.x, tag); f[2] = lo_f32(v.y, tag); f[3] = hi_f32(v.y, tag);
  f[4] = lo_f32(v.z, tag); f[5] = hi_f32(v.z, tag); f[6] = lo_f32(v.w, tag); f[7] = hi_f32(v.w, tag);
}

template <typename T>
__device__ __forceinline__ bool fits(float v) { return rnd1<T>(v) == v; }

// Blend of one 16-byte chunk (8 channels) from its contributors' chunks and the background chunk, with the
// reference's roundings: local = sum_e round(round(b_e * y_e) + local); c = round(local / denom) where sum > 0;
// out = round(round((1 - clamp(sum)) * bg) + round(clamp(sum) * c)).
// Two forms.  `packed`: all of it in packed 16-bit arithmetic, taken when the token's weights are 16-bit values
// (they are when the plan was built for the canvas type); the quotient is local * (1 / denom) -- exact for a
// power-of-two denominator; for any other denominator of the bfloat16 canvas the fp32 product with the correctly
// rounded reciprocal, rounded once: a quotient of two 8-bit significands stays at least 2^-16 (relative) away from every
// rounding boundary, more than the 2^-23 the product can be off (results below the normal range excepted).  Everything
// else (fp16 canvas with a general denominator, weights that are not 16-bit values) runs the fp32 form with the IEEE
// division.
template <typename T>
struct TokenBlend {
  float b0, b1, bsum, bm, denom, one_minus, rden;
  bool pow2, packed, need_bg;
  uint32_t b0p, b1p, bmp, omp, rdp;

  __device__ __forceinline__ void setup(float b0_, float b1_, float bsum_) {
    T tag{};
    b0 = b0_; b1 = b1_; bsum = bsum_;
    bm = fminf(fmaxf(bsum, 0.0f), 1.0f);
    denom = rnd1<T>(fmaxf(bsum, 1e-8f));
    one_minus = rnd1<T>(1.0f - bm);
    need_bg = one_minus != 0.0f;
    pow2 = (__float_as_uint(denom) & 0x007FFFFFu) == 0u;
    rden = __frcp_rn(denom);
    const bool quot_ok = pow2 ? fits<T>(rden) : std::is_same<T, __nv_bfloat16>::value;
    packed = quot_ok && fits<T>(b0) && fits<T>(b1);
    b0p = pack2(b0, b0, tag); b1p = pack2(b1, b1, tag); bmp = pack2(bm, bm, tag); omp = pack2(one_minus, one_minus, tag);
    rdp = pack2(rden, rden, tag);
  }

  // ---- packed form: `local` holds four packed pairs
  __device__ __forceinline__ void add_packed(uint32_t (&local)[4], const uint4& v, uint32_t bp) const {
    T tag{};
    local[0] = add2(local[0], mul2(bp, v.x, tag), tag); local[1] = add2(local[1], mul2(bp, v.y, tag), tag);
    local[2] = add2(local[2], mul2(bp, v.z, tag), tag); local[3] = add2(local[3], mul2(bp, v.w, tag), tag);
  }
  __device__ __forceinline__ uint32_t quotient_packed(uint32_t l) const {
    T tag{};
    if (!(bsum > 0.0f)) return 0u;
    if (pow2) return mul2(l, rdp, tag);
    return pack2(lo_f32(l, tag) * rden, hi_f32(l, tag) * rden, tag);
  }
  __device__ __forceinline__ void finish_packed(const uint32_t (&local)[4], const uint4& bgv, uint4* dst) const {
    T tag{};
    const uint32_t bgw[4] = {bgv.x, bgv.y, bgv.z, bgv.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t u = mul2(bmp, quotient_packed(local[k]), tag);
      // with a background factor of zero the sum is u itself: u is never -0 here (local starts from +0, so it is +0
      // whenever it is zero), and (+-0) + u == u
      o[k] = need_bg ? add2(mul2(omp, bgw[k], tag), u, tag) : u;
    }
    st_v4(dst, make_uint4(o[0], o[1], o[2], o[3]));
  }

  // ---- fp32 form
  __device__ __forceinline__ void finish(float (&local)[8], const uint4& bgv, uint4* dst) const {
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
    st_v4(dst, o);
  }
  __device__ __forceinline__ void add(float (&local)[8], const uint4& v, float b) const {
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
};

// Tokens come in two kinds:
//   copy   one contributor of weight one (every token inside a leaf).  clamp(sum) = 1, the divisor is 1 and the
//          background factor 1 - clamp(sum) is 0, so the reference's arithmetic reduces to out = 0 + y: the routed row
//          itself with -0 written as +0 (0 * b + u == u for every finite background b; the canvas row is not read).
//          Pure data movement: a whole row of loads in flight per lane.
//   blend  everything else (feathered halo tokens, overlaps): the reference's arithmetic with all its roundings.  A
//          token whose accumulated weight reaches one does not read its canvas row either.
// A block takes kTokPerBlock consecutive tokens of the list.  Its first threads examine one token each (read the
// contributor list, classify, work out the blend weights, rounded where the reference rounds) and file it in one of two
// lists in shared memory; then the warps share the work items: a blend token counts as one item per kBatch x 32 chunks
// (those first: they are the longer ones), a copy token as one item.  Every item issues all its loads before it touches
// the data; only lists of more than two contributors walk the contributors chunk by chunk.
struct BlendToken {
  int tok, r0, r1, nv, e0, e1;
  float b0, b1, bsum;
};
constexpr int kTokPerBlock = 16;

template <typename T>
__global__ void __launch_bounds__(kThreads, 4)
pq_scatter_rows_kernel(const T* __restrict__ y, int64_t ldy, int64_t M_act, const int32_t* __restrict__ tokens,
                       const int32_t* __restrict__ ptr, const int32_t* __restrict__ src,
                       const float* __restrict__ beta, int64_t n_tokens, T* __restrict__ canvas, int64_t ldc,
                       int64_t rows, int nchunk) {
  __shared__ BlendToken blend_list[kTokPerBlock];
  __shared__ int2 copy_list[kTokPerBlock];          // (canvas token, routed row)
  __shared__ int n_blend, n_copy;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { n_blend = 0; n_copy = 0; }
  __syncthreads();
  const int64_t tk = static_cast<int64_t>(blockIdx.x) * kTokPerBlock + threadIdx.x;
  if (threadIdx.x < kTokPerBlock && tk < n_tokens) {
    BlendToken bt;
    bt.tok = tokens[tk]; bt.e0 = ptr[tk]; bt.e1 = ptr[tk + 1];
    bt.r0 = bt.r1 = 0; bt.nv = 0; bt.b0 = bt.b1 = 0.0f; bt.bsum = 0.0f;
    for (int e = bt.e0; e < bt.e1; ++e) {
      const int r = src[e];
      if (r < 0 || r >= M_act) continue;
      const float b = beta[e];
      if (bt.nv == 0) { bt.r0 = r; bt.b0 = b; }
      if (bt.nv == 1) { bt.r1 = r; bt.b1 = b; }
      bt.bsum = rnd1<T>(bt.bsum + b);
      ++bt.nv;
    }
    if (bt.tok >= 0 && bt.tok < rows) {
      if (bt.nv == 1 && bt.b0 == 1.0f) copy_list[atomicAdd(&n_copy, 1)] = make_int2(bt.tok, bt.r0);
      else blend_list[atomicAdd(&n_blend, 1)] = bt;
    }
  }
  __syncthreads();
  const int nbatch = (nchunk + 32 * kBatch - 1) / (32 * kBatch);
  const int blend_items = n_blend * nbatch;
  const int items = blend_items + n_copy;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  for (int it = warp; it < items; it += kWarps) {
    if (it >= blend_items) {
      // ---- copy: a half keeps its sign bit only if its magnitude is non-zero (-0 -> +0), on the packed 16-bit pairs
      const int2 ct = copy_list[it - blend_items];
      const uint4* y0 = reinterpret_cast<const uint4*>(y + static_cast<int64_t>(ct.y) * ldy);
      uint4* crow = reinterpret_cast<uint4*>(canvas + static_cast<int64_t>(ct.x) * ldc);
      for (int base = 0; base < nchunk; base += 32 * kCopyBatch) {
        uint4 v[kCopyBatch];
#pragma unroll
        for (int j = 0; j < kCopyBatch; ++j) {
          const int c = base + j * 32 + lane;
          if (c < nchunk) v[j] = ld_stream_v4(y0 + c);
        }
#pragma unroll
        for (int j = 0; j < kCopyBatch; ++j) {
          const int c = base + j * 32 + lane;
          if (c < nchunk) st_v4(crow + c, make_uint4(plus_zero(v[j].x), plus_zero(v[j].y), plus_zero(v[j].z), plus_zero(v[j].w)));
        }
      }
      continue;
    }
    // ---- blend
    const BlendToken bt = blend_list[it / nbatch];
    const int base = (it % nbatch) * 32 * kBatch;
    TokenBlend<T> tb;
    tb.setup(bt.b0, bt.b1, bt.bsum);
    const bool need_bg = tb.need_bg;
    uint4* crow = reinterpret_cast<uint4*>(canvas + static_cast<int64_t>(bt.tok) * ldc);
    if (bt.nv <= 2) {
      const uint4* y0 = reinterpret_cast<const uint4*>(y + static_cast<int64_t>(bt.r0) * ldy);
      const uint4* y1 = reinterpret_cast<const uint4*>(y + static_cast<int64_t>(bt.r1) * ldy);
      uint4 v0[kBatch], v1[kBatch], bgv[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = base + j * 32 + lane;
        v0[j] = zero4; v1[j] = zero4; bgv[j] = zero4;
        if (c < nchunk) {
          if (bt.nv >= 1) v0[j] = ld_stream_v4(y0 + c);
          if (bt.nv >= 2) v1[j] = ld_stream_v4(y1 + c);
          if (need_bg) bgv[j] = ld_v4(crow + c);
        }
      }
      if (tb.packed) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int c = base + j * 32 + lane;
          if (c >= nchunk) continue;
          uint32_t local[4] = {0u, 0u, 0u, 0u};
          if (bt.nv >= 1) tb.add_packed(local, v0[j], tb.b0p);
          if (bt.nv >= 2) tb.add_packed(local, v1[j], tb.b1p);
          tb.finish_packed(local, bgv[j], crow + c);
        }
      } else {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int c = base + j * 32 + lane;
          if (c >= nchunk) continue;
          float local[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (bt.nv >= 1) tb.add(local, v0[j], tb.b0);
          if (bt.nv >= 2) tb.add(local, v1[j], tb.b1);
          tb.finish(local, bgv[j], crow + c);
        }
      }
    } else {
      for (int j = 0; j < kBatch; ++j) {
        const int c = base + j * 32 + lane;
        if (c >= nchunk) continue;
        float local[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int e = bt.e0; e < bt.e1; ++e) {
          const int64_t r = src[e];
          const float b = beta[e];
          if (r < 0 || r >= M_act) continue;
          tb.add(local, ld_stream_v4(reinterpret_cast<const uint4*>(y + r * ldy) + c), b);
        }
        tb.finish(local, need_bg ? ld_v4(crow + c) : zero4, crow + c);
      }
    }
  }
}

template <typename T>
int launch_scatter(const void* y, int64_t ldy, int64_t M_act, const int32_t* tokens, const int32_t* ptr, const int32_t* src,
                   const float* beta, int64_t n_tokens, void* canvas, int64_t ldc, int64_t rows, int nchunk, cudaStream_t st) {
  const int64_t blocks = (n_tokens + kTokPerBlock - 1) / kTokPerBlock;
  if (blocks > 0x7fffffffLL) return PQ_ERR_SHAPE;
  pq_scatter_rows_kernel<T><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
      static_cast<const T*>(y), ldy, M_act, tokens, ptr, src, beta, n_tokens, static_cast<T*>(canvas), ldc, rows, nchunk);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PQ_DTYPE_BF16)
    return launch_scatter<__nv_bfloat16>(y, ldy, M_act, tokens, ptr, src, beta, n_tokens, canvas, ldc, rows, nchunk, st);
  return launch_scatter<__half>(y, ldy, M_act, tokens, ptr, src, beta, n_tokens, canvas, ldc, rows, nchunk, st);
}

