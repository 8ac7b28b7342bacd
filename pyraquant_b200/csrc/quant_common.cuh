// Device helpers shared by the quantisation kernels: packed absmax, the exact per-token scale and the division-free
// quantisation of a 16-byte chunk.
//
// Arithmetic contract (bit-exact with torch on CPU; deploy/int8_exec.py:508-509 and :83-101):
//   scale = max(absmax, 1e-8) / 127        IEEE fp32 division
//   q     = round_half_even(x / scale)     IEEE fp32 division, clamp to [-127, 127]
#pragma once
#include "common.cuh"

namespace pq {
namespace {

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

}  // namespace
}  // namespace pq
