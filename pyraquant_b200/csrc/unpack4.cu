// Packed 4-bit weight storage for the low tier: the nested 4-bit codes (pyraquant/quantizers_weight.py:182-199,
// values in [-7, 7]) are kept two per byte at rest and expanded to the int8 operand layout the GEMM reads.
// Byte b of a row holds element 2b in its low nibble and element 2b+1 in its high nibble, two's complement.
// HBM-bound: one thread turns 16 packed bytes (32 codes) into 32 int8 bytes.
#include "common.cuh"

namespace pq {
namespace {

constexpr int kThreads = 256;

// four packed bytes (eight nibbles) -> two words of four sign-extended int8 each
__device__ __forceinline__ void expand8(uint32_t w, uint32_t& lo, uint32_t& hi) {
  // bytes of `even`: nibbles 0, 2, 4, 6 (low nibbles); bytes of `odd`: nibbles 1, 3, 5, 7 (high nibbles)
  const uint32_t even = w & 0x0F0F0F0Fu;
  const uint32_t odd = (w >> 4) & 0x0F0F0F0Fu;
  // sign extension of a 4-bit value v held in a byte: (v ^ 8) - 8, per byte without carries between bytes
  const uint32_t se_even = ((even ^ 0x08080808u) | 0x80808080u) - 0x08080808u;
  const uint32_t se_odd = ((odd ^ 0x08080808u) | 0x80808080u) - 0x08080808u;
  // the guard bit 0x80 set before the subtraction absorbs the borrow; flip it back: result byte = (v ^ 8) - 8 mod 256
  const uint32_t e = se_even ^ 0x80808080u;
  const uint32_t o = se_odd ^ 0x80808080u;
  // interleave: output bytes e0 o0 e1 o1 | e2 o2 e3 o3
  lo = __byte_perm(e, o, 0x5140);
  hi = __byte_perm(e, o, 0x7362);
}

__global__ void __launch_bounds__(kThreads)
pq_unpack_int4_kernel(const uint4* __restrict__ packed, int64_t ldp16, uint4* __restrict__ out, int64_t ldo16, int64_t N,
                      int chunks) {
  const int64_t total = N * static_cast<int64_t>(chunks);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t n = i / chunks;
    const int c = static_cast<int>(i - n * chunks);
    const uint4 v = ld_stream_v4(packed + n * ldp16 + c);
    uint4 a, b;
    expand8(v.x, a.x, a.y); expand8(v.y, a.z, a.w);
    expand8(v.z, b.x, b.y); expand8(v.w, b.z, b.w);
    uint4* o = out + n * ldo16 + 2 * static_cast<int64_t>(c);
    st_v4(o, a);
    st_v4(o + 1, b);
  }
}

}  // namespace
}  // namespace pq

using namespace pq;

extern "C" int pq_unpack_int4(const uint8_t* packed, int64_t ldp, int8_t* out, int64_t ldo, int64_t N, int64_t K,
                              void* stream) {
  if (N < 0 || K <= 0 || K > 0x7fffffffLL || ldp < K / 2 || ldo < K) return PQ_ERR_SHAPE;
  if (N == 0) return PQ_OK;
  if (packed == nullptr || out == nullptr) return PQ_ERR_NULL;
  if (K % 32 != 0 || ldp % 16 != 0 || ldo % 16 != 0 || !aligned_to(packed, 16) || !aligned_to(out, 16)) return PQ_ERR_ALIGN;
  const int chunks = static_cast<int>(K / 32);
  const int64_t total = N * chunks;
  int64_t blocks = (total + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (blocks > cap) blocks = cap;
  pq_unpack_int4_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(packed), ldp / 16, reinterpret_cast<uint4*>(out), ldo / 16, N, chunks);
  PQ_CUDA_TRY(cudaGetLastError());
  return PQ_OK;
}
