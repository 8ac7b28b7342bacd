// pq_int8_linear_noalloc: per-token quantisation + fused INT8 GEMM of one Linear for callers that must not
// allocate device memory.
//
// Who cannot allocate: a serving loop that has handed all device memory to its own pool and treats any
// cudaMalloc as a bug (it synchronises the whole device and can fail or fragment under a full pool); code that
// runs between cudaStreamBeginCapture and EndCapture, where allocation calls are illegal; a plugin loaded into a
// host process whose memory budget is fixed at start-up.  The regular entry points solve this by taking every
// buffer from the caller; this one exists for the case where the caller has no spare buffer for the
// intermediate results either (the int8 codes and the row scales that live between the two kernels).
//
// The intermediates sit in a file-scope __device__ array of fixed size, so every GPU on which this library is
// loaded carries kScratchBytes (about 16 MiB) until the process exits, and shapes that need more are rejected.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kStatusBytes = 256;                          // word 0: status word of the GEMM
constexpr size_t kMaxRows = PQ_NOALLOC_MAX_ROWS;              // row scales: 4 bytes each
constexpr size_t kMaxCodeBytes = PQ_NOALLOC_MAX_CODE_BYTES;   // int8 codes: M * K bytes
constexpr size_t kScalesOff = kStatusBytes;
constexpr size_t kCodesOff = kScalesOff + kMaxRows * sizeof(float);
constexpr size_t kScratchBytes = kCodesOff + kMaxCodeBytes;

// In host code this name is only a handle for the runtime, not an address a kernel can use: the device address
// is obtained below with cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[64] = {nullptr};

// Device address of g_scratch on the current device (looked up on first use, cached afterwards).
int scratch_address(void** out) {
  int dev = 0;
  PQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PQ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    PQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_scratch));
    if (p == nullptr) return PQ_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return PQ_OK;
}

}  // namespace

extern "C" size_t pq_noalloc_scratch_bytes(void) { return kScratchBytes; }

extern "C" int pq_int8_linear_noalloc(const void* x, int dtype, int64_t ldx, const int8_t* w, int64_t ldw,
                                      const float* s_col, const float* bias, void* out, int64_t ldo, int64_t M,
                                      int64_t N, int64_t K, void** status_word, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return PQ_ERR_SHAPE;
  // the fixed scratch bounds the problem: refuse anything larger instead of overrunning it
  if (static_cast<uint64_t>(M) > kMaxRows) return PQ_ERR_WORKSPACE;
  if (static_cast<uint64_t>(M) * static_cast<uint64_t>(K) > kMaxCodeBytes) return PQ_ERR_WORKSPACE;
  void* base = nullptr;
  int rc = scratch_address(&base);
  if (rc != PQ_OK) return rc;
  unsigned char* b = static_cast<unsigned char*>(base);
  if (status_word != nullptr) *status_word = b;
  if (M == 0) return PQ_OK;
  float* scales = reinterpret_cast<float*>(b + kScalesOff);
  int8_t* codes = reinterpret_cast<int8_t*>(b + kCodesOff);
  // The array keeps whatever the previous call left.  Codes and scales are fully overwritten for the rows in
  // use; the status word must read zero unless THIS call fails, so it is cleared first (cudaMemsetAsync
  // allocates nothing).
  PQ_CUDA_TRY(cudaMemsetAsync(b, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)));
  rc = pq_quant_rows(x, dtype, M, K, ldx, codes, scales, stream);
  if (rc != PQ_OK) return rc;
  return pq_int8_gemm(codes, K, scales, w, ldw, s_col, bias, nullptr, 0, nullptr, 0, nullptr, 0, dtype, out, dtype, ldo, M, N,
                      K,
                      b, kStatusBytes, nullptr, stream);
}
