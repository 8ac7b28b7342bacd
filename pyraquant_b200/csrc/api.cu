// Library-wide pieces of libpq_b200: version, status strings, option table, device queries and the
// status-word reader.
#include <cstring>

#include "common.cuh"

namespace pq {

thread_local int g_last_cuda_error = 0;

Options& options() {
  static Options o;
  return o;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace pq

using namespace pq;

extern "C" int pq_version(void) { return 100; }

extern "C" const char* pq_status_str(int status) {
  switch (status) {
    case PQ_OK: return "ok";
    case PQ_ERR_NULL: return "a required pointer is NULL";
    case PQ_ERR_SHAPE: return "invalid size or leading dimension";
    case PQ_ERR_ALIGN: return "pointer, size or leading dimension breaks the alignment rule";
    case PQ_ERR_DTYPE: return "unknown dtype code";
    case PQ_ERR_CUDA: return "a CUDA call failed";
    case PQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case PQ_ERR_UNSUPPORTED: return "combination of arguments not implemented";
    case PQ_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" int pq_last_cuda_error(void) { return g_last_cuda_error; }

namespace {
int* option_slot(const char* key) {
  Options& o = options();
  if (key == nullptr) return nullptr;
  if (std::strcmp(key, "quant_tpr") == 0) return &o.quant_tpr;
  if (std::strcmp(key, "gemm_stages") == 0) return &o.gemm_stages;
  if (std::strcmp(key, "gemm_block_n") == 0) return &o.gemm_block_n;
  if (std::strcmp(key, "gemm_pm") == 0) return &o.gemm_pm;
  if (std::strcmp(key, "gemm_pn") == 0) return &o.gemm_pn;
  if (std::strcmp(key, "gemm_max_ctas") == 0) return &o.gemm_max_ctas;
  if (std::strcmp(key, "gemm_pair") == 0) return &o.gemm_pair;
  if (std::strcmp(key, "gemm_epi_warps") == 0) return &o.gemm_epi_warps;
  if (std::strcmp(key, "gemm_tma_store") == 0) return &o.gemm_tma_store;
  if (std::strcmp(key, "gemm_debug_timing") == 0) return &o.gemm_debug_timing;
  if (std::strcmp(key, "gemm_tail_pairs") == 0) return &o.gemm_tail_pairs;
  if (std::strcmp(key, "gemm_panel_mb") == 0) return &o.gemm_panel_mb;
  if (std::strcmp(key, "gemm_l2_hints") == 0) return &o.gemm_l2_hints;
  if (std::strcmp(key, "g32_variant") == 0) return &o.g32_variant;
  return nullptr;
}
}  // namespace

extern "C" int pq_set_option(const char* key, int value) {
  int* slot = option_slot(key);
  if (slot == nullptr) return PQ_ERR_UNSUPPORTED;
  *slot = value;
  return PQ_OK;
}

extern "C" int pq_get_option(const char* key, int* value) {
  int* slot = option_slot(key);
  if (slot == nullptr) return PQ_ERR_UNSUPPORTED;
  if (value == nullptr) return PQ_ERR_NULL;
  *value = *slot;
  return PQ_OK;
}

extern "C" int pq_read_status_word(void* workspace, int32_t* raw, int clear, void* stream) {
  if (workspace == nullptr) return PQ_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t word = 0;
  PQ_CUDA_TRY(cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, st));
  PQ_CUDA_TRY(cudaStreamSynchronize(st));
  if (clear && word != 0) {
    PQ_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(word), st));
    PQ_CUDA_TRY(cudaStreamSynchronize(st));
  }
  if (raw != nullptr) *raw = word;
  return word == 0 ? PQ_OK : PQ_ERR_TIMEOUT;
}
