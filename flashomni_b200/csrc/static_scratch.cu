// fo_gemm_q_static: GEMM-Q for callers that cannot obtain device memory at call time.
//
// Some hosts of this library never get to call cudaMalloc on the hot path: an inference server that
// hands the whole device to its own arena at start-up, a plugin running under a framework whose
// allocator it must not touch, or a real-time loop that cannot afford the device-wide synchronisation
// an allocation may imply. fo_gemm_q needs a small scratch region (the list of active output tiles that
// its first kernel compacts from the mask, plus counters and a status word). This variant keeps that
// scratch in a fixed array inside the library image, so the caller passes only inputs and outputs.
//
// Limits and rules:
//   * the array is kStaticScratchBytes (1 MiB) per GPU that loads the library, held until the process
//     exits; it fits work lists of up to 65 534 records (a record covers one or two 128x128 output
//     tiles of one 128-row block, so batch * m/128 * ceil(n/256) must stay below that); larger
//     problems are rejected with FO_ERR_WORKSPACE and a message that names both sizes;
//   * the first call on each device resolves the device address of the array (one cudaGetSymbolAddress,
//     with that device current); make that first call before any stream capture begins;
//   * every call on a device shares the one array: calls that may overlap on the GPU (different
//     streams, or threads launching concurrently) race on it. Serialise them on one stream;
//   * the array keeps the previous call's contents; the words that must start from a known value
//     (tile count, list status, kernel status) are rewritten by every call before they are read;
//   * nothing on this path calls cudaMalloc, cudaFree or any allocating library routine.
#include <mutex>
#include <string>

#include "../../include/flashomni_b200.h"
#include "internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices];   // device address of g_static_scratch, per device ordinal
thread_local std::string g_static_error;

// Host code must not pass `g_static_scratch` itself to a kernel: on the host that name is only a
// stand-in for the symbol. The device address comes from cudaGetSymbolAddress, once per device.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_static_error = "fo_gemm_q_static: cannot identify the current device";
    return FO_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_static_error = std::string("fo_gemm_q_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e);
      return FO_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return FO_OK;
}

}  // namespace

extern "C" {

size_t fo_gemm_q_static_max_bytes(void) { return kStaticScratchBytes; }

const char* fo_gemm_q_static_last_error(void) { return g_static_error.c_str(); }

int fo_gemm_q_static(const void* x, const void* w, void* y, const void* bias, int32_t dtype, int32_t batch,
                     int32_t m, int32_t n, int32_t k, int32_t num_heads, int32_t head_begin, int32_t head_dim,
                     int32_t sparse_q_size, int32_t num_text_tokens, int32_t is_full, const uint8_t* sparse_info,
                     int64_t sparse_info_bytes, const int32_t* sparse_info_indptr, void* stream) {
  g_static_error.clear();
  const size_t need = fo_gemm_workspace_bytes(batch, m, n, k, head_dim);
  if (need > kStaticScratchBytes) {
    g_static_error = "fo_gemm_q_static: this problem needs " + std::to_string(need) +
                     " bytes of scratch but the built-in array holds " + std::to_string(kStaticScratchBytes) +
                     "; use fo_gemm_q with a caller-provided workspace";
    return FO_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != FO_OK) return rc;
  const int rc2 = fo_gemm_q(x, w, y, bias, dtype, batch, m, n, k, num_heads, head_begin, head_dim, sparse_q_size,
                            num_text_tokens, is_full, sparse_info, sparse_info_bytes, sparse_info_indptr, scratch,
                            kStaticScratchBytes, stream);
  if (rc2 != FO_OK) g_static_error = fo_last_error();
  return rc2;
}

}  // extern "C"
