// INT4 forward for callers that cannot hand the library a workspace.
//
// Some hosts of this library own no allocator on the device: an engine that has
// already claimed every free byte of HBM for its KV-cache pool before the first
// forward (the reference sizes that pool from what is left after model load), or a
// binding that is only ever given input and output pointers by its runtime and may
// not call cudaMalloc itself (a call that would also synchronise the whole device in
// the middle of serving).  For them the split-K scratch lives in a fixed array inside
// the library image instead of a caller-provided buffer.
//
// Every GPU that loads the library carries the array (kStaticScratchBytes) until the
// process exits, whether or not this entry point is ever called.
#include <cstdio>
#include <mutex>

#include "internal.cuh"

namespace b200q {

// 128 KiB header (status word, tile counters, argmax keys) + room for the fp32 partials of
// every geometry whose workspace fits: every M <= 64 (the stream-K kernel's partials are
// bounded by the SM count, not by the matrix), larger M while split-K partials fit.
// Larger problems are refused, not truncated.
constexpr size_t kStaticScratchBytes = 16u << 20;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device
// address.  The address is looked up once per device, with that device current.
static void* static_scratch_for_current_device(int* status) {
  static void* ptrs[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_error("cudaGetDevice", e);
    *status = B200Q_ERR_CUDA;
    return nullptr;
  }
  std::lock_guard<std::mutex> g(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error("cudaGetSymbolAddress(g_static_scratch)", e);
      *status = B200Q_ERR_CUDA;
      return nullptr;
    }
    // Nothing is cleared here: a __device__ array is zero-filled when the library image is
    // loaded onto the device, and the kernels return counters, keys and the status word to
    // zero themselves.  (A memset at this point would not be ordered with a forward launched
    // on a non-blocking stream.)
    ptrs[dev] = p;
  }
  *status = B200Q_OK;
  return ptrs[dev];
}

}  // namespace b200q

using namespace b200q;

extern "C" {

size_t b200q_static_scratch_bytes(void) { return kStaticScratchBytes; }

int b200q_w4a16_forward_static_scratch(const void* x, int64_t ldx, int act_dtype,
                                       const void* packed, int64_t ldw, int layout,
                                       const void* scales, const void* zeros, int group,
                                       const void* bias, void* y, int64_t ldy, int M, int N,
                                       int K, int kernel, void* stream) {
  if (M < 0 || N < 0 || K <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N == 0) return B200Q_OK;
  const size_t need = b200q_workspace_bytes(4, M, N, K);
  if (need > kStaticScratchBytes) {
    char text[200];
    std::snprintf(text, sizeof(text),
                  "static scratch holds %zu bytes but M=%d N=%d K=%d needs %zu: use "
                  "b200q_w4a16_forward with a caller-owned workspace",
                  kStaticScratchBytes, M, N, K, need);
    set_last_error_text(text);
    return B200Q_ERR_WORKSPACE;
  }
  int status = B200Q_OK;
  void* scratch = static_scratch_for_current_device(&status);
  if (scratch == nullptr) return status;
  return b200q_w4a16_forward(x, ldx, act_dtype, packed, ldw, layout, scales, zeros, group, bias, y,
                             ldy, M, N, K, scratch, kStaticScratchBytes, kernel, stream);
}

}  // extern "C"
