// The C ABI of libb200q: argument validation, kernel selection, bookkeeping.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "internal.cuh"

namespace b200q {

static std::atomic<uint64_t> g_launches{0};
static thread_local char g_last_error[256] = "";

void set_last_error_text(const char* text) {
  std::snprintf(g_last_error, sizeof(g_last_error), "%s", text);
}
void set_last_error(const char* what, cudaError_t e) {
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
}

int note_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("kernel launch", e);
    return B200Q_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200Q_OK;
}

// The tensor-core kernel serves every M it supports: even at M = 1 the dequantisation, not the
// multiply, is what costs instructions, and handing the multiply-accumulate to the (otherwise
// idle) tensor cores leaves the CUDA cores half the work of the all-CUDA-core kernel.  The
// CUDA-core split-K kernel remains for geometries the tensor-core kernel does not take (group
// sizes other than 128, K not a multiple of 64), on request (B200Q_KERNEL_SIMT), and for a
// single int8 row, where there is hardly any unpacking and it measured faster.
constexpr int kSimtMaxRowsW4 = 0;
constexpr int kSimtMaxRowsW8 = 1;

static int run_forward(ForwardArgs& a, int kernel_and_flags) {
  a.static_weights = (kernel_and_flags & B200Q_FLAG_STATIC_WEIGHTS) != 0;
  const int kernel = kernel_and_flags & 0xFF;
  if (a.argmax) {
    // the row-wise argmax epilogue exists in the tensor-core kernel (A operand in tensor
    // memory) only, and not together with the gated pairs
    if (a.swiglu || (kernel != B200Q_KERNEL_AUTO && kernel != B200Q_KERNEL_TC)) return B200Q_ERR_UNSUPPORTED;
    return launch_forward_tc(a);
  }
  if (a.swiglu) {
    // the gated-pair epilogue exists in the tensor-core kernel only
    if (kernel != B200Q_KERNEL_AUTO && kernel != B200Q_KERNEL_TC && kernel != B200Q_KERNEL_STREAMK)
      return B200Q_ERR_UNSUPPORTED;
    a.force_streamk = kernel == B200Q_KERNEL_STREAMK;
    return launch_forward_tc(a);
  }
  if (kernel == B200Q_KERNEL_SIMT) return launch_forward_simt(a);
  if (kernel == B200Q_KERNEL_TC) return launch_forward_tc(a);
  if (kernel == B200Q_KERNEL_STREAMK) {
    a.force_streamk = true;
    return launch_forward_tc(a);
  }
  if (kernel != B200Q_KERNEL_AUTO) return B200Q_ERR_INVALID;
  const int simt_rows = a.format == FMT_W8 ? kSimtMaxRowsW8 : kSimtMaxRowsW4;
  if (a.M <= simt_rows || !tc_supported(a)) return launch_forward_simt(a);
  return launch_forward_tc(a);
}

// Two ways to deliver a column-parallel forward's output to the peers.  The epilogue form (every
// block of the forward stores its tile into every rank's buffer) hides the peer stores behind
// other blocks' compute, but a single SM sustains only a few GB/s of them: with few, large tiles
// the stores of (world - 1) x tile bytes per block dominate.  The push form (a plain forward into
// this rank's own buffer — every kernel and routing rule available — then a kernel that copies
// the slab to the peers from hundreds of blocks) costs about 6 us more in fixed latency.
// Measured on 2 and 4 GPUs (B200, NVLink): push wins at M = 256..512 with N_local <= 3072
// (28 against 34 us, 34 against 41 us) and for the single-row int8 GEMV, the epilogue everywhere
// else.  B200Q_FLAG_GATHER_EPILOGUE / B200Q_FLAG_GATHER_PUSH force one form.
static bool push_preferred(int format, int M, int n_local, int K, int world, int flags) {
  if (world < 2 || n_local % 8) return false;                   // the push moves whole 16-byte chunks
  if (flags & B200Q_FLAG_GATHER_EPILOGUE) return false;
  if (flags & B200Q_FLAG_GATHER_PUSH) return true;
  if (format == FMT_W8 && M <= kSimtMaxRowsW8) return true;      // the CUDA-core kernel has no gather epilogue
  const int tiles = tc_output_tiles(format, M, n_local, K);
  const long long per_block = static_cast<long long>(tc_tile_bytes(format, M, n_local, K)) * (world - 1);
  return tiles > 0 && tiles <= 32 && per_block >= 96 * 1024;
}

static bool gather_by_push(const ForwardArgs& a, const b200q_gather* g, int flags) {
  if (a.ldy % 8) return false;
  for (int r = 0; r < g->world; ++r)
    if (reinterpret_cast<uintptr_t>(g->y_peer[r]) % 16) return false;
  return push_preferred(a.format, a.M, a.N, a.K, g->world, flags);
}

static int forward_then_push(ForwardArgs& a, const b200q_gather* g, int tiles, int flags) {
  if (tiles <= 0) return B200Q_ERR_UNSUPPORTED;
  a.gather = nullptr;
  a.announce = g;
  a.y = static_cast<unsigned char*>(g->y_peer[g->rank]) + static_cast<size_t>(g->rank) * a.N * 2;
  if (int st = run_forward(a, B200Q_KERNEL_AUTO | (flags & B200Q_FLAG_STATIC_WEIGHTS))) return st;
  return launch_gather_push(g, a.ldy, a.M, a.N, tiles, a.stream);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_version(void) { return 100; }

const char* b200q_status_string(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_INVALID: return "invalid argument";
    case B200Q_ERR_UNSUPPORTED: return "unsupported geometry for this kernel";
    case B200Q_ERR_ALIGNMENT: return "pointer or leading dimension is not 16-byte aligned";
    case B200Q_ERR_WORKSPACE: return "workspace missing or too small";
    case B200Q_ERR_CUDA: return "CUDA call failed";
    case B200Q_ERR_DEVICE_WAIT: return "a bounded device-side wait expired";
    default: return "unknown status";
  }
}

uint64_t b200q_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* b200q_last_error(void) { return g_last_error; }

int b200q_quantize_w8_per_channel(const void* w, int w_dtype, int64_t ldw, int N, int K, int mode,
                                  int8_t* q, void* scales, void* stream) {
  if (!w || !q || !scales || N < 0 || K <= 0 || ldw < K) return B200Q_ERR_INVALID;
  if (mode != B200Q_W8_SCALE_F16 && mode != B200Q_W8_SCALE_F32) return B200Q_ERR_INVALID;
  if (N == 0) return B200Q_OK;
  return launch_quantize_w8(w, w_dtype, ldw, N, K, mode, q, scales, static_cast<cudaStream_t>(stream));
}

int b200q_quantize_rows_int8(const void* x, int64_t ldx, int act_dtype, int M, int K, int8_t* q, int64_t ldq,
                             float* scales, void* stream) {
  if (!x || !q || !scales || M < 0 || K <= 0 || ldx < K || ldq < K) return B200Q_ERR_INVALID;
  if (M == 0) return B200Q_OK;
  return launch_quantize_rows_int8(x, ldx, act_dtype, M, K, q, ldq, scales, static_cast<cudaStream_t>(stream));
}

int b200q_w8a8_forward(const int8_t* qx, int64_t ldq, const float* act_scales, const int8_t* qweight, int64_t ldw,
                       const void* weight_scales, int weight_scale_dtype, void* y, int64_t ldy, int out_dtype, int M,
                       int N, int K, void* workspace, size_t workspace_bytes, void* stream) {
  if (!qx || !act_scales || !qweight || !weight_scales || !y) return B200Q_ERR_INVALID;
  if (M < 0 || N < 0 || K <= 0 || ldq < K || ldw < K || ldy < N) return B200Q_ERR_INVALID;
  if (weight_scale_dtype != B200Q_F16 && weight_scale_dtype != B200Q_F32) return B200Q_ERR_INVALID;
  if (out_dtype != B200Q_F16 && out_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (workspace != nullptr && workspace_bytes < 256) return B200Q_ERR_WORKSPACE;
  if (M == 0 || N == 0) return B200Q_OK;
  return launch_forward_w8a8(qx, ldq, act_scales, qweight, ldw, weight_scales, weight_scale_dtype, y, ldy, out_dtype,
                             M, N, K, static_cast<unsigned*>(workspace), static_cast<cudaStream_t>(stream));
}

int b200q_quantize_w4_grouped(const void* w, int w_dtype, int64_t ldw, int N, int K, int group,
                              int layout, void* packed, void* scales, void* zeros, void* stream) {
  if (!w || !packed || !scales || N < 0 || K <= 0 || ldw < K) return B200Q_ERR_INVALID;
  if (group <= 0 || (group & 1) || K % group) return B200Q_ERR_INVALID;
  if (layout == B200Q_W4_REF_SPLIT_HALF_SYM) {
    if (zeros) return B200Q_ERR_INVALID;
  } else if (layout == B200Q_W4_ASYM_ZP_INT32) {
    if (!zeros || group % 8) return B200Q_ERR_INVALID;
  } else {
    return B200Q_ERR_INVALID;
  }
  if (N == 0) return B200Q_OK;
  return launch_quantize_w4(w, w_dtype, ldw, N, K, group, layout, packed, scales, zeros,
                            static_cast<cudaStream_t>(stream));
}

int b200q_w4_dequant(const void* packed, const void* scales, const void* zeros, int layout, int N,
                     int K, int group, void* out, int64_t ldo, void* stream) {
  if (!packed || !scales || !out || N < 0 || K <= 0 || ldo < K) return B200Q_ERR_INVALID;
  if (group <= 0 || (group & 1) || K % group) return B200Q_ERR_INVALID;
  if (layout == B200Q_W4_ASYM_ZP_INT32 && !zeros) return B200Q_ERR_INVALID;
  if (layout != B200Q_W4_ASYM_ZP_INT32 && layout != B200Q_W4_REF_SPLIT_HALF_SYM)
    return B200Q_ERR_INVALID;
  if (N == 0) return B200Q_OK;
  return launch_dequant_w4(packed, scales, zeros, layout, N, K, group, out, ldo,
                           static_cast<cudaStream_t>(stream));
}

size_t b200q_workspace_bytes(int format, int M, int N, int K) {
  if (format != 8 && format != 4) return 0;
  return tc_workspace_bytes(format == 8 ? FMT_W8 : FMT_W4_REF, M, N, K);
}

int b200q_describe_plan(int format, int layout, int M, int N, int K, int group, char* text, size_t size) {
  if (!text || size == 0) return B200Q_ERR_INVALID;
  if (format != 8 && format != 4) return B200Q_ERR_INVALID;
  const int fmt = format == 8 ? FMT_W8 : (layout == B200Q_W4_ASYM_ZP_INT32 ? FMT_W4_ASYM : FMT_W4_REF);
  const bool tc = format == 8 ? (K % 64 == 0) : (group == 128 && K % 128 == 0);
  if (!tc || M <= (format == 8 ? kSimtMaxRowsW8 : kSimtMaxRowsW4)) {
    std::snprintf(text, size, "wq_gemv_simt_kernel<%s>", format == 8 ? "w8" : "w4");
    return B200Q_OK;
  }
  tc_describe_plan(fmt, M, N, K, text, size);
  return B200Q_OK;
}

int b200q_workspace_status(const void* workspace, void* stream) {
  if (!workspace) return B200Q_ERR_INVALID;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    set_last_error("b200q_workspace_status", e);
    return B200Q_ERR_CUDA;
  }
  return word == 0 ? B200Q_OK : B200Q_ERR_DEVICE_WAIT;
}

int b200q_w8a16_forward(const void* x, int64_t ldx, int act_dtype, const int8_t* qweight,
                        int64_t ldw, const void* scales, int scale_dtype, const void* bias,
                        void* y, int64_t ldy, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, int kernel, void* stream) {
  if (M < 0 || N < 0 || K <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N == 0) return B200Q_OK;
  if (!x || !qweight || !scales || !y) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (scale_dtype != B200Q_F16 && scale_dtype != B200Q_F32) return B200Q_ERR_INVALID;
  const bool swiglu = (kernel & B200Q_FLAG_SWIGLU_PAIRS) != 0;
  if (swiglu && (N & 1)) return B200Q_ERR_INVALID;
  const bool argmax = (kernel & B200Q_FLAG_ARGMAX) != 0;
  if (ldx < K || ldw < K || (!argmax && ldy < (swiglu ? N / 2 : N))) return B200Q_ERR_INVALID;
  if (argmax && reinterpret_cast<uintptr_t>(y) % 8) return B200Q_ERR_ALIGNMENT;
  if (K % 16) return B200Q_ERR_UNSUPPORTED;
  ForwardArgs a{};
  a.swiglu = swiglu;
  a.argmax = argmax;
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = qweight; a.ldw = ldw; a.format = FMT_W8;
  a.scales = scales; a.scale_dtype = scale_dtype; a.zeros = nullptr; a.group = 0;
  a.bias = bias; a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_forward(a, kernel);
}

int b200q_w4a16_forward(const void* x, int64_t ldx, int act_dtype, const void* packed, int64_t ldw,
                        int layout, const void* scales, const void* zeros, int group,
                        const void* bias, void* y, int64_t ldy, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, int kernel, void* stream) {
  if (M < 0 || N < 0 || K <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N == 0) return B200Q_OK;
  if (!x || !packed || !scales || !y) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (layout == B200Q_W4_ASYM_ZP_INT32) {
    if (!zeros) return B200Q_ERR_INVALID;
  } else if (layout != B200Q_W4_REF_SPLIT_HALF_SYM) {
    return B200Q_ERR_INVALID;
  }
  if (group <= 0 || K % group) return B200Q_ERR_INVALID;
  if (group % 32) return B200Q_ERR_UNSUPPORTED;
  const bool swiglu = (kernel & B200Q_FLAG_SWIGLU_PAIRS) != 0;
  if (swiglu && (N & 1)) return B200Q_ERR_INVALID;
  const bool argmax = (kernel & B200Q_FLAG_ARGMAX) != 0;
  if (ldx < K || ldw < K / 2 || (!argmax && ldy < (swiglu ? N / 2 : N))) return B200Q_ERR_INVALID;
  if (argmax && reinterpret_cast<uintptr_t>(y) % 8) return B200Q_ERR_ALIGNMENT;
  ForwardArgs a{};
  a.swiglu = swiglu;
  a.argmax = argmax;
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = packed; a.ldw = ldw;
  a.format = layout == B200Q_W4_ASYM_ZP_INT32 ? FMT_W4_ASYM : FMT_W4_REF;
  a.scales = scales; a.scale_dtype = B200Q_F16; a.zeros = zeros; a.group = group;
  a.bias = bias; a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_forward(a, kernel);
}

static int check_gather(const b200q_gather* g, int64_t ldy, int n_local) {
  if (!g || g->world < 1 || g->world > 8 || g->rank < 0 || g->rank >= g->world) return B200Q_ERR_INVALID;
  if (ldy < static_cast<int64_t>(g->world) * n_local) return B200Q_ERR_INVALID;
  for (int r = 0; r < g->world; ++r) {
    if (!g->y_peer[r] || !g->signal_peer[r]) return B200Q_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(g->signal_peer[r]) % 8) return B200Q_ERR_ALIGNMENT;
  }
  return B200Q_OK;
}

int b200q_gather_tiles(int format, int M, int N_local, int K, int group) {
  if (format == 8) return (K % 64 == 0) ? tc_output_tiles(FMT_W8, M, N_local, K) : 0;
  if (format == 4) return (group == 128 && K % 128 == 0) ? tc_output_tiles(FMT_W4_REF, M, N_local, K) : 0;
  return 0;
}

int b200q_gather_form(int format, int M, int N_local, int K, int group, int world, int flags) {
  if (b200q_gather_tiles(format, M, N_local, K, group) <= 0 || world < 1 || world > 8) return -1;
  return push_preferred(format == 8 ? FMT_W8 : FMT_W4_REF, M, N_local, K, world, flags) ? 1 : 0;
}

int b200q_w4a16_forward_gather(const void* x, int64_t ldx, int act_dtype, const void* packed,
                               int64_t ldw, int layout, const void* scales, const void* zeros,
                               int group, const void* bias, const b200q_gather* gather, int64_t ldy,
                               int M, int N_local, int K, void* workspace, size_t workspace_bytes,
                               int flags, void* stream) {
  if (M < 0 || N_local < 0 || K <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N_local == 0) return B200Q_OK;
  if (!x || !packed || !scales) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (layout == B200Q_W4_ASYM_ZP_INT32) {
    if (!zeros) return B200Q_ERR_INVALID;
  } else if (layout != B200Q_W4_REF_SPLIT_HALF_SYM) {
    return B200Q_ERR_INVALID;
  }
  if (group <= 0 || K % group) return B200Q_ERR_INVALID;
  if (ldx < K || ldw < K / 2) return B200Q_ERR_INVALID;
  if (flags & (B200Q_FLAG_SWIGLU_PAIRS | B200Q_FLAG_ARGMAX)) return B200Q_ERR_INVALID;
  if (int st = check_gather(gather, ldy, N_local)) return st;
  ForwardArgs a{};
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = packed; a.ldw = ldw;
  a.format = layout == B200Q_W4_ASYM_ZP_INT32 ? FMT_W4_ASYM : FMT_W4_REF;
  a.scales = scales; a.scale_dtype = B200Q_F16; a.zeros = zeros; a.group = group;
  a.bias = bias; a.y = gather->y_peer[gather->rank]; a.ldy = ldy; a.M = M; a.N = N_local; a.K = K;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.gather = gather;
  a.static_weights = (flags & B200Q_FLAG_STATIC_WEIGHTS) != 0;
  a.stream = static_cast<cudaStream_t>(stream);
  if (gather_by_push(a, gather, flags))
    return forward_then_push(a, gather, b200q_gather_tiles(4, M, N_local, K, group), flags);
  return launch_forward_tc(a);
}

int b200q_w8a16_forward_gather(const void* x, int64_t ldx, int act_dtype, const int8_t* qweight,
                               int64_t ldw, const void* scales, int scale_dtype, const void* bias,
                               const b200q_gather* gather, int64_t ldy, int M, int N_local, int K,
                               void* workspace, size_t workspace_bytes, int flags, void* stream) {
  if (M < 0 || N_local < 0 || K <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N_local == 0) return B200Q_OK;
  if (!x || !qweight || !scales) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (scale_dtype != B200Q_F16 && scale_dtype != B200Q_F32) return B200Q_ERR_INVALID;
  if (ldx < K || ldw < K) return B200Q_ERR_INVALID;
  if (flags & (B200Q_FLAG_SWIGLU_PAIRS | B200Q_FLAG_ARGMAX)) return B200Q_ERR_INVALID;
  if (int st = check_gather(gather, ldy, N_local)) return st;
  ForwardArgs a{};
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = qweight; a.ldw = ldw; a.format = FMT_W8;
  a.scales = scales; a.scale_dtype = scale_dtype; a.zeros = nullptr; a.group = 0;
  a.bias = bias; a.y = gather->y_peer[gather->rank]; a.ldy = ldy; a.M = M; a.N = N_local; a.K = K;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.gather = gather;
  a.static_weights = (flags & B200Q_FLAG_STATIC_WEIGHTS) != 0;
  a.stream = static_cast<cudaStream_t>(stream);
  if (gather_by_push(a, gather, flags))
    return forward_then_push(a, gather, b200q_gather_tiles(8, M, N_local, K, 0), flags);
  return launch_forward_tc(a);
}

static int check_reduce(const b200q_reduce* r, int64_t ldy, int n) {
  if (!r || r->world < 1 || r->world > 8 || r->rank < 0 || r->rank >= r->world) return B200Q_ERR_INVALID;
  if (ldy < n || n % r->world || (n / r->world) % 128) return B200Q_ERR_INVALID;
  for (int i = 0; i < r->world; ++i) {
    if (!r->y_peer[i] || !r->signal_peer[i] || !r->inbox_peer[i]) return B200Q_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(r->signal_peer[i]) % 8 || reinterpret_cast<uintptr_t>(r->inbox_peer[i]) % 4)
      return B200Q_ERR_ALIGNMENT;
  }
  return B200Q_OK;
}

int b200q_reduce_tiles(int format, int M, int N, int K_local, int group, int world) {
  if (format == 8) return (K_local % 64 == 0) ? tc_reduce_tiles(FMT_W8, M, N, K_local, world) : 0;
  if (format == 4) return (group == 128 && K_local % 128 == 0) ? tc_reduce_tiles(FMT_W4_REF, M, N, K_local, world) : 0;
  return 0;
}

int b200q_w4a16_forward_reduce(const void* x, int64_t ldx, int act_dtype, const void* packed,
                               int64_t ldw, int layout, const void* scales, const void* zeros,
                               int group, const void* bias, const b200q_reduce* reduce, int64_t ldy,
                               int M, int N, int K_local, void* workspace, size_t workspace_bytes,
                               int flags, void* stream) {
  if (M < 0 || N < 0 || K_local <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N == 0) return B200Q_OK;
  if (!x || !packed || !scales) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (layout == B200Q_W4_ASYM_ZP_INT32) {
    if (!zeros) return B200Q_ERR_INVALID;
  } else if (layout != B200Q_W4_REF_SPLIT_HALF_SYM) {
    return B200Q_ERR_INVALID;
  }
  if (group <= 0 || K_local % group) return B200Q_ERR_INVALID;
  if (ldx < K_local || ldw < K_local / 2) return B200Q_ERR_INVALID;
  if (flags & (B200Q_FLAG_SWIGLU_PAIRS | B200Q_FLAG_ARGMAX)) return B200Q_ERR_INVALID;
  if (int st = check_reduce(reduce, ldy, N)) return st;
  if (b200q_reduce_tiles(4, M, N, K_local, group, reduce->world) == 0) return B200Q_ERR_UNSUPPORTED;
  ForwardArgs a{};
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = packed; a.ldw = ldw;
  a.format = layout == B200Q_W4_ASYM_ZP_INT32 ? FMT_W4_ASYM : FMT_W4_REF;
  a.scales = scales; a.scale_dtype = B200Q_F16; a.zeros = zeros; a.group = group;
  a.bias = bias; a.y = reduce->y_peer[reduce->rank]; a.ldy = ldy; a.M = M; a.N = N; a.K = K_local;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.reduce = reduce;
  a.static_weights = (flags & B200Q_FLAG_STATIC_WEIGHTS) != 0;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_forward_tc(a);
}

int b200q_w8a16_forward_reduce(const void* x, int64_t ldx, int act_dtype, const int8_t* qweight,
                               int64_t ldw, const void* scales, int scale_dtype, const void* bias,
                               const b200q_reduce* reduce, int64_t ldy, int M, int N, int K_local,
                               void* workspace, size_t workspace_bytes, int flags, void* stream) {
  if (M < 0 || N < 0 || K_local <= 0) return B200Q_ERR_INVALID;
  if (M == 0 || N == 0) return B200Q_OK;
  if (!x || !qweight || !scales) return B200Q_ERR_INVALID;
  if (act_dtype != B200Q_F16 && act_dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (scale_dtype != B200Q_F16 && scale_dtype != B200Q_F32) return B200Q_ERR_INVALID;
  if (ldx < K_local || ldw < K_local) return B200Q_ERR_INVALID;
  if (flags & (B200Q_FLAG_SWIGLU_PAIRS | B200Q_FLAG_ARGMAX)) return B200Q_ERR_INVALID;
  if (int st = check_reduce(reduce, ldy, N)) return st;
  if (b200q_reduce_tiles(8, M, N, K_local, 0, reduce->world) == 0) return B200Q_ERR_UNSUPPORTED;
  ForwardArgs a{};
  a.x = x; a.ldx = ldx; a.act_dtype = act_dtype;
  a.w = qweight; a.ldw = ldw; a.format = FMT_W8;
  a.scales = scales; a.scale_dtype = scale_dtype; a.zeros = nullptr; a.group = 0;
  a.bias = bias; a.y = reduce->y_peer[reduce->rank]; a.ldy = ldy; a.M = M; a.N = N; a.K = K_local;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.reduce = reduce;
  a.static_weights = (flags & B200Q_FLAG_STATIC_WEIGHTS) != 0;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_forward_tc(a);
}

int b200q_reduce_wait(const b200q_reduce* reduce, int tiles_per_rank, void* stream) {
  if (!reduce || reduce->world < 1 || reduce->world > 8 || tiles_per_rank <= 0) return B200Q_ERR_INVALID;
  if (reduce->rank < 0 || reduce->rank >= reduce->world || !reduce->signal_peer[reduce->rank])
    return B200Q_ERR_INVALID;
  b200q_gather g{};
  g.rank = reduce->rank;
  g.world = reduce->world;
  for (int i = 0; i < 8; ++i) g.signal_peer[i] = reduce->signal_peer[i];
  return launch_gather_wait(&g, static_cast<unsigned long long>(tiles_per_rank) * reduce->world,
                            static_cast<cudaStream_t>(stream));
}

int b200q_gather_wait(const b200q_gather* gather, int tiles_per_rank, void* stream) {
  if (!gather || gather->world < 1 || gather->world > 8 || tiles_per_rank <= 0) return B200Q_ERR_INVALID;
  if (gather->rank < 0 || gather->rank >= gather->world || !gather->signal_peer[gather->rank])
    return B200Q_ERR_INVALID;
  return launch_gather_wait(gather, static_cast<unsigned long long>(tiles_per_rank) * gather->world,
                            static_cast<cudaStream_t>(stream));
}

}  // extern "C"
