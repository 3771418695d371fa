// Declarations shared by the translation units of libb200q.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200q.h"
#include "convert.cuh"

namespace b200q {

enum Format { FMT_W8 = 0, FMT_W4_REF = 1, FMT_W4_ASYM = 2 };

// Everything a forward kernel needs, format-agnostic.
struct ForwardArgs {
  const void* x;        // [M, ldx] activations (f16 / bf16)
  int64_t ldx;          // elements
  int act_dtype;        // B200Q_F16 / B200Q_BF16
  const void* w;        // packed weights
  int64_t ldw;          // BYTES per weight row
  int format;           // Format
  const void* scales;   // W8: [N] f16|f32; W4: [N, K/group] f16
  int scale_dtype;      // W8 only
  const void* zeros;    // W4 ASYM: [N, K/group] f16
  int group;            // W4 only
  const void* bias;     // [N] act dtype or null
  void* y;              // [M, ldy]
  int64_t ldy;          // elements
  int M, N, K;
  void* workspace;
  size_t workspace_bytes;
  bool static_weights;  // weights/scales/zeros/bias were written long before this call
  bool swiglu;          // rows are interleaved (gate, up) pairs; y has N/2 columns of silu(gate) * up
  bool argmax;          // y is u64 keys[M], zeroed by the caller: row-wise maximum and its channel
  bool force_streamk;   // B200Q_KERNEL_STREAMK: the persistent stream-K variant or nothing
  const b200q_gather* gather;  // fused all-gather destinations, or null
  const b200q_reduce* reduce;  // fused all-reduce of a row-parallel forward, or null
  const b200q_gather* announce;  // a push kernel follows: announce the call to these peers early, or null
  cudaStream_t stream;
};

// Records a launch (and any launch error) — returns a b200q_status.
int note_launch();
void set_last_error(const char* what, cudaError_t e);
void set_last_error_text(const char* text);

// quantize.cu
int launch_quantize_w8(const void* w, int w_dtype, int64_t ldw, int N, int K, int mode, int8_t* q,
                       void* scales, cudaStream_t stream);
int launch_quantize_w4(const void* w, int w_dtype, int64_t ldw, int N, int K, int group,
                       int layout, void* packed, void* scales, void* zeros, cudaStream_t stream);
int launch_dequant_w4(const void* packed, const void* scales, const void* zeros, int layout,
                      int N, int K, int group, void* out, int64_t ldo, cudaStream_t stream);

// gemv_simt.cu — CUDA-core path, any M (rows are processed four at a time).
int launch_forward_simt(const ForwardArgs& a);

// gemm_tc.cu — tcgen05 path.
bool tc_supported(const ForwardArgs& a);
size_t tc_workspace_bytes(int format, int M, int N, int K);
int launch_forward_tc(const ForwardArgs& a);
int tc_output_tiles(int format, int M, int N, int K);
int tc_tile_bytes(int format, int M, int N, int K);
int tc_reduce_tiles(int format, int M, int N, int K_local, int world);
void tc_describe_plan(int format, int M, int N, int K, char* text, size_t size);
int launch_gather_wait(const b200q_gather* g, unsigned long long expected, cudaStream_t stream);
int launch_gather_push(const b200q_gather* g, int64_t ldy, int M, int n_local, int tiles, cudaStream_t stream);

// gemm_i8.cu — W8A8: per-row activation quantisation and the int8 x int8 tensor-core GEMM.
int launch_quantize_rows_int8(const void* x, int64_t ldx, int act_dtype, int M, int K, int8_t* q, int64_t ldq,
                              float* scales, cudaStream_t stream);
int launch_forward_w8a8(const int8_t* qx, int64_t ldq, const float* a_scales, const int8_t* qw, int64_t ldw,
                        const void* w_scales, int w_scale_dtype, void* y, int64_t ldy, int out_dtype, int M, int N,
                        int K, unsigned* status, cudaStream_t stream);

}  // namespace b200q
