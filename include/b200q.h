/*
 * b200q — weight-only quantized linear forward for NVIDIA B200 (sm_100a).
 *
 * C ABI of libb200q.so.  Plain pointers and sizes only: every pointer is a
 * DEVICE pointer unless its comment says otherwise, `stream` is a
 * cudaStream_t passed as void*, and every function returns a b200q_status
 * (0 = ok).  Nothing here allocates device memory, synchronises the device
 * or reads results back to the host, so every call may be recorded into a
 * CUDA graph.
 *
 * Each entry point names the interface of the reference project
 * (Vaibhav7711/full-inference-engine, paths relative to its root) that a
 * binding would replace with it.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200q_status {
  B200Q_OK = 0,
  B200Q_ERR_INVALID = 1,      /* bad geometry, null pointer, unknown enum            */
  B200Q_ERR_UNSUPPORTED = 2,  /* legal request this build has no kernel for          */
  B200Q_ERR_ALIGNMENT = 3,    /* pointer or leading dimension not 16-byte aligned    */
  B200Q_ERR_WORKSPACE = 4,    /* workspace missing or smaller than workspace_bytes() */
  B200Q_ERR_CUDA = 5,         /* a CUDA runtime/driver call failed                   */
  B200Q_ERR_DEVICE_WAIT = 6   /* a bounded device-side wait expired (status word)    */
} b200q_status;

/* element types of activations, outputs, scales and quantizer inputs */
typedef enum b200q_dtype {
  B200Q_F16 = 0,
  B200Q_BF16 = 1,
  B200Q_F32 = 2
} b200q_dtype;

/* INT4 container layouts */
typedef enum b200q_w4_layout {
  /* The reference layout (engine/kernels/w4a16_format.py:32-50): symmetric
   * values in [-7,7] stored +8, two per uint8, split-half inside each group:
   * byte j of a group holds input j (low nibble) and input j+G/2 (high
   * nibble).  packed [N, K/2] uint8, scales [N, K/G] fp16, no zero-points. */
  B200Q_W4_REF_SPLIT_HALF_SYM = 0,
  /* Asymmetric 4-bit, eight nibbles per int32, fp16 scale and fp16 zero-point
   * per group.  Word w holds inputs 8w..8w+7; nibble position p (bits 4p..4p+3)
   * holds input 8w + {0,2,4,6,1,3,5,7}[p], i.e. input i sits at position
   * (i & 1) * 4 + (i >> 1): the two nibbles 16 bits apart are neighbours in K,
   * which is what a half2 unpack wants.
   * packed [N, K/8] int32, scales [N, K/G] fp16, zeros [N, K/G] fp16.
   * The reference has no such layout; its definition is this library's.    */
  B200Q_W4_ASYM_ZP_INT32 = 1
} b200q_w4_layout;

/* which kernel family a forward call may use */
typedef enum b200q_kernel {
  B200Q_KERNEL_AUTO = 0,  /* pick by M                                         */
  B200Q_KERNEL_SIMT = 1,  /* CUDA-core split-K GEMV (decode rows)              */
  B200Q_KERNEL_TC = 2,    /* tcgen05 tensor-core GEMM, weights on the M side:
                             AUTO's choice between its two variants             */
  B200Q_KERNEL_STREAMK = 3 /* the persistent stream-K variant of the tensor-core
                             kernel (M <= 64, K a multiple of 1024 for INT4);
                             B200Q_ERR_UNSUPPORTED for other geometries.  AUTO
                             takes it where it measured faster: INT4, M <= 16,
                             weight tiles shared by few blocks                  */
} b200q_kernel;

/* OR-ed into the `kernel` argument of a forward call.
 * STATIC_WEIGHTS: the weights, scales, zero-points and bias of this call were last
 * written before the PREVIOUS kernel of the stream was launched (module buffers
 * set at install time).  The kernel may then start streaming them while that
 * previous kernel is still draining (programmatic dependent launch); activations,
 * outputs and the workspace always stay in stream order.  Without the flag
 * everything stays in stream order.                                            */
#define B200Q_FLAG_STATIC_WEIGHTS 0x100
/* SWIGLU_PAIRS: the weight rows are (gate, up) pairs of a gated feed-forward, interleaved:
 * row 2c is gate channel c and row 2c+1 is up channel c (scales, zero-points and bias
 * interleaved the same way).  The call then writes N/2 columns,
 *   y[m, c] = silu(acc[m, 2c]) * acc[m, 2c+1]       (acc includes the scale and bias),
 * evaluated in fp32 and rounded once to the activation dtype; ldy >= N/2, N even.  It fuses
 * the reference's gate_proj + up_proj + silu(gate) * up (engine/kernels/swiglu.py:65-83,
 * 86-107: FusedGateUpProjection followed by triton_swiglu), which the reference can only
 * build from fp16 `.weight`s, not from quantized modules.  Tensor-core kernel only
 * (B200Q_ERR_UNSUPPORTED with B200Q_KERNEL_SIMT or an unsupported geometry); not accepted
 * by the *_forward_gather entry points.                                                   */
#define B200Q_FLAG_SWIGLU_PAIRS 0x200
/* ARGMAX: instead of the [M, N] outputs the call writes, for every row, the channel of its
 * largest output (greedy decoding over a quantized output head; the reference runs lm_head
 * and then torch.argmax over the [M, vocab] logits).  `y` points at M int64 values; `ldy` is
 * ignored.  Every output is rounded to the activation dtype exactly as the plain call would
 * store it before it is compared, and among equal values the smallest channel wins, so the
 * result equals argmax over the plain call's own output.  One launch: per-row keys live in a
 * region of the workspace that nothing else uses (zero before the first call, like the
 * counters) and the last block of the grid converts them and puts them back to zero.  At most
 * 8192 rows per call (B200Q_ERR_UNSUPPORTED beyond).  Tensor-core kernel only; not with
 * SWIGLU_PAIRS, not in the *_forward_gather entry points.                                   */
#define B200Q_FLAG_ARGMAX 0x400
/*
 * With the *_forward_gather entry points only: how the output reaches the peers.
 * EPILOGUE: from the forward kernel's epilogue (every block stores its tile into every rank's
 * buffer).  PUSH: a plain forward into this rank's own buffer, then a push kernel that copies
 * the rank's columns to the peers from as many blocks as the slab is worth.  Neither flag: the
 * library picks by geometry (few large tiles and single-row int8 calls are pushed).  Both forms
 * count the same b200q_gather_tiles() arrivals and are followed by b200q_gather_wait; every
 * rank must pass the same flags for a call.
 */
#define B200Q_FLAG_GATHER_EPILOGUE 0x800
#define B200Q_FLAG_GATHER_PUSH 0x1000

/* W8 quantizer flavours */
typedef enum b200q_w8_mode {
  /* engine/kernels/w8a16_linear.py:43-47: scale = fp16(max|w|.clamp_min(1e-8)/127),
   * q = round(w / float(scale_fp16)); scales written as fp16.                */
  B200Q_W8_SCALE_F16 = 0,
  /* engine/quantization/int8.py:19-20: scale = max|w|.clamp_min(FLT_EPSILON)/127
   * kept fp32, q = round(w / scale); scales written as fp32.                 */
  B200Q_W8_SCALE_F32 = 1
} b200q_w8_mode;

/* Library identification and diagnostics (host-only, no reference counterpart). */
int b200q_version(void);
const char* b200q_status_string(int status);
/* Kernels this library has launched since load (all devices, all streams). */
uint64_t b200q_launch_count(void);
/* Last CUDA error text seen by a failing call on this thread ("" if none). */
const char* b200q_last_error(void);

/*
 * Quantize [N,K] weights per output channel to int8 + one scale per row.
 * Replaces quantize_weight_per_channel (engine/kernels/w8a16_linear.py:43-47)
 * and the constructor arithmetic of Int8Linear (engine/quantization/int8.py:16-21).
 *   w        [N, ldw] of w_dtype (f16/bf16/f32), row-major
 *   q        [N, K] int8, contiguous
 *   scales   [N] fp16 (mode SCALE_F16) or fp32 (mode SCALE_F32)
 * A row whose scale rounds to zero (all-zero row in SCALE_F16 mode) gets q = 0.
 */
int b200q_quantize_w8_per_channel(const void* w, int w_dtype, int64_t ldw,
                                  int N, int K, int mode,
                                  int8_t* q, void* scales, void* stream);

/*
 * W8A8 linear (engine/kernels/w8a8_linear.py:35-50), in two calls so that the quantised
 * activations can be reused by every projection that reads the same input.
 *
 * b200q_quantize_rows_int8 is the reference's per-row dynamic quantisation (lines 43-45):
 *   scales[m] = max_k |float(x[m,k])| clamp_min 1e-8, / 127      (fp32, IEEE division)
 *   q[m,k]    = clamp(rint(float(x[m,k]) / scales[m]), -127, 127)
 *     x       [M, ldx] of act_dtype (f16 / bf16 / f32)
 *     q       [M, ldq] int8; for b200q_w8a8_forward q must be 16-byte aligned with ldq % 16 == 0
 *     scales  [M] fp32
 *
 * b200q_w8a8_forward replaces torch._int_mm and the scaling of lines 46-48:
 *   y[m,n] = out_dtype( (float(sum_k qx[m,k] * qweight[n,k]) * act_scales[m]) * float(weight_scales[n]) )
 * with the sum exact in int32 (tcgen05.mma kind::i8).
 *     qweight        [N, ldw] int8 row-major (the [N,K] matrix quantize_weight_per_channel
 *                    returns, NOT the transposed copy pack_w8a8_weight makes for cuBLAS),
 *                    16-byte aligned, ldw % 16 == 0
 *     weight_scales  [N] f16 or f32
 *     y              [M, ldy] f16 or bf16
 *     workspace      optional: when non-null (>= 256 bytes) an expired device-side wait is
 *                    recorded in its status word; no other scratch is used
 * K must be a multiple of 16 (B200Q_ERR_UNSUPPORTED otherwise); any M and N.
 */
int b200q_quantize_rows_int8(const void* x, int64_t ldx, int act_dtype, int M, int K,
                             int8_t* q, int64_t ldq, float* scales, void* stream);
int b200q_w8a8_forward(const int8_t* qx, int64_t ldq, const float* act_scales,
                       const int8_t* qweight, int64_t ldw,
                       const void* weight_scales, int weight_scale_dtype,
                       void* y, int64_t ldy, int out_dtype, int M, int N, int K,
                       void* workspace, size_t workspace_bytes, void* stream);

/*
 * Quantize [N,K] weights to 4 bits in groups of `group` along K and pack.
 * REF layout replaces quantize_weight_w4_grouped
 * (engine/kernels/w4a16_format.py:32-50) bit for bit; `zeros` must be NULL.
 * ASYM layout: per group lo=min(min w,0), hi=max(max w,0),
 * s=max((hi-lo)/15,1e-8), zp=clamp(rint(-lo/s),0,15), q=clamp(rint(w/s)+zp,0,15),
 * scale=fp16(s), zero=fp16(zp).
 * Requires group even and K % group == 0 (ASYM: group % 8 == 0).
 */
int b200q_quantize_w4_grouped(const void* w, int w_dtype, int64_t ldw,
                              int N, int K, int group, int layout,
                              void* packed, void* scales, void* zeros,
                              void* stream);

/*
 * Dequantize packed 4-bit weights into a caller-owned [N, ldo] fp16 matrix:
 * out[n,k] = fp16(nibble - zp) * fp16(scale), the product taken in fp16
 * (one rounding).  Replaces w4_dequantize_into
 * (engine/kernels/w4a16_linear.py:245-274) and is bit-identical to
 * unpack_w4_reference (engine/kernels/w4a16_format.py:53-69) for the REF layout.
 */
int b200q_w4_dequant(const void* packed, const void* scales, const void* zeros,
                     int layout, int N, int K, int group,
                     void* out, int64_t ldo, void* stream);

/*
 * Bytes of workspace a forward call of this geometry may use (0 = none).
 * `format`: 8 for W8A16, 4 for either INT4 layout.  Layout: [0, 256) a status
 * word, [256, 64 KiB) tile counters, [64 KiB, 128 KiB) the row keys of the fused
 * argmax, [128 KiB, 128 KiB + 5 MiB) the partial exchange of the decode kernel,
 * then fp32 split-K partial sums.  The workspace must be zero-filled once when it
 * is allocated; every call leaves status, counters, keys and the exchange region
 * at zero again, and the split-K partials are always written before they are
 * read, so graph replays need no memset and calls of any kind may follow one
 * another on the same workspace.
 * Calls that may overlap on the GPU (different streams) need a workspace each:
 * counters, partials and keys of two running kernels must not share memory.
 * A call with B200Q_FLAG_ARGMAX needs only the first 128 KiB.
 */
size_t b200q_workspace_bytes(int format, int M, int N, int K);

/*
 * One line of text naming the kernel instantiation and tiling that a plain forward of
 * this geometry takes on the current device with B200Q_KERNEL_AUTO ("wq_gemm_sk_kernel<w4_asym>
 * tok=16 ...").  Host-only diagnostic, no reference counterpart; `layout` and `group` are
 * ignored for format 8.
 */
int b200q_describe_plan(int format, int layout, int M, int N, int K, int group,
                        char* text, size_t size);

/*
 * Wait for `stream`, then read the status word a forward call keeps at the
 * start of its workspace: B200Q_OK, or B200Q_ERR_DEVICE_WAIT if a kernel gave
 * up on one of its bounded waits (its output is then undefined).  This call
 * synchronises and copies four bytes to the host: for tests and diagnostics,
 * never inside a graph capture.  No reference counterpart.
 */
int b200q_workspace_status(const void* workspace, void* stream);

/*
 * y[M,N] = x[M,K] . (q[N,K] * scales[N])^T (+ bias), fp32 accumulation,
 * y in the activation dtype.  Replaces w8a16_linear
 * (engine/kernels/w8a16_linear.py:50-69) and the arithmetic of
 * Int8Linear.forward (engine/quantization/int8.py:30-33).
 *   x       [M, ldx]  act_dtype (f16 or bf16)
 *   qweight [N, ldw]  int8      (ldw % 16 == 0, K % 16 == 0)
 *   scales  [N]       scale_dtype (f16 or f32)
 *   bias    [N]       act_dtype, or NULL
 *   y       [M, ldy]  act_dtype
 *   workspace/workspace_bytes: see b200q_workspace_bytes; may be NULL when 0.
 */
int b200q_w8a16_forward(const void* x, int64_t ldx, int act_dtype,
                        const int8_t* qweight, int64_t ldw,
                        const void* scales, int scale_dtype,
                        const void* bias,
                        void* y, int64_t ldy,
                        int M, int N, int K,
                        void* workspace, size_t workspace_bytes,
                        int kernel, void* stream);

/*
 * y[M,N] = x[M,K] . dequant(packed, scales, zeros)^T (+ bias), fp32
 * accumulation.  Replaces w4a16_linear / w4a16_gemv
 * (engine/kernels/w4a16_linear.py:77-117, 180-209) and the CUDA branches of
 * W4A16Linear.forward (engine/quantization/w4a16.py:132-178).
 *   packed  REF: [N, ldw] uint8 with ldw >= K/2 bytes;
 *           ASYM: [N, ldw/4] int32 — ldw is always in BYTES (ldw % 16 == 0)
 *   scales  [N, K/group] fp16 contiguous; zeros likewise (ASYM) or NULL (REF)
 *   group   multiple of 32 dividing K
 */
int b200q_w4a16_forward(const void* x, int64_t ldx, int act_dtype,
                        const void* packed, int64_t ldw, int layout,
                        const void* scales, const void* zeros, int group,
                        const void* bias,
                        void* y, int64_t ldy,
                        int M, int N, int K,
                        void* workspace, size_t workspace_bytes,
                        int kernel, void* stream);

/*
 * Fused column-parallel forward + all-gather (no reference counterpart: the reference
 * is single-GPU).  Rank `rank` of `world` (<= 8) holds N_local = N/world output rows
 * of the weights; instead of writing y[M, N_local] and calling a collective, the
 * kernel's epilogue stores every finished tile into the full [M, ldy] output of
 * EVERY rank at columns [rank*N_local, (rank+1)*N_local) through peer-mapped
 * pointers (plain stores over NVLink; no multicast loads anywhere).
 *   y_peer[r]       peer-mapped base of rank r's full output buffer (same shape on all ranks)
 *   signal_peer[r]  peer-mapped base of rank r's signal block: >= 256 bytes, 8-byte
 *                   aligned, zero-filled once when the buffer is created, never
 *                   touched by the host afterwards
 * Protocol per call: the rank announces "entered the call" to all ranks, waits (bounded)
 * for the same announcement from a rank before its first store into that rank's buffer,
 * and counts its b200q_gather_tiles() delivered tiles on every rank (signal word 3 of a
 * rank's own block counts the finished blocks of its push kernel and is zero between calls).
 * b200q_gather_wait, enqueued after the forward on the same stream, waits (bounded)
 * until all world * b200q_gather_tiles() tiles have arrived, which makes the full
 * output safe to read by later work in the stream.  Every rank must make the same
 * sequence of calls on a given buffer.  A bounded wait that expires sets the status
 * word of the signal block (64-bit word 2) instead of hanging.
 * The tensor-core kernel serves these calls: geometries it does not take
 * (b200q_gather_tiles() == 0) must use a separate collective.
 */
typedef struct b200q_gather {
  int rank;
  int world;
  void* y_peer[8];
  void* signal_peer[8];
} b200q_gather;

/* Output tiles one rank's forward of this geometry delivers (0: not supported fused). */
int b200q_gather_tiles(int format, int M, int N_local, int K, int group);

/* Which form such a call takes for 16-byte aligned buffers: 0 the forward's epilogue, 1 the push
 * kernel, -1 not supported.  A function of the geometry, the world size and the GATHER flags
 * only, so every rank answers alike. */
int b200q_gather_form(int format, int M, int N_local, int K, int group, int world, int flags);

int b200q_w4a16_forward_gather(const void* x, int64_t ldx, int act_dtype,
                               const void* packed, int64_t ldw, int layout,
                               const void* scales, const void* zeros, int group,
                               const void* bias,
                               const b200q_gather* gather, int64_t ldy,
                               int M, int N_local, int K,
                               void* workspace, size_t workspace_bytes,
                               int flags, void* stream);

int b200q_w8a16_forward_gather(const void* x, int64_t ldx, int act_dtype,
                               const int8_t* qweight, int64_t ldw,
                               const void* scales, int scale_dtype,
                               const void* bias,
                               const b200q_gather* gather, int64_t ldy,
                               int M, int N_local, int K,
                               void* workspace, size_t workspace_bytes,
                               int flags, void* stream);

int b200q_gather_wait(const b200q_gather* gather, int tiles_per_rank, void* stream);

/*
 * Fused row-parallel forward + all-reduce (no reference counterpart: the reference is
 * single-GPU).  The pairing of the column-parallel forward above: rank `rank` of `world`
 * holds the K_local = K/world INPUT columns [rank*K_local, (rank+1)*K_local) of the
 * weights (all N rows; for INT4 whole groups, with their scales) and the matching slice
 * of the activations, which is exactly what a column-parallel gate/up or q/k/v projection
 * leaves on it, so a feed-forward needs ONE exchange instead of a gather per layer.
 * Each rank computes a partial [M, N]; the rank that owns a block of N/world output
 * columns receives the other ranks' partials of those columns in its inbox (peer stores of
 * self-validating fp32 words: no flag, no collective), adds them in rank order (a fixed
 * order: results are reproducible), adds the bias, rounds once and stores the finished
 * tile into the [M, ldy] output of EVERY rank.
 *   y_peer[r]       peer-mapped base of rank r's full output buffer
 *   signal_peer[r]  as for b200q_gather (>= 256 bytes, zero-filled once)
 *   inbox_peer[r]   peer-mapped base of rank r's inbox: world * M * (N/world) 32-bit
 *                   words, zero-filled once when created; every call leaves it zero
 * Enqueue b200q_reduce_wait after the forward (same stream) before anything reads y.
 * Every rank makes the same sequence of calls.  N % world == 0 and (N/world) % 128 == 0;
 * b200q_reduce_tiles() == 0 means the geometry must use a separate collective.  Bias is
 * added once, by the owner.  Not with SWIGLU_PAIRS or ARGMAX.
 */
typedef struct b200q_reduce {
  int rank;
  int world;
  void* y_peer[8];
  void* signal_peer[8];
  void* inbox_peer[8];
} b200q_reduce;

/* Output tiles one rank owns in such a call (0: not supported fused). */
int b200q_reduce_tiles(int format, int M, int N, int K_local, int group, int world);

int b200q_w4a16_forward_reduce(const void* x, int64_t ldx, int act_dtype,
                               const void* packed, int64_t ldw, int layout,
                               const void* scales, const void* zeros, int group,
                               const void* bias,
                               const b200q_reduce* reduce, int64_t ldy,
                               int M, int N, int K_local,
                               void* workspace, size_t workspace_bytes,
                               int flags, void* stream);

int b200q_w8a16_forward_reduce(const void* x, int64_t ldx, int act_dtype,
                               const int8_t* qweight, int64_t ldw,
                               const void* scales, int scale_dtype,
                               const void* bias,
                               const b200q_reduce* reduce, int64_t ldy,
                               int M, int N, int K_local,
                               void* workspace, size_t workspace_bytes,
                               int flags, void* stream);

int b200q_reduce_wait(const b200q_reduce* reduce, int tiles_per_rank, void* stream);

/*
 * The INT4 forward for callers that have no device memory to give: same
 * arguments and results as b200q_w4a16_forward, minus the workspace.  It has no
 * counterpart in the reference.  It exists for hosts that cannot allocate on the
 * GPU at the point of the call: an engine that has already handed all free HBM
 * to its KV-cache pool, or a binding whose runtime passes it nothing but input
 * and output pointers and forbids cudaMalloc (which would stall the device
 * mid-serving).  The split-K scratch is a fixed array inside the library image
 * (b200q_static_scratch_bytes(), 16 MiB, resident on every GPU that loads the
 * library until the process exits); nothing is allocated, by this call or by
 * anything it calls.
 *
 *  - Geometries whose b200q_workspace_bytes() exceeds the array are refused with
 *    B200Q_ERR_WORKSPACE (b200q_last_error() names both sizes).
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress): make that first call before starting any stream
 *    capture on that device.  Nothing is cleared: the array is zero when the library
 *    image is loaded and the kernels return its counters to zero themselves.
 *  - All calls on a device share the one array and it keeps what the last call
 *    left in it (the kernels return its counters to zero themselves).  Calls that
 *    overlap on the GPU — different streams, or b200q_w4a16_forward given this same
 *    memory — race on it: keep them in one stream order.
 */
size_t b200q_static_scratch_bytes(void);
int b200q_w4a16_forward_static_scratch(const void* x, int64_t ldx, int act_dtype,
                                       const void* packed, int64_t ldw, int layout,
                                       const void* scales, const void* zeros, int group,
                                       const void* bias,
                                       void* y, int64_t ldy,
                                       int M, int N, int K,
                                       int kernel, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
