// Pieces shared by the two tcgen05 kernels (gemm_tc.cu: one block per output tile, every
// M; gemm_sk.cu: persistent stream-K blocks for decode-sized M): tile constants, bounded
// waits, register-level dequantisation into the fp16 MMA operand, epilogue conversions,
// the workspace layout and the host-side tensor-map cache.
//
// Dequantised INT4 weights are computed as the reference computes them: exact (nibble - zero)
// and ONE fp16 multiply by the fp16 scale (unpack_w4_reference,
// engine/kernels/w4a16_format.py:53-69).  For fp16 activations that fp16 value is the MMA
// operand; for bf16 activations it is converted once to bf16, which is exactly the
// reference's `.to(rows.dtype)` (engine/quantization/w4a16.py:168).  (kind::f16 wants both
// operands in one format: an fp16 A against a bf16 B is an illegal instruction on sm_100a.)
// int8 weights are exact in either format.
#pragma once
#include <type_traits>

#include "internal.cuh"
#include "ptx.cuh"

namespace b200q {

constexpr int kBlockN = 128;                 // output channels per tile (UMMA M)
constexpr int kBlockK = 128;                 // K elements per pipeline step

// Workspace layout (fixed, so that calls of different geometry or kernel never see one
// another's leftovers as counters, keys or partials):
//   [0, 256)                 status word
//   [256, 64 KiB)            split-K tile counters of the tile kernel, zero between launches
//   [64 KiB, 128 KiB)        row keys of the fused argmax (8 bytes per row), zero between launches
//   [128 KiB, 128 KiB+5 MiB) partial exchange of the stream-K kernel (one slot per block,
//                            64 rows x 128 channels x 4 bytes), all zero between launches
//   [128 KiB + 5 MiB, ...)   fp32 split-K partials of the tile kernel (always written before
//                            they are read: no zeroing needed)
constexpr size_t kWsCountersOffset = 256;
constexpr size_t kWsKeysOffset = 64 * 1024;
constexpr size_t kWsExchangeOffset = 128 * 1024;
constexpr size_t kWsExchangeBytes = 5 * 1024 * 1024;
constexpr size_t kWsPartialOffset = kWsExchangeOffset + kWsExchangeBytes;
constexpr int kMaxSplitTiles = static_cast<int>((kWsKeysOffset - kWsCountersOffset) / sizeof(unsigned));
constexpr int kMaxArgmaxRows = static_cast<int>((kWsExchangeOffset - kWsKeysOffset) / sizeof(unsigned long long));

template <int FMT>
struct PackedStage {
  // bytes of packed weights per K block of 128: [128 rows x 64 B], two such for int8
  static constexpr int kBytes = (FMT == FMT_W8) ? kBlockN * 128 : kBlockN * 64;
};

// Abort-aware bounded wait: gives up when the poll budget is spent or when another role has
// already flagged the block as failed.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort) {
  for (uint32_t i = 0; i < kMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0x3FF) == 0x3FF && *abort) return false;
  }
  return false;
}

__device__ __forceinline__ void flag_failure(volatile int* abort, unsigned* status, unsigned code) {
  *abort = 1;
  atomicOr(status, code);
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "r"(addr));
  return r;
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Two floats -> one 32-bit word of two T (first in the low half), one packed conversion.
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  return as_u32(__floats2half2_rn(lo, hi));
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  return as_u32(__floats2bfloat162_rn(lo, hi));
}

// SiLU-gated product of one (gate, up) pair in fp32: gate * sigmoid(gate) * up.
__device__ __forceinline__ float swiglu_pair(float gate, float up) {
  return gate * __frcp_rn(1.0f + __expf(-gate)) * up;
}

// ---------------------------------------------------------------- 4-bit unpack
// Per-(row, group) constants, prepared once per K block: the subtrahends of the two nibble
// encodings and the scale, as fp16x2 bit patterns.
struct PairConsts {
  uint32_t bias_lo;    // 1024 + zero
  uint32_t nbias_hi;   // -(64 + zero): after the x1/16 of the high-nibble encoding
  uint32_t scale;
};

__device__ __forceinline__ PairConsts make_pair_consts(__half scale, float zero) {
  PairConsts g;
  g.bias_lo = as_u32(__float2half2_rn(1024.0f + zero));
  g.nbias_hi = as_u32(__float2half2_rn(-(64.0f + zero)));
  g.scale = as_u32(__half2half2(scale));
  return g;
}

// fp16x2 weights -> the MMA operand format of activation type T.
template <typename T>
__device__ __forceinline__ uint32_t pack_operand(__half2 h);
template <>
__device__ __forceinline__ uint32_t pack_operand<__half>(__half2 h) {
  return as_u32(h);
}
template <>
__device__ __forceinline__ uint32_t pack_operand<__nv_bfloat16>(__half2 h) {
  return h2_to_bf162(h);   // rounded to nearest even: what tensor.to(bf16) does
}

// Two nibbles 16 bits apart -> (n - zero) * scale for both.  The low nibble of a byte is
// encoded in place as 0x6400 | n = 1024 + n; the high nibble in place as 1024 + 16 n, and
// (1024 + 16 n) / 16 - (64 + zero) is exact in fp16.  One fp16 multiply by the scale follows:
// the format's contract.
template <typename T>
__device__ __forceinline__ uint32_t deq_lo(uint32_t u, const PairConsts& g) {
  const __half2 e = as_h2(lop3_and_or(u, 0x000F000Fu, 0x64006400u));
  return pack_operand<T>(__hmul2(__hsub2(e, as_h2(g.bias_lo)), as_h2(g.scale)));
}
template <typename T>
__device__ __forceinline__ uint32_t deq_hi(uint32_t u, const PairConsts& g) {
  const __half2 e = as_h2(lop3_and_or(u, 0x00F000F0u, 0x64006400u));
  return pack_operand<T>(__hmul2(__hfma2(e, __float2half2_rn(0.0625f), as_h2(g.nbias_hi)), as_h2(g.scale)));
}

// Scales (and zero-points) of one weight row, eight groups per 16-byte load.
__device__ __forceinline__ __half pick_half(const uint4& v, int idx) {
  const uint32_t w = (idx & 4) ? ((idx & 2) ? v.w : v.z) : ((idx & 2) ? v.y : v.x);
  return __ushort_as_half(static_cast<unsigned short>((idx & 1) ? (w >> 16) : (w & 0xFFFFu)));
}

// Column-count generic TMEM store of one thread's lane.
template <int NCOL>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&r)[NCOL]);
template <>
__device__ __forceinline__ void tmem_st_cols<8>(uint32_t taddr, const uint32_t (&r)[8]) {
  tmem_st_x8(taddr, r);
}
template <>
__device__ __forceinline__ void tmem_st_cols<16>(uint32_t taddr, const uint32_t (&r)[16]) {
  tmem_st_x16(taddr, r);
}
template <>
__device__ __forceinline__ void tmem_st_cols<32>(uint32_t taddr, const uint32_t (&r)[32]) {
  tmem_st_x32(taddr, r);
}

// ---------------------------------------------------------------- fused all-gather signals
// Signal block of the fused all-gather, one per rank per output buffer (64-bit words):
//   [0]     arrivals: +1 for every unit of output a rank has delivered everywhere
//   [1]     generation: calls completed on this rank (advanced by gather_wait_kernel)
//   [2]     status: non-zero if a bounded wait of the protocol expired on this rank
//   [3]     blocks of the push kernel that have finished (this rank only; zero between calls)
//   [8 + r] ready[r]: rank r has entered call number ready[r] (so its previous output is consumed)
constexpr int kSigArrivals = 0, kSigGeneration = 1, kSigStatus = 2, kSigPushBlocks = 3, kSigReady = 8;

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Bounded system-scope poll: quick at first, then about a microsecond per look, roughly five
// seconds in all.  Ranks are separate processes, so benign host-side skew (a first-call
// set-up, a garbage collection) has to fit inside the bound; a rank that never arrives makes
// the caller record a status and move on instead of hanging.
__device__ __forceinline__ bool poll_at_least(const unsigned long long* p, unsigned long long target) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (ld_acquire_sys(p) >= target) return true;
    __nanosleep(i < 4096 ? 40 : 1000);
  }
  return false;
}

// ---------------------------------------------------------------- host side
// Rank-3 tensor maps {d0, d1, d2} with byte pitches {ld1, ld2} and box {b0, b1, b2}; pure
// functions of their arguments, cached (gemm_tc.cu).  Encoding is a host-only driver call,
// legal while a stream is capturing.
bool get_tensor_map(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t d0,
                    uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2, uint32_t b0, uint32_t b1,
                    uint32_t b2, CUtensorMapSwizzle swz);

// B200Q_DEBUG_PLAN=1 prints the tiling of every tensor-core launch to stderr.
bool debug_plan_enabled();

// gemm_sk.cu: persistent stream-K kernel for token tiles of at most 64 rows.
bool sk_supported(const ForwardArgs& a);
bool sk_preferred(int format, int M, int N, int K);
size_t sk_workspace_bytes(int format, int M, int N, int K);
int sk_gather_arrivals(int format, int M, int N, int K);
int launch_forward_sk(const ForwardArgs& a);
bool sk_describe(int format, int M, int N, int K, char* text, size_t size);

}  // namespace b200q
