// Tensor-core weight-only linear for sm_100a: tcgen05.mma with the WEIGHTS on
// the M side of the MMA and the tokens on the N side.
//
//   D[128 channels, TOK tokens] (fp32, TMEM) += Wd[128, 16] * X[TOK, 16]^T
//
// so a tile never pads the token count to 128: TOK is any multiple of 16 up to
// 256 and is chosen per call.  One block owns 128 output channels x TOK tokens
// x a K range (split-K over blockIdx.z when there are too few tiles to fill
// the GPU).
//
// Warp roles (320 threads):
//   warp 0     TMA producer: packed weights [128 x 64 B] boxes (no swizzle) and
//              activation boxes [TOK x 64 elements] (128-byte swizzle)
//   warp 1     TMEM allocation, tcgen05.mma issue (one elected thread), commits
//   warps 2-9  dequantise the packed stage out of shared memory into the
//              128-byte-swizzled K-major A operand stage, later the epilogue:
//              tcgen05.ld, scale/bias, store (or split-K partials + last block
//              reduces, counters reset for the next launch)
//
// Three rings step once per 128-wide K block: packed weights (P), dequantised
// A operand (two 64-wide swizzle atoms) and activations (X, two atoms).
//
// Reference counterparts: _w4a16_linear_kernel (engine/kernels/w4a16_linear.py:27-74),
// _w8a16_linear_kernel (engine/kernels/w8a16_linear.py:10-40) and the dense
// dequantise-then-cuBLAS branch of W4A16Linear (engine/quantization/w4a16.py:158-178).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>
#include <unordered_map>

#include "internal.cuh"
#include "ptx.cuh"

namespace b200q {

// Block = 2 service warps (TMA producer, MMA issuer) + DW dequantise warps (8 or 16).
constexpr int kBlockN = 128;                 // output channels per block (UMMA M)
constexpr int kBlockK = 128;                 // K elements per pipeline step
constexpr int kAtomBytesA = kBlockN * 128;   // one 64-wide K atom of the A operand: 16 KB
constexpr int kStageBytesA = 2 * kAtomBytesA;
constexpr int kMaxRing = 16;
constexpr int kSmemBudget = 226 * 1024;      // dynamic shared memory we ask for at most

struct TcParams {
  const void* scales;
  int scale_is_f32;
  const __half* zeros;
  const void* bias;
  void* y;
  int64_t ldy;
  int M, N, K;
  int groups;        // K / 128 for the 4-bit formats
  int tok;           // tokens per tile
  int tmem_cols;
  int a_col0;        // first TMEM column of the A operand stages (A-in-TMEM variant)
  uint32_t idesc;
  int kb_total;      // ceil(K / 128)
  int kb_per_split;
  int splits;
  int cluster_reduce;  // split-K partials are summed over distributed shared memory (cluster = the splits of a tile)
  int np, na, nx;    // ring depths: weight groups, operand stages, activation chunks
  int pg, xg;        // K blocks per weight group / per activation chunk (one TMA each)
  float* partial;    // [splits, M, N] fp32 (split-K only)
  int static_weights;  // weights/scales/bias may be read ahead of the stream order
  int swiglu;          // rows are (gate, up) pairs: y[m, c] = silu(row 2c) * row 2c+1; N/2 output columns
  int y_tma;           // finished tiles leave shared memory through one TMA store (tm_y is valid)
  int argmax;          // y is int64 channel[M]: per row the channel of the largest output
  unsigned long long* row_keys;  // [M] in the workspace, zero between launches (argmax only)
  // fused all-gather (g_world > 1): every output tile is stored into the [M, ldy] buffer of
  // every rank at column offset g_col0, through peer-mapped pointers
  int g_world, g_rank, g_col0;
  void* g_y[8];
  unsigned long long* g_sig[8];   // each rank's signal block (see GatherSignal)
  unsigned* counters;  // [m_tiles * n_tiles], zero between launches
  unsigned* status;    // device status word (non-zero: a bounded wait expired)
};

template <int FMT>
struct PackedStage {
  // bytes of packed weights per K block of 128
  static constexpr int kBytes = (FMT == FMT_W8) ? kBlockN * 128 : kBlockN * 64;
};

// Abort-aware bounded wait: gives up when the poll budget is spent or when
// another role has already flagged the block as failed.
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

__device__ __forceinline__ uint32_t swizzled_chunk_offset(int row, int chunk) {
  // 128-byte rows, 16-byte chunks XOR-ed with the row index inside each 8-row atom
  return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 + (((chunk ^ (row & 7)) & 7) << 4));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "r"(addr));
  return r;
}

template <typename T>
__device__ __forceinline__ uint32_t pack_operand(__half2 h);
template <>
__device__ __forceinline__ uint32_t pack_operand<__half>(__half2 h) {
  return as_u32(h);
}
template <>
__device__ __forceinline__ uint32_t pack_operand<__nv_bfloat16>(__half2 h) {
  return h2_to_bf162(h);   // fp16 dequant value, then rounded to bf16 (what .to(bf16) does)
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

#ifdef B200Q_TRACE
// Debug builds only: per-block cycle stamps of the pipeline phases.
__device__ unsigned long long g_trace[1024 * 64];
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define B200Q_STAMP(slot)                                                              \
  do {                                                                                 \
    if (trace_cta < 1024 && (slot) < 64) g_trace[trace_cta * 64 + (slot)] = clock64(); \
  } while (0)
// cumulative per-phase cycle counters of one dequantise warp (slots 40..47)
#define B200Q_TIMER_DECL long long tmr_last = clock64(), tmr_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define B200Q_TIMER_LAP(k)                  \
  {                                         \
    const long long tmr_now = clock64();    \
    tmr_acc[k] += tmr_now - tmr_last;       \
    tmr_last = tmr_now;                     \
  }
#define B200Q_TIMER_RESET(on)                  \
  if (on) {                                    \
    for (int k = 0; k < 8; ++k) tmr_acc[k] = 0; \
  }
#define B200Q_TIMER_FLUSH(on)                                                                \
  if (on) {                                                                                  \
    for (int k = 0; k < 8; ++k) g_trace[(trace_cta & 1023) * 64 + 40 + k] = tmr_acc[k];      \
  }
#define B200Q_TIMER_FLUSH_EPI(on)                                                            \
  if (on) {                                                                                  \
    for (int k = 0; k < 4; ++k) g_trace[(trace_cta & 1023) * 64 + 52 + k] = tmr_acc[k];      \
  }
#define B200Q_TIMER_FLUSH_MMA                                                                \
  {                                                                                          \
    for (int k = 0; k < 4; ++k) g_trace[(trace_cta & 1023) * 64 + 48 + k] = tmr_acc[k];      \
  }
#define B200Q_STAMP_NS(slot)                                                             \
  do {                                                                                   \
    if (trace_cta < 1024 && (slot) < 64) g_trace[trace_cta * 64 + (slot)] = global_ns(); \
  } while (0)
#else
#define B200Q_STAMP(slot)
#define B200Q_STAMP_NS(slot)
#define B200Q_TIMER_DECL
#define B200Q_TIMER_LAP(k)
#define B200Q_TIMER_RESET(on)
#define B200Q_TIMER_FLUSH(on)
#define B200Q_TIMER_FLUSH_EPI(on)
#define B200Q_TIMER_FLUSH_MMA
#endif

// Per-(row, group) parameters of the 4-bit formats, fetched eight groups at a time
// (one 16-byte load per row) one chunk ahead of use, so that their latency never sits
// between two pipeline stages.  When K/128 is not a multiple of 8 a chunk is one group.
struct GroupChunk {
  uint4 s[2];   // scales of the thread's two rows
  uint4 z[2];   // zero-points (asymmetric layout only)
};

__device__ __forceinline__ __half pick_half(const uint4& v, int idx) {
  const uint32_t w = (idx & 4) ? ((idx & 2) ? v.w : v.z) : ((idx & 2) ? v.y : v.x);
  return __ushort_as_half(static_cast<unsigned short>((idx & 1) ? (w >> 16) : (w & 0xFFFFu)));
}

// Per-stage constants of one row's group, prepared once: subtrahends for the two nibble
// encodings and the scale, as fp16x2 or bf16x2 bit patterns.
struct PairConsts {
  uint32_t bias_lo;    // 1024 + zero (fp16)  or 128 + zero (bf16)
  uint32_t nbias_hi;   // -(64 + zero) (fp16) or -(8 + zero) (bf16): after the x1/16 of the high encoding
  uint32_t scale;
};

// enc holds two encoded nibbles (kh = 0: magic + n; kh = 1: magic + 16 n).  Returns
// (n - zero) * scale for both, in the operand dtype.
template <bool BF16>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t enc, int kh, const PairConsts& g) {
  if (BF16) {
    __nv_bfloat162 e = *reinterpret_cast<__nv_bfloat162*>(&enc);
    const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&g.scale);
    __nv_bfloat162 c;
    if (kh == 0) {
      c = __hsub2(e, *reinterpret_cast<const __nv_bfloat162*>(&g.bias_lo));
    } else {
      // 128 + 16 n: times 1/16 is 8 + n, exact
      c = __hfma2(e, __float2bfloat162_rn(0.0625f), *reinterpret_cast<const __nv_bfloat162*>(&g.nbias_hi));
    }
    c = __hmul2(c, s);
    return *reinterpret_cast<uint32_t*>(&c);
  } else {
    __half2 e = as_h2(enc);
    __half2 c;
    if (kh == 0) {
      c = __hsub2(e, as_h2(g.bias_lo));
    } else {
      c = __hfma2(e, __float2half2_rn(0.0625f), as_h2(g.nbias_hi));
    }
    c = __hmul2(c, as_h2(g.scale));
    return as_u32(c);
  }
}

// Low / high nibble pair of a 32-bit word laid out as (.., n_hi, n_lo, .., n_hi, n_lo).
// fp16: 0x6400 | n = 1024 + n, and the high nibble in place is 1024 + 16 n.  bf16 has only
// seven mantissa bits, so the high nibble is shifted down and encoded as 128 + n.
template <bool BF16>
__device__ __forceinline__ uint32_t deq_lo(uint32_t u, const PairConsts& g) {
  return dequant_pair<BF16>(lop3_and_or(u, 0x000F000Fu, BF16 ? 0x43004300u : 0x64006400u), 0, g);
}
template <bool BF16>
__device__ __forceinline__ uint32_t deq_hi(uint32_t u, const PairConsts& g) {
  if (BF16) return dequant_pair<true>(lop3_and_or(u >> 4, 0x000F000Fu, 0x43004300u), 0, g);
  return dequant_pair<false>(lop3_and_or(u, 0x00F000F0u, 0x64006400u), 1, g);
}

template <int FMT>
__device__ __forceinline__ void load_group_chunk(GroupChunk& g, const TcParams& p, int chunk,
                                                 bool vec, int n0, int n1) {
  const int rows[2] = {n0, n1};
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    g.s[j] = make_uint4(0u, 0u, 0u, 0u);
    g.z[j] = make_uint4(0u, 0u, 0u, 0u);
    if (rows[j] < p.N) {
      const int64_t base = static_cast<int64_t>(rows[j]) * p.groups;
      const __half* sp = reinterpret_cast<const __half*>(p.scales) + base;
      if (vec) {
        g.s[j] = __ldg(reinterpret_cast<const uint4*>(sp + chunk * 8));
        if (FMT == FMT_W4_ASYM) g.z[j] = __ldg(reinterpret_cast<const uint4*>(p.zeros + base + chunk * 8));
      } else {
        g.s[j].x = __half_as_ushort(__ldg(sp + chunk));
        if (FMT == FMT_W4_ASYM) g.z[j].x = __half_as_ushort(__ldg(p.zeros + base + chunk));
      }
    }
  }
}

// Signal block of the fused all-gather, one per rank per output buffer (64-bit words):
//   [0]     arrivals: +1 from every block of every rank that has stored a finished tile everywhere
//   [1]     generation: calls completed on this rank (advanced by gather_wait_kernel)
//   [2]     status: non-zero if a bounded wait of the protocol expired on this rank
//   [8 + r] ready[r]: rank r has entered call number ready[r] (so its previous output is consumed)
constexpr int kSigArrivals = 0, kSigGeneration = 1, kSigStatus = 2, kSigReady = 8;

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

// After the forward of call `gen` on this rank: wait (bounded) until every block of every rank
// has delivered its tiles here, then publish the new generation.
__global__ void gather_wait_kernel(unsigned long long* sig, unsigned long long expected) {
  if (threadIdx.x != 0) return;
  // Launched with programmatic stream serialization so that the kernel AFTER it may begin its
  // prologue (and stream static weights) at once; that kernel's griddepcontrol.wait still
  // holds it until this one has finished.  This kernel itself first waits for the forward
  // before it to complete: the generation word it reads is written by the previous wait
  // kernel, which that forward was ordered behind.
  grid_launch_dependents();
  grid_dependency_wait();
  const unsigned long long gen = sig[kSigGeneration] + 1;
  if (!poll_at_least(sig + kSigArrivals, gen * expected)) sig[kSigStatus] = 1ull;
  sig[kSigGeneration] = gen;
  __threadfence_system();
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

template <int FMT, typename T, bool ATM, int DW>
__global__ void __launch_bounds__(64 + 32 * DW, (ATM && DW == 8) ? 2 : 1)
wq_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_y, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled operand tiles
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int x_atom_bytes = p.tok * 128;                  // one 64-wide K atom of [tok x 128 B]
  const uint32_t a_ring = smem_base;
  const uint32_t x_ring = a_ring + (ATM ? 0 : p.na * kStageBytesA);
  const int x_chunk_bytes = p.xg * 2 * x_atom_bytes;     // xg K blocks of two atoms each
  const int p_group_bytes = p.pg * PackedStage<FMT>::kBytes;
  const uint32_t p_ring = x_ring + p.nx * x_chunk_bytes;
  const uint32_t bars = p_ring + p.np * p_group_bytes;
  // barrier slots (8 bytes each)
  const uint32_t p_full = bars;
  const uint32_t p_empty = p_full + 8 * kMaxRing;
  const uint32_t a_full = p_empty + 8 * kMaxRing;
  const uint32_t a_empty = a_full + 8 * kMaxRing;
  const uint32_t x_full = a_empty + 8 * kMaxRing;
  const uint32_t x_empty = x_full + 8 * kMaxRing;
  const uint32_t acc_full = x_empty + 8 * kMaxRing;
  const uint32_t tmem_slot = acc_full + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  const uint32_t last_slot = abort_slot + 4;
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_p =
      reinterpret_cast<volatile uint32_t*>(generic_base + (tmem_slot - smem_base));
  volatile int* abort_p = reinterpret_cast<volatile int*>(generic_base + (abort_slot - smem_base));
  volatile int* last_p = reinterpret_cast<volatile int*>(generic_base + (last_slot - smem_base));

  constexpr int kDequantWarps = DW;
  constexpr int kDequantThreads = 32 * DW;
  constexpr int kSplit = DW / 4;                // K slices per weight row (2 or 4)
  static_assert(ATM || DW == 8, "the shared-memory operand variant uses eight dequantise warps");
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  const int nkb = max(kb1 - kb0, 0);
#ifdef B200Q_TRACE
  const int trace_cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  if (threadIdx.x == 0) {
    B200Q_STAMP(0);
    B200Q_STAMP_NS(1);
  }
#endif

  // barrier set-up spread over the lanes of warp 0 (one ring slot per lane)
  if (warp == 0) {
    if (lane < kMaxRing) {
      mbar_init(p_full + 8 * lane, 1);
      mbar_init(p_empty + 8 * lane, kDequantWarps);
      mbar_init(a_full + 8 * lane, kDequantWarps);
      mbar_init(a_empty + 8 * lane, 1);
      mbar_init(x_full + 8 * lane, 1);
      mbar_init(x_empty + 8 * lane, 1);
    }
    if (lane == 0) {
      mbar_init(acc_full, 1);
      *abort_p = 0;
      *last_p = 0;
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      if (p.y_tma) tma_prefetch_desc(&tm_y);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_p;
  if (threadIdx.x == 0) {
    B200Q_STAMP(2);
    // Let the next kernel in the stream begin its own set-up; it orders itself behind
    // this grid with griddepcontrol.wait before it touches anything this grid writes.
    grid_launch_dependents();
  }
  // With static weights the weight stream may start before the previous kernel in the
  // stream has finished; activations, outputs and the workspace always wait for it.
  if (!p.static_weights) grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // One thread feeds two independent rings, polling whichever has a free slot: packed
    // weights (one stage per K block) and activations (one 64-wide atom per slot).
    if (elect_one()) {
      // ring positions are advanced incrementally (slot, phase): no division in the loops
      int ip = 0, ix = 0;                       // weight groups / activation chunks issued
      int sp = 0, sx = 0;                       // their ring slots
      uint32_t p_phase = 1, x_phase = 1;        // parity to wait for on the empty barriers
      const int np_total = (nkb + p.pg - 1) / p.pg;
      const int nx_total = (nkb + p.xg - 1) / p.xg;
      bool waited = !p.static_weights;
      bool ok = true;
      uint32_t idle = 0;
      while (ip < np_total || ix < nx_total) {
        bool progress = false;
        if (ip < np_total) {
          if (mbar_test_wait(p_empty + 8 * sp, p_phase)) {
            // one instruction brings pg K blocks: [pg (x2 for int8)] x [128 rows] x [64 B]
            const int kb = kb0 + ip * p.pg;
            mbar_arrive_expect_tx(p_full + 8 * sp, static_cast<uint32_t>(p_group_bytes));
            tma_load_3d(p_ring + sp * p_group_bytes, &tm_w, p_full + 8 * sp, 0, n_tile * kBlockN,
                        (FMT == FMT_W8) ? 2 * kb : kb);
            if (ip == 0) B200Q_STAMP(3);
            ++ip;
            if (++sp == p.np) {
              sp = 0;
              p_phase ^= 1;
            }
            progress = true;
          }
        }
        if (!waited && (ip >= np_total || ip >= p.np)) {
          // the weight ring is as far ahead as it can get: now order behind the stream
          grid_dependency_wait();
          waited = true;
          progress = true;
        }
        if (waited && ix < nx_total) {
          if (mbar_test_wait(x_empty + 8 * sx, x_phase)) {
            // xg K blocks of activations: [2 xg atoms] x [tok rows] x [64 elements]
            mbar_arrive_expect_tx(x_full + 8 * sx, static_cast<uint32_t>(x_chunk_bytes));
            tma_load_3d(x_ring + sx * x_chunk_bytes, &tm_x, x_full + 8 * sx, 0, m_tile * p.tok,
                        2 * (kb0 + ix * p.xg));
            ++ix;
            if (++sx == p.nx) {
              sx = 0;
              x_phase ^= 1;
            }
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
        } else {
          // nothing to do: step aside so this poll loop does not take issue slots from the
          // dequantising warps that share the scheduler
          __nanosleep(64);
          if (++idle > kMaxPolls || ((idle & 0x3FF) == 0 && *abort_p)) {
            ok = false;
            break;
          }
        }
      }
      B200Q_STAMP(4);
      if (!ok) flag_failure(abort_p, p.status, 1u);
      if (*abort_p) {
        // let the copies already in flight land before the block's shared memory is released
        for (int i = max(0, ip - p.np); i < ip; ++i) mbar_wait(p_full + 8 * (i % p.np), (i / p.np) & 1);
        for (int i = max(0, ix - p.nx); i < ix; ++i) mbar_wait(x_full + 8 * (i % p.nx), (i / p.nx) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      if (p.g_world > 1 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        // Fused all-gather: tell every rank that this rank has entered call `gen`, i.e. that
        // whatever read its previous output has finished (it precedes us in the stream).
        grid_dependency_wait();
        const unsigned long long gen = p.g_sig[p.g_rank][kSigGeneration] + 1;
        // Relaxed: the announcement publishes no data of this kernel, only that the kernels
        // before it in the stream have finished (they have: griddepcontrol.wait returned).  A
        // release store per peer would serialise one NVLink round trip per rank.
        for (int d = 0; d < p.g_world; ++d) st_relaxed_sys(p.g_sig[d] + kSigReady + p.g_rank, gen);
      }
      bool ok = true;
      int sa = 0, sx = 0, xs = 0;                // operand stage, activation chunk slot, block in chunk
      uint32_t a_phase = 0, x_phase = 0;
      B200Q_TIMER_DECL
      for (int i = 0; i < nkb && ok; ++i) {
        B200Q_TIMER_LAP(3)
        B200Q_TIMER_RESET(i == 1)
        if (xs == 0) {
          ok = wait_or_abort(x_full + 8 * sx, x_phase, abort_p);
          if (!ok) break;
        }
        B200Q_TIMER_LAP(0)
        ok = wait_or_abort(a_full + 8 * sa, a_phase, abort_p);
        if (!ok) break;
        B200Q_TIMER_LAP(1)
        tc_fence_after_sync();
        if (i < 6) B200Q_STAMP(8 + 2 * i);
        const uint32_t a_stage = a_ring + sa * kStageBytesA;
        const uint32_t x_stage = x_ring + sx * x_chunk_bytes + xs * 2 * x_atom_bytes;
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
          const uint64_t adesc = umma_desc_sw128(a_stage + atom * kAtomBytesA);
          const uint64_t bdesc = umma_desc_sw128(x_stage + atom * x_atom_bytes);
          // A in tensor memory: stage sa holds 128 K elements as 64 columns, 8 per MMA
          const uint32_t a_tmem = tmem_base + p.a_col0 + sa * 64 + atom * 32;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzle atom
            const uint32_t acc = (i > 0 || atom > 0 || k > 0) ? 1u : 0u;
            if (ATM) {
              umma_f16_ts(tmem_base, a_tmem + 8 * k, bdesc + 2 * k, p.idesc, acc);
            } else {
              umma_f16_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, p.idesc, acc);
            }
          }
        }
        umma_commit(a_empty + 8 * sa);
        if (xs == p.xg - 1 || i == nkb - 1) umma_commit(x_empty + 8 * sx);
        if (i < 6) B200Q_STAMP(9 + 2 * i);
        B200Q_TIMER_LAP(2)
        if (++sa == p.na) {
          sa = 0;
          a_phase ^= 1;
        }
        if (++xs == p.xg) {
          xs = 0;
          if (++sx == p.nx) {
            sx = 0;
            x_phase ^= 1;
          }
        }
      }
      B200Q_TIMER_FLUSH_MMA
      if (!ok) flag_failure(abort_p, p.status, 2u);
      umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------ dequant warps
    const int td = threadIdx.x - 64;          // 0..255
    const int q = td & 3;                      // 16-byte vector inside a 64-byte packed row
    const int r_base = td >> 2;                // 0..63
    // A-in-TMEM mapping: a warp may only touch TMEM lanes 32*(warp%4)..+31
    const int atm_row = (warp & 3) * 32 + lane;
    const int atm_kq = (warp - 2) >> 2;                 // which K slice of the row
    const uint32_t atm_taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + p.a_col0;
    const int row_n0 = n_tile * kBlockN + (ATM ? atm_row : r_base);
    const int row_n1 = ATM ? p.N : row_n0 + 64;
    const bool vec = (p.groups & 7) == 0;
    const int chunk_shift = vec ? 3 : 0;
    GroupChunk cur, nxt;
    int cur_chunk = kb0 >> chunk_shift;
    const int last_chunk = (kb1 - 1) >> chunk_shift;
    if (FMT != FMT_W8 && nkb > 0) {
      load_group_chunk<FMT>(cur, p, cur_chunk, vec, row_n0, row_n1);
      if (cur_chunk < last_chunk) load_group_chunk<FMT>(nxt, p, cur_chunk + 1, vec, row_n0, row_n1);
    }
    bool ok = true;
    int sp = 0, ps = 0, sa = 0;                  // weight group slot, block in group, operand stage
    uint32_t p_phase = 0, a_phase = 1;           // parities: p_full, a_empty
    B200Q_TIMER_DECL
    for (int i = 0; i < nkb && ok; ++i) {
      B200Q_TIMER_LAP(4)
      const int kb = kb0 + i;
      __half2 scale2[2];
      __half2 bias_lo[2], nbias_hi[2];
      if (FMT != FMT_W8) {
        const int chunk = kb >> chunk_shift;
        if (chunk != cur_chunk) {
          cur = nxt;
          cur_chunk = chunk;
          if (chunk < last_chunk) load_group_chunk<FMT>(nxt, p, chunk + 1, vec, row_n0, row_n1);
        }
        const int idx = vec ? (kb & 7) : 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float zp = (FMT == FMT_W4_ASYM) ? __half2float(pick_half(cur.z[j], idx)) : 8.0f;
          scale2[j] = __half2half2(pick_half(cur.s[j], idx));
          bias_lo[j] = __float2half2_rn(1024.0f + zp);
          nbias_hi[j] = __float2half2_rn(-(64.0f + zp));
        }
      }
      if (td == 0 && i == 3) B200Q_STAMP(5);
      B200Q_TIMER_LAP(7)
      PairConsts gp{0u, 0u, 0u};
      if (ATM && FMT != FMT_W8) {
        const int idx = ((p.groups & 7) == 0) ? (kb & 7) : 0;
        const __half sh = pick_half(cur.s[0], idx);
        const float zp = (FMT == FMT_W4_ASYM) ? __half2float(pick_half(cur.z[0], idx)) : 8.0f;
        if (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
          gp.bias_lo = as_u32(__float2bfloat162_rn(128.0f + zp));
          gp.nbias_hi = as_u32(__float2bfloat162_rn(-(8.0f + zp)));
          gp.scale = as_u32(__float2bfloat162_rn(__half2float(sh)));
        } else {
          gp.bias_lo = as_u32(__float2half2_rn(1024.0f + zp));
          gp.nbias_hi = as_u32(__float2half2_rn(-(64.0f + zp)));
          gp.scale = as_u32(__half2half2(sh));
        }
      }
      B200Q_TIMER_LAP(0)
      if (ps == 0) ok = wait_or_abort(p_full + 8 * sp, p_phase, abort_p);
      B200Q_TIMER_LAP(1)
      if (td == 0 && i == 3) B200Q_STAMP(6);
      ok = ok && wait_or_abort(a_empty + 8 * sa, a_phase, abort_p);
      if (!ok) break;
      B200Q_TIMER_LAP(2)
      if (td == 0 && i < 4) B200Q_STAMP(32 + 2 * i);
      const uint32_t p_stage = p_ring + sp * p_group_bytes + ps * PackedStage<FMT>::kBytes;
      const uint32_t a_stage = a_ring + sa * kStageBytesA;
      if (td == 0 && i == 3) B200Q_STAMP(7);
      if (ATM) {
        // One thread = one output channel (its TMEM lane) x one 64-wide half of the K block.
        // The packed stage is read row-wise; the TMA 64-byte swizzle keeps that conflict-free.
        const uint32_t prow = p_stage + atm_row * 64;
        const int xr = (atm_row >> 1) & 3;
        // fp16 activations: (1024 + n) - (1024 + zero) is exact, then ONE fp16 multiply by the
        // scale (the format's contract).  bf16 activations: the same in bf16, (128 + n) - (128 +
        // zero) exact, one bf16 multiply by the scale rounded to bf16.
        constexpr bool kBf = sizeof(T) == 2 && !std::is_same<T, __half>::value;
        const uint32_t a_stage_t = atm_taddr + sa * 64;
        if (td == 0 && i == 3) B200Q_STAMP(61);
        if (FMT == FMT_W4_REF) {
          // This thread unpacks bytes [B*kq, B*kq + B) of its row, B = 64 / kSplit: low nibbles
          // are K offsets B*kq + j (columns B/2*kq ..), high nibbles K offsets 64 + B*kq + j
          // (columns 32 + B/2*kq ..).
          constexpr int kVec = 4 / kSplit;               // 16-byte loads per thread
          constexpr int kCols = 8 * kVec;                // columns per nibble half
          uint32_t lo[kCols], hi[kCols];
#pragma unroll
          for (int c = 0; c < kVec; ++c) {
            const uint4 v = ld_shared_v4(prow + (((kVec * atm_kq + c) ^ xr) << 4));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              // bytes (b0,b1,b2,b3) -> (b0,b2,b1,b3): the masks then pick (b0,b1) from the word
              // and (b2,b3) from the word shifted by 8
              const uint32_t u = prmt(words[w], 0u, 0x3120);
              lo[(c * 4 + w) * 2] = deq_lo<kBf>(u, gp);
              lo[(c * 4 + w) * 2 + 1] = deq_lo<kBf>(u >> 8, gp);
              hi[(c * 4 + w) * 2] = deq_hi<kBf>(u, gp);
              hi[(c * 4 + w) * 2 + 1] = deq_hi<kBf>(u >> 8, gp);
            }
          }
          tmem_st_cols<kCols>(a_stage_t + kCols * atm_kq, lo);
          tmem_st_cols<kCols>(a_stage_t + 32 + kCols * atm_kq, hi);
        } else if (FMT == FMT_W4_ASYM) {
          // words [W*kq, W*kq + W) of the row, W = 16 / kSplit: 8 W consecutive K; the layout's
          // nibble order makes every lop3 pair a pair of K neighbours
          constexpr int kVec = 4 / kSplit;
          constexpr int kCols = 16 * kVec;
          uint32_t out[kCols];
#pragma unroll
          for (int c = 0; c < kVec; ++c) {
            const uint4 v = ld_shared_v4(prow + (((kVec * atm_kq + c) ^ xr) << 4));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const uint32_t u = words[w];
              out[(c * 4 + w) * 4 + 0] = deq_lo<kBf>(u, gp);        // inputs 0,1
              out[(c * 4 + w) * 4 + 1] = deq_hi<kBf>(u, gp);        // inputs 2,3
              out[(c * 4 + w) * 4 + 2] = deq_lo<kBf>(u >> 8, gp);   // inputs 4,5
              out[(c * 4 + w) * 4 + 3] = deq_hi<kBf>(u >> 8, gp);   // inputs 6,7
            }
          }
          tmem_st_cols<kCols>(a_stage_t + kCols * atm_kq, out);
        } else {
          // W8: the stage is two [128 x 64 B] sub-tiles (K 0..63, 64..127); this thread takes
          // 128 / kSplit consecutive K of its row
          constexpr int kVec = 8 / kSplit;               // 16 int8 per load
          constexpr int kCols = 8 * kVec;
          uint32_t out[kCols];
          const int k_first = atm_kq * (128 / kSplit);   // first K of this thread's slice
          const uint32_t sub = p_stage + (k_first >> 6) * (kBlockN * 64) + atm_row * 64;
#pragma unroll
          for (int c = 0; c < kVec; ++c) {
            const uint4 v = ld_shared_v4(sub + (((((k_first & 63) >> 4) + c) ^ xr) << 4));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              __half2 k01, k23;
              int8x4_to_h2(words[w], k01, k23);
              out[(c * 4 + w) * 2] = pack_operand<T>(k01);
              out[(c * 4 + w) * 2 + 1] = pack_operand<T>(k23);
            }
          }
          tmem_st_cols<kCols>(a_stage_t + kCols * atm_kq, out);
        }
        if (td == 0 && i == 3) B200Q_STAMP(62);
        B200Q_TIMER_LAP(3)
        tmem_st_wait();
        if (td == 0 && i == 3) B200Q_STAMP(63);
        tc_fence_before_sync();
      } else if (FMT == FMT_W4_REF) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int row = r_base + 64 * j;
          const uint4 v = ld_shared_v4(p_stage + (row * 4 + q) * 16);
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            W4Quad d = dequant_w4_word_splithalf(words[w], bias_lo[j], nbias_hi[j], scale2[j]);
            lo[2 * w] = pack_operand<T>(d.lo01);
            lo[2 * w + 1] = pack_operand<T>(d.lo23);
            hi[2 * w] = pack_operand<T>(d.hi01);
            hi[2 * w + 1] = pack_operand<T>(d.hi23);
          }
          // low nibbles: K offsets 16q..16q+15 of atom 0; high nibbles: same of atom 1
          const uint32_t o0 = swizzled_chunk_offset(row, 2 * q);
          const uint32_t o1 = swizzled_chunk_offset(row, 2 * q + 1);
          st_shared_v4(a_stage + o0, lo[0], lo[1], lo[2], lo[3]);
          st_shared_v4(a_stage + o1, lo[4], lo[5], lo[6], lo[7]);
          st_shared_v4(a_stage + kAtomBytesA + o0, hi[0], hi[1], hi[2], hi[3]);
          st_shared_v4(a_stage + kAtomBytesA + o1, hi[4], hi[5], hi[6], hi[7]);
        }
      } else if (FMT == FMT_W4_ASYM) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int row = r_base + 64 * j;
          const uint4 v = ld_shared_v4(p_stage + (row * 4 + q) * 16);
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
          // 32 consecutive K: offsets 32q.. -> atom q/2, chunks 4(q%2)..4(q%2)+3
          const uint32_t atom = a_stage + (q >> 1) * kAtomBytesA;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            W4Oct o = dequant_w4_word_seq(words[w], bias_lo[j], nbias_hi[j], scale2[j]);
            st_shared_v4(atom + swizzled_chunk_offset(row, 4 * (q & 1) + w), pack_operand<T>(o.k01),
                         pack_operand<T>(o.k23), pack_operand<T>(o.k45), pack_operand<T>(o.k67));
          }
        }
      } else {
        // W8: two [128 x 64 B] sub-tiles; sub-tile h holds K offsets 64h..64h+63
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int h = j >> 1;
          const int row = r_base + 64 * (j & 1);
          const uint4 v = ld_shared_v4(p_stage + h * (kBlockN * 64) + (row * 4 + q) * 16);
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
          uint32_t out[8];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            __half2 k01, k23;
            int8x4_to_h2(words[w], k01, k23);
            out[2 * w] = pack_operand<T>(k01);
            out[2 * w + 1] = pack_operand<T>(k23);
          }
          const uint32_t atom = a_stage + h * kAtomBytesA;
          st_shared_v4(atom + swizzled_chunk_offset(row, 2 * q), out[0], out[1], out[2], out[3]);
          st_shared_v4(atom + swizzled_chunk_offset(row, 2 * q + 1), out[4], out[5], out[6], out[7]);
        }
      }
      // make the generic-proxy writes visible to the tensor core (async proxy)
      if (!ATM) fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full + 8 * sa);
        if (ps == p.pg - 1 || i == nkb - 1) mbar_arrive(p_empty + 8 * sp);
      }
      if (td == 0 && i < 4) B200Q_STAMP(33 + 2 * i);
      B200Q_TIMER_LAP(5)
      if (++sa == p.na) {
        sa = 0;
        a_phase ^= 1;
      }
      if (++ps == p.pg) {
        ps = 0;
        if (++sp == p.np) {
          sp = 0;
          p_phase ^= 1;
        }
      }
      B200Q_TIMER_LAP(6)
      B200Q_TIMER_RESET(i == 0)
    }
    B200Q_TIMER_FLUSH(td == 0)
    if (!ok) flag_failure(abort_p, p.status, 4u);

    // ------------------------------------------------------------ epilogue
    bool acc_ok = wait_or_abort(acc_full, 0, abort_p);
    if (!acc_ok) flag_failure(abort_p, p.status, 8u);
    tc_fence_after_sync();
    if (td == 0) B200Q_STAMP(56);
    acc_ok = __all_sync(0xffffffffu, acc_ok && !*abort_p) != 0;
    grid_dependency_wait();            // outputs and workspace belong to the stream order
    const int lane_quarter = warp & 3;                   // TMEM lanes this warp may read
    const int col_half = (warp - 2) >> 2;                // which slice of the token columns
    const int ch = lane_quarter * 32 + lane;             // channel inside the tile
    const int n = n_tile * kBlockN + ch;
    const int half_cols = p.tok / kSplit;
    const int c_begin = col_half * half_cols;
    const int m_base = m_tile * p.tok;
    const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(lane_quarter * 32) << 16);
    // destinations: this rank's y, or with the fused all-gather the same tile in every rank's y
    const bool gather = p.g_world > 1;
    const int ndst = gather ? p.g_world : 1;
    const int col0 = gather ? p.g_col0 : 0;
    T* ydst[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) ydst[d] = gather ? static_cast<T*>(p.g_y[d]) : static_cast<T*>(p.y);
    // Before the first store into another rank's buffer: that rank must have entered this call
    // (its consumer of the previous call is done).  Bounded; one lane per peer polls, the rest
    // wait at the named barrier.
    auto gather_wait_ready = [&]() {
      if (td < p.g_world && td != p.g_rank) {       // one lane per peer, polled side by side
        unsigned long long* mine = p.g_sig[p.g_rank];
        const unsigned long long gen = mine[kSigGeneration] + 1;
        if (!poll_at_least(mine + kSigReady + td, gen)) mine[kSigStatus] = 2ull;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
    };
    // After the last store: make the tile visible system-wide, then count it on every rank.
    // The block barrier orders every thread's stores before thread 0's system-scope fence
    // (fences are cumulative), so one fence per block covers the whole tile.
    auto gather_signal_done = [&]() {
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      if (td == 0) {
        __threadfence_system();
        for (int d = 0; d < p.g_world; ++d) red_add_relaxed_sys(p.g_sig[d] + kSigArrivals, 1ull);
      }
    };
    float ch_scale = 1.0f, ch_bias = 0.0f;
    if (n < p.N) {
      if (FMT == FMT_W8)
        ch_scale = p.scale_is_f32 ? reinterpret_cast<const float*>(p.scales)[n]
                                  : __half2float(reinterpret_cast<const __half*>(p.scales)[n]);
      if (p.bias != nullptr) ch_bias = static_cast<float>(static_cast<const T*>(p.bias)[n]);
    }
    if (p.argmax) {
      // Row-wise argmax instead of the outputs (greedy decoding over an output head): every
      // value is rounded to the activation dtype exactly as the plain path would store it,
      // mapped to an order-preserving 16-bit code, and reduced warp -> block (shared-memory
      // atomics) -> grid (one 64-bit atomicMax per row and tile on keys in the workspace).
      // Key = code << 32 | (0xFFFFFFFF - channel): the largest value wins, ties go to the
      // smallest channel.
      volatile uint32_t* best = reinterpret_cast<volatile uint32_t*>(generic_base + (x_ring - smem_base));
      for (int t = td; t < p.tok; t += kDequantThreads) best[t] = 0u;
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      if (acc_ok && nkb > 0) {
        for (int c = 0; c < half_cols; c += 8) {
          uint32_t r[8];
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const uint32_t two = pack_pair<T>(__uint_as_float(r[j]) * ch_scale + ch_bias,
                                              __uint_as_float(r[j + 1]) * ch_scale + ch_bias);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t bits = h ? (two >> 16) : (two & 0xFFFFu);
              const uint32_t code = (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
              const uint32_t key = (n < p.N) ? ((code << 16) | static_cast<uint32_t>(kBlockN - 1 - ch)) : 0u;
              const uint32_t top = __reduce_max_sync(0xffffffffu, key);
              if (lane == 0 && top != 0u)
                atomicMax(const_cast<uint32_t*>(best) + (c_begin + c + j + h), top);
            }
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      const int rows = min(p.tok, p.M - m_base);
      for (int t = td; t < rows; t += kDequantThreads) {
        const uint32_t top = best[t];
        if (top != 0u) {
          const uint32_t channel = static_cast<uint32_t>(n_tile * kBlockN + (kBlockN - 1 - static_cast<int>(top & 0xFFFFu)));
          const unsigned long long key64 =
              (static_cast<unsigned long long>(top >> 16) << 32) | (0xFFFFFFFFull - channel);
          atomicMax(p.row_keys + (m_base + t), key64);
        }
      }
      if (td == 0) B200Q_STAMP(57);
      // The last block of the grid to get here turns the keys into channel indices and puts
      // keys and counter back to zero for the next launch (same protocol as split-K).
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      if (td == 0) {
        const unsigned prev = atomicAdd(p.counters, 1u);
        *last_p = (prev == gridDim.x * gridDim.y - 1u) ? 1 : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      if (*last_p) {
        __threadfence();
        long long* out = static_cast<long long*>(p.y);
        for (int t = td; t < p.M; t += kDequantThreads) {
          const unsigned long long key = __ldcg(p.row_keys + t);
          out[t] = static_cast<long long>(0xFFFFFFFFull - (key & 0xFFFFFFFFull)) * (key != 0ull);
          p.row_keys[t] = 0ull;
        }
        if (td == 0) *p.counters = 0u;
      }
    } else if (p.splits == 1) {
      if (gather) gather_wait_ready();
      // accumulators -> output dtype -> shared memory as dense rows [token][tile_out channels]
      // (the operand rings are idle by now), then either ONE TMA store of the whole tile
      // (rows/columns beyond M/N are clipped by the tensor map) or 16-byte row stores
      const uint32_t stage = x_ring;
      const int tile_out = p.swiglu ? kBlockN / 2 : kBlockN;   // output columns per tile
      const int pitch = 2 * tile_out;                          // bytes per staged row
      const bool vec_out = (p.ldy % 8 == 0) && (col0 % 8 == 0) &&
                           (reinterpret_cast<uintptr_t>(ydst[0]) % 16 == 0) &&
                           (p.nx * x_chunk_bytes >= p.tok * 256);
      const bool tma_out = vec_out && p.y_tma != 0;
      B200Q_TIMER_DECL
      if (acc_ok && nkb > 0) {
        for (int c = 0; c < half_cols; c += 8) {
          uint32_t r[8];
          B200Q_TIMER_LAP(1)
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
          B200Q_TIMER_LAP(0)
          // Two columns per conversion instruction (the packed float -> half2 / bfloat162 form;
          // the scalar conversion is several times slower).  The plain and the gated-pair
          // forms are separate loops: the plain one is the prefill hot path.
          auto put2 = [&](int col, int out_ch, int out_n, bool keep, uint32_t two) {
            if (vec_out) {
              const uint32_t at = stage + col * pitch + out_ch * 2;
              if (keep) {
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(static_cast<unsigned short>(two & 0xFFFFu))
                             : "memory");
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + pitch), "h"(static_cast<unsigned short>(two >> 16))
                             : "memory");
              }
            } else if (keep && n < p.N) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int m = m_base + col + h;
                const unsigned short bits = static_cast<unsigned short>(h ? (two >> 16) : (two & 0xFFFFu));
                if (m < p.M)
                  for (int d = 0; d < ndst; ++d)
                    reinterpret_cast<unsigned short*>(ydst[d])[static_cast<int64_t>(m) * p.ldy + col0 + out_n] = bits;
              }
            }
          };
          if (!p.swiglu && vec_out) {
            // the prefill hot path, spelled out: constant row pitch, no predicates
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const uint32_t two = pack_pair<T>(__uint_as_float(r[j]) * ch_scale + ch_bias,
                                                __uint_as_float(r[j + 1]) * ch_scale + ch_bias);
              const uint32_t at = stage + (c_begin + c + j) * 256 + ch * 2;
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(static_cast<unsigned short>(two & 0xFFFFu))
                           : "memory");
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + 256), "h"(static_cast<unsigned short>(two >> 16))
                           : "memory");
            }
          } else if (!p.swiglu) {
#pragma unroll
            for (int j = 0; j < 8; j += 2)
              put2(c_begin + c + j, ch, n, true,
                   pack_pair<T>(__uint_as_float(r[j]) * ch_scale + ch_bias,
                                __uint_as_float(r[j + 1]) * ch_scale + ch_bias));
          } else {
            // gated pairs: neighbouring lanes hold the gate (even row) and the up (odd row) of
            // one output channel; the even lane keeps silu(gate) * up
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float f0 = __uint_as_float(r[j]) * ch_scale + ch_bias;
              const float f1 = __uint_as_float(r[j + 1]) * ch_scale + ch_bias;
              const float g0 = swiglu_pair(f0, __shfl_xor_sync(0xffffffffu, f0, 1));
              const float g1 = swiglu_pair(f1, __shfl_xor_sync(0xffffffffu, f1, 1));
              put2(c_begin + c + j, ch >> 1, n >> 1, (lane & 1) == 0, pack_pair<T>(g0, g1));
            }
          }
        }
      }
      B200Q_TIMER_LAP(1)
      if (vec_out) {
        if (tma_out) fence_proxy_async_smem();   // staged rows -> visible to the TMA engine
        asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
        B200Q_TIMER_LAP(2)
        if (tma_out) {
          if (td == 0 && acc_ok && nkb > 0) {
            tma_store_3d(&tm_y, stage, n_tile * tile_out, m_base, 0);
            tma_store_commit_and_wait_read();
          }
        } else if (acc_ok && nkb > 0) {
          const int chunk = td & 15;                       // 8 channels = 16 bytes
          const int n_out = p.swiglu ? p.N / 2 : p.N;
          const int n_c = n_tile * tile_out + chunk * 8;
          const int rows = min(p.tok, p.M - m_base);
          for (int r = td >> 4; r < rows && chunk * 8 < tile_out; r += kDequantThreads / 16) {
            const uint4 v = ld_shared_v4(stage + r * pitch + chunk * 16);
            const int64_t off = static_cast<int64_t>(m_base + r) * p.ldy + col0 + n_c;
            for (int d = 0; d < ndst; ++d) {
              T* dst = ydst[d] + off;
              if (n_c + 8 <= n_out) {
                *reinterpret_cast<uint4*>(dst) = v;
              } else {
                const T* e = reinterpret_cast<const T*>(&v);
                for (int k = 0; k < 8; ++k)
                  if (n_c + k < n_out) dst[k] = e[k];
              }
            }
          }
        }
      }
      B200Q_TIMER_LAP(3)
      B200Q_TIMER_FLUSH_EPI(td == 0)
      if (gather) gather_signal_done();
      if (td == 0) B200Q_STAMP(57);
    } else if (p.cluster_reduce) {
      // Split-K inside a cluster: the blocks of one tile (cluster = its K splits) each park
      // their fp32 partial in their own shared memory as [token][128 channels]; after a
      // cluster barrier block r sums rows r, r + splits, ... over every block's copy (in split
      // order, so the result equals the workspace path bit for bit) and stores them.  The
      // rings are idle: every MMA of this block has completed and every copy has landed.
      const uint32_t park = x_ring;
      for (int c = 0; c < half_cols; c += 8) {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (acc_ok && nkb > 0) {
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(park + (c_begin + c + j) * 512 + ch * 4), "r"(r[j])
                       : "memory");
      }
      if (td == 0) B200Q_STAMP(57);
      cluster_arrive_release();
      cluster_wait_acquire();
      {
        const int n_base = n_tile * kBlockN;
        const int q4 = td & 31;                           // float4 index inside the row
        const int nq = n_base + 4 * q4;
        const int rows = min(p.tok, p.M - m_base);
        const bool vec4 = (p.N % 4 == 0) && (nq + 4 <= p.N);
        float sc[4] = {1.0f, 1.0f, 1.0f, 1.0f}, bs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (nq + e < p.N) {
            if (FMT == FMT_W8)
              sc[e] = p.scale_is_f32 ? reinterpret_cast<const float*>(p.scales)[nq + e]
                                     : __half2float(reinterpret_cast<const __half*>(p.scales)[nq + e]);
            if (p.bias != nullptr) bs[e] = static_cast<float>(static_cast<const T*>(p.bias)[nq + e]);
          }
        }
        constexpr int kMaxCluster = 8;
        uint32_t peer[kMaxCluster];
#pragma unroll
        for (int z = 0; z < kMaxCluster; ++z)
          peer[z] = map_to_cluster_rank(park + q4 * 16, static_cast<uint32_t>(z < p.splits ? z : 0));
        for (int r = split + p.splits * (td >> 5); r < rows; r += p.splits * kDequantWarps) {
          float4 t[kMaxCluster];
#pragma unroll
          for (int z = 0; z < kMaxCluster; ++z) {
            t[z] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (z < p.splits) t[z] = ld_cluster_shared_f4(peer[z] + r * 512);
          }
          float4 a = t[0];
#pragma unroll
          for (int z = 1; z < kMaxCluster; ++z) {
            if (z < p.splits) {
              a.x += t[z].x;
              a.y += t[z].y;
              a.z += t[z].z;
              a.w += t[z].w;
            }
          }
          const int64_t off = static_cast<int64_t>(m_base + r) * p.ldy + nq;
          const float v[4] = {a.x, a.y, a.z, a.w};
          if (p.swiglu) {
            // channels nq..nq+3 are two (gate, up) pairs -> output columns nq/2, nq/2 + 1
            T* dst2 = static_cast<T*>(p.y) + static_cast<int64_t>(m_base + r) * p.ldy + (nq >> 1);
            if (nq + 1 < p.N)
              dst2[0] = from_float<T>(swiglu_pair(v[0] * sc[0] + bs[0], v[1] * sc[1] + bs[1]));
            if (nq + 3 < p.N)
              dst2[1] = from_float<T>(swiglu_pair(v[2] * sc[2] + bs[2], v[3] * sc[3] + bs[3]));
            continue;
          }
          alignas(8) T o[4];
          reinterpret_cast<uint32_t*>(o)[0] = pack_pair<T>(v[0] * sc[0] + bs[0], v[1] * sc[1] + bs[1]);
          reinterpret_cast<uint32_t*>(o)[1] = pack_pair<T>(v[2] * sc[2] + bs[2], v[3] * sc[3] + bs[3]);
          T* dst = static_cast<T*>(p.y) + off;
          if (vec4 && reinterpret_cast<uintptr_t>(dst) % 8 == 0) {
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (nq + e < p.N) dst[e] = o[e];
          }
        }
      }
      // no block may leave (and release its shared memory) while a peer still reads it
      cluster_arrive_release();
      cluster_wait_acquire();
    } else {
      if (acc_ok && nkb > 0) {
        for (int c = 0; c < half_cols; c += 8) {
          uint32_t r[8];
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int m = m_base + c_begin + c + j;
              if (m < p.M)
                p.partial[(static_cast<int64_t>(split) * p.M + m) * p.N + n] = __uint_as_float(r[j]);
            }
          }
        }
      }
      if (td == 0) B200Q_STAMP(57);
      // last block to arrive for this tile sums the partials in split order
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      unsigned* counter = p.counters + (m_tile * gridDim.x + n_tile);
      if (td == 0) {
        const unsigned prev = atomicAdd(counter, 1u);
        *last_p = (prev == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
      if (*last_p) {
        __threadfence();
        if (gather) gather_wait_ready();
        // Sum the partials of this tile in split order.  Flat mapping: a row of the tile is
        // 128 channels = 32 float4, one row per warp (the partials sit in L2).
        const int n_base = n_tile * kBlockN;
        const int q4 = td & 31;                           // float4 index inside the row
        const int nq = n_base + 4 * q4;
        const int rows = min(p.tok, p.M - m_base);
        const bool vec4 = (p.N % 4 == 0) && (nq + 4 <= p.N);
        float sc[4] = {1.0f, 1.0f, 1.0f, 1.0f}, bs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (nq + e < p.N) {
            if (FMT == FMT_W8)
              sc[e] = p.scale_is_f32 ? reinterpret_cast<const float*>(p.scales)[nq + e]
                                     : __half2float(reinterpret_cast<const __half*>(p.scales)[nq + e]);
            if (p.bias != nullptr) bs[e] = static_cast<float>(static_cast<const T*>(p.bias)[nq + e]);
          }
        }
        // kRowsInFlight rows x kSplitBatch splits of independent 16-byte loads are issued before
        // any is consumed, so a tile costs one L2 round trip per batch, not one per split.
        constexpr int kRowsInFlight = 2, kSplitBatch = 4;
        for (int r0 = td >> 5; r0 < rows; r0 += kRowsInFlight * kDequantWarps) {
          float4 acc[kRowsInFlight];
#pragma unroll
          for (int u = 0; u < kRowsInFlight; ++u) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          for (int z0 = 0; z0 < p.splits; z0 += kSplitBatch) {
            float4 t[kSplitBatch][kRowsInFlight];
#pragma unroll
            for (int zz = 0; zz < kSplitBatch; ++zz) {
#pragma unroll
              for (int u = 0; u < kRowsInFlight; ++u) {
                const int r = r0 + kDequantWarps * u;
                t[zz][u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (z0 + zz < p.splits && r < rows) {
                  const float* src =
                      p.partial + (static_cast<int64_t>(z0 + zz) * p.M + m_base + r) * p.N + nq;
                  if (vec4) {
                    t[zz][u] = __ldcg(reinterpret_cast<const float4*>(src));
                  } else {
                    if (nq + 0 < p.N) t[zz][u].x = __ldcg(src + 0);
                    if (nq + 1 < p.N) t[zz][u].y = __ldcg(src + 1);
                    if (nq + 2 < p.N) t[zz][u].z = __ldcg(src + 2);
                    if (nq + 3 < p.N) t[zz][u].w = __ldcg(src + 3);
                  }
                }
              }
            }
            // absent splits contribute +0.0f, which leaves the running sum unchanged
#pragma unroll
            for (int zz = 0; zz < kSplitBatch; ++zz) {
#pragma unroll
              for (int u = 0; u < kRowsInFlight; ++u) {
                acc[u].x += t[zz][u].x;
                acc[u].y += t[zz][u].y;
                acc[u].z += t[zz][u].z;
                acc[u].w += t[zz][u].w;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < kRowsInFlight; ++u) {
            const int r = r0 + kDequantWarps * u;
            if (r < rows) {
              const int64_t off = static_cast<int64_t>(m_base + r) * p.ldy + col0 + nq;
              const float v[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
              if (p.swiglu) {
                // channels nq..nq+3 are two (gate, up) pairs -> output columns nq/2, nq/2 + 1
                const int64_t off2 = static_cast<int64_t>(m_base + r) * p.ldy + col0 + (nq >> 1);
                const T o0 = from_float<T>(swiglu_pair(v[0] * sc[0] + bs[0], v[1] * sc[1] + bs[1]));
                const T o1 = from_float<T>(swiglu_pair(v[2] * sc[2] + bs[2], v[3] * sc[3] + bs[3]));
                for (int d = 0; d < ndst; ++d) {
                  if (nq + 1 < p.N) ydst[d][off2] = o0;
                  if (nq + 3 < p.N) ydst[d][off2 + 1] = o1;
                }
                continue;
              }
              alignas(8) T o[4];
              reinterpret_cast<uint32_t*>(o)[0] = pack_pair<T>(v[0] * sc[0] + bs[0], v[1] * sc[1] + bs[1]);
              reinterpret_cast<uint32_t*>(o)[1] = pack_pair<T>(v[2] * sc[2] + bs[2], v[3] * sc[3] + bs[3]);
              const bool vec_store = vec4 && ((off * sizeof(T)) % 8 == 0);
              for (int d = 0; d < ndst; ++d) {
                if (vec_store && reinterpret_cast<uintptr_t>(ydst[d]) % 8 == 0) {
                  *reinterpret_cast<uint2*>(ydst[d] + off) = *reinterpret_cast<const uint2*>(o);
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (nq + e < p.N) ydst[d][off + e] = o[e];
                }
              }
            }
          }
        }
        if (gather) gather_signal_done();
        if (td == 0) *counter = 0u;      // ready for the next launch / graph replay
      }
    }
  }

  if (threadIdx.x == 64) B200Q_STAMP(58);
  if (p.cluster_reduce && warp < 2) {
    // the producer and MMA warps only take part in the epilogue's two cluster barriers
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    B200Q_STAMP(59);
    B200Q_STAMP_NS(60);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

#ifdef B200Q_TRACE
extern "C" int b200q_trace_clear() {
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_trace) != cudaSuccess) return 1;
  return static_cast<int>(cudaMemset(sym, 0, sizeof(g_trace)));
}
extern "C" int b200q_trace_read(unsigned long long* host, size_t count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace, count * sizeof(unsigned long long)));
}
#endif

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2, ld1, ld2;
  uint32_t b0, b1, b2, kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && ld1 == o.ld1 && ld2 == o.ld2 &&
           b0 == o.b0 && b1 == o.b1 && b2 == o.b2 && kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    auto mix = [&h](uint64_t v) { h ^= (v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2)); };
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.ld1); mix(k.ld2);
    mix((static_cast<uint64_t>(k.b0) << 40) ^ (static_cast<uint64_t>(k.b1) << 20) ^ k.b2);
    mix(k.kind);
    return static_cast<size_t>(h);
  }
};

// Rank-3 tensor maps {d0, d1, d2} with byte pitches {ld1, ld2} and box {b0, b1, b2}.  They are
// pure functions of their arguments: cached.  Encoding is a host-only driver call, legal while
// a stream is capturing.
static bool get_tensor_map(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t d0,
                           uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2, uint32_t b0,
                           uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, d0, d1, d2, ld1, ld2, b0, b1, b2,
             static_cast<uint32_t>(dt) * 16u + static_cast<uint32_t>(swz)};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error_text("cuTensorMapEncodeTiled entry point not found");
    return false;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1, ld2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char text[160];
    std::snprintf(text, sizeof(text), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    set_last_error_text(text);
    return false;
  }
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// Workspace layout (fixed, so that calls of different geometry never see one another's
// leftovers as counters): [0,256) status word, [256, 64 KiB) split-K tile counters (always
// zero between launches), then the fp32 partials.
constexpr size_t kWsHeaderBytes = 64 * 1024;
constexpr int kMaxSplitTiles = static_cast<int>((kWsHeaderBytes - 256) / sizeof(unsigned));

struct TcPlan {
  int tok, m_tiles, n_tiles, kb_total, splits, kb_per_split, np, na, nx, pg, xg, tmem_cols, a_col0;
  int dw;            // dequantise warps per block: 8, or 16 for wide tiles (one block per SM)
  bool atm;          // A operand in tensor memory (default) or in shared memory
  size_t smem_bytes;
};

static int packed_stage_bytes(int format) { return format == FMT_W8 ? kBlockN * 128 : kBlockN * 64; }

// B200Q_TC_OPERAND=smem selects the variant that stages the dequantised A operand in
// shared memory; the default keeps it in tensor memory.
static bool use_tmem_operand() {
  static const bool v = []() {
    const char* e = std::getenv("B200Q_TC_OPERAND");
    return !(e && std::strcmp(e, "smem") == 0);
  }();
  return v;
}

// Most weight tiles a problem may have for its 33..64-token tiles to take the wide block shape.
// B200Q_TC_WIDE_SMALL=<n> overrides it (0: never).
static int wide_small_max_tiles() {
  static const int n = [] {
    const char* v = std::getenv("B200Q_TC_WIDE_SMALL");
    return v != nullptr ? std::atoi(v) : 74;
  }();
  return n;
}

static int forced_dequant_warps() {
  static const int v = [] {
    const char* e = std::getenv("B200Q_TC_DW");
    const int n = e ? std::atoi(e) : 0;
    return (n == 8 || n == 16) ? n : 0;
  }();
  return v;
}

static TcPlan make_plan(int format, int M, int N, int K, bool no_split = false) {
  TcPlan pl{};
  pl.atm = use_tmem_operand();
  // Token tile: as few tiles as cover M, except that a problem of at most two waves (148
  // blocks at a time) may take a narrower tile that fills its last wave; with more waves the
  // widest tile measured best.  Cost model per candidate count of token
  // tiles: waves x (tile width + fixed set-up/epilogue worth ~40 columns), a tile narrower than
  // 128 columns being dequantise-bound; a problem under half a wave will be split along K.
  int mt = (M + 255) / 256;
  if (pl.atm && M > 256 && mt * ((N + kBlockN - 1) / kBlockN) <= 2 * 148) {
    const int n_tiles = (N + kBlockN - 1) / kBlockN;
    const int kb_total = (K + kBlockK - 1) / kBlockK;
    double best_cost = 0.0;
    int best_mt = mt;
    for (int c = mt; c <= mt + 4; ++c) {
      const int tok_c = ((M + c - 1) / c + 15) / 16 * 16;
      if (tok_c < 96) break;
      const int tiles = c * n_tiles;
      const int waves = (tiles + 147) / 148;
      int s = 1;
      if (2 * tiles <= 148) s = std::max(1, std::min(std::min(148 / tiles, kb_total / 8), 8));
      const double cost = waves * (std::max(tok_c, 128) + 40.0) / s + (s > 1 ? 16.0 : 0.0);
      if (c == mt || cost < 0.97 * best_cost) {   // more tiles must pay for themselves
        best_cost = cost;
        best_mt = c;
      }
    }
    mt = best_mt;
  }
  int tok = ((M + mt - 1) / mt + 15) / 16 * 16;
  if (tok < 16) tok = 16;
  // Wide tiles own the whole SM: sixteen dequantise warps halve the latency of a dequantise
  // stage there.  Each of their four column slices must be whole groups of 8 columns.
  // Large prefill problems (many waves) are MMA-bound and measured no better with them.
  pl.dw = 8;
  const int forced_dw = forced_dequant_warps();      // B200Q_TC_DW=8|16 overrides (experiments)
  // "Wide" blocks own an SM (512 TMEM columns, up to 227 KB of shared memory).  Token tiles
  // above 64 always are; a tile of 33..64 tokens also takes that shape when the problem has so
  // few weight tiles (at most half a wave) that a K split inside a cluster fits in one wave:
  // its partials (tok x 128 fp32 per block) then never leave the SMs.  Measured at M = 64:
  // 4096x4096 16.3 -> 9.9 us, 4096->8192 16.3 -> 13.5 us, 12288->4096 23.9 -> 19.2 us; a full
  // wave of unsplit wide tiles (4096->12288) ties with the narrow shape, and at 16 tokens two
  // blocks per SM stay ahead (14.1 against 18.2 us), so those keep the narrow shape.
  const int tiles0 = mt * ((N + kBlockN - 1) / kBlockN);
  const bool wide = tok > 64 || (pl.atm && tok > 32 && tiles0 <= wide_small_max_tiles() &&
                                 (K + kBlockK - 1) / kBlockK >= 32);
  if (pl.atm && wide && (forced_dw ? forced_dw == 16 : mt < 4)) {
    tok = (tok + 31) / 32 * 32;
    pl.dw = 16;
  }
  pl.tok = tok;
  pl.m_tiles = (M + tok - 1) / tok;
  pl.n_tiles = (N + kBlockN - 1) / kBlockN;
  pl.kb_total = (K + kBlockK - 1) / kBlockK;

  // Rings.  One TMA instruction fills a weight GROUP of `pg` K blocks and another an
  // activation CHUNK of `xg` K blocks, so that the single producer thread and the single MMA
  // thread touch a barrier once per group/chunk instead of once per block.
  const int pbytes = packed_stage_bytes(format);
  const int xbytes = tok * 256;                    // activations of one K block (two atoms)
  const size_t a_stage_smem = pl.atm ? 0 : kStageBytesA;
  pl.xg = tok <= 16 ? 4 : (tok <= 32 ? 2 : 1);
  pl.pg = wide ? 1 : 2;
  auto total = [&](int np, int na, int nx) {
    return static_cast<size_t>(na) * a_stage_smem + static_cast<size_t>(nx) * pl.xg * xbytes +
           static_cast<size_t>(np) * pl.pg * pbytes + 1024 /*alignment*/ + 8 * kMaxRing * 6 + 64;
  };
  const size_t half_sm = 115712;                   // (228 KiB - 2 x 1 KiB reserved) / 2
  const size_t budget = static_cast<size_t>(kSmemBudget);
  bool two_per_sm;
  pl.na = 2;
  pl.nx = 2;
  pl.np = 2;
  if (pl.atm) {
    // TMEM columns: accumulator [0, tok), then `na` operand stages of 64 columns each.
    // Two resident blocks need <= 256 columns each: narrow tiles (decode, HBM-bound) take
    // that shape so one block's set-up and epilogue overlap the other's weight stream.
    pl.a_col0 = (tok + 63) / 64 * 64;
    two_per_sm = !wide && total(2, 0, 2) <= half_sm;
    if (two_per_sm) {
      pl.na = (256 - pl.a_col0) / 64;              // 3 for tok <= 64
      pl.nx = 3;
      while (total(pl.np, 0, pl.nx) > half_sm && pl.nx > 2) --pl.nx;
      while (pl.np < 6 && total(pl.np + 1, 0, pl.nx) <= half_sm) ++pl.np;
      pl.tmem_cols = 256;
    } else {
      pl.na = (512 - pl.a_col0) / 64;
      if (pl.na > 4) pl.na = 4;
      const int wish[][2] = {{1, 3}, {2, 3}, {2, 4}, {1, 4}, {2, 6}, {2, 8}};
      for (const auto& w : wish) {
        int nx = pl.nx, np = pl.np;
        (w[0] == 1 ? nx : np) = w[1];
        if (nx >= pl.nx && np >= pl.np && total(np, 0, nx) <= budget) {
          pl.nx = nx;
          pl.np = np;
        }
      }
      pl.tmem_cols = 512;
    }
  } else {
    int cols = 32;
    while (cols < tok) cols <<= 1;
    pl.tmem_cols = cols;
    pl.a_col0 = 0;
    two_per_sm = tok <= 32 && total(2, 2, 2) <= half_sm;
    if (two_per_sm) {
      while (pl.np < 4 && total(pl.np + 1, pl.na, pl.nx) <= half_sm) ++pl.np;
    } else {
      const int wish[][2] = {{0, 3}, {2, 3}, {1, 3}, {2, 4}, {0, 4}, {2, 6}};
      for (const auto& w : wish) {
        int na = pl.na, nx = pl.nx, np = pl.np;
        (w[0] == 0 ? na : (w[0] == 1 ? nx : np)) = w[1];
        if (na >= pl.na && nx >= pl.nx && np >= pl.np && total(np, na, nx) <= budget) {
          pl.na = na;
          pl.nx = nx;
          pl.np = np;
        }
      }
    }
  }
  pl.smem_bytes = total(pl.np, pl.na, pl.nx);

  // split-K: choose the smallest split count that fills the resident slots well.  Wide token
  // tiles pay for a split with tok x 128 fp32 partials per block written and re-read, so they
  // split only when less than half of the GPU would otherwise have work, and never into a
  // second wave.
  const int tiles = pl.m_tiles * pl.n_tiles;
  const int slots = 148 * (two_per_sm ? 2 : 1);
  int max_splits = pl.kb_total / 4;          // at least four K blocks per split
  if (max_splits > 16) max_splits = 16;
  if (max_splits < 1) max_splits = 1;
  int best = 1;
  if (wide) {
    if (2 * tiles <= slots) {
      best = slots / tiles;
      const int cap = pl.kb_total / 8;         // a wide tile's split must be worth its reduction
      if (best > cap) best = cap;
      if (best > max_splits) best = max_splits;
    }
  } else {
    double best_eff = 0.0;
    for (int s = 1; s <= max_splits; ++s) {
      const int ctas = tiles * s;
      const int waves = (ctas + slots - 1) / slots;
      const double eff = static_cast<double>(ctas) / (static_cast<double>(waves) * slots);
      if (eff > best_eff + 0.05) {
        best_eff = eff;
        best = s;
      }
      if (eff >= 0.9) break;
    }
  }
  if (tiles >= slots || tiles > kMaxSplitTiles || best < 1 || no_split) best = 1;
  pl.kb_per_split = (pl.kb_total + best - 1) / best;
  pl.splits = (pl.kb_total + pl.kb_per_split - 1) / pl.kb_per_split;
  return pl;
}

size_t tc_workspace_bytes(int format, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  TcPlan pl = make_plan(format, M, N, K);
  size_t bytes = kWsHeaderBytes + 8 * static_cast<size_t>(M);    // header + the argmax keys
  if (pl.splits > 1) bytes += sizeof(float) * static_cast<size_t>(pl.splits) * M * N;
  return bytes;
}

bool tc_supported(const ForwardArgs& a) {
  if (a.format != FMT_W8 && a.group != 128) return false;
  // K must be whole 64-element atoms (the tensor maps' third dimension walks them)
  if (a.format == FMT_W8 ? (a.K % 64 != 0) : (a.K % 128 != 0)) return false;
  if (reinterpret_cast<uintptr_t>(a.x) % 16 || (a.ldx * 2) % 16) return false;
  if (reinterpret_cast<uintptr_t>(a.w) % 16 || a.ldw % 16) return false;
  return true;
}

// B200Q_DEBUG_PLAN=1 prints the tiling of every tensor-core launch to stderr.
static bool debug_plan_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200Q_DEBUG_PLAN");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}

// B200Q_TILE_STORE=rows keeps the per-thread 16-byte row stores of a finished tile instead of
// the TMA store (for comparison).
static bool tma_store_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200Q_TILE_STORE");
    return !(v != nullptr && std::strcmp(v, "rows") == 0);
  }();
  return on;
}

static bool cluster_reduce_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200Q_SPLIT_REDUCE");
    return !(v != nullptr && std::strcmp(v, "workspace") == 0);
  }();
  return on;
}

static bool cluster_reduce_forced() {
  static const bool on = [] {
    const char* v = std::getenv("B200Q_SPLIT_REDUCE");
    return v != nullptr && std::strcmp(v, "cluster") == 0;
  }();
  return on;
}

template <int FMT, typename T, bool ATM, int DW>
static int launch_tc_typed(const ForwardArgs& a, const TcPlan& pl) {
  static bool attr_set_dev[64] = {};
  static std::mutex attr_mu;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    bool& attr_set = attr_set_dev[dev & 63];
    std::lock_guard<std::mutex> g(attr_mu);
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(wq_gemm_tc_kernel<FMT, T, ATM, DW>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
      if (e != cudaSuccess) {
        set_last_error("cudaFuncSetAttribute", e);
        return B200Q_ERR_CUDA;
      }
      // ask for the largest shared-memory carve-out so that two blocks fit an SM (also what the
      // cluster occupancy query assumes)
      (void)cudaFuncSetAttribute(wq_gemm_tc_kernel<FMT, T, ATM, DW>,
                                 cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
      (void)cudaGetLastError();
      attr_set = true;
    }
  }
  CUtensorMap tm_w, tm_x;
  // Packed weights as {64 B, N rows, K chunks of 64 B}: the third coordinate walks K, so a
  // box of depth pg (2 pg for int8, whose K block is two 64-byte chunks) is a weight group.
  // The A-in-TMEM variant reads a stage one row per thread: 64-byte swizzle.
  const uint64_t w_row_bytes = (FMT == FMT_W8) ? static_cast<uint64_t>(a.K) : static_cast<uint64_t>(a.K / 2);
  if (!get_tensor_map(&tm_w, a.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 64, static_cast<uint64_t>(a.N),
                      w_row_bytes / 64, static_cast<uint64_t>(a.ldw), 64, 64, kBlockN,
                      static_cast<uint32_t>((FMT == FMT_W8 ? 2 : 1) * pl.pg),
                      ATM ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE))
    return B200Q_ERR_CUDA;
  // Activations as {64 elements, M rows, K atoms}: a box of depth 2 xg is an activation chunk.
  const CUtensorMapDataType xdt = (a.act_dtype == B200Q_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!get_tensor_map(&tm_x, a.x, xdt, 64, static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K / 64),
                      static_cast<uint64_t>(a.ldx) * 2, 128, 64, static_cast<uint32_t>(pl.tok),
                      static_cast<uint32_t>(2 * pl.xg), CU_TENSOR_MAP_SWIZZLE_128B))
    return B200Q_ERR_CUDA;

  // Output as {N_out, M, 1}: a finished tile [tok rows x tile_out columns] leaves shared memory
  // through one TMA store.  Needs 16-byte aligned rows of whole 16-byte units; the fused
  // all-gather (peer pointers, one copy per rank) and split-K keep their own store paths.
  CUtensorMap tm_y{};
  const bool gathering = a.gather != nullptr && a.gather->world > 1;
  const int n_out = a.swiglu ? a.N / 2 : a.N;
  // (The TMA engine clips the innermost dimension in 16-byte units: measured, a 500-column fp16
  // output had columns 500..503 written.  So the row width must be whole 16-byte units too.)
  const bool y_tma = ATM && !gathering && !a.argmax && pl.splits == 1 && (a.ldy % 8 == 0) && (n_out % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(a.y) % 16 == 0) && tma_store_enabled();
  if (y_tma) {
    const CUtensorMapDataType ydt = (a.act_dtype == B200Q_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (!get_tensor_map(&tm_y, a.y, ydt, static_cast<uint64_t>(n_out), static_cast<uint64_t>(a.M), 1,
                        static_cast<uint64_t>(a.ldy) * 2, static_cast<uint64_t>(a.ldy) * 2 * a.M,
                        static_cast<uint32_t>(a.swiglu ? kBlockN / 2 : kBlockN),
                        static_cast<uint32_t>(pl.tok), 1, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200Q_ERR_CUDA;
  }

  TcParams p{};
  p.y_tma = y_tma ? 1 : 0;
  p.scales = a.scales;
  p.scale_is_f32 = a.scale_dtype == B200Q_F32;
  p.zeros = static_cast<const __half*>(a.zeros);
  p.bias = a.bias;
  p.y = a.y;
  p.ldy = a.ldy;
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.groups = (FMT == FMT_W8) ? 1 : a.K / 128;
  p.tok = pl.tok;
  p.tmem_cols = pl.tmem_cols;
  p.a_col0 = pl.a_col0;
  p.idesc = umma_idesc_f16(a.act_dtype == B200Q_F16 ? 0u : 1u, 128u, static_cast<uint32_t>(pl.tok));
  p.kb_total = pl.kb_total;
  p.kb_per_split = pl.kb_per_split;
  p.splits = pl.splits;
  p.np = pl.np;
  p.na = pl.na;
  p.nx = pl.nx;
  p.pg = pl.pg;
  p.xg = pl.xg;
  p.static_weights = a.static_weights ? 1 : 0;
  p.swiglu = a.swiglu ? 1 : 0;
  p.argmax = a.argmax ? 1 : 0;
  p.g_world = 0;
  if (a.gather != nullptr && a.gather->world > 1) {
    p.g_world = a.gather->world;
    p.g_rank = a.gather->rank;
    p.g_col0 = a.gather->rank * a.N;
    for (int d = 0; d < 8; ++d) {
      p.g_y[d] = d < a.gather->world ? a.gather->y_peer[d] : nullptr;
      p.g_sig[d] = d < a.gather->world ? static_cast<unsigned long long*>(a.gather->signal_peer[d]) : nullptr;
    }
  }
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  p.status = reinterpret_cast<unsigned*>(ws);
  p.counters = reinterpret_cast<unsigned*>(ws + 256);
  p.partial = reinterpret_cast<float*>(ws + kWsHeaderBytes);
  p.row_keys = reinterpret_cast<unsigned long long*>(ws + kWsHeaderBytes);   // argmax never splits K

  // Programmatic dependent launch: this grid may begin its set-up (and, with static
  // weights, its weight stream) while the previous kernel of the stream drains; the
  // kernel orders itself with griddepcontrol.wait before touching x, y or the workspace.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.n_tiles, pl.m_tiles, pl.splits);
  cfg.blockDim = dim3(64 + 32 * DW);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // Split-K over distributed shared memory: the splits of a tile form a cluster (z direction)
  // when every cluster of the grid can be resident at once; otherwise, with the fused
  // all-gather, or on request (B200Q_SPLIT_REDUCE=workspace) the partials go through the
  // workspace and the last block to arrive sums them.
  p.cluster_reduce = 0;
  int resident_clusters = -1;
  const size_t ring_bytes = static_cast<size_t>(pl.nx) * pl.xg * pl.tok * 256 +
                            static_cast<size_t>(pl.np) * pl.pg * packed_stage_bytes(a.format);
  if (ATM && pl.splits > 1 && pl.splits <= 8 && p.g_world == 0 && cluster_reduce_enabled() &&
      ring_bytes >= static_cast<size_t>(pl.tok) * 512) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = static_cast<unsigned>(pl.splits);
    cfg.numAttrs = 2;
    static std::map<std::tuple<int, size_t, int>, int> resident;   // (device, smem, splits) -> clusters
    static std::mutex resident_mu;
    int dev = 0;
    cudaGetDevice(&dev);
    int clusters = 0;
    {
      std::lock_guard<std::mutex> g(resident_mu);
      const auto key = std::make_tuple(dev, pl.smem_bytes, pl.splits);
      auto it = resident.find(key);
      if (it == resident.end()) {
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, wq_gemm_tc_kernel<FMT, T, ATM, DW>, &cfg) != cudaSuccess) {
          (void)cudaGetLastError();
          n = 0;
        }
        it = resident.emplace(key, n).first;
      }
      clusters = it->second;
    }
    resident_clusters = clusters;
    if (clusters >= pl.n_tiles * pl.m_tiles || (clusters > 0 && cluster_reduce_forced())) {
      p.cluster_reduce = 1;
    } else {
      cfg.numAttrs = 1;
    }
  }
  if (debug_plan_enabled())
    std::fprintf(stderr,
                 "b200q plan: fmt %d M %d N %d K %d | tok %d tiles %dx%d splits %d (kb %d/%d) dw %d | "
                 "rings p %dx%d x %dx%d a %d | smem %zu tmem %d | split reduce: %s (resident clusters %d)\n",
                 FMT, a.M, a.N, a.K, pl.tok, pl.m_tiles, pl.n_tiles, pl.splits, pl.kb_per_split,
                 pl.kb_total, DW, pl.np, pl.pg, pl.nx, pl.xg, pl.na, pl.smem_bytes, pl.tmem_cols,
                 pl.splits == 1 ? "none" : (p.cluster_reduce ? "cluster" : "workspace"), resident_clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, wq_gemm_tc_kernel<FMT, T, ATM, DW>, tm_w, tm_x, tm_y, p);
  if (e != cudaSuccess) {
    set_last_error("cudaLaunchKernelEx", e);
    return B200Q_ERR_CUDA;
  }
  return note_launch();
}

template <int FMT, typename T>
static int launch_tc_operand(const ForwardArgs& a, const TcPlan& pl) {
  if (!pl.atm) return launch_tc_typed<FMT, T, false, 8>(a, pl);
  return pl.dw == 16 ? launch_tc_typed<FMT, T, true, 16>(a, pl) : launch_tc_typed<FMT, T, true, 8>(a, pl);
}

int tc_output_tiles(int format, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const TcPlan pl = make_plan(format, M, N, K);
  return pl.m_tiles * pl.n_tiles;
}

int launch_gather_wait(const b200q_gather* g, unsigned long long expected, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gather_wait_kernel,
                                     static_cast<unsigned long long*>(g->signal_peer[g->rank]), expected);
  if (e != cudaSuccess) {
    set_last_error("cudaLaunchKernelEx(gather_wait)", e);
    return B200Q_ERR_CUDA;
  }
  return note_launch();
}

int launch_forward_tc(const ForwardArgs& a) {
  if (a.M <= 0 || a.N <= 0) return B200Q_OK;
  if (!tc_supported(a)) return B200Q_ERR_UNSUPPORTED;
  const TcPlan pl = make_plan(a.format, a.M, a.N, a.K, a.argmax);
  const size_t need = tc_workspace_bytes(a.format, a.M, a.N, a.K);
  if (a.workspace == nullptr || a.workspace_bytes < need) return B200Q_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a.workspace) % 256) return B200Q_ERR_ALIGNMENT;
  const bool h = a.act_dtype == B200Q_F16;
  switch (a.format) {
    case FMT_W8:
      return h ? launch_tc_operand<FMT_W8, __half>(a, pl) : launch_tc_operand<FMT_W8, __nv_bfloat16>(a, pl);
    case FMT_W4_REF:
      return h ? launch_tc_operand<FMT_W4_REF, __half>(a, pl)
               : launch_tc_operand<FMT_W4_REF, __nv_bfloat16>(a, pl);
    case FMT_W4_ASYM:
      return h ? launch_tc_operand<FMT_W4_ASYM, __half>(a, pl)
               : launch_tc_operand<FMT_W4_ASYM, __nv_bfloat16>(a, pl);
    default:
      return B200Q_ERR_INVALID;
  }
}

}  // namespace b200q
