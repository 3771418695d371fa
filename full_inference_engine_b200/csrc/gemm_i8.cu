// W8A8 linear for sm_100a: per-row dynamic int8 quantisation of the activations and an
// int8 x int8 -> int32 GEMM on the tensor cores (tcgen05.mma kind::i8), dequantised in the
// epilogue exactly as the reference does it on its own device:
//
//   a_scale[m] = (max_k |x[m,k]| (fp32) clamp_min 1e-8) * fp32(1 / 127)
//   qx[m,k]    = clamp(rint(x[m,k] / a_scale[m]), -127, 127)
//   y[m,n]     = T( (float(sum_k qx[m,k] * qw[n,k]) * a_scale[m]) * float(w_scale[n]) )
//
// (engine/kernels/w8a8_linear.py:35-50; the reference hands the integer GEMM to torch._int_mm.)
// The "/ 127.0" of the reference is a tensor divided by a Python scalar, which torch's CUDA
// kernel evaluates as a multiplication by the fp32 reciprocal; the reference only accepts CUDA
// tensors, so that is its arithmetic.  "x / a_scale" is tensor by tensor: an IEEE division.
// The integer accumulation is exact, so the result is a pure function of the inputs.
//
// GEMM kernel: persistent, one block per SM walking output tiles.  Weights on the M side of the
// MMA (128 output channels per tile), tokens on the N side (TOK = a multiple of 32 up to 256),
// K in blocks of 128 int8 (TMA zero-fills a ragged last block).  Neither operand needs
// unpacking, so both go straight from TMA (128-byte swizzle) to the MMA, and the accumulator
// is double-buffered in tensor memory so that a tile's epilogue runs under the next tile's MMAs:
//   warp 0     TMA producer: per K block one [128 x 128 B] box of weights and one [TOK x 128 B]
//              box of quantised activations into one ring stage
//   warp 1     TMEM allocation, tcgen05.mma issue (four K = 32 MMAs per block), commits
//   warps 2-9  epilogue, two groups of four warps that take alternate 32-token chunks of a tile:
//              tcgen05.ld of the int32 accumulators, the two scales, the chunk staged in shared
//              memory and written by TMA (direct stores when y is not 16-byte aligned)
// Consecutive tiles share a weight tile (token tiles vary fastest), so the blocks running at
// one time read a handful of weight tiles and all the token tiles: both stay in L2.
#include <algorithm>
#include <cstdio>
#include <mutex>

#include "tc_common.cuh"

namespace b200q {

constexpr int kI8EpilogueGroups = 2;
constexpr int kI8GroupThreads = 32 * 4;                  // one warp per TMEM lane quarter
constexpr int kI8EpilogueThreads = kI8EpilogueGroups * kI8GroupThreads;
constexpr int kI8Threads = 64 + kI8EpilogueThreads;
constexpr int kI8MaxStages = 8;
constexpr int kI8ChunkTokens = 32;                       // tokens per staged store
constexpr int kI8ChunkBytes = kI8ChunkTokens * kBlockN * 2;
constexpr int kI8MaxTok = 256;
constexpr size_t kI8SmemBudget = 227 * 1024;             // the per-block maximum (the kernel has no static variables)
// after the ring: two staging chunks per epilogue group, the tile's activation scales, barriers
constexpr size_t kI8FixedBytes =
    2 * kI8EpilogueGroups * kI8ChunkBytes + kI8MaxTok * 4 + 8 * (2 * kI8MaxStages + 4) + 16;

struct I8Params {
  const float* a_scales;     // [M]
  const void* w_scales;      // [N] fp16 or fp32
  int w_scale_is_f32;
  void* y;
  int64_t ldy;
  int M, N;
  int tok;                   // tokens per tile (UMMA N)
  int m_tiles, total_tiles;
  int kb_total;              // ceil(K / 128)
  int stages;
  int acc_cols;              // TMEM columns per accumulator (two are allocated)
  int tma_out;               // y is written by TMA stores
  uint32_t idesc;
  unsigned* status;          // may be null: no workspace is needed otherwise
};

// Instruction descriptor, kind::i8: signed 8-bit A and B (both K-major), int32 accumulate.
__host__ __device__ __forceinline__ uint32_t umma_idesc_i8(uint32_t m, uint32_t n) {
  return (2u << 4)            // D format s32
         | (1u << 7)          // A format signed 8-bit
         | (1u << 10)         // B format signed 8-bit
         | ((n >> 3) << 17)   // N
         | ((m >> 4) << 24);  // M
}

__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void epilogue_barrier() {           // every epilogue warp
  asm volatile("bar.sync 1, %0;" ::"n"(kI8EpilogueThreads) : "memory");
}
__device__ __forceinline__ void group_barrier(int group) {     // the four warps of one group
  asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "n"(kI8GroupThreads) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kI8Threads, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ CUtensorMap tm_y, const I8Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int kWBytes = kBlockN * 128;                 // [128 channels x 128 int8]
  const int stage_bytes = kWBytes + p.tok * 128;         // + [tok x 128 int8]
  const uint32_t ring = smem_base;
  const uint32_t staging = ring + p.stages * stage_bytes;
  const uint32_t scale_buf = staging + 2 * kI8EpilogueGroups * kI8ChunkBytes;
  const uint32_t full = scale_buf + kI8MaxTok * 4;
  const uint32_t empty = full + 8 * kI8MaxStages;
  const uint32_t acc_full = empty + 8 * kI8MaxStages;    // two
  const uint32_t acc_empty = acc_full + 16;              // two
  const uint32_t tmem_slot = acc_empty + 16;
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(generic_base + (tmem_slot - smem_base));
  volatile int* abort_p = reinterpret_cast<volatile int*>(generic_base + (abort_slot - smem_base));
  float* const scale_p = reinterpret_cast<float*>(generic_base + (scale_buf - smem_base));
  // without a workspace the status word is a private one that nobody reads
  unsigned* const local_status = reinterpret_cast<unsigned*>(generic_base + (abort_slot + 4 - smem_base));
  unsigned* status = p.status != nullptr ? p.status : local_status;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nkb = p.kb_total;
  const int my_tiles = (p.total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);

  if (warp == 0) {
    if (lane < kI8MaxStages) {
      mbar_init(full + 8 * lane, 1);
      mbar_init(empty + 8 * lane, 1);
    }
    if (lane < 2) {
      mbar_init(acc_full + 8 * lane, 1);
      mbar_init(acc_empty + 8 * lane, kI8EpilogueThreads / 32);
    }
    if (lane == 0) {
      *abort_p = 0;
      *local_status = 0u;
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      if (p.tma_out) tma_prefetch_desc(&tm_y);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(2 * p.acc_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_p;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      int s = 0, issued = 0;
      uint32_t phase = 1;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int tile = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = wait_or_abort(empty + 8 * s, phase, abort_p);
          if (!ok) break;
          mbar_arrive_expect_tx(full + 8 * s, static_cast<uint32_t>(stage_bytes));
          tma_load_3d(ring + s * stage_bytes, &tm_w, full + 8 * s, kb * 128, n_tile * kBlockN, 0);
          tma_load_3d(ring + s * stage_bytes + kWBytes, &tm_x, full + 8 * s, kb * 128, m_tile * p.tok, 0);
          ++issued;
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) flag_failure(abort_p, status, 1u);
      // copies still in flight must land before the block's shared memory is released
      if (*abort_p)
        for (int j = max(0, issued - p.stages); j < issued; ++j) mbar_wait(full + 8 * (j % p.stages), (j / p.stages) & 1);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = true;
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int b = i & 1;
        // the epilogue has drained this accumulator (first use of each: passes at once)
        ok = wait_or_abort(acc_empty + 8 * b, ((i >> 1) & 1) ^ 1, abort_p);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(b * p.acc_cols);
        for (int kb = 0; kb < nkb; ++kb) {
          ok = wait_or_abort(full + 8 * s, phase, abort_p);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t adesc = umma_desc_sw128(ring + s * stage_bytes);
          const uint64_t bdesc = umma_desc_sw128(ring + s * stage_bytes + kWBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)          // 32 int8 = 32 bytes along K per MMA
            umma_i8_ss(acc, adesc + 2 * k, bdesc + 2 * k, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + 8 * s);
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(acc_full + 8 * b);
      }
      if (!ok) flag_failure(abort_p, status, 2u);
    }
  } else {
    // a warp may only touch TMEM lane quarter warp % 4; the group is the other index
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int ch = quarter * 32 + lane;
    const int et = static_cast<int>(threadIdx.x) - (kI8Threads - kI8EpilogueThreads);
    const bool issuer = (et & (kI8GroupThreads - 1)) == 0;       // one thread per group issues its stores
    const uint32_t my_staging = staging + static_cast<uint32_t>(group) * 2 * kI8ChunkBytes;
    T* const y = static_cast<T*>(p.y);
    int chunk_no = 0;
    for (int i = 0; i < my_tiles; ++i) {
      const int tile = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      const int b = i & 1;
      const int n = n_tile * kBlockN + ch;
      const int m_base = m_tile * p.tok;
      float w_scale = 0.0f;
      if (n < p.N)
        w_scale = p.w_scale_is_f32 ? __ldg(reinterpret_cast<const float*>(p.w_scales) + n)
                                   : __half2float(__ldg(reinterpret_cast<const __half*>(p.w_scales) + n));
      epilogue_barrier();                                  // the previous tile's scales are no longer read
      for (int t = et; t < p.tok; t += kI8EpilogueThreads)
        scale_p[t] = (m_base + t < p.M) ? __ldg(p.a_scales + m_base + t) : 0.0f;
      epilogue_barrier();
      bool ok = wait_or_abort(acc_full + 8 * b, (i >> 1) & 1, abort_p);
      if (!ok) flag_failure(abort_p, status, 8u);
      ok = __all_sync(0xffffffffu, ok && !*abort_p) != 0;
      tc_fence_after_sync();
      const uint32_t acc_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(b * p.acc_cols);
      const int tok_here = min(p.tok, (p.M - m_base + kI8ChunkTokens - 1) / kI8ChunkTokens * kI8ChunkTokens);
      const int stride = kI8EpilogueGroups * kI8ChunkTokens;
      bool released = false;
      for (int c = group * kI8ChunkTokens; c < tok_here; c += stride, ++chunk_no) {
        uint32_t r[kI8ChunkTokens];
#pragma unroll
        for (int j = 0; j < kI8ChunkTokens; ++j) r[j] = 0u;
        if (ok) {
#pragma unroll
          for (int q = 0; q < kI8ChunkTokens / 8; ++q)
            tmem_ld_x8(acc_addr + c + 8 * q, *reinterpret_cast<uint32_t(*)[8]>(&r[8 * q]));
          tmem_ld_wait();
        }
        if (c + stride >= tok_here) {
          // this group's share of the accumulator is in registers: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty + 8 * b);
          released = true;
        }
        if (p.tma_out) {
          const uint32_t buf = my_staging + static_cast<uint32_t>(chunk_no & 1) * kI8ChunkBytes;
          if (issuer) tma_store_wait_read<1>();            // the store that last used this buffer has read it
          group_barrier(group);
#pragma unroll
          for (int j = 0; j < kI8ChunkTokens; j += 2) {
            // the reference's order: (float(acc) * activation scale) * weight scale, one rounding to T
            const uint32_t two = pack_pair<T>((static_cast<float>(static_cast<int>(r[j])) * scale_p[c + j]) * w_scale,
                                              (static_cast<float>(static_cast<int>(r[j + 1])) * scale_p[c + j + 1]) * w_scale);
            const uint32_t at = buf + j * (kBlockN * 2) + ch * 2;
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(at), "h"(static_cast<unsigned short>(two & 0xFFFFu)) : "memory");
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(at + kBlockN * 2), "h"(static_cast<unsigned short>(two >> 16))
                         : "memory");
          }
          fence_proxy_async_smem();                        // staged rows -> visible to the TMA engine
          group_barrier(group);
          if (issuer && ok) {
            tma_store_3d(&tm_y, buf, n_tile * kBlockN, m_base + c, 0);   // rows >= M and channels >= N are clipped
            tma_store_commit();
          }
        } else if (ok && n < p.N) {
#pragma unroll
          for (int j = 0; j < kI8ChunkTokens; ++j) {
            const int m = m_base + c + j;
            if (m < p.M)
              y[static_cast<int64_t>(m) * p.ldy + n] =
                  from_float<T>((static_cast<float>(static_cast<int>(r[j])) * scale_p[c + j]) * w_scale);
          }
        }
      }
      if (!released) {
        // a short last tile left this group without a chunk: it still owes its arrivals
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8 * b);
      }
    }
    if (issuer) tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(2 * p.acc_cols));
  }
}

// One block per activation row: fp32 max |x|, then the quantised row.
template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_int8_kernel(const T* __restrict__ x, int64_t ldx, int K,
                                                                 int8_t* __restrict__ q, int64_t ldq,
                                                                 float* __restrict__ scales) {
  const int m = blockIdx.x;
  const T* row = x + static_cast<int64_t>(m) * ldx;
  float peak = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) peak = fmaxf(peak, fabsf(static_cast<float>(row[k])));
  for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  __shared__ float warp_peak[8];
  if ((threadIdx.x & 31) == 0) warp_peak[threadIdx.x >> 5] = peak;
  __syncthreads();
  peak = warp_peak[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) peak = fmaxf(peak, warp_peak[w]);
  const float scale = fmaxf(peak, 1e-8f) * (1.0f / 127.0f);   // tensor / scalar on the reference's device
  if (threadIdx.x == 0) scales[m] = scale;
  int8_t* out = q + static_cast<int64_t>(m) * ldq;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float v = rintf(__fdiv_rn(static_cast<float>(row[k]), scale));
    out[k] = static_cast<int8_t>(fminf(fmaxf(v, -127.0f), 127.0f));
  }
}

// The same for 16-bit activations with 16-byte aligned rows: eight values per load, the row kept
// in registers between the two passes (rows longer than 256 x 8 x kHeld values re-read the
// rest, which the L2 still holds), eight int8 per store.
constexpr int kQuantHeld = 6;

template <typename T>
__device__ __forceinline__ float2 pair_to_float2(uint32_t w);
template <>
__device__ __forceinline__ float2 pair_to_float2<__half>(uint32_t w) {
  return __half22float2(as_h2(w));
}
template <>
__device__ __forceinline__ float2 pair_to_float2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

__device__ __forceinline__ uint32_t quantise4(float a, float b, float c, float d, float scale) {
  auto one = [scale](float v) {
    return static_cast<uint32_t>(static_cast<int>(fminf(fmaxf(rintf(__fdiv_rn(v, scale)), -127.0f), 127.0f))) & 0xFFu;
  };
  return one(a) | (one(b) << 8) | (one(c) << 16) | (one(d) << 24);
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_int8_vec_kernel(const T* __restrict__ x, int64_t ldx, int K,
                                                                     int8_t* __restrict__ q, int64_t ldq,
                                                                     float* __restrict__ scales) {
  const int m = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(m) * ldx);
  const int vecs = K / 8;
  uint4 held[kQuantHeld];
  float peak = 0.0f;
  auto absmax = [&peak](const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = pair_to_float2<T>(w[i]);
      peak = fmaxf(peak, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  };
#pragma unroll
  for (int h = 0; h < kQuantHeld; ++h) {
    const int v = threadIdx.x + h * 256;
    held[h] = v < vecs ? __ldg(row + v) : make_uint4(0u, 0u, 0u, 0u);
    absmax(held[h]);
  }
  for (int v = threadIdx.x + kQuantHeld * 256; v < vecs; v += 256) absmax(__ldg(row + v));
  for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  __shared__ float warp_peak[8];
  if ((threadIdx.x & 31) == 0) warp_peak[threadIdx.x >> 5] = peak;
  __syncthreads();
  peak = warp_peak[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) peak = fmaxf(peak, warp_peak[w]);
  const float scale = fmaxf(peak, 1e-8f) * (1.0f / 127.0f);   // tensor / scalar on the reference's device
  if (threadIdx.x == 0) scales[m] = scale;
  uint2* out = reinterpret_cast<uint2*>(q + static_cast<int64_t>(m) * ldq);
  auto emit = [&](int v, const uint4& in) {
    const float2 a = pair_to_float2<T>(in.x), b = pair_to_float2<T>(in.y);
    const float2 c = pair_to_float2<T>(in.z), d = pair_to_float2<T>(in.w);
    out[v] = make_uint2(quantise4(a.x, a.y, b.x, b.y, scale), quantise4(c.x, c.y, d.x, d.y, scale));
  };
#pragma unroll
  for (int h = 0; h < kQuantHeld; ++h) {
    const int v = threadIdx.x + h * 256;
    if (v < vecs) emit(v, held[h]);
  }
  for (int v = threadIdx.x + kQuantHeld * 256; v < vecs; v += 256) emit(v, __ldg(row + v));
}

// Short rows (at most 32 x 8 x kQuantWarpHeld values): one WARP per row, eight rows per block, the
// whole row in registers, no block barrier.
constexpr int kQuantWarpHeld = 8;

template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_int8_warp_kernel(const T* __restrict__ x, int64_t ldx, int M, int K,
                                                                      int8_t* __restrict__ q, int64_t ldq,
                                                                      float* __restrict__ scales) {
  const int m = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(m) * ldx);
  const int vecs = K / 8;
  uint4 held[kQuantWarpHeld];
  float peak = 0.0f;
#pragma unroll
  for (int h = 0; h < kQuantWarpHeld; ++h) {
    const int v = lane + h * 32;
    held[h] = v < vecs ? __ldg(row + v) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t w[4] = {held[h].x, held[h].y, held[h].z, held[h].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = pair_to_float2<T>(w[i]);
      peak = fmaxf(peak, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  const float scale = fmaxf(peak, 1e-8f) * (1.0f / 127.0f);   // tensor / scalar on the reference's device
  if (lane == 0) scales[m] = scale;
  uint2* out = reinterpret_cast<uint2*>(q + static_cast<int64_t>(m) * ldq);
#pragma unroll
  for (int h = 0; h < kQuantWarpHeld; ++h) {
    const int v = lane + h * 32;
    if (v < vecs) {
      const float2 a = pair_to_float2<T>(held[h].x), b = pair_to_float2<T>(held[h].y);
      const float2 c = pair_to_float2<T>(held[h].z), d = pair_to_float2<T>(held[h].w);
      out[v] = make_uint2(quantise4(a.x, a.y, b.x, b.y, scale), quantise4(c.x, c.y, d.x, d.y, scale));
    }
  }
}

template <typename T>
static void launch_quantize_rows_16bit(const void* x, int64_t ldx, int M, int K, int8_t* q, int64_t ldq, float* scales,
                                       cudaStream_t stream) {
  const bool vec = K % 8 == 0 && ldx % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && ldq % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(q) % 8 == 0;
  if (vec && K <= 32 * 8 * kQuantWarpHeld && M >= 64)
    quantize_rows_int8_warp_kernel<T><<<(M + 7) / 8, 256, 0, stream>>>(static_cast<const T*>(x), ldx, M, K, q, ldq,
                                                                      scales);
  else if (vec)
    quantize_rows_int8_vec_kernel<T><<<M, 256, 0, stream>>>(static_cast<const T*>(x), ldx, K, q, ldq, scales);
  else
    quantize_rows_int8_kernel<T><<<M, 256, 0, stream>>>(static_cast<const T*>(x), ldx, K, q, ldq, scales);
}

int launch_quantize_rows_int8(const void* x, int64_t ldx, int act_dtype, int M, int K, int8_t* q, int64_t ldq,
                              float* scales, cudaStream_t stream) {
  if (act_dtype == B200Q_F16)
    launch_quantize_rows_16bit<__half>(x, ldx, M, K, q, ldq, scales, stream);
  else if (act_dtype == B200Q_BF16)
    launch_quantize_rows_16bit<__nv_bfloat16>(x, ldx, M, K, q, ldq, scales, stream);
  else if (act_dtype == B200Q_F32)
    quantize_rows_int8_kernel<float><<<M, 256, 0, stream>>>(static_cast<const float*>(x), ldx, K, q, ldq, scales);
  else
    return B200Q_ERR_INVALID;
  return note_launch();
}

static int i8_sm_count() {
  static int counts[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148;
    }
    counts[dev] = n;
  }
  return counts[dev];
}

template <typename T>
static int launch_w8a8_typed(const I8Params& base, const int8_t* qx, int64_t ldq, const int8_t* qw, int64_t ldw,
                             int K, size_t smem, int grid, cudaStream_t stream) {
  static bool attr_set_dev[64] = {};
  static std::mutex attr_mu;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> g(attr_mu);
    if (!attr_set_dev[dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kI8SmemBudget));
      if (e != cudaSuccess) {
        set_last_error("cudaFuncSetAttribute", e);
        return B200Q_ERR_CUDA;
      }
      attr_set_dev[dev & 63] = true;
    }
  }
  CUtensorMap tm_w, tm_x, tm_y;
  // both operands as {K int8, rows}: a box is one 128-byte K block of a tile, 128-byte swizzle;
  // bytes past K (a ragged last block) and rows past the matrix read as zero
  if (!get_tensor_map(&tm_w, qw, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<uint64_t>(K),
                      static_cast<uint64_t>(base.N), 1, static_cast<uint64_t>(ldw),
                      static_cast<uint64_t>(ldw) * base.N, 128, kBlockN, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200Q_ERR_CUDA;
  if (!get_tensor_map(&tm_x, qx, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<uint64_t>(K),
                      static_cast<uint64_t>(base.M), 1, static_cast<uint64_t>(ldq),
                      static_cast<uint64_t>(ldq) * base.M, 128, static_cast<uint32_t>(base.tok), 1,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return B200Q_ERR_CUDA;
  tm_y = tm_x;
  if (base.tma_out) {
    const CUtensorMapDataType ydt =
        std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    // output as {N channels, M rows}: a box is one staged chunk, [32 tokens x 128 channels]
    if (!get_tensor_map(&tm_y, base.y, ydt, static_cast<uint64_t>(base.N), static_cast<uint64_t>(base.M), 1,
                        static_cast<uint64_t>(base.ldy) * 2, static_cast<uint64_t>(base.ldy) * 2 * base.M, kBlockN,
                        kI8ChunkTokens, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200Q_ERR_CUDA;
  }
  w8a8_gemm_kernel<T><<<grid, kI8Threads, smem, stream>>>(tm_w, tm_x, tm_y, base);
  return note_launch();
}

int launch_forward_w8a8(const int8_t* qx, int64_t ldq, const float* a_scales, const int8_t* qw, int64_t ldw,
                        const void* w_scales, int w_scale_dtype, void* y, int64_t ldy, int out_dtype, int M, int N,
                        int K, unsigned* status, cudaStream_t stream) {
  if (K % 16) return B200Q_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(qx) % 16 || ldq % 16 || reinterpret_cast<uintptr_t>(qw) % 16 || ldw % 16)
    return B200Q_ERR_ALIGNMENT;
  I8Params p{};
  p.a_scales = a_scales;
  p.w_scales = w_scales;
  p.w_scale_is_f32 = w_scale_dtype == B200Q_F32;
  p.y = y;
  p.ldy = ldy;
  p.M = M;
  p.N = N;
  // token tiles of equal size, a multiple of the 32-token store chunk
  p.m_tiles = (M + kI8MaxTok - 1) / kI8MaxTok;
  p.tok = ((M + p.m_tiles - 1) / p.m_tiles + kI8ChunkTokens - 1) / kI8ChunkTokens * kI8ChunkTokens;
  p.m_tiles = (M + p.tok - 1) / p.tok;
  const int n_tiles = (N + kBlockN - 1) / kBlockN;
  if (static_cast<int64_t>(p.m_tiles) * n_tiles > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;
  p.total_tiles = p.m_tiles * n_tiles;
  p.kb_total = (K + 127) / 128;
  const size_t stage = static_cast<size_t>(kBlockN) * 128 + static_cast<size_t>(p.tok) * 128;
  p.stages = static_cast<int>(std::min<size_t>(kI8MaxStages, (kI8SmemBudget - 1024 - kI8FixedBytes) / stage));
  int cols = 32;
  while (cols < p.tok) cols <<= 1;
  p.acc_cols = cols;
  p.tma_out = (reinterpret_cast<uintptr_t>(y) % 16 == 0 && ldy % 8 == 0) ? 1 : 0;
  p.idesc = umma_idesc_i8(128u, static_cast<uint32_t>(p.tok));
  p.status = status;
  const size_t smem = 1024 + static_cast<size_t>(p.stages) * stage + kI8FixedBytes;
  const int grid = std::min(p.total_tiles, i8_sm_count());
  if (debug_plan_enabled())
    std::fprintf(stderr,
                 "b200q plan: w8a8 kernel M %d N %d K %d | tok %d tiles %dx%d on %d blocks, stages %d smem %zu tmem %d "
                 "%s\n",
                 M, N, K, p.tok, p.m_tiles, n_tiles, grid, p.stages, smem, 2 * p.acc_cols,
                 p.tma_out ? "tma stores" : "direct stores");
  return out_dtype == B200Q_F16 ? launch_w8a8_typed<__half>(p, qx, ldq, qw, ldw, K, smem, grid, stream)
                                : launch_w8a8_typed<__nv_bfloat16>(p, qx, ldq, qw, ldw, K, smem, grid, stream);
}

}  // namespace b200q
