// Persistent stream-K weight-only linear for decode-sized token counts (M <= 64) on sm_100a.
//
// The problem is cut into UNITS of one weight tile x one K block (128 output channels x 128
// K: 8 KB of packed int4, 16 KB of int8).  The grid is at most one block per SM and block b
// owns the contiguous unit range [b U / G, (b + 1) U / G) in (tile, K block) order, so every
// block streams the same number of weight bytes whatever the shape: there is no tail wave and
// no split-K plan.  A run of a block's units inside one tile is a SEGMENT; a segment that
// covers the tile's whole K is stored directly.  Otherwise the first block of the tile (the
// one whose range ENDS in it, so it gets there last) owns the output: it adds the partials of
// the tile's other blocks to its own accumulator in block order — fixed order, so results are
// reproducible — and stores.  The others park their fp32 partials in the workspace as
// self-validating words (a word of 0 means "not written"), which the owner polls directly:
// no fence, no flag, no atomic, because under a saturated memory system every dependent trip
// to L2 costs about a microsecond.  An owner only ever waits for higher-numbered blocks of its
// own grid (bounded), and the grid is at most one block per SM, so they are resident.
//
// A block uses at most half of an SM (448 threads, <= 72 registers, <= 113 KB of shared
// memory when the ring allows it, 256 TMEM columns), so the NEXT kernel of the stream
// (programmatic dependent launch) becomes resident beside it and pre-fills its own weight
// ring while this one drains: the HBM stream does not stop at kernel boundaries.
//
// Warp roles:
//   warp 0       TMA producer feeding three rings: per unit one box of packed weights
//                (64-byte swizzle); per eight K blocks of a tile one box of scales (and
//                zero-points) [128 rows x 8 groups]; per unit one box of activations ([2 atoms]
//                x [TOK rows] x [64 elements], 128-byte swizzle).  With static weights the
//                weight and scale rings fill BEFORE the stream-order wait, and the dequantise
//                groups already unpack them into tensor memory; only the activations wait
//   warp 1       TMEM allocation, tcgen05.mma issue (one elected thread), commits
//   warps 2-5    epilogue: tcgen05.ld of a finished segment (the accumulator is handed back
//                to the MMA warp as soon as it is in registers), then park the partial, or
//                collect the other blocks' partials, scale/bias and store
//   warps 6-13   two dequantise groups of four warps; a group takes every other unit, each
//                thread one output channel (its TMEM lane) x the unit's 128 K: packed row out
//                of shared memory, unpack in registers, A operand (activation dtype) into tensor memory
//
// D[128 channels, TOK] (fp32, TMEM) += Wd[128, 16] (TMEM) * X[TOK, 16]^T (smem).
//
// Reference counterparts: _w4a16_gemv_kernel / _w4a16_linear_kernel
// (engine/kernels/w4a16_linear.py:27-74, 120-177) and _w8a16_linear_kernel
// (engine/kernels/w8a16_linear.py:10-40) at decode widths.
#include <algorithm>
#include <cstdio>
#include <mutex>

#include "tc_common.cuh"

namespace b200q {

constexpr int kSkGroups = 2;                                   // dequantise groups
constexpr int kSkThreads = 32 * (2 + 4 + 4 * kSkGroups);       // 448
constexpr int kSkMaxStages = 16;                               // weight ring
constexpr int kSkXStages = 4;                                  // activation ring (most; wide token tiles take two)
constexpr int kSkSStages = 3;                                  // scale-chunk ring (4-bit formats)
constexpr int kSkAStages = 3;                                  // operand stages in tensor memory
constexpr int kSkMaxTok = 64;
constexpr int kSkTmemCols = 256;                               // accumulator [0, 64), operand stages [64, 256)
constexpr int kSkACol0 = 64;
constexpr int kSkBarrierBytes = 512;
static_assert(8 * (2 * kSkMaxStages + 2 * kSkXStages + 2 * kSkSStages + 2 * kSkAStages + 3) + 16 <= kSkBarrierBytes,
              "the barrier region holds every ring's barriers");
static_assert(kSkACol0 + 64 * kSkAStages <= kSkTmemCols, "operand stages fit the tensor memory allocation");
constexpr int kSkMaxGrid = 160;                                // blocks the exchange region has slots for
static_assert(static_cast<size_t>(kSkMaxGrid) * kSkMaxTok * kBlockN * sizeof(uint32_t) <= kWsExchangeBytes,
              "the exchange region holds one partial per block");
constexpr size_t kSkHalfSm = 115712;                           // (228 KiB - 2 x 1 KiB reserved) / 2
constexpr size_t kSkFullSm = 226 * 1024;
constexpr int kSkChunkBytes = kBlockN * 16;                    // eight fp16 group parameters of 128 rows

struct SkParams {
  const void* scales;
  int scale_is_f32;
  const void* bias;
  void* y;
  int64_t ldy;
  int M, N, K;
  int tok;               // UMMA N: token rows per tile, multiple of 16, <= 64
  int kb_total;          // K / 128
  uint32_t total_units;  // weight tiles x K blocks
  int stages;            // weight ring depth
  int x_stages;          // activation ring depth
  uint32_t idesc;
  int static_weights;
  int swiglu;
  uint32_t* exchange;    // [grid][tok][128] encoded fp32 partials, all zero between launches
  unsigned* status;
};

__device__ __forceinline__ uint32_t sk_owner(uint32_t unit, uint32_t grid, uint32_t units) {
  // the block whose range [b U / G, (b + 1) U / G) holds `unit`
  return static_cast<uint32_t>(((static_cast<uint64_t>(unit) + 1) * grid - 1) / units);
}
__device__ __forceinline__ uint32_t sk_first_unit(uint32_t block, uint32_t grid, uint32_t units) {
  return static_cast<uint32_t>(static_cast<uint64_t>(block) * units / grid);
}

// Partials travel between blocks as self-validating words: an fp32 value v is stored as
// bits(v + 0.0f) ^ 0x80000000, which is never 0 (v + 0.0f turns -0.0 into +0.0, so the only
// pattern that would map to 0 cannot occur), and 0 means "not written yet".  The reader polls
// the data itself, so the writer needs no fence and no flag, and puts the word back to 0.
__device__ __forceinline__ uint32_t sk_encode(float v) { return __float_as_uint(v + 0.0f) ^ 0x80000000u; }
__device__ __forceinline__ float sk_decode(uint32_t w) { return __uint_as_float(w ^ 0x80000000u); }
constexpr uint32_t kSkExchangePolls = 1u << 15;          // x ~1 us per look: gives up after tens of milliseconds
__device__ __forceinline__ uint32_t ld_relaxed_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Untiled bulk copy global -> shared of this block (both 16-byte aligned, size a multiple of
// 16 bytes), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// AND of a predicate over the 128 epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool mine) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.and.pred p, 1, 128, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(mine))
      : "memory");
  return out != 0;
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int FMT, typename T>
__global__ void __launch_bounds__(kSkThreads, 2)
wq_gemm_sk_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_z,
                  const SkParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int kWBytes = PackedStage<FMT>::kBytes;
  constexpr bool kGroups = FMT != FMT_W8;                          // per-group scales to fetch
  constexpr int kSBytes = kGroups ? kSkChunkBytes * (FMT == FMT_W4_ASYM ? 2 : 1) : 0;
  const int x_atom_bytes = p.tok * 128;                            // one 64-wide K atom of [tok x 128 B]
  const int x_bytes = 2 * x_atom_bytes;
  const int S = p.stages;
  const uint32_t x_ring = smem_base;                               // 1024-byte aligned atoms
  const uint32_t w_ring = x_ring + p.x_stages * x_bytes;
  const uint32_t s_ring = w_ring + S * kWBytes;
  const uint32_t bars = s_ring + kSkSStages * kSBytes;
  const uint32_t w_full = bars;                                    // [kSkMaxStages]
  const uint32_t w_empty = w_full + 8 * kSkMaxStages;              // 4 arrivals: the warps of one group
  const uint32_t x_full = w_empty + 8 * kSkMaxStages;              // [kSkXStages]
  const uint32_t x_empty = x_full + 8 * kSkXStages;                // MMA commit
  const uint32_t s_full = x_empty + 8 * kSkXStages;                // [kSkSStages]
  const uint32_t s_empty = s_full + 8 * kSkSStages;                // 8 arrivals: every dequantise warp
  const uint32_t a_full = s_empty + 8 * kSkSStages;                // [kSkAStages], 4 arrivals
  const uint32_t a_empty = a_full + 8 * kSkAStages;                // MMA commit
  const uint32_t acc_full = a_empty + 8 * kSkAStages;              // MMA commit
  const uint32_t acc_empty = acc_full + 8;                         // 4 arrivals: the epilogue warps
  const uint32_t xg_full = acc_empty + 8;                          // staged partials of other blocks landed
  const uint32_t tmem_slot = xg_full + 8;
  const uint32_t abort_slot = tmem_slot + 4;
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(generic_base + (tmem_slot - smem_base));
  volatile int* abort_p = reinterpret_cast<volatile int*>(generic_base + (abort_slot - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t U = p.total_units, G = gridDim.x;
  const uint32_t u0 = sk_first_unit(blockIdx.x, G, U);
  const uint32_t u1 = sk_first_unit(blockIdx.x + 1, G, U);
  const int n_units = static_cast<int>(u1 - u0);
  const int KB = p.kb_total;
  const int tile0 = static_cast<int>(u0 / static_cast<uint32_t>(KB));
  const int kbi0 = static_cast<int>(u0 - static_cast<uint32_t>(tile0) * KB);

  if (warp == 0) {
    if (lane < kSkMaxStages) {
      mbar_init(w_full + 8 * lane, 1);
      mbar_init(w_empty + 8 * lane, 4);
    }
    if (lane < kSkXStages) {
      mbar_init(x_full + 8 * lane, 1);
      mbar_init(x_empty + 8 * lane, 1);
    }
    if (lane < kSkSStages) {
      mbar_init(s_full + 8 * lane, 1);
      mbar_init(s_empty + 8 * lane, 4 * kSkGroups);
    }
    if (lane < kSkAStages) {
      mbar_init(a_full + 8 * lane, 4);
      mbar_init(a_empty + 8 * lane, 1);
    }
    if (lane == 0) {
      mbar_init(acc_full, 1);
      mbar_init(acc_empty, 4);
      mbar_init(xg_full, 1);
      *abort_p = 0;
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      if (kGroups) tma_prefetch_desc(&tm_s);
      if (FMT == FMT_W4_ASYM) tma_prefetch_desc(&tm_z);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kSkTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_p;
  // Let the next kernel of the stream become resident now; it orders itself behind this grid
  // with griddepcontrol.wait before it touches anything this grid writes.
  if (threadIdx.x == 0) grid_launch_dependents();
  // With static weights the weight stream (and its dequantisation into tensor memory) may
  // start before the previous kernel in the stream has finished; activations, outputs and the
  // workspace always wait for it.
  if (!p.static_weights) grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // One thread feeds three rings, polling whichever has a free slot: packed weights (one
    // unit per slot), the scale chunks of the 4-bit formats (eight groups x 128 rows, fetched
    // when a unit begins a new chunk) and activations (one K block per slot; only after the
    // stream-order wait).
    if (elect_one()) {
      int iw = 0, ix = 0, ic = 0;                    // units with weights / activations issued, chunks issued
      int sw = 0, sx = 0, sc = 0;                    // ring slots
      uint32_t pw = 1, px = 1, pc = 1;               // parity to wait for on the empty barriers
      int w_tile = tile0, w_kb = kbi0, x_kb = kbi0;
      bool chunk_done = false;                       // the chunk that unit iw begins has been issued
      bool waited = !p.static_weights;
      bool ok = true;
      uint32_t idle = 0;
      while (iw < n_units || ix < n_units) {
        bool progress = false;
        if (iw < n_units) {
          const bool chunk_start = kGroups && (iw == 0 || (w_kb & 7) == 0);
          if (chunk_start && !chunk_done && mbar_test_wait(s_empty + 8 * sc, pc)) {
            mbar_arrive_expect_tx(s_full + 8 * sc, static_cast<uint32_t>(kSBytes));
            tma_load_3d(s_ring + sc * kSBytes, &tm_s, s_full + 8 * sc, (w_kb >> 3) * 8, w_tile * kBlockN, 0);
            if (FMT == FMT_W4_ASYM)
              tma_load_3d(s_ring + sc * kSBytes + kSkChunkBytes, &tm_z, s_full + 8 * sc, (w_kb >> 3) * 8,
                          w_tile * kBlockN, 0);
            chunk_done = true;
            ++ic;
            if (++sc == kSkSStages) {
              sc = 0;
              pc ^= 1;
            }
            progress = true;
          }
          if ((!chunk_start || chunk_done) && mbar_test_wait(w_empty + 8 * sw, pw)) {
            mbar_arrive_expect_tx(w_full + 8 * sw, static_cast<uint32_t>(kWBytes));
            tma_load_3d(w_ring + sw * kWBytes, &tm_w, w_full + 8 * sw, 0, w_tile * kBlockN,
                        (FMT == FMT_W8) ? 2 * w_kb : w_kb);
            ++iw;
            chunk_done = false;
            if (++w_kb == KB) {
              w_kb = 0;
              ++w_tile;
            }
            if (++sw == S) {
              sw = 0;
              pw ^= 1;
            }
            progress = true;
          }
        }
        if (!waited && (iw == n_units || !progress)) {
          // the weight ring is as far ahead as it can get: now order behind the stream
          grid_dependency_wait();
          waited = true;
          progress = true;
        }
        if (waited && ix < n_units && mbar_test_wait(x_empty + 8 * sx, px)) {
          mbar_arrive_expect_tx(x_full + 8 * sx, static_cast<uint32_t>(x_bytes));
          tma_load_3d(x_ring + sx * x_bytes, &tm_x, x_full + 8 * sx, 0, 0, 2 * x_kb);
          ++ix;
          if (++x_kb == KB) x_kb = 0;
          if (++sx == p.x_stages) {
            sx = 0;
            px ^= 1;
          }
          progress = true;
        }
        if (progress) {
          idle = 0;
        } else {
          // nothing to do: step aside so this poll loop does not take issue slots from the
          // dequantising warps that share the scheduler
          __nanosleep(32);
          if (++idle > kMaxPolls || ((idle & 0x3FF) == 0 && *abort_p)) {
            ok = false;
            break;
          }
        }
      }
      if (!ok) flag_failure(abort_p, p.status, 1u);
      if (*abort_p) {
        // let the copies already in flight land before the block's shared memory is released
        for (int j = max(0, iw - S); j < iw; ++j) mbar_wait(w_full + 8 * (j % S), (j / S) & 1);
        for (int j = max(0, ix - p.x_stages); j < ix; ++j) mbar_wait(x_full + 8 * (j % p.x_stages), (j / p.x_stages) & 1);
        for (int j = max(0, ic - kSkSStages); j < ic; ++j) mbar_wait(s_full + 8 * (j % kSkSStages), (j / kSkSStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // One thread, and every instruction of it is on the block's critical path (a dependent
    // scalar sequence issues one instruction every several cycles beside the dequantise warps'
    // bursts): descriptors and ring positions advance incrementally, a segment is counted down.
    if (elect_one()) {
      bool ok = true;
      int sx = 0, as = 0;
      uint32_t x_phase = 0, a_phase = 0, acc_phase = 1;   // acc_phase: parity to wait for on acc_empty
      int seg_left = min(KB - kbi0, n_units);             // units left in the current segment (tile)
      int after_seg = n_units - seg_left;                 // units after it
      bool seg_first = true;
      const uint64_t x_desc0 = umma_desc_sw128(x_ring);
      const uint64_t x_step = static_cast<uint64_t>(x_bytes >> 4), atom_step = static_cast<uint64_t>(x_atom_bytes >> 4);
      uint64_t x_desc = x_desc0;
      const uint32_t a_tmem0 = tmem_base + kSkACol0;
      uint32_t a_tmem = a_tmem0;
      for (int i = 0; i < n_units; ++i) {
        if (seg_first) {
          // the epilogue has read the previous segment out of the accumulator
          ok = wait_or_abort(acc_empty, acc_phase, abort_p);
          if (!ok) break;
          acc_phase ^= 1u;
        }
        ok = wait_or_abort(x_full + 8 * sx, x_phase, abort_p) && wait_or_abort(a_full + 8 * as, a_phase, abort_p);
        if (!ok) break;
        tc_fence_after_sync();
        // operand stage `as` holds 128 K elements as 64 columns, 8 per MMA; two 64-K atoms of activations
        umma_f16_ts(tmem_base, a_tmem, x_desc, p.idesc, seg_first ? 0u : 1u);
#pragma unroll
        for (int k = 1; k < 4; ++k) umma_f16_ts(tmem_base, a_tmem + 8 * k, x_desc + 2 * k, p.idesc, 1u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem_base, a_tmem + 32 + 8 * k, x_desc + atom_step + 2 * k, p.idesc, 1u);
        umma_commit(a_empty + 8 * as);
        umma_commit(x_empty + 8 * sx);
        seg_first = --seg_left == 0;
        if (seg_first) {
          umma_commit(acc_full);
          seg_left = min(KB, after_seg);
          after_seg -= seg_left;
        }
        x_desc += x_step;
        if (++sx == p.x_stages) {
          sx = 0;
          x_phase ^= 1;
          x_desc = x_desc0;
        }
        a_tmem += 64;
        if (++as == kSkAStages) {
          as = 0;
          a_phase ^= 1;
          a_tmem = a_tmem0;
        }
      }
      if (!ok) flag_failure(abort_p, p.status, 2u);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue warps
    grid_dependency_wait();              // outputs and the workspace belong to the stream order
    const int quarter = warp & 3;        // TMEM lanes this warp may read
    const int ch = quarter * 32 + lane;  // channel inside the tile
    const uint32_t acc_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int rows = min(p.tok, p.M);
    T* const y = static_cast<T*>(p.y);
    bool ok = true;
    int tile = tile0, kb = kbi0, left = n_units;
    uint32_t acc_phase = 0, xg_phase = 0;
    // one finished fp32 value of this thread's channel -> the output (all lanes take part)
    auto emit = [&](int m, int n, float v) {
      if (p.swiglu) {
        // neighbouring lanes hold the gate (even row) and the up (odd row) of one output channel
        const float up = __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 1) == 0 && n < p.N) y[static_cast<int64_t>(m) * p.ldy + (n >> 1)] = from_float<T>(swiglu_pair(v, up));
      } else if (n < p.N) {
        y[static_cast<int64_t>(m) * p.ldy + n] = from_float<T>(v);
      }
    };
    while (left > 0) {
      const int len = min(left, KB - kb);
      const int n = tile * kBlockN + ch;
      // Who else works on this tile: blocks b_lo .. b_hi in unit order.  b_lo (for which the
      // tile is the END of its range, so it finishes it last) owns the tile's output and adds
      // the others' partials in block order; every other block parks its partial in its own
      // exchange slot (a block contributes to at most one tile it does not own: the one under
      // way at the start of its range).
      const uint32_t first = static_cast<uint32_t>(tile) * KB;
      const uint32_t b_lo = (len == KB) ? blockIdx.x : sk_owner(first, G, U);
      const uint32_t b_hi = (len == KB) ? blockIdx.x : sk_owner(first + KB - 1, G, U);
      const bool owner = b_lo == blockIdx.x;
      float ch_scale = 1.0f, ch_bias = 0.0f;
      if (owner && n < p.N) {
        if (FMT == FMT_W8)
          ch_scale = p.scale_is_f32 ? reinterpret_cast<const float*>(p.scales)[n]
                                    : __half2float(reinterpret_cast<const __half*>(p.scales)[n]);
        if (p.bias != nullptr) ch_bias = static_cast<float>(static_cast<const T*>(p.bias)[n]);
      }
      const size_t per_slot = static_cast<size_t>(p.tok) * kBlockN;
      uint32_t* mine = p.exchange + static_cast<size_t>(blockIdx.x) * per_slot + ch;
      const bool collect = owner && b_hi > b_lo;   // only ever a block's last segment: the rings drain
      // Up to sixteen token rows: the other blocks' partials are pulled into registers NOW,
      // while this segment's MMAs are still running (the other blocks finished their part of
      // the tile earlier), so that nothing but the addition is left once the accumulator is
      // ready.  Every thread polls its own channel's words (bounded) and empties them.
      const bool early = collect && rows <= 16;
      float others[16];
#pragma unroll
      for (int m = 0; m < 16; ++m) others[m] = 0.0f;
      if (early) {
        for (uint32_t bb = b_lo + 1; bb <= b_hi; ++bb) {
          uint32_t* src = p.exchange + static_cast<size_t>(bb) * per_slot + ch;
          uint32_t v[16];
          bool all = false;
          for (uint32_t tries = 0; !all; ++tries) {
            all = true;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
              v[m] = (m < rows) ? ld_relaxed_gpu_u32(src + m * kBlockN) : 0x80000000u;
              all = all && v[m] != 0u;
            }
            if (!all) {
              if (tries >= kSkExchangePolls || *abort_p) {
                atomicOr(p.status, 16u);
                break;
              }
              __nanosleep(300);
            }
          }
#pragma unroll
          for (int m = 0; m < 16; ++m) {
            others[m] += sk_decode(v[m]);                            // block order; absent rows add +0.0f
            if (m < rows) __stcg(src + m * kBlockN, 0u);             // empty again for the next launch
          }
        }
      }
      if (ok) {
        ok = wait_or_abort(acc_full, acc_phase, abort_p);
        if (!ok) flag_failure(abort_p, p.status, 8u);
      }
      acc_phase ^= 1u;
      tc_fence_after_sync();
      // Read the accumulator out eight columns (token rows) at a time and hand it back to the
      // MMA warp as soon as the last of it is in registers.  A tile of this block alone goes
      // to the output; a partial is parked in this block's exchange slot; an owner's own part
      // goes to shared memory (the idle activation ring) to have the others' added to it.
      const uint32_t sum_buf = x_ring + ch * 4;                    // [token row][128 channels] fp32
      for (int c = 0; c < p.tok; c += 8) {
        uint32_t r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = 0u;
        if (ok) {
          tmem_ld_x8(acc_addr + c, r);
          tmem_ld_wait();
        }
        if (c + 8 >= p.tok) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty);
        }
        if (c >= rows) continue;
        if (collect && !early) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j < rows) st_shared_f32(sum_buf + (c + j) * 512, __uint_as_float(r[j]));
        } else if (owner) {
          // (c is 0 or 8 whenever `others` holds anything; otherwise it is all zeros)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float extra = c == 0 ? others[j] : (c == 8 ? others[8 + j] : 0.0f);
            if (c + j < rows) emit(c + j, n, (__uint_as_float(r[j]) + extra) * ch_scale + ch_bias);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j < rows) __stcg(mine + (c + j) * kBlockN, sk_encode(__uint_as_float(r[j])));
        }
      }
      if (collect && !early) {
        // More than sixteen token rows.  The other blocks' partials, a batch at a time: one bulk copy per block brings its
        // whole slot into the idle weight ring (every byte in flight at once: a look costs one
        // trip to L2 whatever the row count), every thread checks its channel's words, and
        // the look is repeated (bounded) until none reads as "not written".  Then they are
        // added in block order and the slots are put back to zero.
        const uint32_t slot_bytes = static_cast<uint32_t>(rows) * 512u;
        const uint32_t stride = static_cast<uint32_t>(p.tok) * 512u;
        const uint32_t room = static_cast<uint32_t>(S) * kWBytes / stride;
        const uint32_t batch = room < 4u ? (room < 1u ? 1u : room) : 4u;
        for (uint32_t bb = b_lo + 1; bb <= b_hi; bb += batch) {
          const uint32_t nb = min(batch, b_hi - bb + 1);
          bool all = false;
          for (uint32_t tries = 0; !all; ++tries) {
            if (threadIdx.x == 64) {
              mbar_arrive_expect_tx(xg_full, nb * slot_bytes);
              for (uint32_t z = 0; z < nb; ++z)
                bulk_load(w_ring + z * stride, p.exchange + static_cast<size_t>(bb + z) * per_slot, slot_bytes, xg_full);
            }
            bool landed = wait_or_abort(xg_full, xg_phase, abort_p);
            xg_phase ^= 1u;
            bool mine_ok = landed;
            for (uint32_t z = 0; z < nb && mine_ok; ++z)
              for (int m = 0; m < rows; ++m)
                mine_ok = mine_ok && __float_as_uint(ld_shared_f32(w_ring + z * stride + m * 512 + ch * 4)) != 0u;
            all = epilogue_all(mine_ok);
            if (!all) {
              if (tries >= kSkExchangePolls || !landed || *abort_p) {
                if (threadIdx.x == 64) atomicOr(p.status, 16u);
                break;
              }
              __nanosleep(500);
            }
          }
          for (uint32_t z = 0; z < nb; ++z) {
            uint32_t* slot = p.exchange + static_cast<size_t>(bb + z) * per_slot + ch;
            for (int m0 = 0; m0 < rows; m0 += 8) {
              float a[8], b[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const bool in = m0 + j < rows;
                a[j] = in ? ld_shared_f32(sum_buf + (m0 + j) * 512) : 0.0f;
                b[j] = in ? sk_decode(__float_as_uint(ld_shared_f32(w_ring + z * stride + (m0 + j) * 512 + ch * 4))) : 0.0f;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (m0 + j < rows) {
                  st_shared_f32(sum_buf + (m0 + j) * 512, a[j] + b[j]);
                  __stcg(slot + (m0 + j) * kBlockN, 0u);             // empty again for the next launch
                }
              }
            }
          }
          // every thread is done with the staged batch before the next one overwrites it
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        for (int m0 = 0; m0 < rows; m0 += 8) {
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = (m0 + j < rows) ? ld_shared_f32(sum_buf + (m0 + j) * 512) : 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (m0 + j < rows) emit(m0 + j, n, v[j] * ch_scale + ch_bias);
        }
      }
      left -= len;
      kb = 0;
      ++tile;
    }
  } else {
    // ------------------------------------------------------------ dequantise groups
    // A warp visits only the units of its group (ring positions advance by the group count: the
    // bookkeeping of a skipped unit cost as much issue time as it saved); every warp still
    // takes every scale chunk in order (its row's eight scales into registers), so a chunk slot
    // is released by exactly eight arrivals.  Unit j lies in chunk ((kbi0 + j) >> 3) - (kbi0 >> 3):
    // a tile's K blocks are a multiple of eight, so chunks never straddle tiles.
    const int g = (warp - 6) >> 2;                          // group: units g, g + 2, ...
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                    // channel inside the tile = TMEM lane
    const uint32_t row_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kSkACol0;
    const int xr = (row >> 1) & 3;                          // 64-byte swizzle term of this row
    uint4 cs = make_uint4(0u, 0u, 0u, 0u), cz = make_uint4(0u, 0u, 0u, 0u);   // the current chunk
    bool ok = true;
    // positions of this group's first unit (the rings are at least two deep, the operand stages three)
    int kb = kbi0 + g, sw = g, as = g, sc = 0;
    while (kb >= KB) kb -= KB;
    uint32_t w_phase = 0, ae_phase = 1, c_phase = 0;
    int chunks_taken = 0;                                   // scale chunks this warp has consumed
    for (int j = g; j < n_units && ok; j += kSkGroups) {
      if (kGroups) {
        const int chunk = ((kbi0 + j) >> 3) - (kbi0 >> 3);
        while (chunks_taken <= chunk) {                     // at most two steps: a group moves two units at a time
          ok = wait_or_abort(s_full + 8 * sc, c_phase, abort_p);
          if (!ok) break;
          cs = ld_shared_v4(s_ring + sc * kSBytes + row * 16);
          if (FMT == FMT_W4_ASYM) cz = ld_shared_v4(s_ring + sc * kSBytes + kSkChunkBytes + row * 16);
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + 8 * sc);
          if (++sc == kSkSStages) {
            sc = 0;
            c_phase ^= 1;
          }
          ++chunks_taken;
        }
        if (!ok) break;
      }
      {
        PairConsts gp{0u, 0u, 0u};
        if (kGroups)
          gp = make_pair_consts(pick_half(cs, kb & 7),
                                (FMT == FMT_W4_ASYM) ? __half2float(pick_half(cz, kb & 7)) : 8.0f);
        ok = wait_or_abort(w_full + 8 * sw, w_phase, abort_p);
        if (!ok) break;
        const uint32_t w_stage = w_ring + sw * kWBytes;
        const uint32_t a_stage_t = row_taddr + as * 64;
        if (FMT == FMT_W4_REF) {
          // 64 bytes of the row: byte j holds K j (low nibble) and K 64 + j (high nibble)
          const uint32_t prow = w_stage + row * 64;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint4 v = ld_shared_v4(prow + (((2 * h + c) ^ xr) << 4));
              const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                // bytes (b0,b1,b2,b3) -> (b0,b2,b1,b3): the masks then pick (b0,b1) from the
                // word and (b2,b3) from the word shifted by 8
                const uint32_t u = prmt(words[w], 0u, 0x3120);
                lo[(c * 4 + w) * 2] = deq_lo<T>(u, gp);
                lo[(c * 4 + w) * 2 + 1] = deq_lo<T>(u >> 8, gp);
                hi[(c * 4 + w) * 2] = deq_hi<T>(u, gp);
                hi[(c * 4 + w) * 2 + 1] = deq_hi<T>(u >> 8, gp);
              }
            }
            if (h == 0) {
              ok = wait_or_abort(a_empty + 8 * as, ae_phase, abort_p);
              if (!ok) break;
              tc_fence_after_sync();
            }
            tmem_st_x16(a_stage_t + 16 * h, lo);
            tmem_st_x16(a_stage_t + 32 + 16 * h, hi);
          }
        } else if (FMT == FMT_W4_ASYM) {
          // 16 words of the row, word w = K 8w .. 8w+7; the layout's nibble order makes every
          // lop3 pair a pair of K neighbours
          const uint32_t prow = w_stage + row * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v = ld_shared_v4(prow + ((c ^ xr) << 4));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
            uint32_t out[16];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const uint32_t u = words[w];
              out[w * 4 + 0] = deq_lo<T>(u, gp);        // inputs 0,1
              out[w * 4 + 1] = deq_hi<T>(u, gp);        // inputs 2,3
              out[w * 4 + 2] = deq_lo<T>(u >> 8, gp);   // inputs 4,5
              out[w * 4 + 3] = deq_hi<T>(u >> 8, gp);   // inputs 6,7
            }
            if (c == 0) {
              ok = wait_or_abort(a_empty + 8 * as, ae_phase, abort_p);
              if (!ok) break;
              tc_fence_after_sync();
            }
            tmem_st_x16(a_stage_t + 16 * c, out);
          }
        } else {
          // int8: two [128 x 64 B] sub-tiles (K 0..63, 64..127).  The integers enter the MMA
          // unscaled (exact in fp16 and bf16); the channel scale is applied to the accumulator.
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const uint32_t sub = w_stage + (h >> 1) * (kBlockN * 64) + row * 64;
            uint32_t out[16];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint4 v = ld_shared_v4(sub + (((2 * (h & 1) + c) ^ xr) << 4));
              const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                __half2 k01, k23;
                int8x4_to_h2(words[w], k01, k23);
                out[(c * 4 + w) * 2] = pack_operand<T>(k01);
                out[(c * 4 + w) * 2 + 1] = pack_operand<T>(k23);
              }
            }
            if (h == 0) {
              ok = wait_or_abort(a_empty + 8 * as, ae_phase, abort_p);
              if (!ok) break;
              tc_fence_after_sync();
            }
            tmem_st_x16(a_stage_t + 16 * h, out);
          }
        }
        if (!ok) break;
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(a_full + 8 * as);
          mbar_arrive(w_empty + 8 * sw);
        }
      }
      kb += kSkGroups;
      while (kb >= KB) kb -= KB;                          // (a one-block K wraps twice)
      sw += kSkGroups;
      if (sw >= S) {
        sw -= S;
        w_phase ^= 1;
      }
      as += kSkGroups;
      if (as >= kSkAStages) {
        as -= kSkAStages;
        ae_phase ^= 1;
      }
    }
    if (!ok) flag_failure(abort_p, p.status, 4u);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kSkTmemCols);
  }
}

// ---------------------------------------------------------------- host side
struct SkPlan {
  int tok, n_tiles, kb_total, stages, x_stages, grid;
  uint32_t units;
  size_t smem_bytes;
};

static int sm_count() {
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

static bool sk_geometry(int format, int M, int N, int K) {
  if (M <= 0 || M > kSkMaxTok || N <= 0 || K <= 0 || K % kBlockK) return false;
  if ((N + kBlockN - 1) / kBlockN > kMaxSplitTiles) return false;
  // scale chunks are fetched eight groups (16 bytes) at a time: whole chunks per row
  if (format != FMT_W8 && (K / kBlockK) % 8 != 0) return false;
  return true;
}

static SkPlan sk_plan(int format, int M, int N, int K, int sms) {
  SkPlan pl{};
  pl.tok = (M + 15) / 16 * 16;
  pl.n_tiles = (N + kBlockN - 1) / kBlockN;
  pl.kb_total = K / kBlockK;
  pl.units = static_cast<uint32_t>(pl.n_tiles) * static_cast<uint32_t>(pl.kb_total);
  // at least four units per block: a block's set-up must be worth its share
  const uint32_t want = pl.units / 4;
  pl.grid = static_cast<int>(std::max<uint32_t>(1u, std::min<uint32_t>(static_cast<uint32_t>(std::min(sms, kSkMaxGrid)), want)));
  // Shared memory: half an SM when that leaves the weight ring at least six stages (so that
  // the next kernel's block fits beside this one), otherwise the whole SM.
  const size_t w_stage = format == FMT_W8 ? kBlockN * 128 : kBlockN * 64;
  const size_t chunk = format == FMT_W8 ? 0 : static_cast<size_t>(kSkChunkBytes) * (format == FMT_W4_ASYM ? 2 : 1);
  // wide token tiles keep two activation stages (16 KB each at 64 rows; the collecting owner
  // needs rows x 512 bytes of the ring as its summing buffer), so that the block still fits half an SM
  pl.x_stages = pl.tok > 32 ? 2 : kSkXStages;
  const size_t fixed = 1024 + kSkBarrierBytes + static_cast<size_t>(pl.x_stages) * pl.tok * 256 + kSkSStages * chunk;
  int stages = kSkHalfSm > fixed ? static_cast<int>((kSkHalfSm - fixed) / w_stage) : 0;
  if (stages < 6) stages = static_cast<int>((kSkFullSm - fixed) / w_stage);
  pl.stages = std::max(2, std::min(stages, kSkMaxStages));
  pl.smem_bytes = fixed + static_cast<size_t>(pl.stages) * w_stage;
  return pl;
}

size_t sk_workspace_bytes(int format, int M, int N, int K) {
  if (!sk_geometry(format, M, N, K)) return 0;
  return kWsExchangeOffset + kWsExchangeBytes;
}

bool sk_supported(const ForwardArgs& a) {
  if (a.argmax) return false;
  if (a.gather != nullptr && a.gather->world > 1) return false;
  if (a.reduce != nullptr && a.reduce->world > 1) return false;
  if (a.format != FMT_W8) {
    if (a.group != 128) return false;
    if (reinterpret_cast<uintptr_t>(a.scales) % 16) return false;
    if (a.format == FMT_W4_ASYM && reinterpret_cast<uintptr_t>(a.zeros) % 16) return false;
  }
  return sk_geometry(a.format, a.M, a.N, a.K);
}

// Where the stream-K kernel measured faster than the tile kernel (B200, CUDA-graph replay over
// rotating weights): 4-bit weights at up to sixteen token rows when a weight tile is shared by
// few blocks (a block's share of units is at least half a tile's K), e.g. 4096 -> 12288 at
// M = 1 / 16: 12.3 / 14.2 us against 14.1 / 15.0.  It lost on int8 (4096 -> 12288 M = 16: 18.3
// against 16.9 us), on deep K (12288 -> 4096 M = 16: 17.2 against 16.0) and above sixteen rows.
bool sk_preferred(int format, int M, int N, int K) {
  if (format == FMT_W8 || M > 16 || !sk_geometry(format, M, N, K)) return false;
  const SkPlan pl = sk_plan(format, M, N, K, sm_count());
  return 2u * (pl.units / static_cast<uint32_t>(pl.grid)) >= static_cast<uint32_t>(pl.kb_total);
}

int sk_gather_arrivals(int, int, int, int) { return 0; }

bool sk_describe(int format, int M, int N, int K, char* text, size_t size) {
  if (!sk_geometry(format, M, N, K)) return false;
  const SkPlan pl = sk_plan(format, M, N, K, sm_count());
  std::snprintf(text, size, "wq_gemm_sk_kernel<%s> tok=%d units=%u grid=%d ring=%d smem=%zu",
                format == FMT_W8 ? "w8" : (format == FMT_W4_REF ? "w4_ref" : "w4_asym"), pl.tok, pl.units,
                pl.grid, pl.stages, pl.smem_bytes);
  return true;
}

template <int FMT, typename T>
static int launch_sk_typed(const ForwardArgs& a, const SkPlan& pl) {
  static bool attr_set_dev[64] = {};
  static std::mutex attr_mu;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    bool& attr_set = attr_set_dev[dev & 63];
    std::lock_guard<std::mutex> g(attr_mu);
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(wq_gemm_sk_kernel<FMT, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kSkFullSm));
      if (e != cudaSuccess) {
        set_last_error("cudaFuncSetAttribute", e);
        return B200Q_ERR_CUDA;
      }
      (void)cudaFuncSetAttribute(wq_gemm_sk_kernel<FMT, T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
      (void)cudaGetLastError();
      attr_set = true;
    }
  }
  CUtensorMap tm_w, tm_x;
  // Packed weights as {64 B, N rows, K chunks of 64 B}; one box is a unit: [128 rows x 64 B]
  // for int4, two such (K 0..63 and 64..127) for int8.  Read one row per thread: 64-byte swizzle.
  const uint64_t w_row_bytes = (FMT == FMT_W8) ? static_cast<uint64_t>(a.K) : static_cast<uint64_t>(a.K / 2);
  if (!get_tensor_map(&tm_w, a.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 64, static_cast<uint64_t>(a.N),
                      w_row_bytes / 64, static_cast<uint64_t>(a.ldw), 64, 64, kBlockN, (FMT == FMT_W8) ? 2u : 1u,
                      CU_TENSOR_MAP_SWIZZLE_64B))
    return B200Q_ERR_CUDA;
  // Activations as {64 elements, M rows, K atoms}: a box of depth 2 is one K block.
  const CUtensorMapDataType xdt = (a.act_dtype == B200Q_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!get_tensor_map(&tm_x, a.x, xdt, 64, static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K / 64),
                      static_cast<uint64_t>(a.ldx) * 2, 128, 64, static_cast<uint32_t>(pl.tok), 2,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return B200Q_ERR_CUDA;
  // Scales (and zero-points) as {K / 128 groups, N rows, 1} fp16: a box is eight groups of 128
  // rows, 16 bytes per row.
  CUtensorMap tm_s = tm_w, tm_z = tm_w;
  if (FMT != FMT_W8) {
    const uint64_t groups = static_cast<uint64_t>(a.K / 128);
    if (!get_tensor_map(&tm_s, a.scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, groups, static_cast<uint64_t>(a.N), 1,
                        groups * 2, groups * 2 * static_cast<uint64_t>(a.N), 8, kBlockN, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200Q_ERR_CUDA;
    tm_z = tm_s;
    if (FMT == FMT_W4_ASYM &&
        !get_tensor_map(&tm_z, a.zeros, CU_TENSOR_MAP_DATA_TYPE_UINT16, groups, static_cast<uint64_t>(a.N), 1,
                        groups * 2, groups * 2 * static_cast<uint64_t>(a.N), 8, kBlockN, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200Q_ERR_CUDA;
  }

  SkParams p{};
  p.scales = a.scales;
  p.scale_is_f32 = a.scale_dtype == B200Q_F32;
  p.bias = a.bias;
  p.y = a.y;
  p.ldy = a.ldy;
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.tok = pl.tok;
  p.kb_total = pl.kb_total;
  p.total_units = pl.units;
  p.stages = pl.stages;
  p.x_stages = pl.x_stages;
  const uint32_t ab_fmt = a.act_dtype == B200Q_F16 ? 0u : 1u;    // both operands in the activation dtype
  p.idesc = umma_idesc_f16(ab_fmt, ab_fmt, 128u, static_cast<uint32_t>(pl.tok));
  p.static_weights = a.static_weights ? 1 : 0;
  p.swiglu = a.swiglu ? 1 : 0;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  p.status = reinterpret_cast<unsigned*>(ws);
  p.exchange = reinterpret_cast<uint32_t*>(ws + kWsExchangeOffset);

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (debug_plan_enabled())
    std::fprintf(stderr,
                 "b200q plan: stream-K kernel fmt %d M %d N %d K %d | tok %d tiles %d kb %d units %u grid %d | "
                 "weight ring %d stages | smem %zu\n",
                 FMT, a.M, a.N, a.K, pl.tok, pl.n_tiles, pl.kb_total, pl.units, pl.grid, pl.stages, pl.smem_bytes);
  cudaError_t e = cudaLaunchKernelEx(&cfg, wq_gemm_sk_kernel<FMT, T>, tm_w, tm_x, tm_s, tm_z, p);
  if (e != cudaSuccess) {
    set_last_error("cudaLaunchKernelEx", e);
    return B200Q_ERR_CUDA;
  }
  return note_launch();
}

int launch_forward_sk(const ForwardArgs& a) {
  const SkPlan pl = sk_plan(a.format, a.M, a.N, a.K, sm_count());
  if (a.workspace == nullptr || a.workspace_bytes < kWsExchangeOffset + kWsExchangeBytes) return B200Q_ERR_WORKSPACE;
  const bool h = a.act_dtype == B200Q_F16;
  switch (a.format) {
    case FMT_W8:
      return h ? launch_sk_typed<FMT_W8, __half>(a, pl) : launch_sk_typed<FMT_W8, __nv_bfloat16>(a, pl);
    case FMT_W4_REF:
      return h ? launch_sk_typed<FMT_W4_REF, __half>(a, pl) : launch_sk_typed<FMT_W4_REF, __nv_bfloat16>(a, pl);
    case FMT_W4_ASYM:
      return h ? launch_sk_typed<FMT_W4_ASYM, __half>(a, pl) : launch_sk_typed<FMT_W4_ASYM, __nv_bfloat16>(a, pl);
    default:
      return B200Q_ERR_INVALID;
  }
}

}  // namespace b200q
