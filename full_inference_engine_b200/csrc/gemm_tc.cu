// Tensor-core weight-only linear for sm_100a, one block per output tile: tcgen05.mma with
// the WEIGHTS on the M side of the MMA and the tokens on the N side.
//
//   D[128 channels, TOK tokens] (fp32, TMEM) += Wd[128, 16] * X[TOK, 16]^T
//
// so a tile never pads the token count to 128: TOK is any multiple of 16 up to 256 and is
// chosen per call.  One block owns 128 output channels x TOK tokens x a K range (split-K
// over blockIdx.z when there are too few tiles to fill the GPU).  This kernel serves token
// tiles above 64 rows (prefill, mixed steps), the fused argmax and anything the persistent
// stream-K kernel (gemm_sk.cu) does not take.
//
// Warp roles (64 + 32 DW threads, DW = 8 or 16):
//   warp 0      TMA producer: rank-3 boxes of packed weights ([pg] x [128 rows] x [64 B],
//               64-byte swizzle) and of activations ([2 xg atoms] x [TOK rows] x [64 elements],
//               128-byte swizzle); one instruction fills a group of K blocks
//   warp 1      TMEM allocation, tcgen05.mma issue (one elected thread), commits
//   warps 2..   dequantise: each thread owns one output channel (its TMEM lane) and a K
//               slice, unpacks the packed stage out of shared memory in registers and writes
//               the A operand into TENSOR MEMORY (tcgen05.st); the MMA reads A from
//               TMEM and only the activations from shared memory.  Later the epilogue:
//               tcgen05.ld, scale/bias, one TMA store per finished tile (or split-K partials:
//               summed over distributed shared memory inside a cluster, or through the
//               workspace by the last block to arrive; counters reset for the next launch)
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
#include <unordered_map>

#include "tc_common.cuh"

namespace b200q {

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
  // plain forward ahead of a push kernel (a_world > 1, g_world == 0): only the "entered the
  // call" announcement is made here, early, so that the push kernel finds the peers ready
  int a_world, a_rank;
  // fused all-reduce of a row-parallel (K-sharded) forward (reduce != 0, g_world > 1): every
  // rank computes a partial [M, N]; the rank that owns a column block adds the other ranks'
  // partials (delivered into its inbox as self-validating fp32 words) in rank order and
  // stores the finished tile into every rank's y
  int reduce;
  int r_cols;                     // output columns owned by each rank (a multiple of 128)
  uint32_t* r_inbox[8];           // each rank's inbox: [world][M][r_cols] words, all zero between calls
  unsigned* counters;  // [m_tiles * n_tiles], zero between launches
  unsigned* status;    // device status word (non-zero: a bounded wait expired)
};

// Per-(row, group) parameters of the 4-bit formats, fetched eight groups at a time
// (one 16-byte load per row) one chunk ahead of use, so that their latency never sits
// between two pipeline stages.  When K/128 is not a multiple of 8 a chunk is one group.
struct GroupChunk {
  uint4 s;   // scales of the thread's row
  uint4 z;   // zero-points (asymmetric layout only)
};

template <int FMT>
__device__ __forceinline__ void load_group_chunk(GroupChunk& g, const TcParams& p, int chunk,
                                                 bool vec, int row) {
  g.s = make_uint4(0u, 0u, 0u, 0u);
  g.z = make_uint4(0u, 0u, 0u, 0u);
  if (row < p.N) {
    const int64_t base = static_cast<int64_t>(row) * p.groups;
    const __half* sp = reinterpret_cast<const __half*>(p.scales) + base;
    if (vec) {
      g.s = __ldg(reinterpret_cast<const uint4*>(sp + chunk * 8));
      if (FMT == FMT_W4_ASYM) g.z = __ldg(reinterpret_cast<const uint4*>(p.zeros + base + chunk * 8));
    } else {
      g.s.x = __half_as_ushort(__ldg(sp + chunk));
      if (FMT == FMT_W4_ASYM) g.z.x = __half_as_ushort(__ldg(p.zeros + base + chunk));
    }
  }
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

// All-gather by push: after a plain forward has written this rank's [M, n_local] slab into its own
// copy of the full output, every block copies a share of the slab into the same place of every
// peer's copy (16-byte loads, one 16-byte peer store per destination), so the NVLink writes are
// spread over as many SMs as the slab is worth instead of over the few blocks that own output
// tiles.  Protocol, on the same signal block as the epilogue form: announce "entered call g"
// to the peers, wait (bounded) for theirs before the first store into their buffers, and when
// the LAST block of this grid has made its stores visible, count `tiles` arrivals on every rank —
// the number gather_wait_kernel expects from a rank, whichever way the tiles travelled.
struct PushParams {
  unsigned char* y[8];            // peer-mapped bases of every rank's full output
  unsigned long long* sig[8];
  int rank, world;
  int rows;
  long long ld_bytes;             // row pitch of the full output
  long long col0_bytes;           // this rank's slab starts here in every row
  int row_chunks;                 // 16-byte chunks per slab row
  unsigned long long tiles;
};

__global__ void __launch_bounds__(512) gather_push_kernel(const PushParams p) {
  grid_launch_dependents();
  grid_dependency_wait();                                   // the forward that wrote the slab
  unsigned long long* const mine = p.sig[p.rank];
  const unsigned long long gen = mine[kSigGeneration] + 1;
  if (blockIdx.x == 0 && threadIdx.x < p.world && static_cast<int>(threadIdx.x) != p.rank)
    st_relaxed_sys(p.sig[threadIdx.x] + kSigReady + p.rank, gen);
  if (threadIdx.x < p.world && static_cast<int>(threadIdx.x) != p.rank) {
    if (!poll_at_least(mine + kSigReady + threadIdx.x, gen)) mine[kSigStatus] = 2ull;
  }
  __syncthreads();
  const long long total = static_cast<long long>(p.rows) * p.row_chunks;
  const unsigned char* const src = p.y[p.rank];
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / p.row_chunks, c = i - r * p.row_chunks;
    const long long off = r * p.ld_bytes + p.col0_bytes + c * 16;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + off));
#pragma unroll
    for (int d = 0; d < 8; ++d)
      if (d < p.world && d != p.rank) *reinterpret_cast<uint4*>(p.y[d] + off) = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();                                 // this block's peer stores are visible
    unsigned long long* const done = mine + kSigPushBlocks;
    if (atomicAdd(done, 1ull) == gridDim.x - 1) {
      *done = 0ull;                                         // for the next call
      __threadfence_system();                               // cumulative: every block's stores before the counts
      for (int d = 0; d < p.world; ++d) red_add_relaxed_sys(p.sig[d] + kSigArrivals, p.tiles);
    }
  }
}

int launch_gather_push(const b200q_gather* g, int64_t ldy, int M, int n_local, int tiles, cudaStream_t stream) {
  PushParams p{};
  for (int r = 0; r < g->world; ++r) {
    p.y[r] = static_cast<unsigned char*>(g->y_peer[r]);
    p.sig[r] = static_cast<unsigned long long*>(g->signal_peer[r]);
  }
  p.rank = g->rank;
  p.world = g->world;
  p.rows = M;
  p.ld_bytes = ldy * 2;
  p.col0_bytes = static_cast<long long>(g->rank) * n_local * 2;
  p.row_chunks = n_local * 2 / 16;
  p.tiles = static_cast<unsigned long long>(tiles);
  // one block per 4 KiB of peer stores (a single SM sustains only a few GB/s of them), at most
  // four per SM
  const long long out_bytes = static_cast<long long>(M) * n_local * 2 * (g->world - 1);
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(592, (out_bytes + 4095) / 4096)));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(512);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gather_push_kernel, p);
  if (e != cudaSuccess) {
    set_last_error("cudaLaunchKernelEx(gather_push)", e);
    return B200Q_ERR_CUDA;
  }
  return note_launch();
}

template <int FMT, typename T, int DW>
__global__ void __launch_bounds__(64 + 32 * DW, DW == 8 ? 2 : 1)
wq_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_y, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled operand tiles
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int x_atom_bytes = p.tok * 128;                  // one 64-wide K atom of [tok x 128 B]
  const uint32_t x_ring = smem_base;
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
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  const int nkb = max(kb1 - kb0, 0);

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
      if ((p.g_world > 1 || p.a_world > 1) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        // Fused all-gather: tell every rank that this rank has entered call `gen`, i.e. that
        // whatever read its previous output has finished (it precedes us in the stream).
        grid_dependency_wait();
        const int world = p.g_world > 1 ? p.g_world : p.a_world;
        const int rank = p.g_world > 1 ? p.g_rank : p.a_rank;
        const unsigned long long gen = p.g_sig[rank][kSigGeneration] + 1;
        // Relaxed: the announcement publishes no data of this kernel, only that the kernels
        // before it in the stream have finished (they have: griddepcontrol.wait returned).  A
        // release store per peer would serialise one NVLink round trip per rank.
        for (int d = 0; d < world; ++d) st_relaxed_sys(p.g_sig[d] + kSigReady + rank, gen);
      }
      bool ok = true;
      int sa = 0, sx = 0, xs = 0;                // operand stage, activation chunk slot, block in chunk
      uint32_t a_phase = 0, x_phase = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        if (xs == 0) {
          ok = wait_or_abort(x_full + 8 * sx, x_phase, abort_p);
          if (!ok) break;
        }
        ok = wait_or_abort(a_full + 8 * sa, a_phase, abort_p);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t x_stage = x_ring + sx * x_chunk_bytes + xs * 2 * x_atom_bytes;
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
          const uint64_t bdesc = umma_desc_sw128(x_stage + atom * x_atom_bytes);
          // A in tensor memory: stage sa holds 128 K elements as 64 columns, 8 per MMA
          const uint32_t a_tmem = tmem_base + p.a_col0 + sa * 64 + atom * 32;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzle atom
            const uint32_t acc = (i > 0 || atom > 0 || k > 0) ? 1u : 0u;
            umma_f16_ts(tmem_base, a_tmem + 8 * k, bdesc + 2 * k, p.idesc, acc);
          }
        }
        umma_commit(a_empty + 8 * sa);
        if (xs == p.xg - 1 || i == nkb - 1) umma_commit(x_empty + 8 * sx);
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
      if (!ok) flag_failure(abort_p, p.status, 2u);
      umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------ dequant warps
    // One thread = one output channel (its TMEM lane; a warp may only touch TMEM lanes
    // 32 (warp % 4) .. +31) x one K slice of the K block.
    const int td = threadIdx.x - 64;
    const int atm_row = (warp & 3) * 32 + lane;
    const int atm_kq = (warp - 2) >> 2;                 // which K slice of the row
    const uint32_t atm_taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + p.a_col0;
    const int row_n = n_tile * kBlockN + atm_row;
    const bool vec = (p.groups & 7) == 0;
    const int chunk_shift = vec ? 3 : 0;
    GroupChunk cur, nxt;
    int cur_chunk = kb0 >> chunk_shift;
    const int last_chunk = (kb1 - 1) >> chunk_shift;
    if (FMT != FMT_W8 && nkb > 0) {
      load_group_chunk<FMT>(cur, p, cur_chunk, vec, row_n);
      if (cur_chunk < last_chunk) load_group_chunk<FMT>(nxt, p, cur_chunk + 1, vec, row_n);
    }
    bool ok = true;
    int sp = 0, ps = 0, sa = 0;                  // weight group slot, block in group, operand stage
    uint32_t p_phase = 0, a_phase = 1;           // parities: p_full, a_empty
    for (int i = 0; i < nkb && ok; ++i) {
      const int kb = kb0 + i;
      PairConsts gp{0u, 0u, 0u};
      if (FMT != FMT_W8) {
        const int chunk = kb >> chunk_shift;
        if (chunk != cur_chunk) {
          cur = nxt;
          cur_chunk = chunk;
          if (chunk < last_chunk) load_group_chunk<FMT>(nxt, p, chunk + 1, vec, row_n);
        }
        const int idx = vec ? (kb & 7) : 0;
        gp = make_pair_consts(pick_half(cur.s, idx),
                              (FMT == FMT_W4_ASYM) ? __half2float(pick_half(cur.z, idx)) : 8.0f);
      }
      if (ps == 0) ok = wait_or_abort(p_full + 8 * sp, p_phase, abort_p);
      ok = ok && wait_or_abort(a_empty + 8 * sa, a_phase, abort_p);
      if (!ok) break;
      const uint32_t p_stage = p_ring + sp * p_group_bytes + ps * PackedStage<FMT>::kBytes;
      // The packed stage is read row-wise; the TMA 64-byte swizzle keeps that conflict-free.
      const uint32_t prow = p_stage + atm_row * 64;
      const int xr = (atm_row >> 1) & 3;
      const uint32_t a_stage_t = atm_taddr + sa * 64;
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
            lo[(c * 4 + w) * 2] = deq_lo<T>(u, gp);
            lo[(c * 4 + w) * 2 + 1] = deq_lo<T>(u >> 8, gp);
            hi[(c * 4 + w) * 2] = deq_hi<T>(u, gp);
            hi[(c * 4 + w) * 2 + 1] = deq_hi<T>(u >> 8, gp);
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
            out[(c * 4 + w) * 4 + 0] = deq_lo<T>(u, gp);        // inputs 0,1
            out[(c * 4 + w) * 4 + 1] = deq_hi<T>(u, gp);        // inputs 2,3
            out[(c * 4 + w) * 4 + 2] = deq_lo<T>(u >> 8, gp);   // inputs 4,5
            out[(c * 4 + w) * 4 + 3] = deq_hi<T>(u >> 8, gp);   // inputs 6,7
          }
        }
        tmem_st_cols<kCols>(a_stage_t + kCols * atm_kq, out);
      } else {
        // W8: the stage is two [128 x 64 B] sub-tiles (K 0..63, 64..127); this thread takes
        // 128 / kSplit consecutive K of its row.  The integers enter the MMA unscaled (exact
        // in fp16 and bf16); the channel scale is applied to the accumulator.
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
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full + 8 * sa);
        if (ps == p.pg - 1 || i == nkb - 1) mbar_arrive(p_empty + 8 * sp);
      }
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
    }
    if (!ok) flag_failure(abort_p, p.status, 4u);

    // ------------------------------------------------------------ epilogue
    bool acc_ok = wait_or_abort(acc_full, 0, abort_p);
    if (!acc_ok) flag_failure(abort_p, p.status, 8u);
    tc_fence_after_sync();
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
    const bool gather = p.g_world > 1 && !p.reduce;
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
    if (p.reduce) {
      // Row-parallel forward: this block holds the partial of its tile over this rank's K
      // shard.  The tile's columns belong to one owner rank.  Every other rank sends its partial
      // to the owner's inbox through peer memory as self-validating words (an fp32 value v
      // travels as bits(v + 0.0f) ^ 0x80000000, never 0; 0 means "not written"), so the owner
      // needs no flag: it polls the words themselves (bounded), adds the partials in rank
      // order — a fixed order, identical on every run — adds the bias, rounds once, and stores
      // the finished tile into the output of every rank; then it counts the tile on every rank
      // exactly as the fused all-gather does.
      const int owner = (n_tile * kBlockN) / p.r_cols;
      const int n_local = n - owner * p.r_cols;
      if (owner == p.g_rank) gather_wait_ready();          // peers have consumed the previous output
      for (int c = 0; c < half_cols; c += 8) {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (acc_ok && nkb > 0) {
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
        }
        const int m0 = m_base + c_begin + c;
        if (owner != p.g_rank) {
          uint32_t* dst = p.r_inbox[owner] + (static_cast<size_t>(p.g_rank) * p.M + m0) * p.r_cols + n_local;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (m0 + j < p.M && n < p.N)
              dst[static_cast<size_t>(j) * p.r_cols] = __float_as_uint(__uint_as_float(r[j]) + 0.0f) ^ 0x80000000u;
          continue;
        }
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.0f;
        for (int src = 0; src < p.g_world; ++src) {
          if (src == p.g_rank) {
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] += __uint_as_float(r[j]);
            continue;
          }
          uint32_t* from = p.r_inbox[p.g_rank] + (static_cast<size_t>(src) * p.M + m0) * p.r_cols + n_local;
          uint32_t v[8];
          bool all = false;
          for (uint32_t tries = 0; !all; ++tries) {
            all = true;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[j] = 0x80000000u;
              if (m0 + j < p.M && n < p.N)
                asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v[j]) : "l"(from + static_cast<size_t>(j) * p.r_cols) : "memory");
              all = all && v[j] != 0u;
            }
            if (!all) {
              if (tries >= (1u << 22) || *abort_p) {      // about five seconds, like the gather waits
                p.g_sig[p.g_rank][kSigStatus] = 4ull;
                break;
              }
              __nanosleep(tries < 4096 ? 40 : 1000);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sum[j] += __uint_as_float(v[j] ^ 0x80000000u);
            if (m0 + j < p.M && n < p.N) from[static_cast<size_t>(j) * p.r_cols] = 0u;   // empty for the next call
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (m0 + j < p.M && n < p.N) {
            const T out = from_float<T>(sum[j] * ch_scale + ch_bias);
            for (int d = 0; d < p.g_world; ++d)
              static_cast<T*>(p.g_y[d])[static_cast<int64_t>(m0 + j) * p.ldy + n] = out;
          }
        }
      }
      if (owner == p.g_rank) gather_signal_done();     // (a tile has one owner: uniform per block)
    } else if (p.argmax) {
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
      if (acc_ok && nkb > 0) {
        for (int c = 0; c < half_cols; c += 8) {
          uint32_t r[8];
          tmem_ld_x8(tmem_row + (c_begin + c), r);
          tmem_ld_wait();
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
      if (vec_out) {
        if (tma_out) fence_proxy_async_smem();   // staged rows -> visible to the TMA engine
        asm volatile("bar.sync 1, %0;" ::"n"(kDequantThreads) : "memory");
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
      if (gather) gather_signal_done();
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
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}


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

bool get_tensor_map(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t d0,
                    uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2, uint32_t b0, uint32_t b1,
                    uint32_t b2, CUtensorMapSwizzle swz) {
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

bool debug_plan_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200Q_DEBUG_PLAN");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}

struct TcPlan {
  int tok, m_tiles, n_tiles, kb_total, splits, kb_per_split, np, nx, na, pg, xg, tmem_cols, a_col0;
  int dw;            // dequantise warps per block: 8, or 16 for wide tiles (one block per SM)
  size_t smem_bytes;
};

static int packed_stage_bytes(int format) { return format == FMT_W8 ? kBlockN * 128 : kBlockN * 64; }

// Most weight tiles a problem may have for its 33..64-token tiles to take the wide block shape.
constexpr int kWideSmallMaxTiles = 74;

static TcPlan make_plan(int format, int M, int N, int K, bool no_split = false) {
  TcPlan pl{};
  // Token tile: as few tiles as cover M, except that a problem of at most two waves (148
  // blocks at a time) may take a narrower tile that fills its last wave; with more waves the
  // widest tile measured best.  Cost model per candidate count of token tiles: waves x (tile
  // width + fixed set-up/epilogue worth ~40 columns), a tile narrower than 128 columns being
  // dequantise-bound; a problem under half a wave will be split along K.
  int mt = (M + 255) / 256;
  if (M > 256 && mt * ((N + kBlockN - 1) / kBlockN) <= 2 * 148) {
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
  // "Wide" blocks own an SM (512 TMEM columns, up to 227 KB of shared memory).  Token tiles
  // above 64 always are; a tile of 33..64 tokens also takes that shape when the problem has so
  // few weight tiles (at most half a wave) that a K split inside a cluster fits in one wave:
  // its partials (tok x 128 fp32 per block) then never leave the SMs.  Wide tiles of a problem
  // with few token tiles take sixteen dequantise warps, which halve the latency of a
  // dequantise stage; large prefill problems (many waves) are MMA-bound and measured no
  // better with them.  Each of the four column slices must then be whole groups of 8 columns.
  pl.dw = 8;
  const int tiles0 = mt * ((N + kBlockN - 1) / kBlockN);
  const bool wide = tok > 64 || (tok > 32 && tiles0 <= kWideSmallMaxTiles && (K + kBlockK - 1) / kBlockK >= 32);
  if (wide && mt < 4) {
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
  pl.xg = tok <= 16 ? 4 : (tok <= 32 ? 2 : 1);
  pl.pg = wide ? 1 : 2;
  auto total = [&](int np, int nx) {
    return static_cast<size_t>(nx) * pl.xg * xbytes + static_cast<size_t>(np) * pl.pg * pbytes +
           1024 /*alignment*/ + 8 * kMaxRing * 6 + 64;
  };
  const size_t half_sm = 115712;                   // (228 KiB - 2 x 1 KiB reserved) / 2
  const size_t budget = static_cast<size_t>(kSmemBudget);
  pl.nx = 2;
  pl.np = 2;
  // TMEM columns: accumulator [0, tok), then `na` operand stages of 64 columns each.  Two
  // resident blocks need <= 256 columns each: narrow tiles take that shape so one block's
  // set-up and epilogue overlap the other's weight stream.
  pl.a_col0 = (tok + 63) / 64 * 64;
  const bool two_per_sm = !wide && total(2, 2) <= half_sm;
  if (two_per_sm) {
    pl.na = (256 - pl.a_col0) / 64;              // 3 for tok <= 64
    pl.nx = 3;
    while (total(pl.np, pl.nx) > half_sm && pl.nx > 2) --pl.nx;
    while (pl.np < 6 && total(pl.np + 1, pl.nx) <= half_sm) ++pl.np;
    pl.tmem_cols = 256;
  } else {
    pl.na = (512 - pl.a_col0) / 64;
    if (pl.na > 4) pl.na = 4;
    const int wish[][2] = {{1, 3}, {2, 3}, {2, 4}, {1, 4}, {2, 6}, {2, 8}};
    for (const auto& w : wish) {
      int nx = pl.nx, np = pl.np;
      (w[0] == 1 ? nx : np) = w[1];
      if (nx >= pl.nx && np >= pl.np && total(np, nx) <= budget) {
        pl.nx = nx;
        pl.np = np;
      }
    }
    pl.tmem_cols = 512;
  }
  pl.smem_bytes = total(pl.np, pl.nx);

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

// Workspace a forward of this geometry may need, whichever kernel serves it: the fixed
// header (status, counters, argmax keys), the stream-K exchange region for token counts that
// kernel takes, or the tile kernel's split-K partials behind it.
size_t tc_workspace_bytes(int format, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  TcPlan pl = make_plan(format, M, N, K);
  size_t bytes = kWsExchangeOffset;
  if (pl.splits > 1) bytes = kWsPartialOffset + sizeof(float) * static_cast<size_t>(pl.splits) * M * N;
  const size_t sk = sk_workspace_bytes(format, M, N, K);
  return sk > bytes ? sk : bytes;
}

bool tc_supported(const ForwardArgs& a) {
  if (a.format != FMT_W8 && a.group != 128) return false;
  // K must be whole 64-element atoms (the tensor maps' third dimension walks them)
  if (a.format == FMT_W8 ? (a.K % 64 != 0) : (a.K % 128 != 0)) return false;
  if (reinterpret_cast<uintptr_t>(a.x) % 16 || (a.ldx * 2) % 16) return false;
  if (reinterpret_cast<uintptr_t>(a.w) % 16 || a.ldw % 16) return false;
  return true;
}

template <int FMT, typename T, int DW>
static int launch_tc_typed(const ForwardArgs& a, const TcPlan& pl) {
  static bool attr_set_dev[64] = {};
  static std::mutex attr_mu;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    bool& attr_set = attr_set_dev[dev & 63];
    std::lock_guard<std::mutex> g(attr_mu);
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(wq_gemm_tc_kernel<FMT, T, DW>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
      if (e != cudaSuccess) {
        set_last_error("cudaFuncSetAttribute", e);
        return B200Q_ERR_CUDA;
      }
      // ask for the largest shared-memory carve-out so that two blocks fit an SM (also what the
      // cluster occupancy query assumes)
      (void)cudaFuncSetAttribute(wq_gemm_tc_kernel<FMT, T, DW>,
                                 cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
      (void)cudaGetLastError();
      attr_set = true;
    }
  }
  CUtensorMap tm_w, tm_x;
  // Packed weights as {64 B, N rows, K chunks of 64 B}: the third coordinate walks K, so a
  // box of depth pg (2 pg for int8, whose K block is two 64-byte chunks) is a weight group.
  // A stage is read one row per thread: 64-byte swizzle.
  const uint64_t w_row_bytes = (FMT == FMT_W8) ? static_cast<uint64_t>(a.K) : static_cast<uint64_t>(a.K / 2);
  if (!get_tensor_map(&tm_w, a.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 64, static_cast<uint64_t>(a.N),
                      w_row_bytes / 64, static_cast<uint64_t>(a.ldw), 64, 64, kBlockN,
                      static_cast<uint32_t>((FMT == FMT_W8 ? 2 : 1) * pl.pg), CU_TENSOR_MAP_SWIZZLE_64B))
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
  const bool reducing = a.reduce != nullptr && a.reduce->world > 1;
  const int n_out = a.swiglu ? a.N / 2 : a.N;
  // (The TMA engine clips the innermost dimension in 16-byte units: measured, a 500-column fp16
  // output had columns 500..503 written.  So the row width must be whole 16-byte units too.)
  const bool y_tma = !gathering && !reducing && !a.argmax && pl.splits == 1 && (a.ldy % 8 == 0) && (n_out % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(a.y) % 16 == 0);
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
  const uint32_t ab_fmt = a.act_dtype == B200Q_F16 ? 0u : 1u;    // both operands in the activation dtype
  p.idesc = umma_idesc_f16(ab_fmt, ab_fmt, 128u, static_cast<uint32_t>(pl.tok));
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
  if (gathering) {
    p.g_world = a.gather->world;
    p.g_rank = a.gather->rank;
    p.g_col0 = a.gather->rank * a.N;
    for (int d = 0; d < 8; ++d) {
      p.g_y[d] = d < a.gather->world ? a.gather->y_peer[d] : nullptr;
      p.g_sig[d] = d < a.gather->world ? static_cast<unsigned long long*>(a.gather->signal_peer[d]) : nullptr;
    }
  }
  p.a_world = 0;
  if (!gathering && !reducing && a.announce != nullptr && a.announce->world > 1) {
    p.a_world = a.announce->world;
    p.a_rank = a.announce->rank;
    for (int d = 0; d < 8; ++d)
      p.g_sig[d] = d < p.a_world ? static_cast<unsigned long long*>(a.announce->signal_peer[d]) : nullptr;
  }
  p.reduce = 0;
  if (reducing) {
    p.reduce = 1;
    p.g_world = a.reduce->world;
    p.g_rank = a.reduce->rank;
    p.g_col0 = 0;
    p.r_cols = a.N / a.reduce->world;
    for (int d = 0; d < 8; ++d) {
      const bool in = d < a.reduce->world;
      p.g_y[d] = in ? a.reduce->y_peer[d] : nullptr;
      p.g_sig[d] = in ? static_cast<unsigned long long*>(a.reduce->signal_peer[d]) : nullptr;
      p.r_inbox[d] = in ? static_cast<uint32_t*>(a.reduce->inbox_peer[d]) : nullptr;
    }
  }
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  p.status = reinterpret_cast<unsigned*>(ws);
  p.counters = reinterpret_cast<unsigned*>(ws + kWsCountersOffset);
  p.row_keys = reinterpret_cast<unsigned long long*>(ws + kWsKeysOffset);
  p.partial = reinterpret_cast<float*>(ws + kWsPartialOffset);

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
  // when every cluster of the grid can be resident at once; otherwise, or with the fused
  // all-gather, the partials go through the workspace and the last block to arrive sums them.
  p.cluster_reduce = 0;
  int resident_clusters = -1;
  const size_t ring_bytes = static_cast<size_t>(pl.nx) * pl.xg * pl.tok * 256 +
                            static_cast<size_t>(pl.np) * pl.pg * packed_stage_bytes(a.format);
  if (pl.splits > 1 && pl.splits <= 8 && p.g_world == 0 && ring_bytes >= static_cast<size_t>(pl.tok) * 512) {
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
        if (cudaOccupancyMaxActiveClusters(&n, wq_gemm_tc_kernel<FMT, T, DW>, &cfg) != cudaSuccess) {
          (void)cudaGetLastError();
          n = 0;
        }
        it = resident.emplace(key, n).first;
      }
      clusters = it->second;
    }
    resident_clusters = clusters;
    if (clusters >= pl.n_tiles * pl.m_tiles) {
      p.cluster_reduce = 1;
    } else {
      cfg.numAttrs = 1;
    }
  }
  if (debug_plan_enabled())
    std::fprintf(stderr,
                 "b200q plan: tile kernel fmt %d M %d N %d K %d | tok %d tiles %dx%d splits %d (kb %d/%d) dw %d | "
                 "rings p %dx%d x %dx%d a %d | smem %zu tmem %d | split reduce: %s (resident clusters %d)\n",
                 FMT, a.M, a.N, a.K, pl.tok, pl.m_tiles, pl.n_tiles, pl.splits, pl.kb_per_split,
                 pl.kb_total, DW, pl.np, pl.pg, pl.nx, pl.xg, pl.na, pl.smem_bytes, pl.tmem_cols,
                 pl.splits == 1 ? "none" : (p.cluster_reduce ? "cluster" : "workspace"), resident_clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, wq_gemm_tc_kernel<FMT, T, DW>, tm_w, tm_x, tm_y, p);
  if (e != cudaSuccess) {
    set_last_error("cudaLaunchKernelEx", e);
    return B200Q_ERR_CUDA;
  }
  return note_launch();
}

template <int FMT, typename T>
static int launch_tc_width(const ForwardArgs& a, const TcPlan& pl) {
  return pl.dw == 16 ? launch_tc_typed<FMT, T, 16>(a, pl) : launch_tc_typed<FMT, T, 8>(a, pl);
}

// Tiles one rank owns (finishes and announces on every rank) in a fused all-reduce of a
// row-parallel forward over `world` ranks; 0 when the geometry cannot take it.
int tc_reduce_tiles(int format, int M, int N, int K_local, int world) {
  if (M <= 0 || N <= 0 || K_local <= 0 || world < 1 || N % world || (N / world) % kBlockN) return 0;
  const TcPlan pl = make_plan(format, M, N, K_local, true);
  return pl.m_tiles * (pl.n_tiles / world);
}

// Units of output one rank's fused-gather forward of this geometry announces on every rank
// (what b200q_gather_wait must be told): output tiles of the tile kernel.
int tc_output_tiles(int format, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int sk = sk_gather_arrivals(format, M, N, K);
  if (sk > 0) return sk;
  const TcPlan pl = make_plan(format, M, N, K);
  return pl.m_tiles * pl.n_tiles;
}

// Bytes of one output tile of the tile kernel's plan for this geometry (what a block of the
// epilogue form of the all-gather stores into EACH peer).
int tc_tile_bytes(int format, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const TcPlan pl = make_plan(format, M, N, K);
  return pl.tok * kBlockN * 2;
}

// One line naming the kernel instantiation and tiling a plain forward of this geometry takes.
void tc_describe_plan(int format, int M, int N, int K, char* text, size_t size) {
  if (M <= 0 || N <= 0 || K <= 0) {
    std::snprintf(text, size, "nothing to launch");
    return;
  }
  if (sk_preferred(format, M, N, K) && sk_describe(format, M, N, K, text, size)) return;
  const TcPlan pl = make_plan(format, M, N, K);
  std::snprintf(text, size, "wq_gemm_tc_kernel<%s,dw%d> tok=%d tiles=%dx%d splits=%d smem=%zu tmem=%d",
                format == FMT_W8 ? "w8" : (format == FMT_W4_REF ? "w4_ref" : "w4_asym"), pl.dw, pl.tok,
                pl.m_tiles, pl.n_tiles, pl.splits, pl.smem_bytes, pl.tmem_cols);
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
  if (a.workspace == nullptr) return B200Q_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a.workspace) % 256) return B200Q_ERR_ALIGNMENT;
  if (a.force_streamk && !sk_supported(a)) return B200Q_ERR_UNSUPPORTED;
  if (sk_supported(a) && (a.force_streamk || sk_preferred(a.format, a.M, a.N, a.K))) return launch_forward_sk(a);
  // The fused argmax never splits K: it needs the header (counters and row keys) only.
  if (a.argmax && a.M > kMaxArgmaxRows) return B200Q_ERR_UNSUPPORTED;
  // (nor does the fused all-reduce: a rank's K shard is already a K split)
  const TcPlan pl = make_plan(a.format, a.M, a.N, a.K, a.argmax || (a.reduce != nullptr && a.reduce->world > 1));
  size_t need = kWsExchangeOffset;
  if (pl.splits > 1) need = kWsPartialOffset + sizeof(float) * static_cast<size_t>(pl.splits) * a.M * a.N;
  if (a.workspace_bytes < need) return B200Q_ERR_WORKSPACE;
  const bool h = a.act_dtype == B200Q_F16;
  switch (a.format) {
    case FMT_W8:
      return h ? launch_tc_width<FMT_W8, __half>(a, pl) : launch_tc_width<FMT_W8, __nv_bfloat16>(a, pl);
    case FMT_W4_REF:
      return h ? launch_tc_width<FMT_W4_REF, __half>(a, pl) : launch_tc_width<FMT_W4_REF, __nv_bfloat16>(a, pl);
    case FMT_W4_ASYM:
      return h ? launch_tc_width<FMT_W4_ASYM, __half>(a, pl) : launch_tc_width<FMT_W4_ASYM, __nv_bfloat16>(a, pl);
    default:
      return B200Q_ERR_INVALID;
  }
}

}  // namespace b200q
