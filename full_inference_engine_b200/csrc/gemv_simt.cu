// CUDA-core weight-only linear for decode-sized M: y = x . dequant(W)^T.
//
// HBM-bound: every weight byte is read once with 128-bit streaming loads and
// multiplied against activations converted once per thread and reused over
// four output channels.  The K reduction is split over the 128 threads of a
// channel group (split-K inside the block): warp shuffles, then one shared
// memory hop; no global scratch, no atomics, deterministic.
//
// Block = 256 threads = 2 channel groups x 128 threads; a channel group owns
// 4 consecutive output channels; grid = (ceil(N/8), ceil(M/MT)).
//
// Reference counterparts: _w4a16_gemv_kernel (engine/kernels/w4a16_linear.py:120-177)
// and _w8a16_linear_kernel (engine/kernels/w8a16_linear.py:10-40).
#include "internal.cuh"

namespace b200q {

constexpr int kSimtThreads = 256;
constexpr int kGroupThreads = 128;                      // threads sharing a channel group
constexpr int kChanPerGroup = 4;                        // R
constexpr int kChanPerBlock = kChanPerGroup * (kSimtThreads / kGroupThreads);

__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <typename T>
__device__ __forceinline__ float2 act_pair_to_float2(uint32_t u);
template <>
__device__ __forceinline__ float2 act_pair_to_float2<__half>(uint32_t u) {
  return __half22float2(as_h2(u));
}
template <>
__device__ __forceinline__ float2 act_pair_to_float2<__nv_bfloat16>(uint32_t u) {
  // bf16 is the high half of an fp32
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}

// 8 activations (one 16-byte load) -> 8 floats
template <typename T>
__device__ __forceinline__ void load_x8(const T* p, float* dst) {
  uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  float2 a = act_pair_to_float2<T>(v.x), b = act_pair_to_float2<T>(v.y);
  float2 c = act_pair_to_float2<T>(v.z), d = act_pair_to_float2<T>(v.w);
  dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
  dst[4] = c.x; dst[5] = c.y; dst[6] = d.x; dst[7] = d.y;
}

template <int MT>
__device__ __forceinline__ void fma_pair(float (&acc)[MT], __half2 w, const float (&xf)[MT][32],
                                         int i) {
  float2 wf = __half22float2(w);
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    acc[m] = fmaf(wf.x, xf[m][i], acc[m]);
    acc[m] = fmaf(wf.y, xf[m][i + 1], acc[m]);
  }
}

template <int FMT, typename T, int MT>
__global__ void __launch_bounds__(kSimtThreads)
wq_gemv_simt_kernel(const T* __restrict__ x, int64_t ldx, const uint8_t* __restrict__ w,
                    int64_t ldw, const void* __restrict__ scales, int scale_is_f32,
                    const __half* __restrict__ zeros, int group, const T* __restrict__ bias,
                    T* __restrict__ y, int64_t ldy, int M, int N, int K) {
  const int tid = threadIdx.x;
  const int cg = tid / kGroupThreads;          // channel group in the block
  const int tv = tid % kGroupThreads;          // position along K
  const int n0 = blockIdx.x * kChanPerBlock + cg * kChanPerGroup;
  const int m0 = blockIdx.y * MT;
  const int groups = (FMT == FMT_W8) ? 1 : K / group;

  // vectors of 16 bytes per weight row
  const int V = (FMT == FMT_W8) ? (K >> 4) : (K >> 5);

  const uint8_t* wrow[kChanPerGroup];
  int nrow[kChanPerGroup];
#pragma unroll
  for (int r = 0; r < kChanPerGroup; ++r) {
    nrow[r] = min(n0 + r, N - 1);
    wrow[r] = w + static_cast<int64_t>(nrow[r]) * ldw;
  }
  const T* xrow[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) xrow[m] = x + static_cast<int64_t>(min(m0 + m, M - 1)) * ldx;

  float acc[kChanPerGroup][MT];
#pragma unroll
  for (int r = 0; r < kChanPerGroup; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

  for (int v = tv; v < V; v += kGroupThreads) {
    uint4 wv[kChanPerGroup];
#pragma unroll
    for (int r = 0; r < kChanPerGroup; ++r) wv[r] = ld_stream_v4(wrow[r] + (static_cast<int64_t>(v) << 4));

    float xf[MT][32];
    int g = 0;
    if (FMT == FMT_W4_REF) {
      const int half = group >> 1;
      const int b = v << 4;
      g = b / half;
      const int k_lo = g * group + (b - g * half);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        load_x8<T>(xrow[m] + k_lo, &xf[m][0]);
        load_x8<T>(xrow[m] + k_lo + 8, &xf[m][8]);
        load_x8<T>(xrow[m] + k_lo + half, &xf[m][16]);
        load_x8<T>(xrow[m] + k_lo + half + 8, &xf[m][24]);
      }
    } else if (FMT == FMT_W4_ASYM) {
      const int k0 = v << 5;
      g = k0 / group;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int i = 0; i < 4; ++i) load_x8<T>(xrow[m] + k0 + 8 * i, &xf[m][8 * i]);
      }
    } else {
      const int k0 = v << 4;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        load_x8<T>(xrow[m] + k0, &xf[m][0]);
        load_x8<T>(xrow[m] + k0 + 8, &xf[m][8]);
      }
    }

#pragma unroll
    for (int r = 0; r < kChanPerGroup; ++r) {
      const uint32_t words[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
      if (FMT == FMT_W4_REF) {
        const __half2 s = __half2half2(
            reinterpret_cast<const __half*>(scales)[static_cast<int64_t>(nrow[r]) * groups + g]);
        const __half2 bias_lo = __float2half2_rn(1032.0f), nbias_hi = __float2half2_rn(-72.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          W4Quad q = dequant_w4_word_splithalf(words[i], bias_lo, nbias_hi, s);
          fma_pair<MT>(acc[r], q.lo01, xf, 4 * i);
          fma_pair<MT>(acc[r], q.lo23, xf, 4 * i + 2);
          fma_pair<MT>(acc[r], q.hi01, xf, 16 + 4 * i);
          fma_pair<MT>(acc[r], q.hi23, xf, 16 + 4 * i + 2);
        }
      } else if (FMT == FMT_W4_ASYM) {
        const int64_t si = static_cast<int64_t>(nrow[r]) * groups + g;
        const __half2 s = __half2half2(reinterpret_cast<const __half*>(scales)[si]);
        const float zp = __half2float(zeros[si]);
        const __half2 bias_lo = __float2half2_rn(1024.0f + zp);
        const __half2 nbias_hi = __float2half2_rn(-(64.0f + zp));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          W4Oct o = dequant_w4_word_seq(words[i], bias_lo, nbias_hi, s);
          fma_pair<MT>(acc[r], o.k01, xf, 8 * i);
          fma_pair<MT>(acc[r], o.k23, xf, 8 * i + 2);
          fma_pair<MT>(acc[r], o.k45, xf, 8 * i + 4);
          fma_pair<MT>(acc[r], o.k67, xf, 8 * i + 6);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __half2 k01, k23;
          int8x4_to_h2(words[i], k01, k23);
          fma_pair<MT>(acc[r], k01, xf, 4 * i);
          fma_pair<MT>(acc[r], k23, xf, 4 * i + 2);
        }
      }
    }
  }

  // reduce over the 128 threads of the channel group
  __shared__ float red[kSimtThreads / 32][kChanPerGroup][MT];
#pragma unroll
  for (int r = 0; r < kChanPerGroup; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][m] = v;
    }
  const int warp = tid >> 5, lane = tid & 31;
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kChanPerGroup; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) red[warp][r][m] = acc[r][m];
  }
  __syncthreads();
  if (tv < kChanPerGroup * MT) {
    const int r = tv / MT, m = tv % MT;
    const int n = n0 + r, row = m0 + m;
    if (n < N && row < M) {
      const int w0 = cg * (kGroupThreads / 32);
      float v = red[w0][r][m] + red[w0 + 1][r][m] + red[w0 + 2][r][m] + red[w0 + 3][r][m];
      if (FMT == FMT_W8) {
        const float s = scale_is_f32 ? reinterpret_cast<const float*>(scales)[n]
                                     : __half2float(reinterpret_cast<const __half*>(scales)[n]);
        v *= s;
      }
      if (bias != nullptr) v += static_cast<float>(bias[n]);
      y[static_cast<int64_t>(row) * ldy + n] = static_cast<T>(v);
    }
  }
}

template <int FMT, typename T>
static int launch_simt_typed(const ForwardArgs& a) {
  const int mt = a.M == 1 ? 1 : (a.M == 2 ? 2 : 4);
  dim3 grid((a.N + kChanPerBlock - 1) / kChanPerBlock, (a.M + mt - 1) / mt);
  dim3 block(kSimtThreads);
#define B200Q_SIMT_LAUNCH(MT)                                                                   \
  wq_gemv_simt_kernel<FMT, T, MT><<<grid, block, 0, a.stream>>>(                                \
      static_cast<const T*>(a.x), a.ldx, static_cast<const uint8_t*>(a.w), a.ldw, a.scales,     \
      a.scale_dtype == B200Q_F32, static_cast<const __half*>(a.zeros), a.group,                 \
      static_cast<const T*>(a.bias), static_cast<T*>(a.y), a.ldy, a.M, a.N, a.K)
  if (mt == 1) {
    B200Q_SIMT_LAUNCH(1);
  } else if (mt == 2) {
    B200Q_SIMT_LAUNCH(2);
  } else {
    B200Q_SIMT_LAUNCH(4);
  }
#undef B200Q_SIMT_LAUNCH
  return note_launch();
}

int launch_forward_simt(const ForwardArgs& a) {
  if (a.M <= 0 || a.N <= 0) return B200Q_OK;
  // 16-byte loads of activations: base and row pitch must keep 8-element alignment
  if (reinterpret_cast<uintptr_t>(a.x) % 16 || a.ldx % 8) return B200Q_ERR_ALIGNMENT;
  if (reinterpret_cast<uintptr_t>(a.w) % 16 || a.ldw % 16) return B200Q_ERR_ALIGNMENT;
  const bool h = a.act_dtype == B200Q_F16;
  switch (a.format) {
    case FMT_W8:
      return h ? launch_simt_typed<FMT_W8, __half>(a) : launch_simt_typed<FMT_W8, __nv_bfloat16>(a);
    case FMT_W4_REF:
      return h ? launch_simt_typed<FMT_W4_REF, __half>(a)
               : launch_simt_typed<FMT_W4_REF, __nv_bfloat16>(a);
    case FMT_W4_ASYM:
      return h ? launch_simt_typed<FMT_W4_ASYM, __half>(a)
               : launch_simt_typed<FMT_W4_ASYM, __nv_bfloat16>(a);
    default:
      return B200Q_ERR_INVALID;
  }
}

}  // namespace b200q
