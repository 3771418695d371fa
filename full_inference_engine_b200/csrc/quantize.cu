// Weight quantizers and the 4-bit dequantizer.  One-time (install/load) work:
// a thread block per output row, bandwidth-bound, bit-exact against the
// reference's torch arithmetic (IEEE fp32 division, round-half-to-even).
#include "internal.cuh"

namespace b200q {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, int64_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, int64_t i) {
  return p[i];
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, int64_t i) {
  return __half2float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// clamp that maps NaN to 0 (torch's NaN -> int8 conversion yields 0 on the
// reference's CPU path; an all-zero row divides 0 by a zero fp16 scale).
__device__ __forceinline__ float clamp_nan0(float v, float lo, float hi) {
  if (v != v) return 0.0f;
  return fminf(fmaxf(v, lo), hi);
}

// ------------------------------------------------------------------ W8
// engine/kernels/w8a16_linear.py:43-47 (mode 0) and engine/quantization/int8.py:19-20 (mode 1)
template <typename T>
__global__ void __launch_bounds__(256) quantize_w8_kernel(const T* __restrict__ w, int64_t ldw,
                                                          int N, int K, int mode,
                                                          int8_t* __restrict__ q,
                                                          void* __restrict__ scales) {
  __shared__ float red[8];
  __shared__ float s_div;
  const int n = blockIdx.x;
  const T* row = w + static_cast<int64_t>(n) * ldw;
  float m = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) m = fmaxf(m, fabsf(load_as_float(row, k)));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = red[0];
    for (int i = 1; i < (blockDim.x >> 5); ++i) mm = fmaxf(mm, red[i]);
    if (mode == B200Q_W8_SCALE_F16) {
      float s32 = __fdiv_rn(fmaxf(mm, 1e-8f), 127.0f);
      __half sh = __float2half_rn(s32);
      reinterpret_cast<__half*>(scales)[n] = sh;
      s_div = __half2float(sh);
    } else {
      float s32 = __fdiv_rn(fmaxf(mm, 1.1920928955078125e-07f), 127.0f);
      reinterpret_cast<float*>(scales)[n] = s32;
      s_div = s32;
    }
  }
  __syncthreads();
  const float s = s_div;
  int8_t* qrow = q + static_cast<int64_t>(n) * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    float v = rintf(__fdiv_rn(load_as_float(row, k), s));
    qrow[k] = static_cast<int8_t>(static_cast<int>(clamp_nan0(v, -127.0f, 127.0f)));
  }
}

// ------------------------------------------------------------------ W4
// Per (row, group) scale (and zero-point) into shared memory, then pack.
// REF:  engine/kernels/w4a16_format.py:32-50.
template <typename T>
__global__ void __launch_bounds__(256) quantize_w4_kernel(const T* __restrict__ w, int64_t ldw,
                                                          int N, int K, int group, int layout,
                                                          uint8_t* __restrict__ packed,
                                                          __half* __restrict__ scales,
                                                          __half* __restrict__ zeros) {
  extern __shared__ float sm[];  // [groups] scale32, then [groups] zero (ASYM)
  const int groups = K / group;
  float* s_scale = sm;
  float* s_zero = sm + groups;
  const int n = blockIdx.x;
  const T* row = w + static_cast<int64_t>(n) * ldw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nwarps) {
    const T* gp = row + static_cast<int64_t>(g) * group;
    if (layout == B200Q_W4_REF_SPLIT_HALF_SYM) {
      float m = 0.0f;
      for (int j = lane; j < group; j += 32) m = fmaxf(m, fabsf(load_as_float(gp, j)));
      m = warp_max(m);
      if (lane == 0) {
        float s32 = __fdiv_rn(fmaxf(m, 1e-8f), 7.0f);
        s_scale[g] = s32;
        scales[static_cast<int64_t>(n) * groups + g] = __float2half_rn(s32);
      }
    } else {
      float lo = 0.0f, hi = 0.0f;
      for (int j = lane; j < group; j += 32) {
        float v = load_as_float(gp, j);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
      }
      lo = warp_min(lo);
      hi = warp_max(hi);
      if (lane == 0) {
        float s32 = fmaxf(__fdiv_rn(hi - lo, 15.0f), 1e-8f);
        float zp = clamp_nan0(rintf(__fdiv_rn(-lo, s32)), 0.0f, 15.0f);
        s_scale[g] = s32;
        s_zero[g] = zp;
        scales[static_cast<int64_t>(n) * groups + g] = __float2half_rn(s32);
        zeros[static_cast<int64_t>(n) * groups + g] = __float2half_rn(zp);
      }
    }
  }
  __syncthreads();
  if (layout == B200Q_W4_REF_SPLIT_HALF_SYM) {
    const int half = group >> 1;
    uint8_t* prow = packed + static_cast<int64_t>(n) * (K >> 1);
    for (int idx = threadIdx.x; idx < (K >> 1); idx += blockDim.x) {
      const int g = idx / half, j = idx - g * half;
      const float s = s_scale[g];
      const T* gp = row + static_cast<int64_t>(g) * group;
      float a = clamp_nan0(rintf(__fdiv_rn(load_as_float(gp, j), s)), -7.0f, 7.0f) + 8.0f;
      float b = clamp_nan0(rintf(__fdiv_rn(load_as_float(gp, j + half), s)), -7.0f, 7.0f) + 8.0f;
      prow[idx] = static_cast<uint8_t>(static_cast<int>(a) | (static_cast<int>(b) << 4));
    }
  } else {
    uint32_t* prow = reinterpret_cast<uint32_t*>(packed) + static_cast<int64_t>(n) * (K >> 3);
    for (int idx = threadIdx.x; idx < (K >> 3); idx += blockDim.x) {
      const int k0 = idx << 3;
      const int g = k0 / group;
      const float s = s_scale[g], zp = s_zero[g];
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = clamp_nan0(rintf(__fdiv_rn(load_as_float(row, k0 + i), s)) + zp, 0.0f, 15.0f);
        // input i of the word sits at nibble position (i & 1) * 4 + (i >> 1): positions
        // 0..7 hold inputs 0,2,4,6,1,3,5,7
        word |= static_cast<uint32_t>(static_cast<int>(v)) << (4 * ((i & 1) * 4 + (i >> 1)));
      }
      prow[idx] = word;
    }
  }
}

// ------------------------------------------------------------------ dequant
// out[n,k] = fp16(nibble - zero) * fp16(scale), product in fp16.
// REF: engine/kernels/w4a16_format.py:53-69, engine/kernels/w4a16_linear.py:211-242.
// One thread per 32-bit packed word (8 weights).
__global__ void __launch_bounds__(256) dequant_w4_kernel(const uint32_t* __restrict__ packed,
                                                         const __half* __restrict__ scales,
                                                         const __half* __restrict__ zeros,
                                                         int layout, int N, int K, int group,
                                                         __half* __restrict__ out, int64_t ldo) {
  const int words_per_row = K >> 3;
  const int64_t total = static_cast<int64_t>(N) * words_per_row;
  const int groups = K / group;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(t / words_per_row);
    const int wi = static_cast<int>(t - static_cast<int64_t>(n) * words_per_row);
    const uint32_t w = packed[t];
    __half* orow = out + static_cast<int64_t>(n) * ldo;
    if (layout == B200Q_W4_REF_SPLIT_HALF_SYM) {
      const int half = group >> 1;
      const int byte0 = wi << 2;               // first packed byte of this word in the row
      const int g = byte0 / half;
      const int j = byte0 - g * half;
      const __half2 s = __half2half2(scales[static_cast<int64_t>(n) * groups + g]);
      W4Quad q = dequant_w4_word_splithalf(w, __float2half2_rn(1032.0f), __float2half2_rn(-72.0f), s);
      __half2* lo = reinterpret_cast<__half2*>(orow + static_cast<int64_t>(g) * group + j);
      __half2* hi = reinterpret_cast<__half2*>(orow + static_cast<int64_t>(g) * group + half + j);
      lo[0] = q.lo01;
      lo[1] = q.lo23;
      hi[0] = q.hi01;
      hi[1] = q.hi23;
    } else {
      const int k0 = wi << 3;
      const int g = k0 / group;
      const float zp = __half2float(zeros[static_cast<int64_t>(n) * groups + g]);
      const __half2 s = __half2half2(scales[static_cast<int64_t>(n) * groups + g]);
      W4Oct o = dequant_w4_word_seq(w, __float2half2_rn(1024.0f + zp),
                                    __float2half2_rn(-(64.0f + zp)), s);
      __half2* dst = reinterpret_cast<__half2*>(orow + k0);
      dst[0] = o.k01;
      dst[1] = o.k23;
      dst[2] = o.k45;
      dst[3] = o.k67;
    }
  }
}

// Scalar variant for groups whose half is not a multiple of 4 bytes (REF layout only).
__global__ void __launch_bounds__(256) dequant_w4_ref_bytes_kernel(
    const uint8_t* __restrict__ packed, const __half* __restrict__ scales, int N, int K, int group,
    __half* __restrict__ out, int64_t ldo) {
  const int bytes_per_row = K >> 1;
  const int half = group >> 1;
  const int groups = K / group;
  const int64_t total = static_cast<int64_t>(N) * bytes_per_row;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(t / bytes_per_row);
    const int bi = static_cast<int>(t - static_cast<int64_t>(n) * bytes_per_row);
    const int g = bi / half, j = bi - g * half;
    const uint32_t b = packed[t];
    const __half s = scales[static_cast<int64_t>(n) * groups + g];
    __half* orow = out + static_cast<int64_t>(n) * ldo + static_cast<int64_t>(g) * group;
    orow[j] = __hmul(__int2half_rn(static_cast<int>(b & 15u) - 8), s);
    orow[j + half] = __hmul(__int2half_rn(static_cast<int>(b >> 4) - 8), s);
  }
}

// ------------------------------------------------------------------ host launchers
int launch_quantize_w8(const void* w, int w_dtype, int64_t ldw, int N, int K, int mode, int8_t* q,
                       void* scales, cudaStream_t stream) {
  dim3 grid(N), block(256);
  switch (w_dtype) {
    case B200Q_F32:
      quantize_w8_kernel<float><<<grid, block, 0, stream>>>(static_cast<const float*>(w), ldw, N,
                                                            K, mode, q, scales);
      break;
    case B200Q_F16:
      quantize_w8_kernel<__half><<<grid, block, 0, stream>>>(static_cast<const __half*>(w), ldw,
                                                             N, K, mode, q, scales);
      break;
    case B200Q_BF16:
      quantize_w8_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(w), ldw, N, K, mode, q, scales);
      break;
    default:
      return B200Q_ERR_INVALID;
  }
  return note_launch();
}

int launch_quantize_w4(const void* w, int w_dtype, int64_t ldw, int N, int K, int group,
                       int layout, void* packed, void* scales, void* zeros, cudaStream_t stream) {
  dim3 grid(N), block(256);
  const size_t smem = sizeof(float) * 2 * static_cast<size_t>(K / group);
  if (smem > 48 * 1024) return B200Q_ERR_UNSUPPORTED;
  auto p = static_cast<uint8_t*>(packed);
  auto s = static_cast<__half*>(scales);
  auto z = static_cast<__half*>(zeros);
  switch (w_dtype) {
    case B200Q_F32:
      quantize_w4_kernel<float><<<grid, block, smem, stream>>>(static_cast<const float*>(w), ldw,
                                                               N, K, group, layout, p, s, z);
      break;
    case B200Q_F16:
      quantize_w4_kernel<__half><<<grid, block, smem, stream>>>(static_cast<const __half*>(w),
                                                                ldw, N, K, group, layout, p, s, z);
      break;
    case B200Q_BF16:
      quantize_w4_kernel<__nv_bfloat16><<<grid, block, smem, stream>>>(
          static_cast<const __nv_bfloat16*>(w), ldw, N, K, group, layout, p, s, z);
      break;
    default:
      return B200Q_ERR_INVALID;
  }
  return note_launch();
}

int launch_dequant_w4(const void* packed, const void* scales, const void* zeros, int layout,
                      int N, int K, int group, void* out, int64_t ldo, cudaStream_t stream) {
  const bool word_path =
      (layout == B200Q_W4_ASYM_ZP_INT32) ? (group % 8 == 0) : ((group >> 1) % 4 == 0);
  const bool aligned = (reinterpret_cast<uintptr_t>(out) % 4 == 0) && (ldo % 2 == 0) &&
                       (reinterpret_cast<uintptr_t>(packed) % 4 == 0);
  if (word_path && aligned) {
    const int64_t total = static_cast<int64_t>(N) * (K >> 3);
    int blocks = static_cast<int>((total + 255) / 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks < 1) blocks = 1;
    dequant_w4_kernel<<<blocks, 256, 0, stream>>>(
        static_cast<const uint32_t*>(packed), static_cast<const __half*>(scales),
        static_cast<const __half*>(zeros), layout, N, K, group, static_cast<__half*>(out), ldo);
  } else {
    if (layout != B200Q_W4_REF_SPLIT_HALF_SYM) return B200Q_ERR_UNSUPPORTED;
    const int64_t total = static_cast<int64_t>(N) * (K >> 1);
    int blocks = static_cast<int>((total + 255) / 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks < 1) blocks = 1;
    dequant_w4_ref_bytes_kernel<<<blocks, 256, 0, stream>>>(
        static_cast<const uint8_t*>(packed), static_cast<const __half*>(scales), N, K, group,
        static_cast<__half*>(out), ldo);
  }
  return note_launch();
}

}  // namespace b200q
