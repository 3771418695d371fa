// Register-level conversions from packed integers to fp16/bf16 pairs.
//
// The fp16 results reproduce the reference's dequantisation contract
// (engine/kernels/w4a16_format.py:53-69): fp16(nibble - zero) * fp16(scale),
// the product rounded once in fp16.  Integers are turned into floats without
// an int->float instruction: OR-ing a small unsigned integer n into the
// mantissa of fp16 1024.0 (0x6400) gives exactly 1024 + n.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200q {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));  // (a&b)|c
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 h) {
  return *reinterpret_cast<uint32_t*>(&h);
}

// fp16x2 -> bf16x2, each value rounded to nearest even (what tensor.to(bf16) does).
__device__ __forceinline__ uint32_t h2_to_bf162(__half2 h) {
  float2 f = __half22float2(h);
  return as_u32(__floats2bfloat162_rn(f.x, f.y));
}

// One 32-bit word of the split-half layout holds bytes b0..b3; byte bi carries
// input j+i (low nibble) and input j+i+G/2 (high nibble).  Produces the four
// "low" weights and the four "high" weights, each as two fp16x2 in K order,
// already multiplied by the group scale: (nibble - zero) * scale.
//   bias_lo  = 1024 + zero          (subtracted from the 1024+n encoding)
//   bias_hi  = 64 + zero            (after the x16 encoding is scaled by 1/16)
struct W4Quad {
  __half2 lo01, lo23, hi01, hi23;
};
__device__ __forceinline__ W4Quad dequant_w4_word_splithalf(uint32_t w, __half2 bias_lo,
                                                            __half2 neg_bias_hi, __half2 scale) {
  const uint32_t kLoMask = 0x000F000Fu, kHiMask = 0x00F000F0u, kMagic = 0x64006400u;
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  uint32_t w8 = w >> 8;
  // (b0, b2) and (b1, b3) pairs
  __half2 a = __hsub2(as_h2(lop3_and_or(w, kLoMask, kMagic)), bias_lo);
  __half2 c = __hsub2(as_h2(lop3_and_or(w8, kLoMask, kMagic)), bias_lo);
  // high nibbles sit at bits 4..7: the encoding is 1024 + 16 n; (.)/16 - (64+zero) is exact
  __half2 b = __hfma2(as_h2(lop3_and_or(w, kHiMask, kMagic)), sixteenth, neg_bias_hi);
  __half2 d = __hfma2(as_h2(lop3_and_or(w8, kHiMask, kMagic)), sixteenth, neg_bias_hi);
  a = __hmul2(a, scale);
  c = __hmul2(c, scale);
  b = __hmul2(b, scale);
  d = __hmul2(d, scale);
  W4Quad q;
  q.lo01 = as_h2(prmt(as_u32(a), as_u32(c), 0x5410));
  q.lo23 = as_h2(prmt(as_u32(a), as_u32(c), 0x7632));
  q.hi01 = as_h2(prmt(as_u32(b), as_u32(d), 0x5410));
  q.hi23 = as_h2(prmt(as_u32(b), as_u32(d), 0x7632));
  return q;
}

// One 32-bit word of the asymmetric layout.  Its eight nibbles hold inputs 8w+{0,2,4,6,1,3,5,7}
// (input i sits at nibble position (i & 1) * 4 + (i >> 1)): the two 0x000F000F-spaced nibbles
// that one lop3 isolates are then neighbours in K, so no byte permute is needed.  Produces the
// eight weights in K order as four fp16x2, scaled.
struct W4Oct {
  __half2 k01, k23, k45, k67;
};
__device__ __forceinline__ W4Oct dequant_w4_word_seq(uint32_t w, __half2 bias_lo,
                                                     __half2 neg_bias_hi, __half2 scale) {
  const uint32_t kLoMask = 0x000F000Fu, kHiMask = 0x00F000F0u, kMagic = 0x64006400u;
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  uint32_t w8 = w >> 8;
  W4Oct o;
  o.k01 = __hmul2(__hsub2(as_h2(lop3_and_or(w, kLoMask, kMagic)), bias_lo), scale);
  o.k23 = __hmul2(__hfma2(as_h2(lop3_and_or(w, kHiMask, kMagic)), sixteenth, neg_bias_hi), scale);
  o.k45 = __hmul2(__hsub2(as_h2(lop3_and_or(w8, kLoMask, kMagic)), bias_lo), scale);
  o.k67 = __hmul2(__hfma2(as_h2(lop3_and_or(w8, kHiMask, kMagic)), sixteenth, neg_bias_hi), scale);
  return o;
}

// Four int8 in one word -> two fp16x2 in K order, exact (|q| <= 128).
// q ^ 0x80 is q + 128 as an unsigned byte; 0x6400 | u is 1024 + u; minus 1152.
__device__ __forceinline__ void int8x4_to_h2(uint32_t w, __half2& k01, __half2& k23) {
  const __half2 bias = __float2half2_rn(1152.0f);
  uint32_t x = w ^ 0x80808080u;
  k01 = __hsub2(as_h2(prmt(x, 0x64646464u, 0x4140)), bias);
  k23 = __hsub2(as_h2(prmt(x, 0x64646464u, 0x4342)), bias);
}

}  // namespace b200q
