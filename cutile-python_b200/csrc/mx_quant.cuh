// MXFP8 and NVFP4 block arithmetic shared by the quantiser kernels and the quantising GEMM
// epilogues.
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200k {

__device__ __forceinline__ int64_t swizzled_sf_offset(int64_t row, int64_t kblk, int64_t k_atoms) {
  return ((row >> 7) * k_atoms + (kblk >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
         (kblk & 3);
}

// ceil(log2(q)) for q > 0 as the reference computes it in fp32:
// ceil(float(log2(q))).  Away from powers of two this is the exponent of q plus one;
// within a few ulps above a power of two the fp32 rounding of the logarithm decides,
// which the double-precision logarithm rounded to fp32 reproduces.
__device__ __forceinline__ int ceil_log2_f32(float q) {
  const uint32_t bits = __float_as_uint(q);
  int e = static_cast<int>((bits >> 23) & 0xff);
  uint32_t man = bits & 0x7fffff;
  if (e == 0) {  // subnormal: not reachable after the 1e-12 clamp, kept for completeness
    return static_cast<int>(ceilf(static_cast<float>(log2(static_cast<double>(q)))));
  }
  e -= 127;
  if (man == 0) return e;
  if (man > 64) return e + 1;
  return static_cast<int>(ceilf(static_cast<float>(log2(static_cast<double>(q)))));
}

// The scale byte (ue8m0) and the exact reciprocal 2^-e of one block with maximum `amax`;
// NaN or infinity anywhere in the block gives the byte 0xff and a NaN reciprocal, as the
// reference's float arithmetic does.
__device__ __forceinline__ uint8_t block_scale(float amax, bool has_nan, float* inv_scale) {
  if (has_nan || amax == __int_as_float(0x7f800000)) {
    *inv_scale = __int_as_float(0x7fc00000);
    return 0xff;
  }
  float s = __fdiv_rn(amax, 448.0f);
  s = fmaxf(s, 1e-12f);
  const int e = ceil_log2_f32(s);
  // 2^-e, exact: e is in [-39, 120]
  *inv_scale = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
  if (127 - e <= 0) *inv_scale = ldexpf(1.0f, -e);
  return static_cast<uint8_t>(e + 127);
}


// One block of 32 fp32 values -> 32 e4m3 bytes (eight packed words) and the scale byte, with
// the quantiser's exact arithmetic (mxfp8_quantize_kernel produces the same bytes).
__device__ __forceinline__ uint8_t mx_quantize_block32(const float (&v)[32], uint32_t (&packed)[8]) {
  float amax = 0.0f;
  bool has_nan = false;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    amax = fmaxf(amax, fabsf(v[i]));
    has_nan |= (v[i] != v[i]);
  }
  float inv_scale;
  const uint8_t sf_byte = block_scale(amax, has_nan, &inv_scale);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv_scale, v[4 * i + 1] * inv_scale),
                                                __NV_SATFINITE, __NV_E4M3);
    const uint32_t b = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv_scale, v[4 * i + 3] * inv_scale),
                                                __NV_SATFINITE, __NV_E4M3);
    packed[i] = a | (b << 16);
  }
  return sf_byte;
}

// ---- NVFP4 ----
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// One 16-element block: returns the ue4m3 scale byte, packs the sixteen e2m1 codes into
// lo (elements 0..7) and hi (8..15), low nibble = even element.
__device__ __forceinline__ uint8_t nvfp4_block(const float (&v)[16], float six_st, float s_t,
                                               uint32_t* lo_out, uint32_t* hi_out) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  uint8_t sf_byte = 0;
  float denom = 0.0f;
  if (amax > 0.0f && six_st > 0.0f) {
    const float r = __fdiv_rn(amax, six_st);
    sf_byte = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
    denom = __fmul_rn(e4m3_to_f32(sf_byte), s_t);
  }
  // x / denom as x * (1 / denom), both correctly rounded: one reciprocal per block instead
  // of sixteen divisions.  A subnormal denom (reciprocal not finite) keeps the division.
  // One branch per block, not per pair: the three cases run their own straight-line loops.
  uint32_t code[8];
  if (denom >= 1.17549435e-38f) {
    const float inv = __frcp_rn(denom);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      code[i] = __nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(v[2 * i], inv), __fmul_rn(v[2 * i + 1], inv)),
                                         __NV_E2M1, cudaRoundNearest);
  } else if (denom > 0.0f) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      code[i] = __nv_cvt_float2_to_fp4x2(make_float2(__fdiv_rn(v[2 * i], denom), __fdiv_rn(v[2 * i + 1], denom)),
                                         __NV_E2M1, cudaRoundNearest);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) code[i] = 0;     // the codes of (+0, +0)
  }
  // four code bytes per word with three byte permutes
  const uint32_t lo = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
  const uint32_t hi = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
  *lo_out = lo;
  *hi_out = hi;
  return sf_byte;
}

}  // namespace b200k
