// Numeric contract of the paged KV cache: bf16 / e4m3fn / e2m1 / e8m0 conversions and the two block quantisers.
// Storage types are raw integers (bf16 = uint16_t, fp8 = uint8_t). Every operation is a single correctly rounded fp32
// operation or integer arithmetic, so the results do not depend on the compiler as long as fast-math, flush-to-zero
// and approximate division stay off (the build passes none of them, and -fmad=false).
//
// The arithmetic reproduces ewtodd/unholy's src/kernels/dev.hip.hpp:40-127 (conversions), src/kernels/indexer.hip:18-41
// (MXFP4 block: e2m1 codes + one e8m0 scale per 32 values) and src/kernels/ref_elem.hip:18-41 (fp8 block: e4m3 codes +
// one e8m0 scale per 32/64/128 values) bit for bit.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace pkv {

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Round to nearest even; NaN keeps its upper bits and is made quiet.
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40u);
  return uint16_t((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ float e8m0_bits_to_f32(uint32_t e) { return __uint_as_float(e << 23); }

// Exponent byte of the smallest power of two >= v (v positive and normal).
__device__ __forceinline__ uint32_t pow2_ceil_exp(float v) {
  const uint32_t b = __float_as_uint(v);
  return (((b >> 23) & 0xffu) + ((b & 0x7fffffu) ? 1u : 0u)) & 0xffu;
}

// e4m3fn decode.
__device__ __forceinline__ float e4m3_bits_to_f32(uint32_t c) {
  const uint32_t ex = (c >> 3) & 15u, man = c & 7u;
  const float mag = ex == 0 ? float(man) * (1.0f / 512.0f) : __uint_as_float(((ex + 120u) << 23) | (man << 20));
  return (c & 0x80u) ? -mag : mag;
}

// e4m3fn encode of |x| <= 448, round to nearest even. Below 2^-6 the code counts multiples of 2^-9.
__device__ __forceinline__ uint32_t f32_to_e4m3_bits(float x) {
  uint32_t u = __float_as_uint(x);
  const uint32_t sign = (u >> 24) & 0x80u;
  u &= 0x7fffffffu;
  if (int(u >> 23) - 127 < -6) return sign | (uint32_t(rintf(__uint_as_float(u) * 512.0f)) & 0xffu);
  u += 0x7ffffu + ((u >> 20) & 1u);
  return sign | ((((u >> 23) - 120u) << 3) & 0x78u) | ((u >> 20) & 7u);
}

// e2m1 grid: 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign.
__device__ __forceinline__ float e2m1_bits_to_f32(uint32_t nib) {
  const uint32_t m = nib & 7u;
  const float mag = m < 4u ? 0.5f * float(m) : (m == 7u ? 6.0f : float(m - 2u));
  return (nib & 8u) ? -mag : mag;
}

// Nibble of x (already clamped to [-6, 6]) rounded to the nearest grid point, ties to the even code. The sign bit is
// set when x < 0, including when the magnitude rounds to zero; x = -0.0 is not < 0 and gives nibble 0.
__device__ __forceinline__ uint32_t e2m1_nibble(float x) {
  const float a = fabsf(x);
  uint32_t m;
  if (a <= 0.25f) m = 0u;
  else if (a < 0.75f) m = 1u;
  else if (a <= 1.25f) m = 2u;
  else if (a < 1.75f) m = 3u;
  else if (a <= 2.5f) m = 4u;
  else if (a < 3.5f) m = 5u;
  else if (a <= 5.0f) m = 6u;
  else m = 7u;
  return m | (x < 0.0f ? 8u : 0u);
}

// Eight bf16 values of one thread (a 16-byte vector) as floats.
__device__ __forceinline__ void unpack8(const uint4& w, float* v) {
  const uint32_t s[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(s[i] << 16);
    v[2 * i + 1] = __uint_as_float(s[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ float absmax8(const float* v) {
  float a = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(v[i]));
  return a;
}

// Maximum over an aligned group of `group` lanes (4, 8 or 16 lanes: a block of 32, 64 or 128 values at 8 per lane).
// Every lane of the warp must call it.
__device__ __forceinline__ float group_max(float a, int group) {
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
  if (group > 4) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
  if (group > 8) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
  return a;
}

// MXFP4 block scale from the block's absolute maximum: floor 6 * 2^-126, then the power of two >= amax / 6.
__device__ __forceinline__ uint32_t fp4_scale_exp(float amax) {
  return pow2_ceil_exp(fmaxf(amax, 6.0f * 1.1754943508222875e-38f) * (1.0f / 6.0f));
}
// fp8 block scale: floor 1e-4, then the power of two >= amax / 448.
__device__ __forceinline__ uint32_t fp8_scale_exp(float amax) {
  return pow2_ceil_exp(fmaxf(amax, 1e-4f) * (1.0f / 448.0f));
}

// Eight values -> eight e2m1 nibbles packed low-to-high (value 0 in bits 0..3), i.e. 4 bytes of a code row.
__device__ __forceinline__ uint32_t fp4_pack8(const float* v, float sc) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) w |= e2m1_nibble(fminf(fmaxf(v[i] / sc, -6.0f), 6.0f)) << (4 * i);
  return w;
}

// Eight values -> eight e4m3 bytes (value 0 in the lowest byte of .x).
__device__ __forceinline__ uint2 fp8_pack8(const float* v, float sc) {
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i >> 2] |= f32_to_e4m3_bits(fminf(fmaxf(v[i] / sc, -448.0f), 448.0f)) << (8 * (i & 3));
  return make_uint2(w[0], w[1]);
}

// Hadamard transform of one 128-value segment held by 16 consecutive lanes, 8 values each (value j * 8 + e in v[e] of
// lane j of the group), as ewtodd/unholy's hadamard128_kernel does it (src/kernels/ref_elem.hip:111-135): seven
// butterfly stages h = 1 .. 64 in fp32, (a, c) -> (a + c, a - c) for the pair (i, i + h), then * 128^-0.5 and rounding
// to bf16. Stages 1, 2, 4 pair values of one lane; stages 8 .. 64 pair lane j with lane j ^ (h / 8): the lower lane
// keeps own + other, the upper one other - own — the same two operands per result as the reference, so the same
// bits. Every lane of the warp must call it. On return v holds the bf16-rounded values as floats.
__device__ __forceinline__ void hadamard128_lanes(float* v, int j) {
#pragma unroll
  for (int h = 1; h <= 4; h <<= 1)
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = (t / h) * 2 * h + (t % h);
      const float a = v[i], c = v[i + h];
      v[i] = a + c;
      v[i + h] = a - c;
    }
#pragma unroll
  for (int m = 1; m <= 8; m <<= 1) {
    const bool upper = (j & m) != 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float o = __shfl_xor_sync(0xffffffffu, v[e], m);
      v[e] = upper ? o - v[e] : v[e] + o;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = bf16_bits_to_f32(f32_to_bf16_bits(v[e] * 0.08838834764831845f));
}

}  // namespace pkv
