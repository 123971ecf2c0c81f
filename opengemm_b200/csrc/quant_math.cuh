// Arithmetic of block-scaled quantisation shared by the standalone
// quantisation kernel (quantize.cu) and the GEMM epilogue that writes a
// block-scaled C (kernel.cuh): float -> e4m3 / e2m1 codes, exact division by
// a scale, and one scale block end to end.  Bit for bit the reference's torch
// helper (opengemm/python/quant.py:99-122 with pack at :50-70).
#pragma once

#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace og {

enum QFormat { Q_NVFP4 = 0, Q_MXFP8 = 1, Q_MXFP4 = 2 };

// float -> e4m3fn code, nearest even; magnitudes that round past 448 give NaN
// (0x7F) as torch's cast does.  The input is non-negative or signed; NaN -> 0x7F.
__device__ __forceinline__ uint32_t to_e4m3(float x) {
  const uint32_t bits = __float_as_uint(x);
  const uint32_t sign = (bits >> 24) & 0x80u;
  const float mag = fabsf(x);
  if (!(mag < 464.0f)) {
    // 464 itself is the tie between 448 (even mantissa) and the NaN slot: it rounds to 448.
    return sign | ((mag == 464.0f) ? 0x7Eu : 0x7Fu);
  }
  uint32_t code;
  if (mag < 0.015625f) {  // below 2^-6: subnormals, spacing 2^-9
    code = uint32_t(__float2int_rn(mag * 512.0f));  // rn = nearest even; 8 becomes the first normal
  } else {
    const uint32_t m = __float_as_uint(mag);
    // keep 3 mantissa bits: add half of the dropped field with the even tie rule
    const uint32_t rounded = m + 0x7FFFFu + ((m >> 20) & 1u);
    const int exponent = int(rounded >> 23) - 127 + 7;
    code = (uint32_t(exponent) << 3) | ((rounded >> 20) & 7u);
  }
  return sign | code;
}

__device__ __forceinline__ float from_e4m3(uint32_t code) {
  const uint32_t e = (code >> 3) & 15u, m = code & 7u;
  const float mag = e ? __uint_as_float(((e + 120u) << 23) | (m << 20)) : float(m) * 0.001953125f;
  return (code & 0x80u) ? -mag : mag;
}

// Nearest e2m1 code (sign-magnitude, values 0 .5 1 1.5 2 3 4 6), a tie to the
// even code.  A value that rounds to zero is stored as +0, as the reference's
// scan leaves it.
__device__ __forceinline__ uint32_t to_e2m1(float x) {
  const float a = fabsf(x);
  if (!(a < 64.0f)) {
    // Far outside the format (the block's scale underflowed): float32 can no
    // longer tell the distances to the sixteen values apart, and the
    // reference's scan - keep the first best, move to an even code only from
    // an odd one on an exact tie - decides.  Repeat that scan literally.
    const float values[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
    uint32_t code = 0;
    float best = fabsf(__fsub_rn(x, values[0]));
#pragma unroll
    for (uint32_t c = 1; c < 16; ++c) {
      const float d = fabsf(__fsub_rn(x, values[c]));
      if (d < best || (d == best && (c & 1) == 0 && (code & 1) == 1)) best = d, code = c;
    }
    return code;
  }
  uint32_t code = 0;
  code += a > 0.25f;   // tie at .25 stays at code 0 (even)
  code += a >= 0.75f;  // tie at .75 goes up to code 2 (even)
  code += a > 1.25f;   // tie at 1.25 stays at code 2
  code += a >= 1.75f;  // tie goes up to code 4
  code += a > 2.5f;    // tie stays at code 4
  code += a >= 3.5f;   // tie goes up to code 6
  code += a > 5.0f;    // tie stays at code 6
  return (code && x < 0.f) ? (code | 8u) : code;
}

// Eight float32 values -> eight e2m1 codes in one 32-bit word (value 0 in the
// low nibble) with the hardware's packed conversion: nearest even, saturating
// at +-6.  The hardware keeps the sign of a value that rounds to zero; the
// reference stores +0 there, so sign bits of zero magnitudes are cleared.
__device__ __forceinline__ uint32_t pack_e2m1x8(const float* q) {
  uint32_t w = 0;
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    uint32_t byte;
    asm("{\n\t.reg .b8 t;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n\t"
        "cvt.u32.u8 %0, t;\n\t}"
        : "=r"(byte)
        : "f"(q[2 * h]), "f"(q[2 * h + 1]));
    w |= byte << (8 * h);
  }
  const uint32_t magnitude = w & 0x77777777u;
  const uint32_t nonzero = ((magnitude + 0x77777777u) | magnitude) & 0x88888888u;
  return magnitude | (w & nonzero);
}

// Four float32 values -> four e4m3 codes, nearest even (every quotient of a
// block is at most 448 in magnitude, so saturation never differs from torch).
__device__ __forceinline__ uint32_t pack_e4m3x4(const float* q) {
  uint32_t lo, hi;
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}"
      : "=r"(lo) : "f"(q[0]), "f"(q[1]));
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}"
      : "=r"(hi) : "f"(q[2]), "f"(q[3]));
  return lo | (hi << 16);
}

__device__ __forceinline__ float through_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// max(|a|, |b|) of two packed bfloat16 pairs, lane-wise (NaN-propagating like fmaxf is not
// needed: a NaN input already poisons the block's scale through the float path below).
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("{\n\t.reg .b32 x, y;\n\t"
      "abs.bf16x2 x, %1;\n\t"
      "abs.bf16x2 y, %2;\n\t"
      "max.bf16x2 %0, x, y;\n\t}"
      : "=r"(r)
      : "r"(a), "r"(b));
  return r;
}

// x / s, correctly rounded, for a divisor that is a ue4m3 value (at most four
// significant bits).  q0 = x * (1/s) is refined once with the exact residual;
// the true quotient a / b (a < 2^24, b <= 15 after scaling) is either exactly
// representable or at least 2^-30 (relative) away from every float32
// rounding boundary, far more than the refined value's error, so the result
// equals IEEE division.  Tiny numerators, whose quotient could be subnormal,
// take the library division.
__device__ __forceinline__ float divide_exact(float x, float s, float inverse) {
  if (fabsf(x) < 1e-30f) return __fdiv_rn(x, s);
  const float q0 = x * inverse;
  const float residual = __fmaf_rn(-q0, s, x);
  return __fmaf_rn(residual, inverse, q0);
}


// One scale block of a row, end to end: BLOCK values that are exactly
// representable in bfloat16 (16 for nvfp4, 32 for the mx formats) ->
// `stored` (the scale byte) and `words` (the packed codes: BLOCK / 8 words of
// e2m1, or BLOCK / 4 words of e4m3).  The same steps as quantize_kernel takes
// for bfloat16 input.
template <int FORMAT>
__device__ __forceinline__ void quantize_block(const float* v, uint32_t* words, uint32_t& stored) {
  constexpr int BLOCK = FORMAT == Q_NVFP4 ? 16 : 32;
  constexpr bool FP4 = FORMAT != Q_MXFP8;
  constexpr float TOP = FP4 ? 6.0f : 448.0f;
  constexpr float TOP_INVERSE = 1.0f / TOP;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < BLOCK; ++i) amax = fmaxf(amax, fabsf(v[i]));
  bool any_nan = false;
#pragma unroll
  for (int i = 0; i < BLOCK; ++i) any_nan |= (v[i] != v[i]);
  if (any_nan) amax = __uint_as_float(0x7FC00000u);
  const float scale =
      fmaxf((amax > 1e-20f && amax < 1e30f) ? divide_exact(amax, TOP, TOP_INVERSE) : __fdiv_rn(amax, TOP), 1e-30f);
  float divisor, inverse;
  bool exact_inverse;
  if constexpr (FORMAT == Q_NVFP4) {
    stored = to_e4m3(scale);
    divisor = fmaxf(from_e4m3(stored), 1e-30f);
    inverse = __frcp_rn(divisor);
    exact_inverse = false;
  } else {
    const uint32_t bits = __float_as_uint(scale);
    const int exponent = int(bits >> 23) - 127 + ((bits & 0x7FFFFFu) ? 1 : 0);
    stored = uint32_t(exponent + 127);
    divisor = __uint_as_float(stored << 23);
    exact_inverse = exponent <= 126;
    inverse = exact_inverse ? __uint_as_float(uint32_t(127 - exponent) << 23) : 0.f;
  }
  const bool plain = FORMAT == Q_NVFP4 && ((stored & 0x7Fu) == 0x7Fu || (stored & 0x7Fu) == 0u);
  float q[BLOCK];
#pragma unroll
  for (int i = 0; i < BLOCK; i += 2) {
    float pair[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // bfloat16 numerator over a ue4m3 or power-of-two divisor: one multiply
      // by the reciprocal rounds to the same bfloat16 as the exact quotient.
      if (exact_inverse || (FORMAT == Q_NVFP4 && !plain)) pair[h] = v[i + h] * inverse;
      else pair[h] = __fdiv_rn(v[i + h], divisor);
    }
    uint32_t both;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(both) : "f"(pair[1]), "f"(pair[0]));
    q[i] = __uint_as_float(both << 16);
    q[i + 1] = __uint_as_float(both & 0xFFFF0000u);
  }
  if constexpr (FP4) {
    const bool nan_scale = FORMAT == Q_NVFP4 && (stored & 0x7Fu) == 0x7Fu;
    const bool literal = !(amax < 32.0f * divisor);
#pragma unroll
    for (int i = 0; i < BLOCK / 8; ++i) {
      uint32_t w = 0;
      if (literal) {
#pragma unroll
        for (int h = 0; h < 8; ++h) w |= to_e2m1(q[8 * i + h]) << (4 * h);
      } else {
        w = pack_e2m1x8(q + 8 * i);
      }
      words[i] = nan_scale ? 0u : w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < BLOCK / 4; ++i) words[i] = pack_e4m3x4(q + 4 * i);
  }
}

}  // namespace og
