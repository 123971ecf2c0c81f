// Block-scaled quantisation on the GPU: values -> nvfp4 / mxfp8 / mxfp4 storage
// plus scales, written both row-major and in the 128x4 blocked layout the GEMM
// reads, in one pass over the input.
//
// Bit for bit the arithmetic of the reference's torch helper
// (opengemm/python/quant.py:99-122, with pack at :50-70 and to_blocked at
// :82-97), which takes several elementwise passes and a 16-way code scan:
//   scale  = max(amax / top, 1e-30)            top = 6 (e2m1) or 448 (e4m3)
//   ue8m0:   scale = 2^ceil(log2(scale))
//   stored = scale rounded to the scale type   (ue4m3: nearest even)
//   value  = bf16(x / float(stored))           then the nearest element value,
//            a tie going to the even code
//
// One thread owns four consecutive scale blocks of one row (64 values for
// nvfp4, 128 for the mx formats): it reads them with 16-byte loads, writes
// 32-128 contiguous bytes of packed output and one 32-bit word of four scales.
// A CTA of 128 threads covers 128 rows, so its scale words make up exactly
// one 512-byte atom of the blocked layout.  HBM-bound: 2 (bf16) or 4 (f32)
// bytes read and 0.5-1 byte plus 1/16-1/32 byte written per value.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/opengemm_b200.h"

namespace og {
namespace {

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

template <int FORMAT, bool F32_IN>
__global__ void __launch_bounds__(128) quantize_kernel(const void* __restrict__ x, int64_t rows, int64_t k,
                                                       uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                       uint8_t* __restrict__ blocked) {
  constexpr int BLOCK = FORMAT == Q_NVFP4 ? 16 : 32;  // values per scale
  constexpr bool FP4 = FORMAT != Q_MXFP8;
  constexpr float TOP = FP4 ? 6.0f : 448.0f;
  const int64_t k_blocks = k / BLOCK;
  const int64_t k_groups = (k_blocks + 3) / 4;
  const int64_t row = int64_t(blockIdx.y) * 128 + threadIdx.x;
  const int64_t group = blockIdx.x;  // four scale blocks along K
  uint32_t scale_word = 0;
  if (row < rows) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t kb = group * 4 + j;
      if (kb >= k_blocks) break;
      float v[BLOCK];
      const int64_t at = row * k + kb * BLOCK;
      if constexpr (F32_IN) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(x) + at);
#pragma unroll
        for (int i = 0; i < BLOCK / 4; ++i) {
          const float4 q = __ldg(src + i);
          v[4 * i] = q.x, v[4 * i + 1] = q.y, v[4 * i + 2] = q.z, v[4 * i + 3] = q.w;
        }
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + at);
#pragma unroll
        for (int i = 0; i < BLOCK / 8; ++i) {
          const uint4 q = __ldg(src + i);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            v[8 * i + 2 * h] = __uint_as_float(w[h] << 16);
            v[8 * i + 2 * h + 1] = __uint_as_float(w[h] & 0xFFFF0000u);
          }
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < BLOCK; ++i) amax = fmaxf(amax, fabsf(v[i]));
      float scale = fmaxf(__fdiv_rn(amax, TOP), 1e-30f);
      uint32_t stored;
      float stored_value;
      if constexpr (FORMAT == Q_NVFP4) {
        stored = to_e4m3(scale);
        stored_value = from_e4m3(stored);
      } else {
        // 2^ceil(log2(scale)): the exponent, plus one when any mantissa bit is set
        const uint32_t bits = __float_as_uint(scale);
        int exponent = int(bits >> 23) - 127 + ((bits & 0x7FFFFFu) ? 1 : 0);
        if ((bits >> 23) == 0) exponent = -126;  // float32 subnormals: not reachable after the 1e-30 floor
        stored = uint32_t(exponent + 127);
        stored_value = __uint_as_float(stored << 23);
      }
      const float divisor = fmaxf(stored_value, 1e-30f);
      // A ue4m3 scale past the format's range is stored as NaN; dividing by it
      // makes every value NaN, which the reference's nearest-code scan leaves
      // at code 0.
      const bool nan_scale = FORMAT == Q_NVFP4 && (stored & 0x7Fu) == 0x7Fu;
      scale_word |= stored << (8 * j);
      if (scales) scales[row * k_blocks + kb] = uint8_t(stored);
      // quantise through bfloat16, as the reference does
      if constexpr (FP4) {
        uint32_t words[BLOCK / 8];
#pragma unroll
        for (int i = 0; i < BLOCK / 8; ++i) {
          uint32_t w = 0;
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            const float q = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(v[8 * i + h], divisor)));
            w |= to_e2m1(q) << (4 * h);
          }
          words[i] = nan_scale ? 0u : w;
        }
        uint8_t* dst = packed + (row * k + kb * BLOCK) / 2;
        if constexpr (BLOCK == 16) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(words[0], words[1]);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
        }
      } else {
        uint32_t words[BLOCK / 4];
#pragma unroll
        for (int i = 0; i < BLOCK / 4; ++i) {
          uint32_t w = 0;
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float q = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(v[4 * i + h], divisor)));
            w |= to_e4m3(q) << (8 * h);
          }
          words[i] = w;
        }
        uint4* dst = reinterpret_cast<uint4*>(packed + row * k + kb * BLOCK);
        dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
        dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
      }
    }
  }
  if (blocked) {
    // Rows past the end pad the last 128-row block with zero scales.
    const int64_t atom = int64_t(blockIdx.y) * k_groups + group;
    const uint32_t r = threadIdx.x;
    *reinterpret_cast<uint32_t*>(blocked + atom * 512 + (r & 31) * 16 + (r >> 5) * 4) = scale_word;
  }
}

thread_local char quantize_error[256];

int quantize_fail(const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(quantize_error, sizeof quantize_error, format, args);
  va_end(args);
  return OG_ERR_LAUNCH;
}

}  // namespace
}  // namespace og

using namespace og;

extern "C" {

OG_API const char* og_b200_quantize_error(void) { return quantize_error; }

OG_API int32_t og_b200_quantize(const char* format, const void* x, int32_t x_is_f32, int64_t rows, int64_t k,
                                void* packed, void* scales, void* scales_blocked, int32_t device, void* stream) {
  if (!format || !x || !packed) return quantize_fail("format, x and packed must not be null");
  int which = -1;
  if (!std::strcmp(format, "nvfp4")) which = Q_NVFP4;
  else if (!std::strcmp(format, "mxfp8")) which = Q_MXFP8;
  else if (!std::strcmp(format, "mxfp4")) which = Q_MXFP4;
  else return quantize_fail("%.16s is not a block-scaled format: nvfp4, mxfp8 or mxfp4", format);
  const int block = which == Q_NVFP4 ? 16 : 32;
  if (rows <= 0 || k <= 0 || k % block) return quantize_fail("K = %lld must be a positive multiple of %d", (long long)k, block);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed)) & 15)
    return quantize_fail("x and packed must start on 16-byte boundaries");
  if (scales_blocked && (reinterpret_cast<uintptr_t>(scales_blocked) & 3))
    return quantize_fail("the blocked scale buffer must start on a 4-byte boundary");
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return quantize_fail("cudaGetDevice failed");
  if (current != device && cudaSetDevice(device) != cudaSuccess) return quantize_fail("cudaSetDevice(%d) failed", device);
  const int64_t k_groups = (k / block + 3) / 4;
  const int64_t row_blocks = (rows + 127) / 128;
  if (k_groups > 0x7FFFFFFF || row_blocks > 65535) return quantize_fail("the operand is too large for one launch");
  const dim3 grid{unsigned(k_groups), unsigned(row_blocks), 1};
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* p = static_cast<uint8_t*>(packed);
  uint8_t* sc = static_cast<uint8_t*>(scales);
  uint8_t* sb = static_cast<uint8_t*>(scales_blocked);
#define OG_QUANTIZE(F)                                                                      \
  if (x_is_f32) quantize_kernel<F, true><<<grid, 128, 0, s>>>(x, rows, k, p, sc, sb);       \
  else quantize_kernel<F, false><<<grid, 128, 0, s>>>(x, rows, k, p, sc, sb)
  if (which == Q_NVFP4) { OG_QUANTIZE(Q_NVFP4); }
  else if (which == Q_MXFP8) { OG_QUANTIZE(Q_MXFP8); }
  else { OG_QUANTIZE(Q_MXFP4); }
#undef OG_QUANTIZE
  const cudaError_t launched = cudaGetLastError();
  if (launched != cudaSuccess) return quantize_fail("quantize launch failed: %s", cudaGetErrorString(launched));
  return OG_OK;
}

}  // extern "C"
