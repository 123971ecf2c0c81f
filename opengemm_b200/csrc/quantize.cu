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
// One thread quantises one scale block at a time (16 or 32 values) with
// 16-byte loads and stores; the lanes of a warp take consecutive blocks of a
// row, so a warp reads and writes contiguous kilobytes; a CTA covers 128 rows
// x 32 blocks and writes its eight 512-byte atoms of the blocked scale layout
// whole.  HBM-bound: 2 (bf16) or 4 (f32) bytes read and 0.5-1 byte plus
// 1/16-1/32 byte written per value.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/opengemm_b200.h"
#include "quant_math.cuh"

namespace og {
namespace {

constexpr int Q_THREADS = 256;
constexpr int Q_GROUPS = 8;                 // K groups (of four scale blocks) per CTA
constexpr int Q_BLOCKS = Q_GROUPS * 4;      // scale blocks along K per CTA

// A CTA covers 128 rows x 32 scale blocks.  One thread quantises one scale
// block at a time (16 or 32 values, 32-128 bytes of input); the 32 lanes of a
// warp take the 32 consecutive blocks of one row, 1-4 KiB of contiguous
// input, and the CTA's eight warps walk the 128 rows sixteen at a time.  Scale
// bytes collect in shared memory and leave as whole 512-byte atoms.
template <int FORMAT, bool F32_IN>
__global__ void __launch_bounds__(Q_THREADS) quantize_kernel(const void* __restrict__ x, int64_t rows, int64_t k,
                                                             uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                             uint8_t* __restrict__ blocked) {
  constexpr int BLOCK = FORMAT == Q_NVFP4 ? 16 : 32;  // values per scale
  constexpr bool FP4 = FORMAT != Q_MXFP8;
  constexpr float TOP = FP4 ? 6.0f : 448.0f;
  constexpr int VEC = F32_IN ? 4 : 8;                 // values per 16-byte load
  constexpr int LOADS = BLOCK / VEC;                  // loads per scale block
  const int64_t k_blocks = k / BLOCK;
  const int64_t k_groups = (k_blocks + 3) / 4;
  __shared__ uint8_t scale_bytes[128][Q_BLOCKS + 4];  // [row][block]; the pad spreads banks
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t kb = int64_t(blockIdx.x) * Q_BLOCKS + lane;  // this lane's scale block along K
  const bool live_block = kb < k_blocks;

#pragma unroll 2
  for (int step = 0; step < 16; ++step) {
    const int row_in_block = step * 8 + warp;
    const int64_t row = int64_t(blockIdx.y) * 128 + row_in_block;
    uint32_t stored = 0;
    if (row < rows && live_block) {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x) +
                                                        (row * k + kb * BLOCK) * (F32_IN ? 4 : 2));
      uint4 raw[LOADS];
#pragma unroll
      for (int i = 0; i < LOADS; ++i) raw[i] = __ldg(src + i);
      float v[BLOCK];
#pragma unroll
      for (int i = 0; i < LOADS; ++i) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          if constexpr (F32_IN) {
            v[4 * i + h] = __uint_as_float(w[h]);
          } else {
            v[8 * i + 2 * h] = __uint_as_float(w[h] << 16);
            v[8 * i + 2 * h + 1] = __uint_as_float(w[h] & 0xFFFF0000u);
          }
        }
      }
      float amax = 0.f;
      if constexpr (F32_IN) {
#pragma unroll
        for (int i = 0; i < BLOCK; ++i) amax = fmaxf(amax, fabsf(v[i]));
      } else {
        // bfloat16 input: the largest magnitude by packed pairs, two values per
        // instruction; the comparison of magnitudes is exact in any width.
        uint32_t m2 = absmax_bf16x2(raw[0].x, raw[0].y);
        m2 = absmax_bf16x2(m2, absmax_bf16x2(raw[0].z, raw[0].w));
#pragma unroll
        for (int i = 1; i < LOADS; ++i) {
          m2 = absmax_bf16x2(m2, absmax_bf16x2(raw[i].x, raw[i].y));
          m2 = absmax_bf16x2(m2, absmax_bf16x2(raw[i].z, raw[i].w));
        }
        amax = fmaxf(__uint_as_float(m2 << 16), __uint_as_float(m2 & 0xFFFF0000u));
        bool any_nan = false;  // max.bf16x2 drops NaN operands; the reference's amax keeps them
#pragma unroll
        for (int i = 0; i < BLOCK; ++i) any_nan |= (v[i] != v[i]);
        if (any_nan) amax = __uint_as_float(0x7FC00000u);
      }
      // amax / 6 and amax / 448 by the same exact reciprocal refinement (3 and 7
      // are the divisors' odd parts); tiny or huge amax takes the library division.
      constexpr float TOP_INVERSE = 1.0f / TOP;
      const float scale = fmaxf((amax > 1e-20f && amax < 1e30f) ? divide_exact(amax, TOP, TOP_INVERSE) : __fdiv_rn(amax, TOP), 1e-30f);
      float divisor, inverse;
      bool exact_inverse;  // `inverse` is exactly 1 / divisor (a power of two)
      if constexpr (FORMAT == Q_NVFP4) {
        stored = to_e4m3(scale);
        divisor = fmaxf(from_e4m3(stored), 1e-30f);
        inverse = __frcp_rn(divisor);
        exact_inverse = false;
      } else {
        // 2^ceil(log2(scale)): the exponent, plus one when any mantissa bit is
        // set (the 1e-30 floor keeps `scale` a normal float).  Dividing by a
        // power of two is multiplying by its reciprocal, exactly.
        const uint32_t bits = __float_as_uint(scale);
        const int exponent = int(bits >> 23) - 127 + ((bits & 0x7FFFFFu) ? 1 : 0);
        stored = uint32_t(exponent + 127);
        divisor = __uint_as_float(stored << 23);
        exact_inverse = exponent <= 126;
        inverse = exact_inverse ? __uint_as_float(uint32_t(127 - exponent) << 23) : 0.f;
      }
      if (scales) scales[row * k_blocks + kb] = uint8_t(stored);

      // quotients, rounded through bfloat16 as the reference does
      // A ue4m3 scale that underflowed to zero (divisor 1e-30) or overflowed to NaN
      // is rare: those blocks take the library division.
      const bool plain = FORMAT == Q_NVFP4 && ((stored & 0x7Fu) == 0x7Fu || (stored & 0x7Fu) == 0u);
      // bfloat16 values over a ue4m3 divisor: numerator and divisor carry 8 and 4
      // significant bits, so the exact quotient is either a bfloat16 value itself
      // (the divisor's odd part divides the numerator) or a fraction whose binary
      // expansion repeats with a period of at most 12 bits and therefore stays
      // 2^-14 (relative) or more away from every bfloat16 rounding boundary.  The
      // one-multiply estimate x * (1/s) is within 2^-23 of it: rounded to
      // bfloat16 it gives the same value as the correctly rounded float32
      // quotient does (and rounding that to float32 first changes nothing, for
      // the same reason).
      const bool short_quotient = FORMAT == Q_NVFP4 && !F32_IN && !plain;
      float q[BLOCK];
#pragma unroll
      for (int i = 0; i < BLOCK; i += 2) {
        float pair[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (exact_inverse || short_quotient) pair[h] = v[i + h] * inverse;
          else if (FORMAT != Q_NVFP4 || plain) pair[h] = __fdiv_rn(v[i + h], divisor);
          else pair[h] = divide_exact(v[i + h], divisor, inverse);
        }
        uint32_t both;  // two quotients rounded to bfloat16 in one instruction
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(both) : "f"(pair[1]), "f"(pair[0]));
        q[i] = __uint_as_float(both << 16);
        q[i + 1] = __uint_as_float(both & 0xFFFF0000u);
      }

      if constexpr (FP4) {
        // A ue4m3 scale past the format's range is stored as NaN: every quotient
        // is then NaN, which the reference's nearest-code scan leaves at code 0.
        const bool nan_scale = FORMAT == Q_NVFP4 && (stored & 0x7Fu) == 0x7Fu;
        // Quotients far outside +-6 (the scale underflowed) need the literal scan.
        // (amax >= 32 x divisor is a cheap superset of "some quotient reaches 64".)
        const bool literal = !(amax < 32.0f * divisor);
        uint32_t words[BLOCK / 8];
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
        uint8_t* dst = packed + (row * k + kb * BLOCK) / 2;
        if constexpr (BLOCK == 16) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(words[0], words[1]);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
        }
      } else {
        uint32_t words[BLOCK / 4];
#pragma unroll
        for (int i = 0; i < BLOCK / 4; ++i) words[i] = pack_e4m3x4(q + 4 * i);
        uint4* dst = reinterpret_cast<uint4*>(packed + row * k + kb * BLOCK);
        dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
        dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
      }
    }
    scale_bytes[row_in_block][lane] = uint8_t(stored);  // zero for rows and blocks past the end
  }
  if (blocked) {
    // Whole atoms, 128 words each: word w holds the four scales of row
    // (w % 4) * 32 + w / 4 for the atom's four scale blocks.
    __syncthreads();
    const int64_t first_group = int64_t(blockIdx.x) * Q_GROUPS;
    for (int i = threadIdx.x; i < Q_GROUPS * 128; i += Q_THREADS) {
      const int g = i >> 7, word = i & 127;
      if (first_group + g >= k_groups) break;
      const int r = (word & 3) * 32 + (word >> 2);
      const uint8_t* four = &scale_bytes[r][4 * g];
      uint32_t* atom = reinterpret_cast<uint32_t*>(blocked + (int64_t(blockIdx.y) * k_groups + first_group + g) * 512);
      atom[word] = uint32_t(four[0]) | (uint32_t(four[1]) << 8) | (uint32_t(four[2]) << 16) | (uint32_t(four[3]) << 24);
    }
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
  const dim3 grid{unsigned((k_groups + Q_GROUPS - 1) / Q_GROUPS), unsigned(row_blocks), 1};
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* p = static_cast<uint8_t*>(packed);
  uint8_t* sc = static_cast<uint8_t*>(scales);
  uint8_t* sb = static_cast<uint8_t*>(scales_blocked);
#define OG_QUANTIZE(F)                                                                      \
  if (x_is_f32) quantize_kernel<F, true><<<grid, Q_THREADS, 0, s>>>(x, rows, k, p, sc, sb); \
  else quantize_kernel<F, false><<<grid, Q_THREADS, 0, s>>>(x, rows, k, p, sc, sb)
  if (which == Q_NVFP4) { OG_QUANTIZE(Q_NVFP4); }
  else if (which == Q_MXFP8) { OG_QUANTIZE(Q_MXFP8); }
  else { OG_QUANTIZE(Q_MXFP4); }
#undef OG_QUANTIZE
  const cudaError_t launched = cudaGetLastError();
  if (launched != cudaSuccess) return quantize_fail("quantize launch failed: %s", cudaGetErrorString(launched));
  return OG_OK;
}

}  // extern "C"
