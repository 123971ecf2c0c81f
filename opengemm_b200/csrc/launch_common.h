// What every launch entry point shares: the tensor-map encoder with its
// per-thread cache, and the translation of a tile plan plus the caller's
// pointers into the kernel's parameter block.  Included by host.cu (the
// ordinary launches) and no_alloc.cu (the allocation-free one), so a field
// added to GemmParams is filled in one place.
//
// Counterpart of the reference's per-library launch code
// (opengemm/src/mm/launch.cuh:105-150, opengemm/src/smm/launch.cuh:105-120,
// opengemm/src/common/tmap.cuh:7-22), which re-encodes three to five tensor
// maps on every call; here encoded maps are kept in a small per-thread cache
// keyed by pointer and geometry.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>

#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel.cuh"
#include "plan.h"

namespace og {

// cuTensorMapEncodeTiled, resolved through the runtime so that the library
// loads (and bind / plan work) on a machine without a driver.
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

inline EncodeFn tensor_map_encoder() {
  static EncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return EncodeFn(nullptr);
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t dim0, dim1, stride;
  uint32_t box0, box1;
  int type, swizzle, l2;
  bool operator==(const MapKey& o) const {
    return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && stride == o.stride &&
           box0 == o.box0 && box1 == o.box1 && type == o.type && swizzle == o.swizzle && l2 == o.l2;
  }
};

struct MapSlot {
  MapKey key{};
  CUtensorMap map;
};

// 64 sets of four ways: a loop over a few rotating operand sets keeps a dozen
// or two maps alive, and in a direct-mapped table two of those would often
// share a slot and evict each other on every call (a driver call each time).
// A set's four hash tags sit together in half a cache line and are all a
// miss reads: a loop over more buffers than the table holds (benchmarks that
// rotate hundreds of operand sets past L2) then pays one line per look-up
// instead of four keys spread over a dozen lines it has not touched since the
// table last wrapped.
constexpr int MAP_SETS = 64;
constexpr int MAP_WAYS = 4;
struct MapSet {
  uint64_t tag[MAP_WAYS] = {0, 0, 0, 0};  // the slot's full hash with bit 0 set; 0 = empty
  unsigned next = 0;                      // the way the next miss replaces
  MapSlot way[MAP_WAYS];
};
inline thread_local MapSet map_cache[MAP_SETS];

inline uint64_t mix_hash(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  return h;
}

// A 2-D tiled map over `base`: dim0 innermost (elements), rows `stride` bytes
// apart.  Out-of-bounds parts of a box read as zero and are clipped on store.
// Returns OG_OK, or OG_ERR_TENSORMAP with the reason in `why`.
inline int encode_2d(CUtensorMap* out, const void* base, int type, uint64_t dim0, uint64_t dim1,
                     uint64_t stride, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle, int l2,
                     const char* which, char* why, size_t why_cap) {
  const MapKey key{base, dim0, dim1, stride, box0, box1, type, int(swizzle), l2};
  uint64_t h = mix_hash(0, reinterpret_cast<uint64_t>(base));
  h = mix_hash(h, dim0 * 1315423911ull + dim1);
  h = mix_hash(h, (uint64_t(box0) << 32) | box1);
  h = mix_hash(h, stride * 31 + uint64_t(type) * 7 + uint64_t(swizzle) * 3 + uint64_t(l2));
  MapSet& set = map_cache[(h >> 8) % MAP_SETS];
  const uint64_t tag = h | 1;
  for (int w = 0; w < MAP_WAYS; ++w)
    if (set.tag[w] == tag && set.way[w].key == key) {
      *out = set.way[w].map;
      return OG_OK;
    }
  const unsigned victim = set.next++ % MAP_WAYS;
  MapSlot& slot = set.way[victim];
  EncodeFn encode = tensor_map_encoder();
  if (!encode) {
    snprintf(why, why_cap, "cuTensorMapEncodeTiled is not available: no CUDA driver");
    return OG_ERR_TENSORMAP;
  }
  const cuuint64_t dims[2] = {dim0, dim1};
  const cuuint64_t strides[1] = {stride};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUtensorMapL2promotion promo = l2 == 2   ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                       : l2 == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_NONE;
  const CUresult status =
      encode(out, CUtensorMapDataType(type), 2, const_cast<void*>(base), dims, strides, box,
             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) {
    snprintf(why, why_cap,
             "cuTensorMapEncodeTiled failed for %s (driver error %d; dims %llu x %llu, stride %llu, "
             "box %u x %u, type %d)",
             which, int(status), (unsigned long long)dim0, (unsigned long long)dim1,
             (unsigned long long)stride, box0, box1, type);
    return OG_ERR_TENSORMAP;
  }
  slot.key = key;
  slot.map = *out;
  set.tag[victim] = tag;
  return OG_OK;
}

// The caller's pointers, as og_*_launch receives them.
struct LaunchPointers {
  const void* a;
  const void* b;
  const void* sfa;
  const void* sfb;
  void* c;
  const void* bias;  // float32 [n], added to every row of C before it is stored; may be null
  // Block-scaled output: `c` receives packed codes, `c_scales` the blocked scales.
  int out_quant = 0;        // 0 off, else 1 nvfp4, 2 mxfp8, 3 mxfp4
  void* c_scales = nullptr;
};

// Checks every launch entry point makes before touching the device.
inline int check_pointers(const OgGemm& g, const Plan& p, const LaunchPointers& io, const float* alpha,
                          char* why, size_t why_cap) {
  if (g.row != p.variant) {
    snprintf(why, why_cap, "row %d is not the kernel of this OgGemm: bind it first", g.row);
    return OG_ERR_LAUNCH;
  }
  if (!io.a || !io.b || !io.c) {
    snprintf(why, why_cap, "a, b and c must be device pointers, got null");
    return OG_ERR_LAUNCH;
  }
  if (p.format->scaled && (!io.sfa || !io.sfb)) {
    snprintf(why, why_cap, "a block-scaled format takes both sfa and sfb");
    return OG_ERR_LAUNCH;
  }
  if (io.out_quant) {
    if (!io.c_scales) {
      snprintf(why, why_cap, "a block-scaled output takes a scale buffer");
      return OG_ERR_LAUNCH;
    }
    if (p.format->out != OUT_BF16) {
      snprintf(why, why_cap, "dtype %.16s writes no bfloat16: bind a block-scaled format or \"<format>.bf16\" to quantise C", g.dtype);
      return OG_ERR_LAUNCH;
    }
    if (p.swap || p.tile_n % 64 || g.n % 64) {
      snprintf(why, why_cap, "a block-scaled output needs N %% 64 == 0, tiles a multiple of 64 wide and no operand swap "
               "(n = %d, tile width %d, swap_ab = %d)", g.n, p.tile_n, p.swap);
      return OG_ERR_LAUNCH;
    }
  }
  if ((alpha || io.bias) && p.format->out == OUT_S32) {
    snprintf(why, why_cap, "dtype %.16s accumulates integers exactly: its output cannot be scaled or biased", g.dtype);
    return OG_ERR_LAUNCH;
  }
  return OG_OK;
}

// Tensor maps and every plan-derived field of the kernel's parameter block.
// Schedule fields (use_clc, stream_k and its workspace, pdl) are left zero for
// the caller to set.  Returns OG_OK or an error code with `why` filled.
inline int fill_params(const Plan& p, const OgGemm& g, const LaunchPointers& io, int* status_word,
                       const float* alpha, unsigned long long wait_limit_ns, GemmParams* out, char* why,
                       size_t why_cap) {
  GemmParams& params = *out;
  std::memset(&params, 0, sizeof params);
  const void* x = p.swap ? io.b : io.a;
  const void* y = p.swap ? io.a : io.b;
  const void* sfx = p.swap ? io.sfb : io.sfa;
  const void* sfy = p.swap ? io.sfa : io.sfb;
  const uint64_t k = uint64_t(p.k);
  int rc = encode_2d(&params.map_x, x, p.x_map, k, uint64_t(p.rows_m), k * p.x_bits / 8, uint32_t(p.block_k),
                     uint32_t(p.x_rows), CU_TENSOR_MAP_SWIZZLE_128B, p.l2_promo, "the M-side operand", why, why_cap);
  if (rc != OG_OK) return rc;
  rc = encode_2d(&params.map_y, y, p.y_map, k, uint64_t(p.rows_n), k * p.y_bits / 8, uint32_t(p.block_k),
                 uint32_t(p.tile_n / p.cta_group), CU_TENSOR_MAP_SWIZZLE_128B, p.l2_promo, "the N-side operand",
                 why, why_cap);
  if (rc != OG_OK) return rc;
  const bool c_aligned = (reinterpret_cast<uintptr_t>(io.c) & 15) == 0;
  const int epi_staged = p.epi_staged && c_aligned;
  const int epi_tma = p.epi_tma && c_aligned && !io.out_quant;  // block-scaled C is stored by its own path
  if (epi_tma) {
    const int type = p.format->out == OUT_S32    ? int(CU_TENSOR_MAP_DATA_TYPE_INT32)
                     : p.format->out == OUT_BF16 ? int(CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
                     : p.format->out == OUT_F16  ? int(CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
                                                 : int(CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    rc = encode_2d(&params.map_d, io.c, type, uint64_t(g.n), uint64_t(g.m), uint64_t(g.n) * p.out_bytes,
                   uint32_t(128 / p.out_bytes), 32, CU_TENSOR_MAP_SWIZZLE_128B, 0, "the output", why, why_cap);
    if (rc != OG_OK) return rc;
  }
  if (p.format->scaled) {
    const uint64_t atoms_x = uint64_t(ceil_div(p.rows_m, 128)) * p.k_groups;
    const uint64_t atoms_y = uint64_t(ceil_div(p.rows_n, 128)) * p.k_groups;
    rc = encode_2d(&params.map_sfx, sfx, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_x, 256, 256,
                   uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, 0, "the M-side scales", why, why_cap);
    if (rc != OG_OK) return rc;
    rc = encode_2d(&params.map_sfy, sfy, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_y, 256, 256,
                   uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, 0, "the N-side scales", why, why_cap);
    if (rc != OG_OK) return rc;
  }
  params.d = io.c;
  params.bias = static_cast<const float*>(io.bias);
  params.status = status_word;
  params.wait_limit_ns = wait_limit_ns;
  params.rows_m = p.rows_m;
  params.rows_n = p.rows_n;
  params.k = p.k;
  params.ldd = g.n;
  params.transpose_out = p.swap;
  params.out_f16 = p.format->out == OUT_F16 ? 1 : 0;
  params.tile_n = p.tile_n;
  params.block_k = p.block_k;
  params.mma_k = p.mma_k;
  params.k_blocks = p.k_blocks;
  params.stages = p.stages;
  params.x_bytes = p.x_bytes;
  params.y_bytes = p.y_bytes;
  params.stage_bytes = p.stage_bytes;
  params.tx_bytes = p.tx_bytes;
  params.tiles_m = p.tiles_m;
  params.tiles_n = p.tiles_n;
  params.num_tiles = p.num_tiles;
  params.group = p.group;
  params.walk = p.walk;
  params.cluster_k = p.cluster_k;
  params.acc_int = p.format->out == OUT_S32;
  params.idesc = p.idesc;
  params.acc_slots = p.acc_slots;
  params.acc_stride = p.acc_stride;
  params.sf_col = p.sf_col;
  params.sf_slots = p.sf_slots;
  params.sf_cols = p.sf_cols;
  params.tmem_cols = p.tmem_cols;
  params.epi_staged = epi_staged;
  params.epi_tma = epi_tma;
  params.vec_ok = (c_aligned && (int64_t(g.n) * p.out_bytes) % 16 == 0) ? 1 : 0;
  params.sf_atoms = p.sf_atoms;
  params.sf_yblocks = p.sf_yblocks;
  params.k_groups = p.k_groups;
  if (alpha) {
    params.scale_out = 1;
    params.alpha = *alpha;
  }
  if (io.out_quant) {
    params.out_quant = io.out_quant;
    params.out_scales = static_cast<uint8_t*>(io.c_scales);
    params.out_k_groups = ceil_div(g.n, io.out_quant == 1 ? 64 : 128);
  }
  return OG_OK;
}

// The limit of device-side waits set by og_b200_set_wait_limit_ms (host.cu).
unsigned long long current_wait_limit_ns();

}  // namespace og
