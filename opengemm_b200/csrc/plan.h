// Host-side planning: the format table, validation of an OgGemm, and the
// translation of its configs.json knobs into the native tile plan the kernel
// runs.  No CUDA calls: this header also compiles with a plain C++ compiler.
//
// It covers what the reference spreads over its registries and launchers:
// the element tables (opengemm/src/mm/types.cuh:9-33, opengemm/src/smm/types.cuh:8-37),
// dtype names (opengemm/src/mm/registry.cuh:120-140, opengemm/src/smm/registry.cuh:15-16),
// bind (opengemm/src/mm/launch.cuh:41-64, opengemm/src/smm/launch.cuh:38-57) and the
// compile-time geometry (opengemm/src/mm/types.cuh:102-231, opengemm/src/smm/types.cuh:96-182),
// which here is computed at bind time because the kernel takes it as run-time data.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/opengemm_b200.h"

namespace og {

enum OutType { OUT_F32 = 0, OUT_S32 = 1, OUT_BF16 = 2, OUT_F16 = 3 };

// Tensor-map element types, numbered like CUtensorMapDataType so this header
// needs no CUDA include.
enum MapType {
  MAP_U8 = 0,
  MAP_F16 = 6,
  MAP_BF16 = 9,
  MAP_TF32 = 11,
  MAP_16U4_ALIGN8B = 13,   // packed fp4 kept packed (block-scaled kinds)
  MAP_16U4_ALIGN16B = 14,  // packed fp4 expanded to one byte per value by TMA
  MAP_16U6_ALIGN16B = 15,  // packed fp6 expanded likewise
};

struct Element {
  const char* name;
  int kind;        // og::Kind of the dense path; block-scaled kinds are chosen per format
  int format;      // instruction-descriptor code
  int value_bits;  // in global memory
  int smem_bits;   // per value in shared memory
  int map_type;
};

// kind numbers follow og::Kind in ptx.cuh: 0 f16, 1 tf32, 2 i8, 3 f8f6f4.
constexpr Element ELEMENTS[] = {
    {"bf16", 0, 1, 16, 16, MAP_BF16},          {"f16", 0, 0, 16, 16, MAP_F16},
    {"tf32", 1, 2, 32, 32, MAP_TF32},          {"s8", 2, 1, 8, 8, MAP_U8},
    {"u8", 2, 0, 8, 8, MAP_U8},                {"e4m3", 3, 0, 8, 8, MAP_U8},
    {"e5m2", 3, 1, 8, 8, MAP_U8},              {"e3m2", 3, 4, 6, 8, MAP_16U6_ALIGN16B},
    {"e2m3", 3, 3, 6, 8, MAP_16U6_ALIGN16B},   {"e2m1", 3, 5, 4, 8, MAP_16U4_ALIGN16B},
};

struct Format {
  const char* name;
  bool scaled;
  const char* a;  // element names
  const char* b;
  int kind;       // og::Kind
  int out;        // OutType
  int sf_block;   // values per scale (0 for dense)
  int sf_format;  // 0 ue4m3, 1 ue8m0
};

constexpr Format FORMATS[] = {
    {"bf16", false, "bf16", "bf16", 0, OUT_F32, 0, 0},
    {"f16", false, "f16", "f16", 0, OUT_F32, 0, 0},
    {"tf32", false, "tf32", "tf32", 1, OUT_F32, 0, 0},
    {"s8", false, "s8", "s8", 2, OUT_S32, 0, 0},
    {"u8", false, "u8", "u8", 2, OUT_S32, 0, 0},
    {"e4m3", false, "e4m3", "e4m3", 3, OUT_F32, 0, 0},
    {"e5m2", false, "e5m2", "e5m2", 3, OUT_F32, 0, 0},
    {"e3m2", false, "e3m2", "e3m2", 3, OUT_F32, 0, 0},
    {"e2m3", false, "e2m3", "e2m3", 3, OUT_F32, 0, 0},
    {"e2m1", false, "e2m1", "e2m1", 3, OUT_F32, 0, 0},
    {"e4m3xe5m2", false, "e4m3", "e5m2", 3, OUT_F32, 0, 0},
    {"nvfp4", true, "e2m1", "e2m1", 6, OUT_BF16, 16, 0},
    {"mxfp8", true, "e4m3", "e4m3", 4, OUT_BF16, 32, 1},
    {"mxfp4", true, "e2m1", "e2m1", 5, OUT_BF16, 32, 1},
    // Additions with no counterpart in the reference: the dense float formats
    // with the f32 accumulator rounded to bfloat16 on the way out
    // ("<format>.bf16"), which halves the bytes of C.
    {"bf16.bf16", false, "bf16", "bf16", 0, OUT_BF16, 0, 0},
    {"f16.bf16", false, "f16", "f16", 0, OUT_BF16, 0, 0},
    {"tf32.bf16", false, "tf32", "tf32", 1, OUT_BF16, 0, 0},
    {"e4m3.bf16", false, "e4m3", "e4m3", 3, OUT_BF16, 0, 0},
    {"e5m2.bf16", false, "e5m2", "e5m2", 3, OUT_BF16, 0, 0},
    {"e3m2.bf16", false, "e3m2", "e3m2", 3, OUT_BF16, 0, 0},
    {"e2m3.bf16", false, "e2m3", "e2m3", 3, OUT_BF16, 0, 0},
    {"e2m1.bf16", false, "e2m1", "e2m1", 3, OUT_BF16, 0, 0},
    {"e4m3xe5m2.bf16", false, "e4m3", "e5m2", 3, OUT_BF16, 0, 0},
    // ... or to IEEE half ("<format>.f16"), through the same kernels.
    {"bf16.f16", false, "bf16", "bf16", 0, OUT_F16, 0, 0},
    {"f16.f16", false, "f16", "f16", 0, OUT_F16, 0, 0},
    {"tf32.f16", false, "tf32", "tf32", 1, OUT_F16, 0, 0},
    {"e4m3.f16", false, "e4m3", "e4m3", 3, OUT_F16, 0, 0},
    {"e5m2.f16", false, "e5m2", "e5m2", 3, OUT_F16, 0, 0},
    {"e3m2.f16", false, "e3m2", "e3m2", 3, OUT_F16, 0, 0},
    {"e2m3.f16", false, "e2m3", "e2m3", 3, OUT_F16, 0, 0},
    {"e2m1.f16", false, "e2m1", "e2m1", 3, OUT_F16, 0, 0},
    {"e4m3xe5m2.f16", false, "e4m3", "e5m2", 3, OUT_F16, 0, 0},
};
constexpr int NUM_REFERENCE_FORMATS = 14;  // the leading rows are the reference's fourteen
constexpr int NUM_FORMATS = sizeof(FORMATS) / sizeof(FORMATS[0]);

inline const Element* element(const char* name) {
  for (const Element& e : ELEMENTS)
    if (std::strcmp(e.name, name) == 0) return &e;
  return nullptr;
}

inline const Format* format_named(const char (&dtype)[16]) {
  for (const Format& f : FORMATS)
    if (std::strncmp(f.name, dtype, sizeof dtype) == 0) return &f;
  return nullptr;
}

// Everything the launcher needs beyond pointers: filled by make_plan.
struct Plan {
  const Format* format = nullptr;
  int variant = -1;  // which compiled kernel: kind * 2 + (cta_group - 1); 14 + ... for dense formats with 2-byte output
  int cta_group = 1;
  int swap = 0;
  int rows_m = 0, rows_n = 0, k = 0;  // MMA-side extents (after swap)
  int tile_m = 128, tile_n = 128, block_k = 64, mma_k = 16, k_blocks = 0, stages = 0;
  int x_bytes = 0, y_bytes = 0, sf_bytes = 0, stage_bytes = 0, tx_bytes = 0;
  int tiles_m = 0, tiles_n = 0, num_tiles = 0, group = 1;
  int cluster_k = 1;  // one-CTA MMAs only: CTAs of a cluster that share each tile along K (1, 2, 4 or 8)
  int walk = 0;       // rasterisation order (raster.h)
  int x_rows = 128;   // rows of the M-side box one CTA loads per stage
  uint32_t idesc = 0;
  int acc_slots = 2, acc_stride = 0, sf_col = 0, sf_slots = 1, sf_cols = 0, tmem_cols = 32;
  int epi_staged = 0, epi_tma = 0, out_bytes = 4;
  int epi = 0;        // 0 each thread stores its own row, 1 rows staged in shared memory, 2 staged and stored by TMA
  int smem_bits = 8;  // bits per value in shared memory
  int sf_atoms = 0, sf_yblocks = 0, k_groups = 0;
  int smem_bytes = 0;
  int x_bits = 0, y_bits = 0;        // global bits per value of the X / Y operand
  int x_map = 0, y_map = 0;          // MapType of each
  int l2_promo = 0;
};

constexpr int SMEM_LIMIT = 227 * 1024;   // dynamic shared memory a CTA may opt into
constexpr int SMEM_RESERVE = 1024 + 512; // alignment slack + static barriers
constexpr int PLAN_MAX_STAGES = 16;
constexpr int EPI_BUF_BYTES_HOST = 32 * 128;  // one staging buffer: 32 rows of one 128-byte swizzle row

inline int round_up(int x, int to) { return (x + to - 1) / to * to; }
inline int ceil_div(int x, int by) { return (x + by - 1) / by; }
inline int pow2_at_least(int x) {
  int p = 32;
  while (p < x) p *= 2;
  return p;
}

// The part of a tile plan that does not depend on the problem's extents: what
// follows from the MMA kind, the pair size, the output width, the tile width
// and the epilogue path alone.  make_plan derives these fields here, and the
// kernels that are compiled for one such plan (kernels_fixed.cu) fold the same
// values in at compile time, so the two cannot drift apart.
struct TileShape {
  int tile_n = 0, block_k = 0, mma_k = 0;
  int x_bytes = 0, y_bytes = 0, sf_bytes = 0, stage_bytes = 0;
  int sf_atoms = 0, sf_yblocks = 0, sf_cols = 0;
  int epi_staged = 0, epi_tma = 0, stages = 0;
  int acc_slots = 0, acc_stride = 0, sf_col = 0, sf_slots = 0, tmem_cols = 0;
  int smem_bytes = 0;
};

// `smem_bits`: bits per value in shared memory (16 f16/bf16, 32 tf32, 8 for
// every 8-bit container, 4 for packed fp4); `sf_block`: values per scale, 0
// for a dense kind; `epi`: 0 each thread stores its own row, 1 rows staged in
// shared memory, 2 staged and stored by TMA; `cluster_k`: CTAs sharing a tile
// along K, whose accumulators land in (cluster_k - 1) x tile_n x 512 bytes of
// rank 0's shared memory.
constexpr TileShape tile_shape(int smem_bits, int sf_block, int cta_group, int out_bytes, int tile_n, int epi,
                               int cluster_k = 1) {
  TileShape t;
  t.tile_n = tile_n;
  t.block_k = 1024 / smem_bits;
  t.mma_k = t.block_k / 4;
  t.x_bytes = 128 * 128;
  t.y_bytes = tile_n / cta_group * 128;
  if (sf_block > 0) {
    t.sf_atoms = t.block_k / (4 * sf_block);
    t.sf_yblocks = tile_n > 128 ? 2 : 1;
    t.sf_bytes = t.sf_atoms * 512 * (1 + t.sf_yblocks);
    t.sf_cols = 4 * t.sf_atoms * (1 + t.sf_yblocks);
  }
  t.stage_bytes = (t.x_bytes + t.y_bytes + t.sf_bytes + 1023) / 1024 * 1024;
  t.epi_staged = epi >= 1 ? 1 : 0;
  t.epi_tma = epi == 2 ? 1 : 0;
  const int epi_bytes = (t.epi_staged ? 4 * (t.epi_tma ? 2 : 1) * (32 * 128) : 0) + (cluster_k - 1) * tile_n * 512;
  const int fit = (227 * 1024 - (1024 + 512) - epi_bytes) / t.stage_bytes;
  t.stages = fit < 16 ? fit : 16;
  t.smem_bytes = t.stages * t.stage_bytes + epi_bytes + 1024;
  t.acc_stride = tile_n;
  t.acc_slots = (2 * tile_n + t.sf_cols <= 512) ? 2 : 1;
  t.sf_col = t.acc_slots * t.acc_stride;
  t.sf_slots = (t.sf_cols && t.sf_col + 2 * t.sf_cols <= 512) ? 2 : 1;
  int cols = 32;
  while (cols < t.sf_col + t.sf_slots * t.sf_cols) cols *= 2;
  t.tmem_cols = cols;
  return t;
}

// K granularity a format accepts: TMA addresses rows 16 bytes at a time, the
// expanding tensor maps of the dense sub-byte elements want whole 128-value
// groups (opengemm/src/mm/launch.cuh:47-53); block-scaled formats need whole
// scale blocks (opengemm/src/smm/launch.cuh:44-47) and 16-byte rows.
inline int k_multiple(const Format& f) {
  const Element* e = element(f.a);
  if (f.scaled) return std::max(f.sf_block, 128 / e->value_bits);
  return e->value_bits < 8 ? 128 : 128 / e->value_bits;
}

// The widest MMA N this path can use for a format.
inline int legal_tile_n(const Format& f, int cta_group, int want, int rows_n) {
  int n = std::min(std::max(want, 16), 256);
  n = round_up(n, 16);
  if (cta_group == 2) n = std::max(n, 32);
  if (f.scaled) {
    // Scale atoms cover 128 rows; a tile may start 0 or 64 rows into one, so
    // tiles are multiples of 64 wide unless one tile spans all of N.
    if (!(n < 64 && rows_n <= n)) n = round_up(n, 64);
  }
  return std::min(n, 256);
}

// Validate `g` and derive the plan.  Returns OG_OK or an error code with
// `why` filled.  `sm_count` sizes the persistent grid.
inline int make_plan(const OgGemm& g, int sm_count, Plan* out, char* why, size_t why_cap) {
  Plan p;
  const Format* f = format_named(g.dtype);
  if (!f) {
    snprintf(why, why_cap, "dtype %.16s names no element pair this build serves", g.dtype);
    return OG_ERR_BIND;
  }
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) {
    snprintf(why, why_cap, "m, n and k must be positive, got %d, %d, %d", g.m, g.n, g.k);
    return OG_ERR_BIND;
  }
  const int multiple = k_multiple(*f);
  if (g.k % multiple) {
    snprintf(why, why_cap, "K = %d is not a multiple of %d, which the tensor map for %s requires",
             g.k, multiple, f->name);
    return OG_ERR_BIND;
  }
  p.format = f;
  p.cta_group = g.use_2cta ? 2 : 1;
  p.swap = g.swap_ab ? 1 : 0;
  p.variant = f->kind * 2 + (p.cta_group - 1);
  if (!f->scaled && (f->out == OUT_BF16 || f->out == OUT_F16))  // kinds 0, 1, 3 (no integer kind) -> 14..19
    p.variant = 14 + (f->kind == 3 ? 2 : f->kind) * 2 + (p.cta_group - 1);
  const Element* ea = element(f->a);
  const Element* eb = element(f->b);
  const Element* ex = p.swap ? eb : ea;
  const Element* ey = p.swap ? ea : eb;
  p.rows_m = p.swap ? g.n : g.m;
  p.rows_n = p.swap ? g.m : g.n;
  p.k = g.k;
  p.tile_m = 128 * p.cta_group;
  p.tile_n = legal_tile_n(*f, p.cta_group, g.output_n > 0 ? g.output_n : 128, p.rows_n);
  const bool packed4 = f->scaled && ea->value_bits == 4;
  const int smem_bits = packed4 ? 4 : ex->smem_bits;
  p.out_bytes = (f->out == OUT_BF16 || f->out == OUT_F16) ? 2 : 4;
  p.k_blocks = ceil_div(p.k, 1024 / smem_bits);
  const int64_t ldd = g.n;              // C is [m, n] row-major whichever way the MMA runs
  // Staged rows leave by TMA store (32 rows x 128 bytes a time, two buffers per
  // warp) wherever a tile is whole 128-byte chunks wide: measured against plain
  // 16-byte stores of the same staged rows it is level on a single tile and up
  // to 1.3x faster where the stores are the work (bf16 8192x8192x32: 67.7 ->
  // 52.8 us, 2048x2048x128: 6.9 -> 5.7 us).  16-bit output behind a long K loop
  // keeps the plain stores: nothing waits for them there, and the second
  // buffer would cost the widest block-scaled tiles a ring stage.
  // epi_direct: 0 as above, 1 every thread stores its own row, 2 TMA stores
  // for 16-bit output too, whatever the length of the K loop.
  const bool staged = g.epi_direct != 1 && !p.swap && (ldd * p.out_bytes) % 16 == 0;
  const bool by_tma = staged && (p.out_bytes == 4 ? p.tile_n % 32 == 0
                                                  : p.tile_n % 64 == 0 && (p.k_blocks <= 16 || g.epi_direct == 2));
  p.epi = by_tma ? 2 : staged ? 1 : 0;
  // Cluster-K: the requested power of two, no more ways than there are K
  // blocks, halved until the landing zone leaves room for a three-stage ring.
  p.cluster_k = 1;
  if (p.cta_group == 1 && g.cluster_k > 1 && !g.use_clc && g.split_k < 2) {
    int ways = 1;
    while (ways * 2 <= std::min<int>(g.cluster_k, 8) && ways * 2 <= p.k_blocks) ways *= 2;
    while (ways > 1 && tile_shape(smem_bits, f->scaled ? f->sf_block : 0, 1, p.out_bytes, p.tile_n, p.epi, ways).stages < 3)
      ways /= 2;
    p.cluster_k = ways;
  }
  const TileShape t =
      tile_shape(smem_bits, f->scaled ? f->sf_block : 0, p.cta_group, p.out_bytes, p.tile_n, p.epi, p.cluster_k);
  p.block_k = t.block_k;
  p.mma_k = t.mma_k;
  p.x_bits = ex->value_bits;
  p.y_bits = ey->value_bits;
  p.x_map = packed4 ? MAP_16U4_ALIGN8B : ex->map_type;
  p.y_map = packed4 ? MAP_16U4_ALIGN8B : ey->map_type;
  const int y_rows = p.tile_n / p.cta_group;
  p.x_bytes = t.x_bytes;
  p.y_bytes = t.y_bytes;
  p.sf_atoms = t.sf_atoms;
  p.sf_yblocks = t.sf_yblocks;
  p.sf_bytes = t.sf_bytes;
  p.sf_cols = t.sf_cols;
  if (f->scaled) p.k_groups = ceil_div(p.k, 4 * f->sf_block);
  p.stage_bytes = t.stage_bytes;
  // Bytes TMA credits per stage: the packed global size for expanding maps.
  const int x_tx = 128 * p.block_k * (packed4 ? 4 : p.x_bits) / 8;
  const int y_tx = y_rows * p.block_k * (packed4 ? 4 : p.y_bits) / 8;
  p.tx_bytes = p.cta_group * (x_tx + y_tx + p.sf_bytes);

  p.epi_staged = t.epi_staged;
  p.epi_tma = t.epi_tma;
  p.tiles_m = ceil_div(p.rows_m, p.tile_m);
  p.tiles_n = ceil_div(p.rows_n, p.tile_n);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.stages = t.stages;
  if (g.stages > 0) p.stages = std::min(p.stages, std::max(2, (int)g.stages));
  if (p.stages < 2) {
    snprintf(why, why_cap, "a %d-wide tile of %s leaves no room for a two-stage ring", p.tile_n, f->name);
    return OG_ERR_NO_KERNEL;
  }
  p.smem_bytes = t.smem_bytes - (t.stages - p.stages) * t.stage_bytes;

  p.acc_stride = t.acc_stride;
  p.acc_slots = t.acc_slots;
  p.sf_col = t.sf_col;
  p.sf_slots = t.sf_slots;
  p.tmem_cols = t.tmem_cols;
  if (p.tmem_cols > 512) {
    snprintf(why, why_cap, "a %d-wide tile of %s does not fit tensor memory", p.tile_n, f->name);
    return OG_ERR_NO_KERNEL;
  }
  p.smem_bits = smem_bits;

  p.walk = (g.walk >= 0 && g.walk <= 4) ? g.walk : 0;
  {
    // Bands run along N, except in the row-band walk, where they run along M.
    const int extent = p.walk == 4 ? p.tiles_m : p.tiles_n;
    p.group = std::max(1, std::min<int>(g.supergroup > 0 ? g.supergroup : 8, extent));
  }
  p.l2_promo = g.l2_promo;

  const uint32_t n_field = uint32_t(p.tile_n >> 3) << 17;
  const uint32_t m_field = uint32_t(p.tile_m >> 4) << 24;
  if (f->scaled) {
    const uint32_t fmt = packed4 ? 1u : uint32_t(ex->format);  // packed e2m1 is code 1 in the mxf4 kinds
    const uint32_t fmt_y = packed4 ? 1u : uint32_t(ey->format);
    p.idesc = (fmt << 7) | (fmt_y << 10) | n_field | (uint32_t(f->sf_format) << 23) | m_field;
  } else {
    const uint32_t c_fmt = f->out == OUT_S32 ? 2u : 1u;
    p.idesc = (c_fmt << 4) | (uint32_t(ex->format) << 7) | (uint32_t(ey->format) << 10) | n_field | m_field;
  }
  (void)sm_count;
  *out = p;
  return OG_OK;
}

// The candidate configurations og_*_kernel enumerates for tuners: per format,
// pair size x tile width x operand swap.  Every row binds.
struct MenuRow {
  int format;  // index into FORMATS
  int use_2cta, output_n, swap_ab;
};

inline int menu_rows(bool scaled, MenuRow* rows, int cap) {
  static const int dense_n[] = {16, 32, 64, 96, 128, 160, 192, 224, 256};
  static const int scaled_n[] = {16, 32, 64, 128, 192, 256};
  int count = 0;
  for (int fi = 0; fi < NUM_REFERENCE_FORMATS; ++fi) {  // the menu a reference-side tuner walks: its own formats
    if (FORMATS[fi].scaled != scaled) continue;
    for (int two = 0; two < 2; ++two)
      for (int swap = 0; swap < 2; ++swap) {
        const int* ns = scaled ? scaled_n : dense_n;
        const int nn = scaled ? 6 : 9;
        for (int i = 0; i < nn; ++i) {
          if (two && ns[i] < 32) continue;
          if (rows && count < cap) rows[count] = {fi, two, ns[i], swap};
          ++count;
        }
      }
  }
  return count;
}

}  // namespace og
