// Host side of libopengemm_b200.so: the extern "C" surface, tensor-map
// construction with a per-thread cache, and the launch.
//
// Replaces, for both of the reference's libraries at once,
// opengemm/src/{mm,smm}/capi.cu (exports), opengemm/src/{mm,smm}/launch.cuh
// (bind, launch_cfg), opengemm/src/{mm,smm}/tmap.cuh and
// opengemm/src/common/{launch,tmap}.cuh.  Where the reference re-encodes
// three to five tensor maps on every call (mm/launch.cuh:105-150,
// smm/launch.cuh:105-120), encoded maps are kept here in a small per-thread
// cache keyed by pointer and geometry.
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel.cuh"
#include "plan.h"

namespace og {

// Implemented in kernels_dense.cu (variants 0-7 and 14-19) and kernels_scaled.cu (8-13).
cudaError_t configure_dense(int variant, int smem_bytes);
cudaError_t configure_scaled(int variant, int smem_bytes);
cudaError_t launch_dense(int variant, const GemmParams& params, int grid, int smem_bytes,
                         cudaStream_t stream, bool pdl);
cudaError_t launch_scaled(int variant, const GemmParams& params, int grid, int smem_bytes,
                          cudaStream_t stream, bool pdl);

inline cudaError_t configure_variant(int variant, int smem_bytes) {
  return (variant < 8 || variant >= 14) ? configure_dense(variant, smem_bytes) : configure_scaled(variant, smem_bytes);
}
inline cudaError_t launch_variant(int variant, const GemmParams& params, int grid, int smem_bytes,
                                  cudaStream_t stream, bool pdl) {
  return (variant < 8 || variant >= 14) ? launch_dense(variant, params, grid, smem_bytes, stream, pdl)
                     : launch_scaled(variant, params, grid, smem_bytes, stream, pdl);
}

namespace {

thread_local char error_text[320];
std::atomic<long long> wait_limit_ns{2000ll * 1000 * 1000};
std::atomic<int> independent_inputs{0};

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(error_text, sizeof error_text, format, args);
  va_end(args);
  return code;
}

// cuTensorMapEncodeTiled, resolved through the runtime so that the library
// loads (and bind / plan work) on a machine without a driver.
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encoder() {
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
  bool used = false;
};

constexpr int MAP_SLOTS = 256;
thread_local MapSlot map_cache[MAP_SLOTS];

uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  return h;
}

// A 2-D tiled map over `base`: dim0 innermost (elements), rows `stride` bytes
// apart.  Out-of-bounds parts of a box read as zero and are clipped on store.
int encode_2d(CUtensorMap* out, const void* base, int type, uint64_t dim0, uint64_t dim1,
              uint64_t stride, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle, int l2,
              const char* which) {
  const MapKey key{base, dim0, dim1, stride, box0, box1, type, int(swizzle), l2};
  uint64_t h = mix(0, reinterpret_cast<uint64_t>(base));
  h = mix(h, dim0 * 1315423911ull + dim1);
  h = mix(h, (uint64_t(box0) << 32) | box1);
  h = mix(h, stride * 31 + uint64_t(type) * 7 + uint64_t(swizzle) * 3 + uint64_t(l2));
  MapSlot& slot = map_cache[h % MAP_SLOTS];
  if (slot.used && slot.key == key) {
    *out = slot.map;
    return OG_OK;
  }
  EncodeFn encode = encoder();
  if (!encode) return fail(OG_ERR_TENSORMAP, "cuTensorMapEncodeTiled is not available: no CUDA driver");
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
  if (status != CUDA_SUCCESS)
    return fail(OG_ERR_TENSORMAP,
                "cuTensorMapEncodeTiled failed for %s (driver error %d; dims %llu x %llu, stride %llu, "
                "box %u x %u, type %d)",
                which, int(status), (unsigned long long)dim0, (unsigned long long)dim1,
                (unsigned long long)stride, box0, box1, type);
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return OG_OK;
}

// Stream-K scratch: partial sums of tiles shared by two clusters, and the
// flags that publish them.  One region per epilogue warp of a full grid;
// WORKSPACES of them are used round-robin by successive launches so that a
// launch never reuses the buffers of one that may still be running (each
// launch fills the GPU, so no more than two or three can overlap).
constexpr int WORKSPACES = 4;
constexpr size_t REGION_BYTES = 32 * 256 * 4;

struct DeviceInfo {
  int sm_count = 0;
  uint64_t configured = 0;  // bit per kernel variant
  float* partial[WORKSPACES] = {};
  int* flags[WORKSPACES] = {};
};
std::atomic<unsigned> launch_epoch{0};
std::mutex device_mutex;
DeviceInfo devices[64];

int follow_device(int device) {
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return fail(OG_ERR_LAUNCH, "cudaGetDevice failed");
  if (current != device) {
    const cudaError_t moved = cudaSetDevice(device);
    if (moved != cudaSuccess) return fail(OG_ERR_LAUNCH, "cudaSetDevice: %s", cudaGetErrorString(moved));
  }
  return OG_OK;
}

std::atomic<int> sm_count_fast[64];
std::atomic<uint64_t> configured_fast[64];

int sm_count_of(int device) {
  if (device < 0) return 148;
  if (const int known = sm_count_fast[device & 63].load(std::memory_order_relaxed)) return known;
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device & 63];
  if (!info.sm_count) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    info.sm_count = count;
  }
  sm_count_fast[device & 63].store(info.sm_count, std::memory_order_relaxed);
  return info.sm_count;
}

int ensure_configured(int device, int variant, int smem_bytes) {
  const uint64_t bit = 1ull << variant;
  if (configured_fast[device & 63].load(std::memory_order_acquire) & bit) return OG_OK;
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device & 63];
  if (info.configured & bit) return OG_OK;
  const cudaError_t status = configure_variant(variant, SMEM_LIMIT - 1024);  // static barriers take the rest
  if (status != cudaSuccess)
    return fail(OG_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(status));
  (void)smem_bytes;
  info.configured |= bit;
  configured_fast[device & 63].fetch_or(bit, std::memory_order_release);
  return OG_OK;
}

// The workspace for one stream-K launch on `device` (allocated on first use;
// flags start at zero and are matched against a per-launch epoch, so they
// are never cleared).
int workspace_for(int device, int sm_count, unsigned epoch, float** partial, int** flags) {
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device & 63];
  const int slot = int(epoch % WORKSPACES);
  if (!info.partial[slot]) {
    const size_t regions = size_t(sm_count) * 4;
    void* data = nullptr;
    void* words = nullptr;
    if (cudaMalloc(&data, regions * REGION_BYTES) != cudaSuccess ||
        cudaMalloc(&words, regions * sizeof(int)) != cudaSuccess ||
        cudaMemset(words, 0, regions * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      if (data) cudaFree(data);
      if (words) cudaFree(words);
      return fail(OG_ERR_LAUNCH, "cannot allocate the %zu-byte stream-K workspace", regions * REGION_BYTES);
    }
    info.partial[slot] = static_cast<float*>(data);
    info.flags[slot] = static_cast<int*>(words);
  }
  *partial = info.partial[slot];
  *flags = info.flags[slot];
  return OG_OK;
}

// Stream-K applies when the tiles do not fill a whole number of waves: the
// tiles of the partial wave are then cut along K across all clusters.
bool use_stream_k(const OgGemm& g, const Plan& p, int grid) {
  const int clusters = grid / p.cta_group;
  return g.split_k >= 2 && p.num_tiles % clusters != 0 && p.k_blocks > 1;
}

int grid_for(const Plan& p, int sm_count, bool fill = false) {
  // `fill`: a stream-K launch occupies every SM even with fewer tiles than SMs.
  const int all = std::max(1, sm_count / p.cta_group);
  const int clusters = fill ? std::min(all, std::max(1, p.num_tiles * p.k_blocks)) : std::max(1, std::min(p.num_tiles, all));
  return clusters * p.cta_group;
}

int bind_impl(OgGemm* g, bool scaled) {
  Plan plan;
  char why[256];
  const int status = make_plan(*g, 148, &plan, why, sizeof why);
  if (status != OG_OK) return fail(status, "%s", why);
  if (plan.format->scaled != scaled)
    return fail(OG_ERR_BIND, "dtype %.16s is a %s format: bind it through og_%s_bind", g->dtype,
                plan.format->scaled ? "block-scaled" : "dense", plan.format->scaled ? "smm" : "mm");
  // split-K is served by the persistent schedule; the request is recorded as
  // the reference clamps it (mm/registry.cuh:149-153) so stored entries round-trip.
  if (!scaled) {
    if (g->epi_double == 1 || g->split_k <= 1) g->split_k = 1;
    else g->split_k = std::min<int>(g->split_k, (g->k + 127) / 128);
  }
  g->row = plan.variant;
  return OG_OK;
}

// The plan of the OgGemm this thread launched last: launches of one bound
// GEMM in a loop skip re-deriving it.
struct PlanMemo {
  OgGemm key;
  Plan plan;
  bool valid = false;
};
thread_local PlanMemo plan_memo;

int launch_impl(const OgGemm* g, const void* a, const void* b, const void* sfa, const void* sfb,
                void* c, int device, void* stream, int* status_word, int want_scaled, const float* alpha = nullptr) {
  if (!g) return fail(OG_ERR_LAUNCH, "null OgGemm");
  if (!plan_memo.valid || std::memcmp(&plan_memo.key, g, sizeof(OgGemm)) != 0) {
    char why[256];
    plan_memo.valid = false;
    const int planned = make_plan(*g, 148, &plan_memo.plan, why, sizeof why);
    if (planned != OG_OK) return fail(planned, "%s", why);
    plan_memo.key = *g;
    plan_memo.valid = true;
  }
  const Plan& p = plan_memo.plan;
  if (g->row != p.variant)
    return fail(OG_ERR_LAUNCH, "row %d is not the kernel of this OgGemm: bind it first", g->row);
  if (want_scaled >= 0 && int(p.format->scaled) != want_scaled)
    return fail(OG_ERR_LAUNCH, "dtype %.16s does not belong to this library", g->dtype);
  if (!a || !b || !c) return fail(OG_ERR_LAUNCH, "a, b and c must be device pointers, got null");
  if (p.format->scaled && (!sfa || !sfb))
    return fail(OG_ERR_LAUNCH, "a block-scaled format takes both sfa and sfb");
  if (alpha && p.format->out == OUT_S32)
    return fail(OG_ERR_LAUNCH, "dtype %.16s accumulates integers exactly: its output cannot be scaled", g->dtype);
  const int followed = follow_device(device);
  if (followed != OG_OK) return followed;
  const int configured = ensure_configured(device, p.variant, p.smem_bytes);
  if (configured != OG_OK) return configured;

  GemmParams params;
  std::memset(&params, 0, sizeof params);
  const void* x = p.swap ? b : a;
  const void* y = p.swap ? a : b;
  const void* sfx = p.swap ? sfb : sfa;
  const void* sfy = p.swap ? sfa : sfb;
  const uint64_t k = uint64_t(p.k);
  int rc = encode_2d(&params.map_x, x, p.x_map, k, uint64_t(p.rows_m), k * p.x_bits / 8,
                     uint32_t(p.block_k), 128, CU_TENSOR_MAP_SWIZZLE_128B, p.l2_promo, "the M-side operand");
  if (rc != OG_OK) return rc;
  rc = encode_2d(&params.map_y, y, p.y_map, k, uint64_t(p.rows_n), k * p.y_bits / 8,
                 uint32_t(p.block_k), uint32_t(p.tile_n / p.cta_group), CU_TENSOR_MAP_SWIZZLE_128B,
                 p.l2_promo, "the N-side operand");
  if (rc != OG_OK) return rc;
  const bool c_aligned = (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  const int epi_staged = p.epi_staged && c_aligned;
  const int epi_tma = p.epi_tma && c_aligned;
  if (epi_tma) {
    const int type = p.format->out == OUT_S32 ? int(CU_TENSOR_MAP_DATA_TYPE_INT32) : int(CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    rc = encode_2d(&params.map_d, c, type, uint64_t(g->n), uint64_t(g->m), uint64_t(g->n) * p.out_bytes,
                   uint32_t(128 / p.out_bytes), 32, CU_TENSOR_MAP_SWIZZLE_128B, 0, "the output");
    if (rc != OG_OK) return rc;
  }
  if (p.format->scaled) {
    const uint64_t atoms_x = uint64_t(ceil_div(p.rows_m, 128)) * p.k_groups;
    const uint64_t atoms_y = uint64_t(ceil_div(p.rows_n, 128)) * p.k_groups;
    rc = encode_2d(&params.map_sfx, sfx, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_x, 256, 256,
                   uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, 0, "the M-side scales");
    if (rc != OG_OK) return rc;
    rc = encode_2d(&params.map_sfy, sfy, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_y, 256, 256,
                   uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, 0, "the N-side scales");
    if (rc != OG_OK) return rc;
  }
  params.d = c;
  params.status = status_word;
  params.wait_limit_ns = (unsigned long long)wait_limit_ns.load();
  params.rows_m = p.rows_m;
  params.rows_n = p.rows_n;
  params.k = p.k;
  params.ldd = g->n;
  params.transpose_out = p.swap;
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
  params.idesc = p.idesc;
  params.acc_slots = p.acc_slots;
  params.acc_stride = p.acc_stride;
  params.sf_col = p.sf_col;
  params.sf_slots = p.sf_slots;
  params.sf_cols = p.sf_cols;
  params.tmem_cols = p.tmem_cols;
  params.epi_staged = epi_staged;
  params.epi_tma = epi_tma;
  params.vec_ok = (c_aligned && (int64_t(g->n) * p.out_bytes) % 16 == 0) ? 1 : 0;
  params.sf_atoms = p.sf_atoms;
  params.sf_yblocks = p.sf_yblocks;
  params.k_groups = p.k_groups;
  if (alpha) {
    params.scale_out = 1;
    params.alpha = *alpha;
  }
  static const bool pdl_enabled = [] { const char* e = getenv("OPENGEMM_PDL"); return !(e && e[0] == '0'); }();
  params.pdl = pdl_enabled ? (independent_inputs.load(std::memory_order_relaxed) ? 2 : 1) : 0;

  const int sm_count = sm_count_of(device);
  int grid = grid_for(p, sm_count);
  if (g->use_clc && g->split_k < 2) {
    // Cluster launch control: one cluster per tile; running clusters take over
    // the tiles of those that have not started.
    params.use_clc = 1;
    grid = p.num_tiles * p.cta_group;
  }
  if (g->split_k >= 2 && use_stream_k(*g, p, grid_for(p, sm_count, true))) {
    grid = grid_for(p, sm_count, true);
    unsigned epoch = ++launch_epoch;
    if ((epoch & 0x7FFFFFFFu) == 0) epoch = ++launch_epoch;  // the tag is never 0
    const int got = workspace_for(device, sm_count, epoch, &params.partial, &params.flags);
    if (got != OG_OK) return got;
    params.stream_k = 1;
    {
      // split_k is the most ways a tile of the partial wave is cut: that many
      // clusters per leftover tile share its K blocks, the rest sit the wave out.
      const int clusters = grid / p.cta_group;
      const int leftover = p.num_tiles % clusters;
      params.sk_clusters = std::min<long long>(clusters, (long long)leftover * std::min<int>(g->split_k, p.k_blocks));
    }
    params.epoch = int(epoch & 0x7FFFFFFFu);
    params.acc_int = p.format->out == OUT_S32;
  }
  const cudaError_t launched =
      launch_variant(p.variant, params, grid, p.smem_bytes, static_cast<cudaStream_t>(stream), params.pdl != 0);
  if (launched != cudaSuccess)
    return fail(OG_ERR_LAUNCH, "kernel launch failed: %s", cudaGetErrorString(launched));
  return OG_OK;
}

int describe_row(bool scaled, int i, OgGemm* out) {
  static MenuRow rows[2][1024];
  static int counts[2] = {menu_rows(false, rows[0], 1024), menu_rows(true, rows[1], 1024)};
  const int which = scaled ? 1 : 0;
  if (!out) return fail(OG_ERR_BIND, "null OgGemm");
  if (i < 0 || i >= counts[which]) return fail(OG_ERR_NO_KERNEL, "kernel index %d out of range 0..%d", i, counts[which] - 1);
  const MenuRow& row = rows[which][i];
  std::memset(out, 0, sizeof *out);
  std::strncpy(out->dtype, FORMATS[row.format].name, sizeof out->dtype - 1);
  out->use_2cta = row.use_2cta;
  out->output_n = row.output_n;
  out->swap_ab = row.swap_ab;
  out->cluster_m = row.use_2cta ? 2 : 1;
  out->cluster_n = 1;
  out->cluster_k = 1;
  out->block_m = 128;
  out->split_k = 1;
  out->persistent = 1;
  return OG_OK;
}

}  // namespace
}  // namespace og

using namespace og;

extern "C" {

OG_API int32_t og_mm_abi(void) { return OG_ABI_VERSION; }
OG_API const char* og_mm_error(void) { return error_text; }
OG_API int32_t og_mm_kernels(void) { return menu_rows(false, nullptr, 0); }
OG_API int32_t og_mm_kernel(int32_t i, OgGemm* out) { return describe_row(false, i, out); }
OG_API int32_t og_mm_bind(OgGemm* g) {
  if (!g) return fail(OG_ERR_BIND, "null OgGemm");
  return bind_impl(g, false);
}
OG_API int32_t og_mm_launch(const OgGemm* g, const void* a, const void* b, const void* sfa,
                            const void* sfb, void* c, int32_t device, void* stream) {
  (void)sfa;
  (void)sfb;
  return launch_impl(g, a, b, nullptr, nullptr, c, device, stream, nullptr, 0);
}

OG_API int32_t og_smm_abi(void) { return OG_ABI_VERSION; }
OG_API const char* og_smm_error(void) { return error_text; }
OG_API int32_t og_smm_kernels(void) { return menu_rows(true, nullptr, 0); }
OG_API int32_t og_smm_kernel(int32_t i, OgGemm* out) { return describe_row(true, i, out); }
OG_API int32_t og_smm_bind(OgGemm* g) {
  if (!g) return fail(OG_ERR_BIND, "null OgGemm");
  return bind_impl(g, true);
}
OG_API int32_t og_smm_launch(const OgGemm* g, const void* a, const void* b, const void* sfa,
                             const void* sfb, void* c, int32_t device, void* stream) {
  return launch_impl(g, a, b, sfa, sfb, c, device, stream, nullptr, 1);
}

OG_API int32_t og_b200_plan(const OgGemm* g, int32_t device, OgPlan* out) {
  if (!g || !out) return fail(OG_ERR_BIND, "null argument");
  Plan p;
  char why[256];
  const int status = make_plan(*g, 148, &p, why, sizeof why);
  if (status != OG_OK) return fail(status, "%s", why);
  out->cta_group = p.cta_group;
  out->tile_m = p.tile_m;
  out->tile_n = p.tile_n;
  out->block_k = p.block_k;
  out->stages = p.stages;
  out->swap = p.swap;
  out->epi_staged = p.epi_staged;
  out->epi_tma = p.epi_tma;
  out->acc_slots = p.acc_slots;
  out->tmem_cols = p.tmem_cols;
  out->smem_bytes = p.smem_bytes;
  out->tiles = p.num_tiles;
  out->grid = grid_for(p, sm_count_of(device));
  out->group = p.group;
  out->use_clc = 0;
  if (g->use_clc && g->split_k < 2) {
    out->use_clc = 1;
    out->grid = p.num_tiles * p.cta_group;
  }
  out->stream_k = 0;
  if (g->split_k >= 2 && use_stream_k(*g, p, grid_for(p, sm_count_of(device), true))) {
    out->grid = grid_for(p, sm_count_of(device), true);
    out->stream_k = 1;
  }
  return OG_OK;
}

OG_API int32_t og_b200_launch_checked(const OgGemm* g, const void* a, const void* b,
                                      const void* sfa, const void* sfb, void* c, int32_t device,
                                      void* stream, int32_t* status) {
  return launch_impl(g, a, b, sfa, sfb, c, device, stream, status, -1);
}

OG_API int32_t og_b200_launch_alpha(const OgGemm* g, const void* a, const void* b, const void* sfa,
                                    const void* sfb, void* c, int32_t device, void* stream, float alpha) {
  return launch_impl(g, a, b, sfa, sfb, c, device, stream, nullptr, -1, &alpha);
}

OG_API int32_t og_b200_describe(const OgGemm* g, int32_t sm_count, char* out, int32_t cap) {
  if (!g || !out || cap <= 0) return fail(OG_ERR_BIND, "null argument");
  Plan p;
  char why[256];
  const int status = make_plan(*g, sm_count, &p, why, sizeof why);
  if (status != OG_OK) return fail(status, "%s", why);
  const int grid = grid_for(p, sm_count > 0 ? sm_count : 148);
  const int wrote = snprintf(
      out, size_t(cap),
      "{\"scaled\":%d,\"variant\":%d,\"kind\":%d,\"cta_group\":%d,\"swap\":%d,\"rows_m\":%d,\"rows_n\":%d,\"k\":%d,"
      "\"tile_m\":%d,\"tile_n\":%d,\"block_k\":%d,\"mma_k\":%d,\"k_blocks\":%d,\"stages\":%d,\"x_bytes\":%d,"
      "\"y_bytes\":%d,\"sf_bytes\":%d,\"stage_bytes\":%d,\"tx_bytes\":%d,\"tiles_m\":%d,\"tiles_n\":%d,"
      "\"num_tiles\":%d,\"group\":%d,\"idesc\":%u,\"acc_slots\":%d,\"acc_stride\":%d,\"sf_col\":%d,\"sf_slots\":%d,"
      "\"sf_cols\":%d,\"tmem_cols\":%d,\"epi_staged\":%d,\"epi_tma\":%d,\"out_bytes\":%d,\"out\":%d,\"sf_atoms\":%d,\"sf_yblocks\":%d,"
      "\"k_groups\":%d,\"smem_bytes\":%d,\"x_bits\":%d,\"y_bits\":%d,\"x_map\":%d,\"y_map\":%d,\"l2_promo\":%d,"
      "\"grid\":%d,\"m\":%d,\"n\":%d}",
      int(p.format->scaled), p.variant, p.format->kind, p.cta_group, p.swap, p.rows_m, p.rows_n, p.k, p.tile_m,
      p.tile_n, p.block_k, p.mma_k, p.k_blocks, p.stages, p.x_bytes, p.y_bytes, p.sf_bytes, p.stage_bytes,
      p.tx_bytes, p.tiles_m, p.tiles_n, p.num_tiles, p.group, p.idesc, p.acc_slots, p.acc_stride, p.sf_col,
      p.sf_slots, p.sf_cols, p.tmem_cols, p.epi_staged, p.epi_tma, p.out_bytes, p.format->out, p.sf_atoms, p.sf_yblocks,
      p.k_groups, p.smem_bytes, p.x_bits, p.y_bits, p.x_map, p.y_map, p.l2_promo, grid, g->m, g->n);
  if (wrote < 0 || wrote >= cap) return fail(OG_ERR_BIND, "the buffer of %d bytes is too small for the description", cap);
  return OG_OK;
}

OG_API void og_b200_set_independent_inputs(int32_t yes) { independent_inputs.store(yes ? 1 : 0); }

OG_API void og_b200_set_wait_limit_ms(int32_t ms) {
  wait_limit_ns.store((long long)std::max(1, (int)ms) * 1000000ll);
}

}  // extern "C"
