// og_b200_launch_no_alloc: the stream-K GEMM for callers that must not
// allocate.
//
// Some users of this library cannot tolerate a device allocation inside a
// launch call: a serving process that sized its memory pool at start-up and
// must never fail (or implicitly synchronise the device, as cudaMalloc does)
// in the middle of a request; code running under a framework's caching
// allocator that owns every remaining byte; a latency-critical loop where an
// allocation on first use is an unacceptable hiccup.  The ordinary launch
// path allocates the stream-K schedule's partial-sum workspace with cudaMalloc
// the first time a device needs it.  This entry point never allocates: its
// workspace is the fixed array below, part of the library image, so every GPU
// that loads the library carries it (about 18.5 MiB) until the process exits.
//
// What follows from a fixed, shared array:
//  * Capacity.  It holds one 32 KiB partial-sum region and one flag per
//    epilogue warp of a grid of at most 148 CTAs (592 regions).  The need
//    grows with the number of SMs the launch occupies, not with M, N or K; a
//    device whose grid would need more regions is refused with an error.
//  * One user at a time.  Every call on a device uses the same array, and the
//    array still holds what the previous call left in it.  Each call clears
//    the flag words on its stream before the kernel, so a kernel never
//    mistakes an old partial sum for a fresh one; but two calls whose kernels
//    overlap on the GPU (different streams, or programmatic overlap) would
//    write the same regions and race.  Serialise calls per device.
//  * Set-up.  The array's name is only a host-side handle.  The first call on
//    each device makes that device current and asks the runtime for the
//    array's address there (cudaGetSymbolAddress), once; later calls reuse
//    it.  Make that first call outside any stream capture.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel.cuh"
#include "plan.h"

namespace og {

cudaError_t configure_dense(int variant, int smem_bytes);
cudaError_t configure_scaled(int variant, int smem_bytes);
cudaError_t launch_dense(int variant, const GemmParams& params, int grid, int smem_bytes,
                         cudaStream_t stream, bool pdl);
cudaError_t launch_scaled(int variant, const GemmParams& params, int grid, int smem_bytes,
                          cudaStream_t stream, bool pdl);

namespace {

constexpr int MAX_CTAS = 148;                     // largest grid the fixed workspace serves
constexpr int MAX_REGIONS = MAX_CTAS * 4;         // one per epilogue warp
constexpr size_t REGION_BYTES = 32 * 256 * 4;     // 32 rows x 256 f32 partial sums
constexpr size_t PARTIAL_BYTES = MAX_REGIONS * REGION_BYTES;
constexpr size_t FLAG_BYTES = 4096;               // MAX_REGIONS ints, rounded up
static_assert(MAX_REGIONS * sizeof(int) <= FLAG_BYTES, "flag area too small");

// The workspace itself: partial sums first, flag words after them.  Device
// code could name it directly; host code may only take its address through
// cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char fixed_workspace[PARTIAL_BYTES + FLAG_BYTES];

// Where the current call's error text goes: the caller's buffer, if it gave one.
thread_local char* error_out = nullptr;
thread_local int error_cap = 0;

int refuse(int code, const char* format, ...) {
  if (error_out && error_cap > 0) {
    va_list args;
    va_start(args, format);
    vsnprintf(error_out, size_t(error_cap), format, args);
    va_end(args);
  }
  return code;
}

struct PerDevice {
  unsigned char* workspace = nullptr;  // device address of fixed_workspace on this device
  int sm_count = 0;
  uint64_t configured = 0;             // bit per kernel variant whose smem limit is raised
  unsigned calls = 0;                  // tags successive calls
};
std::mutex setup_mutex;
PerDevice per_device[64];

// Make `device` current and, the first time, find this device's copy of the
// workspace.  Nothing here allocates.
int set_up(int device, PerDevice** out) {
  if (device < 0 || device >= 64) return refuse(OG_ERR_LAUNCH, "device %d is out of range", device);
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return refuse(OG_ERR_LAUNCH, "cudaGetDevice failed");
  if (current != device) {
    const cudaError_t moved = cudaSetDevice(device);
    if (moved != cudaSuccess) return refuse(OG_ERR_LAUNCH, "cudaSetDevice: %s", cudaGetErrorString(moved));
  }
  std::lock_guard<std::mutex> lock(setup_mutex);
  PerDevice& slot = per_device[device];
  if (!slot.workspace) {
    void* address = nullptr;
    const cudaError_t found = cudaGetSymbolAddress(&address, fixed_workspace);
    if (found != cudaSuccess || !address)
      return refuse(OG_ERR_LAUNCH, "cudaGetSymbolAddress for the fixed workspace failed on device %d: %s",
                    device, cudaGetErrorString(found));
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      return refuse(OG_ERR_LAUNCH, "cannot read the SM count of device %d", device);
    slot.workspace = static_cast<unsigned char*>(address);
    slot.sm_count = sms;
  }
  *out = &slot;
  return OG_OK;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

int encode(CUtensorMap* out, const void* base, int type, uint64_t dim0, uint64_t dim1, uint64_t stride,
           uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle, const char* which) {
  static EncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return EncodeFn(nullptr);
    return reinterpret_cast<EncodeFn>(sym);
  }();
  if (!fn) return refuse(OG_ERR_TENSORMAP, "cuTensorMapEncodeTiled is not available: no CUDA driver");
  const cuuint64_t dims[2] = {dim0, dim1};
  const cuuint64_t strides[1] = {stride};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t ones[2] = {1, 1};
  const CUresult status = fn(out, CUtensorMapDataType(type), 2, const_cast<void*>(base), dims, strides, box, ones,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS)
    return refuse(OG_ERR_TENSORMAP, "cuTensorMapEncodeTiled failed for %s (driver error %d)", which, int(status));
  return OG_OK;
}

}  // namespace
}  // namespace og

using namespace og;

extern "C" {

// Same contract as og_mm_launch / og_smm_launch (chosen by g->dtype; `g` bound
// beforehand), always on the stream-K schedule where the shape admits it, and
// without any allocation: see the head of this file for the conditions.  On
// failure the return code is an OG_ERR_* value and, when `error_text` is not
// null, up to `error_text_cap` bytes of explanation are written there.
OG_API int32_t og_b200_launch_no_alloc(const OgGemm* g, const void* a, const void* b, const void* sfa,
                                       const void* sfb, void* c, int32_t device, void* stream,
                                       char* error_text, int32_t error_text_cap) {
  error_out = error_text;
  error_cap = error_text_cap;
  if (error_out && error_cap > 0) error_out[0] = 0;
  if (!g) return refuse(OG_ERR_LAUNCH, "null OgGemm");
  Plan p;
  char why[256];
  const int planned = make_plan(*g, 148, &p, why, sizeof why);
  if (planned != OG_OK) return refuse(planned, "%s", why);
  if (g->row != p.variant)
    return refuse(OG_ERR_LAUNCH, "row %d is not the kernel of this OgGemm: bind it first", g->row);
  if (!a || !b || !c) return refuse(OG_ERR_LAUNCH, "a, b and c must be device pointers, got null");
  if (p.format->scaled && (!sfa || !sfb))
    return refuse(OG_ERR_LAUNCH, "a block-scaled format takes both sfa and sfb");

  PerDevice* dev = nullptr;
  const int ready = set_up(device, &dev);
  if (ready != OG_OK) return ready;

  const int clusters = std::max(1, std::min(p.num_tiles, dev->sm_count / p.cta_group));
  const int grid = clusters * p.cta_group;
  const int regions = grid * 4;
  if (regions > MAX_REGIONS)
    return refuse(OG_ERR_LAUNCH,
                  "this launch needs %d partial-sum regions (a grid of %d CTAs); the fixed workspace holds %d "
                  "(grids of at most %d CTAs): use og_mm_launch / og_smm_launch on this device",
                  regions, grid, MAX_REGIONS, MAX_CTAS);
  {
    std::lock_guard<std::mutex> lock(setup_mutex);
    const uint64_t bit = 1ull << p.variant;
    if (!(dev->configured & bit)) {
      const cudaError_t raised = (p.variant < 8 || p.variant >= 14) ? configure_dense(p.variant, SMEM_LIMIT - 1024)
                                               : configure_scaled(p.variant, SMEM_LIMIT - 1024);
      if (raised != cudaSuccess) return refuse(OG_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(raised));
      dev->configured |= bit;
    }
  }

  GemmParams params;
  std::memset(&params, 0, sizeof params);
  const void* x = p.swap ? b : a;
  const void* y = p.swap ? a : b;
  const uint64_t k = uint64_t(p.k);
  int rc = encode(&params.map_x, x, p.x_map, k, uint64_t(p.rows_m), k * p.x_bits / 8, uint32_t(p.block_k), 128,
                  CU_TENSOR_MAP_SWIZZLE_128B, "the M-side operand");
  if (rc != OG_OK) return rc;
  rc = encode(&params.map_y, y, p.y_map, k, uint64_t(p.rows_n), k * p.y_bits / 8, uint32_t(p.block_k),
              uint32_t(p.tile_n / p.cta_group), CU_TENSOR_MAP_SWIZZLE_128B, "the N-side operand");
  if (rc != OG_OK) return rc;
  const bool c_aligned = (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  const int epi_staged = p.epi_staged && c_aligned;
  const int epi_tma = p.epi_tma && c_aligned;
  if (epi_tma) {
    const int type = p.format->out == OUT_S32 ? int(CU_TENSOR_MAP_DATA_TYPE_INT32) : int(CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    rc = encode(&params.map_d, c, type, uint64_t(g->n), uint64_t(g->m), uint64_t(g->n) * p.out_bytes,
                uint32_t(128 / p.out_bytes), 32, CU_TENSOR_MAP_SWIZZLE_128B, "the output");
    if (rc != OG_OK) return rc;
  }
  if (p.format->scaled) {
    const uint64_t atoms_x = uint64_t(ceil_div(p.rows_m, 128)) * p.k_groups;
    const uint64_t atoms_y = uint64_t(ceil_div(p.rows_n, 128)) * p.k_groups;
    rc = encode(&params.map_sfx, p.swap ? sfb : sfa, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_x, 256,
                256, uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, "the M-side scales");
    if (rc != OG_OK) return rc;
    rc = encode(&params.map_sfy, p.swap ? sfa : sfb, int(CU_TENSOR_MAP_DATA_TYPE_UINT8), 256, 2 * atoms_y, 256,
                256, uint32_t(2 * p.sf_atoms), CU_TENSOR_MAP_SWIZZLE_NONE, "the N-side scales");
    if (rc != OG_OK) return rc;
  }
  params.d = c;
  params.status = nullptr;
  params.wait_limit_ns = 2000ull * 1000 * 1000;
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

  // Stream-K wherever every cluster gets at least a tile's worth of K blocks
  // and the tiles do not already fill whole waves; otherwise the plain
  // schedule, which needs no workspace at all.
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.num_tiles > clusters && p.num_tiles % clusters != 0) {
    unsigned char* flags = dev->workspace + PARTIAL_BYTES;
    // The flag words must not carry a previous call's tags into this one.
    const cudaError_t cleared = cudaMemsetAsync(flags, 0, size_t(regions) * sizeof(int), s);
    if (cleared != cudaSuccess) return refuse(OG_ERR_LAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(cleared));
    unsigned tag;
    {
      std::lock_guard<std::mutex> lock(setup_mutex);
      tag = ++dev->calls;
      if ((tag & 0x7FFFFFFFu) == 0) tag = ++dev->calls;
    }
    params.stream_k = 1;
    params.sk_clusters = clusters;
    params.epoch = int(tag & 0x7FFFFFFFu);
    params.acc_int = p.format->out == OUT_S32;
    params.partial = reinterpret_cast<float*>(dev->workspace);
    params.flags = reinterpret_cast<int*>(flags);
  }
  const cudaError_t launched = (p.variant < 8 || p.variant >= 14) ? launch_dense(p.variant, params, grid, p.smem_bytes, s, false)
                                             : launch_scaled(p.variant, params, grid, p.smem_bytes, s, false);
  if (launched != cudaSuccess) return refuse(OG_ERR_LAUNCH, "kernel launch failed: %s", cudaGetErrorString(launched));
  return OG_OK;
}

}  // extern "C"
