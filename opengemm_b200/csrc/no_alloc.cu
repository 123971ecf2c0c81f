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
#include "launch_common.h"
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
  char why[320];
  const int planned = make_plan(*g, 148, &p, why, sizeof why);
  if (planned != OG_OK) return refuse(planned, "%s", why);
  const LaunchPointers io{a, b, sfa, sfb, c, nullptr};
  int rc = check_pointers(*g, p, io, nullptr, why, sizeof why);
  if (rc != OG_OK) return refuse(rc, "%s", why);

  PerDevice* dev = nullptr;
  const int ready = set_up(device, &dev);
  if (ready != OG_OK) return ready;
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

  // The same parameter block as the ordinary launches build (tensor maps from
  // the shared per-thread cache, the wait limit of og_b200_set_wait_limit_ms).
  GemmParams params;
  rc = fill_params(p, *g, io, nullptr, nullptr, current_wait_limit_ns(), &params, why, sizeof why);
  if (rc != OG_OK) return refuse(rc, "%s", why);

  // Stream-K wherever the tiles leave a partial wave that can be cut along K;
  // otherwise the plain schedule, which touches no workspace at all (and is
  // therefore never refused for its size).
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per_cluster = p.cta_group * p.cluster_k;
  const int clusters = std::max(1, std::min(p.num_tiles, dev->sm_count / per_cluster));
  const int grid = clusters * per_cluster;
  if (p.cluster_k == 1 && p.num_tiles > clusters && p.num_tiles % clusters != 0 && p.k_blocks > 1) {
    const int regions = grid * 4;
    if (regions > MAX_REGIONS)
      return refuse(OG_ERR_LAUNCH,
                    "this launch needs %d partial-sum regions (a grid of %d CTAs); the fixed workspace holds %d "
                    "(grids of at most %d CTAs): use og_mm_launch / og_smm_launch on this device",
                    regions, grid, MAX_REGIONS, MAX_CTAS);
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
    params.partial = reinterpret_cast<float*>(dev->workspace);
    params.flags = reinterpret_cast<int*>(flags);
  }
  // No programmatic overlap with the previous kernel: two of these calls must
  // never run at once, they share the workspace.
  const cudaError_t launched = (p.variant < 8 || p.variant >= 14) ? launch_dense(p.variant, params, grid, p.smem_bytes, s, false)
                                             : launch_scaled(p.variant, params, grid, p.smem_bytes, s, false);
  if (launched != cudaSuccess) return refuse(OG_ERR_LAUNCH, "kernel launch failed: %s", cudaGetErrorString(launched));
  return OG_OK;
}

}  // extern "C"
