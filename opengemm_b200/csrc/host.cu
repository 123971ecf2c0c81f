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
#include <memory>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "kernel.cuh"
#include "kernels_fixed.cuh"
#include "launch_common.h"
#include "plan.h"

namespace og {

// Implemented in kernels_dense.cu (variants 0-7 and 14-19) and kernels_scaled.cu (8-13).
cudaError_t configure_dense(int variant, int smem_bytes);
cudaError_t configure_scaled(int variant, int smem_bytes);
cudaError_t launch_dense(int variant, const GemmParams& params, int grid, int smem_bytes,
                         cudaStream_t stream, bool pdl);
cudaError_t launch_scaled(int variant, const GemmParams& params, int grid, int smem_bytes,
                          cudaStream_t stream, bool pdl);

// Implemented in kernels_fixed_dense.cu and kernels_fixed_scaled.cu.
extern const FixedKernel FIXED_DENSE[];
extern const int FIXED_DENSE_COUNT;
extern const FixedKernel FIXED_SCALED[];
extern const int FIXED_SCALED_COUNT;
// Implemented in kernels_plain_dense.cu and kernels_plain_scaled.cu.
extern const FixedKernel PLAIN_DENSE[];
extern const int PLAIN_DENSE_COUNT;
extern const FixedKernel PLAIN_SCALED[];
extern const int PLAIN_SCALED_COUNT;

// One index space over the specialised kernels: fixed-shape dense, fixed-shape
// scaled, then the feature-free ones.
inline int fixed_count() { return FIXED_DENSE_COUNT + FIXED_SCALED_COUNT; }
inline int specialised_count() { return fixed_count() + PLAIN_DENSE_COUNT + PLAIN_SCALED_COUNT; }
inline const FixedKernel& fixed_kernel(int index) {
  if (index < FIXED_DENSE_COUNT) return FIXED_DENSE[index];
  if (index < fixed_count()) return FIXED_SCALED[index - FIXED_DENSE_COUNT];
  index -= fixed_count();
  return index < PLAIN_DENSE_COUNT ? PLAIN_DENSE[index] : PLAIN_SCALED[index - PLAIN_DENSE_COUNT];
}

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
// Testing aid (og_b200_test_overcredit_next_launch): bytes added to what the
// next launch on this thread credits to every stage barrier.
thread_local int overcredit_next = 0;

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(error_text, sizeof error_text, format, args);
  va_end(args);
  return code;
}

// Stream-K scratch: partial sums of tiles shared by two clusters, and the
// flags that publish them.  One region per epilogue warp of a full grid;
// WORKSPACES of them per device are used round-robin by that device's
// successive stream-K launches.  A launch that takes a slot first makes its
// stream wait for the slot's previous user (an event recorded behind that
// launch), so launches on any number of streams never share a workspace while
// either is running; with one stream the wait is already satisfied.
constexpr int WORKSPACES = 4;
constexpr size_t REGION_BYTES = 32 * 256 * 4;
constexpr int MAX_DEVICES = 64;

struct DeviceInfo {
  int sm_count = 0;
  uint64_t configured = 0;  // bit per kernel variant
  unsigned epoch = 0;       // this device's stream-K launches so far
  float* partial[WORKSPACES] = {};
  int* flags[WORKSPACES] = {};
  cudaEvent_t released[WORKSPACES] = {};  // recorded behind the slot's last user
};
std::mutex device_mutex;
DeviceInfo devices[MAX_DEVICES];

int follow_device(int device) {
  if (device < 0 || device >= MAX_DEVICES)
    return fail(OG_ERR_LAUNCH, "device %d is out of range: this library serves devices 0..%d", device, MAX_DEVICES - 1);
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return fail(OG_ERR_LAUNCH, "cudaGetDevice failed");
  if (current != device) {
    const cudaError_t moved = cudaSetDevice(device);
    if (moved != cudaSuccess) return fail(OG_ERR_LAUNCH, "cudaSetDevice: %s", cudaGetErrorString(moved));
  }
  return OG_OK;
}

std::atomic<int> sm_count_fast[MAX_DEVICES];
std::atomic<uint64_t> configured_fast[MAX_DEVICES];

int sm_count_of(int device) {
  if (device < 0 || device >= MAX_DEVICES) return 148;
  if (const int known = sm_count_fast[device].load(std::memory_order_relaxed)) return known;
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device];
  if (!info.sm_count) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    info.sm_count = count;
  }
  sm_count_fast[device].store(info.sm_count, std::memory_order_relaxed);
  return info.sm_count;
}

// The most specialised kernel that serves this launch: the one compiled for
// exactly its tile shape if there is one, else - when it asks for no optional
// feature - the feature-free build of its variant; its index, else -1.  Every
// value such a kernel has folded in must equal the launch's, and every option
// it was compiled without must be off.
std::atomic<int> fixed_kernels_on{[] { const char* e = getenv("OPENGEMM_FIXED"); return (e && e[0] == '0') ? 0 : 1; }()};

int fixed_kernel_for(const Plan& p, const GemmParams& params) {
  if (!fixed_kernels_on.load(std::memory_order_relaxed)) return -1;
  if (params.use_clc || params.stream_k || params.scale_out || params.bias || params.out_f16 || params.out_quant ||
      params.walk || params.cluster_k > 1)
    return -1;
  const int epi = params.epi_tma ? 2 : params.epi_staged ? 1 : 0;
  for (int i = 0; i < fixed_count() && !params.transpose_out && params.vec_ok; ++i) {
    const FixedKernel& k = fixed_kernel(i);
    if (k.variant != p.variant || k.tile_n != params.tile_n || k.epi != epi) continue;
    const TileShape t = tile_shape(p.smem_bits, p.format->scaled ? p.format->sf_block : 0, p.cta_group,
                                   p.out_bytes, k.tile_n, k.epi);
    if (t.stages == params.stages) return i;
    break;
  }
  for (int i = fixed_count(); i < specialised_count(); ++i)
    if (fixed_kernel(i).variant == p.variant) return i;
  return -1;
}

std::atomic<uint64_t> fixed_configured_fast[MAX_DEVICES];

int ensure_fixed_configured(int device, int index) {
  const uint64_t bit = 1ull << index;
  if (fixed_configured_fast[device].load(std::memory_order_acquire) & bit) return OG_OK;
  std::lock_guard<std::mutex> lock(device_mutex);
  const cudaError_t status = fixed_kernel(index).configure(SMEM_LIMIT - 1024);
  if (status != cudaSuccess)
    return fail(OG_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(status));
  fixed_configured_fast[device].fetch_or(bit, std::memory_order_release);
  return OG_OK;
}

int ensure_configured(int device, int variant, int smem_bytes) {
  const uint64_t bit = 1ull << variant;
  if (configured_fast[device].load(std::memory_order_acquire) & bit) return OG_OK;
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device];
  if (info.configured & bit) return OG_OK;
  const cudaError_t status = configure_variant(variant, SMEM_LIMIT - 1024);  // static barriers take the rest
  if (status != cudaSuccess)
    return fail(OG_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(status));
  (void)smem_bytes;
  info.configured |= bit;
  configured_fast[device].fetch_or(bit, std::memory_order_release);
  return OG_OK;
}

// Allocate `device`'s stream-K workspaces and their guard events, once.
// Flags start at zero and are matched against a per-launch epoch, so they are
// never cleared.  The device must be current.  Caller holds device_mutex.
int allocate_workspaces(DeviceInfo& info, int sm_count) {
  if (info.partial[WORKSPACES - 1]) return OG_OK;
  const size_t regions = size_t(sm_count) * 4;
  for (int slot = 0; slot < WORKSPACES; ++slot) {
    if (info.partial[slot]) continue;
    void* data = nullptr;
    void* words = nullptr;
    cudaEvent_t event = nullptr;
    if (cudaMalloc(&data, regions * REGION_BYTES) != cudaSuccess ||
        cudaMalloc(&words, regions * sizeof(int)) != cudaSuccess ||
        cudaMemset(words, 0, regions * sizeof(int)) != cudaSuccess ||
        cudaEventCreateWithFlags(&event, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      if (data) cudaFree(data);
      if (words) cudaFree(words);
      return fail(OG_ERR_LAUNCH, "cannot allocate the %zu-byte stream-K workspace", regions * REGION_BYTES);
    }
    info.flags[slot] = static_cast<int*>(words);
    info.released[slot] = event;
    info.partial[slot] = static_cast<float*>(data);
  }
  return OG_OK;
}

// Take the next workspace of `device` for a stream-K launch on `stream`:
// returns its buffers and this launch's tag, after making `stream` wait for
// the slot's previous user.  `*slot_out` is handed to release_workspace once
// the kernel is enqueued.
int take_workspace(int device, int sm_count, cudaStream_t stream, float** partial, int** flags, int* tag,
                   int* slot_out) {
  std::lock_guard<std::mutex> lock(device_mutex);
  DeviceInfo& info = devices[device];
  const int ready = allocate_workspaces(info, sm_count);
  if (ready != OG_OK) return ready;
  unsigned epoch = ++info.epoch;
  if ((epoch & 0x7FFFFFFFu) == 0) epoch = ++info.epoch;  // the tag is never 0
  const int slot = int(epoch % WORKSPACES);
  if (epoch > unsigned(WORKSPACES) &&
      cudaStreamWaitEvent(stream, info.released[slot], 0) != cudaSuccess) {
    cudaGetLastError();
    return fail(OG_ERR_LAUNCH, "cudaStreamWaitEvent on the stream-K workspace failed");
  }
  *partial = info.partial[slot];
  *flags = info.flags[slot];
  *tag = int(epoch & 0x7FFFFFFFu);
  *slot_out = slot;
  return OG_OK;
}

void release_workspace(int device, int slot, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(device_mutex);
  if (cudaEventRecord(devices[device].released[slot], stream) != cudaSuccess) cudaGetLastError();
}

// Stream-K applies when the tiles do not fill a whole number of waves: the
// tiles of the partial wave are then cut along K across all clusters.
bool use_stream_k(const OgGemm& g, const Plan& p, int grid) {
  const int clusters = grid / p.cta_group;
  return g.split_k >= 2 && p.cluster_k == 1 && p.num_tiles % clusters != 0 && p.k_blocks > 1;
}

int grid_for(const Plan& p, int sm_count, bool fill = false) {
  // `fill`: a stream-K launch occupies every SM even with fewer tiles than SMs.
  const int per_cluster = p.cta_group * p.cluster_k;
  const int all = std::max(1, sm_count / per_cluster);
  const int clusters = fill ? std::min(all, std::max(1, p.num_tiles * p.k_blocks)) : std::max(1, std::min(p.num_tiles, all));
  return clusters * per_cluster;
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
  unsigned generation = 0;  // changes whenever `plan` does
};
thread_local PlanMemo plan_memo;

// A launch's parameter block is a function of the bound GEMM, the caller's
// pointers and the wait limit.  Loops that run the same buffers again and
// again (serving, benchmarks) find theirs here and skip the pointer checks,
// the tensor-map look-ups and the fill: per thread, 256 blocks indexed by a
// hash of the output address (about 280 KB, allocated by a thread's first
// launch), enough for loops that rotate a hundred-odd buffer sets past L2.
struct ParamsMemo {
  bool valid = false;
  unsigned generation = 0;
  LaunchPointers io{};
  int* status = nullptr;
  bool scaled_out = false;
  float alpha = 1.0f;
  unsigned long long wait_limit = 0;
  GemmParams params;
  bool matches(unsigned gen, const LaunchPointers& o, int* status_word, const float* a, unsigned long long limit) const {
    return valid && generation == gen && io.a == o.a && io.b == o.b && io.sfa == o.sfa && io.sfb == o.sfb &&
           io.c == o.c && io.bias == o.bias && io.out_quant == o.out_quant && io.c_scales == o.c_scales &&
           status == status_word && scaled_out == (a != nullptr) && (!a || alpha == *a) && wait_limit == limit;
  }
};
constexpr unsigned PARAMS_MEMO_BITS = 8;
thread_local std::unique_ptr<ParamsMemo[]> params_memo;

int launch_impl(const OgGemm* g, const LaunchPointers& io, int device, void* stream, int* status_word,
                int want_scaled, const float* alpha = nullptr) {
  if (!g) return fail(OG_ERR_LAUNCH, "null OgGemm");
  if (!plan_memo.valid || std::memcmp(&plan_memo.key, g, sizeof(OgGemm)) != 0) {
    char why[256];
    plan_memo.valid = false;
    const int planned = make_plan(*g, 148, &plan_memo.plan, why, sizeof why);
    if (planned != OG_OK) return fail(planned, "%s", why);
    plan_memo.key = *g;
    plan_memo.valid = true;
    ++plan_memo.generation;
  }
  const Plan& p = plan_memo.plan;
  char why[320];
  if (want_scaled >= 0 && int(p.format->scaled) != want_scaled)
    return fail(OG_ERR_LAUNCH, "dtype %.16s does not belong to this library", g->dtype);
  const unsigned long long wait_limit = current_wait_limit_ns();
  if (!params_memo) params_memo.reset(new ParamsMemo[1u << PARAMS_MEMO_BITS]());
  ParamsMemo& memo =
      params_memo[(uint32_t(reinterpret_cast<uintptr_t>(io.c) >> 9) * 0x9E3779B1u) >> (32 - PARAMS_MEMO_BITS)];
  const bool remembered = memo.matches(plan_memo.generation, io, status_word, alpha, wait_limit);
  if (!remembered) {
    const int rc = check_pointers(*g, p, io, alpha, why, sizeof why);
    if (rc != OG_OK) return fail(rc, "%s", why);
  }
  const int followed = follow_device(device);
  if (followed != OG_OK) return followed;
  const int configured = ensure_configured(device, p.variant, p.smem_bytes);
  if (configured != OG_OK) return configured;

  GemmParams params;
  if (remembered) {
    params = memo.params;
  } else {
    const int rc = fill_params(p, *g, io, status_word, alpha, wait_limit, &params, why, sizeof why);
    if (rc != OG_OK) return fail(rc, "%s", why);
    memo.valid = true, memo.generation = plan_memo.generation, memo.io = io, memo.status = status_word;
    memo.scaled_out = alpha != nullptr, memo.alpha = alpha ? *alpha : 1.0f, memo.wait_limit = wait_limit;
    memo.params = params;
  }
  if (overcredit_next) {  // testing aid: the stage barriers will wait for bytes that never come
    params.tx_bytes += overcredit_next;
    overcredit_next = 0;
  }
  static const bool pdl_enabled = [] { const char* e = getenv("OPENGEMM_PDL"); return !(e && e[0] == '0'); }();
  params.pdl = pdl_enabled ? (independent_inputs.load(std::memory_order_relaxed) ? 2 : 1) : 0;

  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sm_count = sm_count_of(device);
  int grid = grid_for(p, sm_count);
  if (g->use_clc && g->split_k < 2 && p.cluster_k == 1) {
    // Cluster launch control: one cluster per tile; running clusters take over
    // the tiles of those that have not started.
    params.use_clc = 1;
    grid = p.num_tiles * p.cta_group;
  }
  int workspace_slot = -1;
  if (g->split_k >= 2 && use_stream_k(*g, p, grid_for(p, sm_count, true))) {
    grid = grid_for(p, sm_count, true);
    const int got = take_workspace(device, sm_count, s, &params.partial, &params.flags, &params.epoch, &workspace_slot);
    if (got != OG_OK) return got;
    params.stream_k = 1;
    {
      // split_k is the most ways a tile of the partial wave is cut: that many
      // clusters per leftover tile share its K blocks, the rest sit the wave out.
      const int clusters = grid / p.cta_group;
      const int leftover = p.num_tiles % clusters;
      params.sk_clusters = std::min<long long>(clusters, (long long)leftover * std::min<int>(g->split_k, p.k_blocks));
    }
  }
  const int fixed = fixed_kernel_for(p, params);
  if (fixed >= 0) {
    const int ready = ensure_fixed_configured(device, fixed);
    if (ready != OG_OK) return ready;
  }
  const cudaError_t launched =
      fixed >= 0 ? fixed_kernel(fixed).launch(params, grid, p.smem_bytes, s, params.pdl != 0)
                 : launch_variant(p.variant, params, grid, p.smem_bytes, s, params.pdl != 0);
  if (workspace_slot >= 0) release_workspace(device, workspace_slot, s);
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

unsigned long long current_wait_limit_ns() { return (unsigned long long)wait_limit_ns.load(); }

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
  return launch_impl(g, LaunchPointers{a, b, nullptr, nullptr, c, nullptr}, device, stream, nullptr, 0);
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
  return launch_impl(g, LaunchPointers{a, b, sfa, sfb, c, nullptr}, device, stream, nullptr, 1);
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
  if (g->use_clc && g->split_k < 2 && p.cluster_k == 1) {
    out->use_clc = 1;
    out->grid = p.num_tiles * p.cta_group;
  }
  out->stream_k = 0;
  if (g->split_k >= 2 && use_stream_k(*g, p, grid_for(p, sm_count_of(device), true))) {
    out->grid = grid_for(p, sm_count_of(device), true);
    out->stream_k = 1;
  }
  {
    // Which kernel a plain launch into a 16-byte aligned C would run.
    GemmParams probe;
    std::memset(&probe, 0, sizeof probe);
    probe.tile_n = p.tile_n, probe.stages = p.stages, probe.epi_staged = p.epi_staged, probe.epi_tma = p.epi_tma;
    probe.transpose_out = p.swap, probe.walk = p.walk, probe.use_clc = out->use_clc, probe.stream_k = out->stream_k;
    probe.vec_ok = (int64_t(g->n) * p.out_bytes) % 16 == 0;
    probe.cluster_k = p.cluster_k;
    out->cluster_k = p.cluster_k;
    probe.out_f16 = p.format->out == OUT_F16;
    const int special = fixed_kernel_for(p, probe);
    out->fixed_shape = (special >= 0 && special < fixed_count()) ? 1 : 0;
    out->plain = special >= fixed_count() ? 1 : 0;
  }
  return OG_OK;
}

OG_API int32_t og_b200_launch_checked(const OgGemm* g, const void* a, const void* b,
                                      const void* sfa, const void* sfb, void* c, int32_t device,
                                      void* stream, int32_t* status) {
  return launch_impl(g, LaunchPointers{a, b, sfa, sfb, c, nullptr}, device, stream, status, -1);
}

OG_API int32_t og_b200_launch_alpha(const OgGemm* g, const void* a, const void* b, const void* sfa,
                                    const void* sfb, void* c, int32_t device, void* stream, float alpha) {
  return launch_impl(g, LaunchPointers{a, b, sfa, sfb, c, nullptr}, device, stream, nullptr, -1, &alpha);
}

OG_API int32_t og_b200_launch_bias(const OgGemm* g, const void* a, const void* b, const void* sfa,
                                   const void* sfb, void* c, int32_t device, void* stream, float alpha,
                                   const void* bias) {
  const bool scale = alpha != 1.0f;
  return launch_impl(g, LaunchPointers{a, b, sfa, sfb, c, bias}, device, stream, nullptr, -1, scale ? &alpha : nullptr);
}

OG_API int32_t og_b200_launch_quantized(const OgGemm* g, const void* a, const void* b, const void* sfa,
                                        const void* sfb, void* c_packed, void* c_scales, int32_t device,
                                        void* stream, const char* out_format) {
  int which = 0;
  if (out_format && !std::strcmp(out_format, "nvfp4")) which = 1;
  else if (out_format && !std::strcmp(out_format, "mxfp8")) which = 2;
  else if (out_format && !std::strcmp(out_format, "mxfp4")) which = 3;
  else return fail(OG_ERR_LAUNCH, "%.16s is not a block-scaled format: nvfp4, mxfp8 or mxfp4", out_format ? out_format : "(null)");
  LaunchPointers io{a, b, sfa, sfb, c_packed, nullptr};
  io.out_quant = which;
  io.c_scales = c_scales;
  return launch_impl(g, io, device, stream, nullptr, -1);
}

OG_API int32_t og_b200_status(int32_t status_word) {
  if (status_word == 0) return OG_OK;
  static const char* const sites[] = {"none", "producer waiting for a free stage", "MMA waiting for a stage's data",
                                      "MMA waiting for a free accumulator", "epilogue waiting for an accumulator",
                                      "producer draining", "stream-K finisher waiting for a partial sum",
                                      "scheduler answer", "tensor-memory allocation"};
  const int site = status_word & 0xFF;
  return fail(OG_ERR_TIMEOUT, "a device-side wait gave up: site %d (%s) in CTA %d", site,
              site >= 0 && site < int(sizeof sites / sizeof sites[0]) ? sites[site] : "unknown", status_word >> 8);
}

OG_API int32_t og_b200_prepare_device(int32_t device) {
  const int followed = follow_device(device);
  if (followed != OG_OK) return followed;
  for (int variant = 0; variant < 20; ++variant) {
    const int configured = ensure_configured(device, variant, 0);
    if (configured != OG_OK) return configured;
  }
  for (int index = 0; index < specialised_count(); ++index) {
    const int configured = ensure_fixed_configured(device, index);
    if (configured != OG_OK) return configured;
  }
  const int sm_count = sm_count_of(device);
  std::lock_guard<std::mutex> lock(device_mutex);
  return allocate_workspaces(devices[device], sm_count);
}

OG_API int32_t og_b200_tile_order(const OgGemm* g, int32_t* out, int32_t cap) {
  if (!g || !out) return fail(OG_ERR_BIND, "null argument");
  Plan p;
  char why[256];
  const int status = make_plan(*g, 148, &p, why, sizeof why);
  if (status != OG_OK) return fail(status, "%s", why);
  if (cap < 2 * p.num_tiles) return fail(OG_ERR_BIND, "%d tiles need room for %d integers, got %d", p.num_tiles, 2 * p.num_tiles, cap);
  for (int tile = 0; tile < p.num_tiles; ++tile) {
    const TileCoord t = tile_coord_of(tile, p.tiles_m, p.tiles_n, p.group, p.walk);
    out[2 * tile] = t.mi;
    out[2 * tile + 1] = t.ni;
  }
  return p.num_tiles;
}

OG_API void og_b200_test_overcredit_next_launch(int32_t bytes) { overcredit_next = bytes; }

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
      "\"grid\":%d,\"m\":%d,\"n\":%d,\"walk\":%d,\"cluster_k\":%d}",
      int(p.format->scaled), p.variant, p.format->kind, p.cta_group, p.swap, p.rows_m, p.rows_n, p.k, p.tile_m,
      p.tile_n, p.block_k, p.mma_k, p.k_blocks, p.stages, p.x_bytes, p.y_bytes, p.sf_bytes, p.stage_bytes,
      p.tx_bytes, p.tiles_m, p.tiles_n, p.num_tiles, p.group, p.idesc, p.acc_slots, p.acc_stride, p.sf_col,
      p.sf_slots, p.sf_cols, p.tmem_cols, p.epi_staged, p.epi_tma, p.out_bytes, p.format->out, p.sf_atoms, p.sf_yblocks,
      p.k_groups, p.smem_bytes, p.x_bits, p.y_bits, p.x_map, p.y_map, p.l2_promo, grid, g->m, g->n, p.walk, p.cluster_k);
  if (wrote < 0 || wrote >= cap) return fail(OG_ERR_BIND, "the buffer of %d bytes is too small for the description", cap);
  return OG_OK;
}

OG_API void og_b200_set_independent_inputs(int32_t yes) { independent_inputs.store(yes ? 1 : 0); }

OG_API void og_b200_set_fixed_kernels(int32_t yes) { fixed_kernels_on.store(yes ? 1 : 0); }

OG_API void og_b200_set_wait_limit_ms(int32_t ms) {
  wait_limit_ns.store((long long)std::max(1, (int)ms) * 1000000ll);
}

}  // extern "C"
