/* C ABI of libopengemm_b200.so: a B200 (sm_100a) GEMM library that stands in
 * for both of OpenGEMM's kernel libraries.
 *
 * It exports, with the same names, signatures and status codes, the twelve
 * entry points the reference's front end binds through ctypes
 * (opengemm/python/capi.py:86-174): six for the dense library
 * (opengemm/src/mm/capi.h:9-17, opengemm/src/mm/capi.cu:6-32) and six for the
 * block-scaled one (opengemm/src/smm/capi.h:9-17, opengemm/src/smm/capi.cu:6-32).
 * Pointing OPENGEMM_LIB_MM and OPENGEMM_LIB_SMM (opengemm/python/build.py:100-102)
 * at this one file makes the unmodified reference front end run on it.
 *
 * Plain C: pointers and sizes only.  All data pointers are device pointers
 * owned by the caller; the library keeps no reference to them after a call
 * returns.  It allocates no device memory, with one exception: the first launch
 * on a device that asks for the stream-K schedule (split_k >= 2) allocates
 * that schedule's scratch (about 76 MB) for the life of the process, unless
 * og_b200_prepare_device did so earlier.  Launches are asynchronous on the
 * stream given.  Devices 0..63 are served.
 */
#ifndef OPENGEMM_B200_H
#define OPENGEMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define OG_API __declspec(dllexport)
#else
#define OG_API __attribute__((visibility("default")))
#endif

/* opengemm/src/common/abi.h:11 */
#define OG_ABI_VERSION 3

/* Status codes, opengemm/src/common/abi.h:13-19; OG_ERR_TIMEOUT is new. */
enum {
  OG_OK = 0,
  OG_ERR_BIND = -1,      /* unknown dtype, or a K the format cannot take */
  OG_ERR_NO_KERNEL = -2, /* no kernel can serve the configuration */
  OG_ERR_TENSORMAP = -3,
  OG_ERR_LAUNCH = -4,
  OG_ERR_TIMEOUT = -5    /* a device-side wait ran out: what og_b200_status answers for a non-zero status word */
};

/* One GEMM: shape, the configs.json entry that picks and drives the kernel,
 * and the row og_*_bind resolved.  Field for field the reference's struct
 * (opengemm/src/common/abi.h:24-39), 108 bytes, no padding.  The caller fills
 * every field but `row`. */
typedef struct {
  int32_t m, n, k; /* k in values, not bytes */
  char dtype[16];  /* "bf16", "e4m3xe5m2", "nvfp4", ... */

  int32_t use_2cta, output_n, use_clc, swap_ab;
  int32_t cluster_m, cluster_n, cluster_k;
  int32_t block_m, stages, epi_hold, epi_double, epi_direct;
  int32_t epi_trade, deep_stages;

  int32_t supergroup, split_k, walk, l2_promo;
  int32_t persistent;

  int32_t row; /* set by og_*_bind */
} OgGemm;

/* ---- dense library: replaces opengemm/src/mm/capi.cu:6-32 ---------------- */

/* ABI version this library speaks (mm/capi.cu:6). */
OG_API int32_t og_mm_abi(void);
/* Text of the last failure on the calling thread (mm/capi.cu:8). */
OG_API const char* og_mm_error(void);
/* Number of kernel rows og_mm_kernel enumerates (mm/capi.cu:10). */
OG_API int32_t og_mm_kernels(void);
/* Fill `out` with the configuration that binds to row `i` (mm/capi.cu:12-18). */
OG_API int32_t og_mm_kernel(int32_t i, OgGemm* out);
/* Validate dtype / shape / knobs, clamp split_k, set g->row (mm/capi.cu:20, mm/launch.cuh:41-64). */
OG_API int32_t og_mm_bind(OgGemm* g);
/* Enqueue C[m,n] = A[m,k] . B[n,k]^T on `stream` of `device` (mm/capi.cu:22-32, mm/launch.cuh:105-183).
 * sfa and sfb are ignored. */
OG_API int32_t og_mm_launch(const OgGemm* g, const void* a, const void* b, const void* sfa,
                            const void* sfb, void* c, int32_t device, void* stream);

/* ---- block-scaled library: replaces opengemm/src/smm/capi.cu:6-32 -------- */

OG_API int32_t og_smm_abi(void);
OG_API const char* og_smm_error(void);
OG_API int32_t og_smm_kernels(void);
OG_API int32_t og_smm_kernel(int32_t i, OgGemm* out);
/* smm/launch.cuh:38-57 */
OG_API int32_t og_smm_bind(OgGemm* g);
/* sfa / sfb: scales in the 128x4 blocked layout (smm/launch.cuh:87-150, smm/tmap.cuh:21-36). */
OG_API int32_t og_smm_launch(const OgGemm* g, const void* a, const void* b, const void* sfa,
                             const void* sfb, void* c, int32_t device, void* stream);

/* ---- additions with no counterpart in the reference ----------------------- */

/* Output variant: besides the reference's fourteen dtype names, og_mm_bind accepts
 * "<format>.bf16" for every dense float format ("bf16.bf16", "f16.bf16", "tf32.bf16",
 * "e4m3.bf16", "e5m2.bf16", "e3m2.bf16", "e2m3.bf16", "e2m1.bf16", "e4m3xe5m2.bf16"):
 * same operands and tile plans, the f32 accumulator rounded to bfloat16 (nearest
 * even) on the way out, C a row-major bfloat16 [m, n]; and "<format>.f16" for the
 * same nine, C a row-major IEEE half [m, n].  og_mm_kernels / og_mm_kernel
 * enumerate the reference's formats only.
 *
 * Rasterisation: OgGemm.walk selects the order tiles are visited in, with the
 * reference's numbering (opengemm/src/mm/types.cuh:78-84): 0 bands `supergroup`
 * tiles wide along N; 1 the same, serpentine; 2 blocks inside a band; 3 a
 * generalised Hilbert curve; 4 bands along M.  Block-scaled formats, whose
 * reference struct carries no walk, use 0.
 *
 * Cluster-K: OgGemm.cluster_k = 2, 4 or 8 with use_2cta = 0 makes that many CTAs of one
 * thread-block cluster share every output tile, each taking a contiguous slice of K; the
 * slices' accumulators meet in the shared memory of the cluster's first CTA (distributed
 * shared memory, no trip through global memory), which stores the tile.  For shapes with
 * fewer tiles than SMs (small M, decode).  The reference's cluster_k planes add into a
 * zeroed C with atomics instead (opengemm/src/mm/kernel.cuh:29-36,86-96).  The request is
 * lowered to what fits: no more ways than K blocks, and the landing zone of
 * (cluster_k - 1) x tile width x 512 bytes must leave a three-stage ring. */

/* The native tile plan of a bound GEMM, for tuners and reports. */
typedef struct {
  int32_t cta_group; /* CTAs per MMA: 1 or 2 */
  int32_t tile_m, tile_n, block_k, stages;
  int32_t swap;      /* operands exchanged: B rows ride the 128-row MMA side */
  int32_t epi_staged; /* epilogue stages rows in shared memory and stores whole 128-byte lines */
  int32_t epi_tma;    /* ... and they leave by TMA store (32-bit output behind a long K loop) */
  int32_t acc_slots; /* accumulator buffers in tensor memory */
  int32_t tmem_cols, smem_bytes;
  int32_t tiles, grid; /* output tiles; CTAs launched */
  int32_t group;     /* rasterisation band width in tiles */
  int32_t stream_k;  /* partial wave cut along K across clusters (split_k >= 2) */
  int32_t use_clc;   /* tiles handed out by cluster launch control; grid = one cluster per tile */
  int32_t fixed_shape; /* served by a kernel compiled for exactly this tile shape (og_b200_set_fixed_kernels) */
  int32_t cluster_k; /* CTAs of a cluster sharing each tile along K (OgGemm.cluster_k with use_2cta = 0), else 1 */
  int32_t plain;     /* served by the build of the run-time-shaped kernel that has no optional feature compiled in */
} OgPlan;

/* Describe how `g` (already bound by og_mm_bind / og_smm_bind) would run on `device`
 * (pass -1 for "assume 148 SMs", which needs no GPU). */
OG_API int32_t og_b200_plan(const OgGemm* g, int32_t device, OgPlan* out);

/* Launch like og_mm_launch / og_smm_launch (chosen by g->dtype) with a device status
 * word: `status` points to a zero-initialised int32 in device-accessible memory.  A wait
 * that gives up stores (site | cta << 8) there instead of spinning forever; the kernel
 * then leaves through its ordinary teardown and the context stays usable.  Read the word
 * back after synchronising and hand it to og_b200_status. */
OG_API int32_t og_b200_launch_checked(const OgGemm* g, const void* a, const void* b,
                                      const void* sfa, const void* sfb, void* c, int32_t device,
                                      void* stream, int32_t* status);

/* Turns the status word of og_b200_launch_checked into a return code: OG_OK for 0,
 * else OG_ERR_TIMEOUT with og_mm_error() naming the wait (which role, which CTA). */
OG_API int32_t og_b200_status(int32_t status_word);

/* Launch like og_mm_launch / og_smm_launch (chosen by g->dtype) with every output
 * multiplied by `alpha` in float32 before it is stored (the product of per-tensor
 * dequantisation scales of fp8 / fp4 operands, for instance).  Float formats only:
 * s8 and u8 answer OG_ERR_LAUNCH. */
OG_API int32_t og_b200_launch_alpha(const OgGemm* g, const void* a, const void* b,
                                    const void* sfa, const void* sfb, void* c, int32_t device,
                                    void* stream, float alpha);

/* Output variant: C = alpha * (A . B^T) + bias, with `bias` a float32 device vector of
 * n values, one per column of C, added in float32 before the store (alpha = 1 adds the
 * bias only).  Float formats only.  The reference's epilogues store the bare product
 * (opengemm/src/mm/kernel.cuh:410-596, opengemm/src/smm/kernel.cuh:374-598). */
OG_API int32_t og_b200_launch_bias(const OgGemm* g, const void* a, const void* b,
                                   const void* sfa, const void* sfb, void* c, int32_t device,
                                   void* stream, float alpha, const void* bias);

/* Output variant: C leaves block-scaled - quantised along N exactly as the reference's
 * quantize (opengemm/python/quant.py:99-122) followed by to_blocked (quant.py:82-97) would
 * quantise a bfloat16 C - so that it can be the A operand of the next block-scaled GEMM
 * without a round trip through memory in bfloat16.  `out_format` is "nvfp4", "mxfp8" or
 * "mxfp4"; `c_packed` receives m x n/2 bytes (fp4) or m x n bytes (mxfp8), row-major;
 * `c_scales` the 128x4 blocked scales (ceil(m/128)*128 x ceil(n/(4*block))*4 bytes; rows past
 * m are left untouched).  g->dtype must be a block-scaled format or a "<format>.bf16" name;
 * n a multiple of 64, the tile width a multiple of 64, swap_ab 0.  The reference's
 * epilogues write bfloat16 or float32 only (opengemm/src/smm/kernel.cuh:374-598). */
OG_API int32_t og_b200_launch_quantized(const OgGemm* g, const void* a, const void* b,
                                        const void* sfa, const void* sfb, void* c_packed,
                                        void* c_scales, int32_t device, void* stream,
                                        const char* out_format);

/* Do now what launches on `device` do on first use: opt every kernel into its shared
 * memory and allocate the stream-K workspaces.  Call it before capturing launches into
 * a CUDA graph, or to keep the first request of a server free of allocations. */
OG_API int32_t og_b200_prepare_device(int32_t device);

/* The order a bound `g` visits its output tiles in: writes (M index, N index) pairs for
 * tile 0, 1, ... into `out` (room for `cap` integers) and returns the number of tiles,
 * or a negative status.  Needs no GPU. */
OG_API int32_t og_b200_tile_order(const OgGemm* g, int32_t* out, int32_t cap);

/* Testing aid.  The calling thread's next launch credits `bytes` more to each of its
 * stage barriers than its loads deliver, so the first wait for data runs out after the
 * limit of og_b200_set_wait_limit_ms and the launch reports it through its status word.
 * Nothing faults and nothing spins without bound. */
OG_API void og_b200_test_overcredit_next_launch(int32_t bytes);

/* The complete tile plan of a bound `g` for a device of `sm_count` SMs, as one JSON
 * object of integers written to `out` (what the standalone-kernel emitter bakes
 * into the code it writes).  Needs no GPU. */
OG_API int32_t og_b200_describe(const OgGemm* g, int32_t sm_count, char* out, int32_t cap);

/* Block-scaled quantisation on the GPU, the step upstream of every block-scaled GEMM:
 * `x` ([rows, k] bfloat16, or float32 when x_is_f32) -> `packed` (the operand in the
 * format's storage: k/2 bytes per row for nvfp4 / mxfp4, k for mxfp8), `scales`
 * ([rows, k/block] bytes, row-major; may be null) and `scales_blocked` (the 128x4
 * blocked layout og_smm_launch reads, ceil(rows/128)*128 x ceil(k/(4*block))*4 bytes;
 * may be null).  Same arithmetic, bit for bit, as the reference's torch helper
 * (opengemm/python/quant.py:99-122 followed by to_blocked, quant.py:82-97), in one
 * pass.  `format` is "nvfp4", "mxfp8" or "mxfp4".  Errors: og_b200_quantize_error(). */
OG_API int32_t og_b200_quantize(const char* format, const void* x, int32_t x_is_f32, int64_t rows,
                                int64_t k, void* packed, void* scales, void* scales_blocked,
                                int32_t device, void* stream);
OG_API const char* og_b200_quantize_error(void);

/* Launches use programmatic dependent launch: the next kernel of a stream may start
 * while this one drains.  By default every global-memory access of a kernel first
 * waits for the previous kernel to complete, so chained GEMMs (C of one feeding the
 * next) are safe.  With `yes` != 0 the caller vouches, process-wide, that no earlier
 * kernel in the stream writes the A / B / scale operands of a launch (weights and
 * inputs already resident, as in a benchmark loop): operand loads then start without
 * waiting, and only the stores wait - which is the only mode the reference has
 * (opengemm/src/mm/kernel.cuh:209,479-483).  Default 0. */
OG_API void og_b200_set_independent_inputs(int32_t yes);

/* Specialised builds of the kernel.  The hot tile shapes (pairs of CTAs on 256-row tiles,
 * the decode tile) also exist as kernels compiled for that one shape, with the plan's
 * constants folded in; and every variant exists once more with a run-time tile shape but
 * none of the optional features (stream-K, cluster launch control, cluster-K, bias, alpha,
 * half or block-scaled output, the non-default tile walks) compiled in, which is what a
 * launch that asks for none of them runs when no fixed-shape kernel matches its plan: a
 * GEMM of a tile or two per CTA runs its code once, from a cold instruction cache, and is
 * timed by the amount of code on its path.  All builds compute the same bits.  `yes` = 0
 * sends every launch to the full run-time kernel (default 1; the environment variable
 * OPENGEMM_FIXED=0 sets the default to 0). */
OG_API void og_b200_set_fixed_kernels(int32_t yes);

/* Limit of every device-side wait in milliseconds (default 2000).  Waits for a whole
 * accumulator, which sit behind a K loop of the others, allow twice as long. */
OG_API void og_b200_set_wait_limit_ms(int32_t ms);

/* No counterpart in the reference.  The same launch as og_mm_launch / og_smm_launch
 * (by g->dtype; bind `g` first) for callers that must not allocate device memory
 * inside a launch: processes that fixed their memory budget at start-up, code
 * running under an allocator that owns the rest of the GPU, latency-critical loops
 * that cannot absorb cudaMalloc's implicit device synchronisation.  It runs the
 * stream-K schedule out of a fixed workspace that is part of the library image
 * (about 18.5 MiB held by every GPU that loads the library, until exit) and calls
 * no allocating routine.  Limits: grids of at most 148 CTAs (a device needing more
 * partial-sum regions is refused with OG_ERR_LAUNCH and a message); one call at a
 * time per device, because all calls share the workspace: kernels of two calls
 * that overlap on the GPU race.  The first call on each device looks up the
 * workspace's address on that device; make it before any stream capture.
 * `error_text` (may be null) receives up to `error_text_cap` bytes on failure. */
OG_API int32_t og_b200_launch_no_alloc(const OgGemm* g, const void* a, const void* b,
                                       const void* sfa, const void* sfb, void* c, int32_t device,
                                       void* stream, char* error_text, int32_t error_text_cap);

#ifdef __cplusplus
}
#endif
#endif /* OPENGEMM_B200_H */
