// One persistent, warp-specialised GEMM kernel for sm_100a that serves the
// dense formats and the block-scaled ones:  D[rows_m, rows_n] = X . Y^T with
// both operands K-major.
//
//   warp 0      TMA producer: one elected thread streams X/Y (and scale)
//               tiles into a ring of shared-memory stages
//   warp 1      owns tensor memory; one elected thread of the pair's leader
//               copies scale atoms into tensor memory and issues tcgen05.mma
//   warps 2-5   epilogue: tcgen05.ld the accumulator, convert, and store
//               either each thread its own row, or through a swizzled
//               staging buffer per warp from which every store instruction
//               writes four rows x 128 contiguous bytes (or, for 32-bit
//               output behind a long K loop, a TMA store takes the buffer)
//
// It takes the place of the reference's two kernels, mm_gemm_kernel
// (opengemm/src/mm/kernel.cuh:38-601) and smm_gemm_kernel
// (opengemm/src/smm/kernel.cuh:6-607).  Differences by design: the tile
// width, stage count, rasterisation and tensor-memory plan are run-time
// values carried in GemmParams (the instruction and matrix descriptors are
// register operands, so only the MMA kind and the pair size are compile
// time); scales travel in the same stage and on the same barrier as the
// operand tiles; a pair's CTAs each fetch every byte they need with plain
// TMA loads (no cluster multicast); every wait is bounded.
#pragma once

#include "ptx.cuh"
#include "quant_math.cuh"
#include "raster.h"
#ifndef OG_FIXED_PLAN
#include "plan.h"
#endif

namespace og {

constexpr int MAX_STAGES = 16;
constexpr int THREADS = 192;
constexpr int SWIZZLE_ALIGN = 1024;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows of one 128-byte swizzle row
constexpr int CLC_SLOTS = 3;             // answers in flight between the fastest and the slowest role
constexpr int CLC_READERS = 6;           // per CTA: producer, warp 1's thread, four epilogue warps

struct alignas(64) GemmParams {
  CUtensorMap map_x;    // MMA-M side operand, [rows_m, K]
  CUtensorMap map_y;    // MMA-N side operand, [rows_n, K]
  CUtensorMap map_d;    // output, boxes of 32 rows x 128 bytes (TMA-store epilogue only)
  CUtensorMap map_sfx;  // scales of the M side, blocked layout seen as [atoms*2, 256] bytes
  CUtensorMap map_sfy;  // scales of the N side
  void* d;              // output base pointer
  int* status;          // device word a timed-out wait reports into (may be null)
  unsigned long long wait_limit_ns;
  int rows_m, rows_n, k;  // extents in MMA terms (after any operand swap)
  int ldd;                // elements between consecutive output rows
  int transpose_out;      // 1: D is written transposed (MMA row -> output column)
  int tile_n;             // MMA N: multiple of 16, at most 256
  int block_k, mma_k;     // K values per stage and per MMA
  int k_blocks;           // stages of K per tile
  int stages;
  int x_bytes, y_bytes;   // shared-memory bytes of one stage's X and Y tiles (per CTA)
  int stage_bytes;        // stride between stages, a multiple of 1024
  int tx_bytes;           // bytes credited to a stage's barrier, whole pair
  int tiles_m, tiles_n, num_tiles, group;
  unsigned idesc;
  int acc_slots, acc_stride;   // accumulator ring in tensor memory
  int sf_col, sf_slots, sf_cols;  // scale ring in tensor memory
  int tmem_cols;
  int epi_staged;         // 1: rows staged in shared memory, stored as whole 128-byte lines; 0: each thread stores its own row
  int epi_tma;            // 1 (32-bit output, long K loops): the staged rows leave by TMA store instead of st.global
  int vec_ok;             // direct stores may use 16-byte vectors
  int sf_atoms;           // 512-byte scale atoms per stage per 128-row block
  int sf_yblocks;         // 128-row blocks of N-side scales per tile (1 or 2)
  int k_groups;           // atoms along K of the global scale buffers
  int pdl;                // 1: every global access waits for the previous grid; 2: only the stores do
                          // (the caller vouches that no earlier kernel of the stream writes the operands)
  // Stream-K: the (tile, K-block) units are dealt out in equal contiguous
  // ranges, so a range may begin or end inside a tile.  See WorkIter.
  int use_clc;            // tiles come from cluster launch control instead of a fixed stride
  int stream_k;
  int sk_clusters;        // clusters that share the partial wave's units (the rest only run whole tiles)
  int acc_int;            // accumulators are s32 (partials add as integers)
  int scale_out;          // 1: float accumulators are multiplied by `alpha` before they are stored
  float alpha;
  int epoch;              // this launch's tag in `flags` (never 0)
  float* partial;         // per epilogue warp: 32 rows x 256 columns of f32 partial sums
  int* flags;             // per epilogue warp: epoch of the partial it last published
  int walk;               // rasterisation order (og::Walk)
  int out_f16;            // 2-byte output is IEEE half instead of bfloat16
  const float* bias;      // float32 [columns of C], added to every row before the store; may be null
  // Block-scaled output (2-byte-output kernels only): C leaves quantised along
  // N, ready to be the A operand of the next block-scaled GEMM.  `d` then
  // receives the packed values and `out_scales` the 128x4 blocked scales.
  // Cluster-K (one-CTA MMAs only): `cluster_k` CTAs of a cluster share every
  // tile, each taking a contiguous slice of its K blocks; ranks above 0 send
  // their accumulators to rank 0's shared memory, which adds them and stores.
  int cluster_k;          // 1 off, else 2, 4 or 8
  int out_quant;          // 0 off, else 1 + QFormat: 1 nvfp4, 2 mxfp8, 3 mxfp4
  int out_k_groups;       // 512-byte scale atoms along N of `out_scales`
  uint8_t* out_scales;
};

// Second, unused kernel argument.  On B200 with driver 580 the host cost of
// cudaLaunchKernelEx depends on the size of the parameter block modulo 64: an
// empty kernel launches in 1.7 us per call with 416, 480, 544, ... 928 or 992
// bytes of parameters and in 2.0-2.2 us with any multiple of 64 from 448 to
// 1024 (measured back to back on three machines).  GemmParams is a multiple of
// 64 because tensor maps are 64-byte aligned; these 32 bytes move the block to
// the cheap residue, which is the difference a launch-bound GEMM sees.
struct LaunchPad {
  unsigned long long words[4];
};
static_assert((sizeof(GemmParams) + sizeof(LaunchPad)) % 64 == 32, "parameter block should be an odd multiple of 32 bytes");

// Tiles are visited in the order `walk` names (raster.h); the default is bands
// `group` tiles wide along N, N fastest inside a band, so concurrently running
// clusters share X rows and Y rows in L2.
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int tile) {
  return tile_coord_of(tile, p.tiles_m, p.tiles_n, p.group, p.walk);
}

// One piece of work for a cluster: K blocks [kb0, kb1) of an output tile.
struct Work {
  int tile, kb0, kb1;
};

// The sequence of work of one cluster; all three roles walk it identically.
//
// Static schedule: whole tiles cluster, cluster + clusters, ...
//
// Stream-K schedule: the whole waves of tiles are still dealt out statically
// (neighbouring clusters then work on neighbouring tiles, which keeps operand
// panels shared in L2).  Only the tiles of the last, partial wave are cut
// along K: their units u = tile * k_blocks + kb are split into `clusters`
// equal contiguous ranges, so such a tile is shared by two or more
// consecutive clusters.  The cluster holding a tile's first K blocks
// (kb0 == 0) finishes it: it adds the partial sums of the clusters after it
// and writes the output.  Every other sharer contributes: it publishes raw
// f32/s32 partial sums in its own workspace region and never waits, so the
// schedule cannot deadlock while all clusters are resident.  A range starts
// inside at most one tile, so a cluster contributes at most once per launch.
//
// Cluster launch control (use_clc): the grid has one cluster per tile; a
// running cluster takes over the tile of a cluster that has not started yet.
// The pair leader's producer thread asks for one at the start of every tile
// (clc_request); every role reads the answer when it finishes the tile
// (inside next).  In a pair the leader forwards the answer to its peer through
// distributed shared memory; nothing is multicast.
struct ClcState {
  uint32_t full, empty_leader, answers;  // barrier arrays and answer slots (shared-memory addresses)
  uint32_t rank;
  bool forwards;                          // this thread is the leader's producer
  bool arrives;                           // this thread reports having read an answer
  const WaitCtx* ctx;
};

struct WorkIter {
  int slice_kb0, slice_kb1;  // this CTA's K blocks of every tile (all of them unless cluster-K splits K)
  int stream_k, k_blocks, clusters, cluster, step;
  int tile, static_tiles;
  long long total, u, u_end;
  int use_clc, cta_group, answered;
  ClcState clc;
  // `clusters` below is the number of clusters that share the partial wave
  // (p.sk_clusters, at most the grid's); `step` is the grid's cluster count.
  __device__ __forceinline__ WorkIter(const GemmParams& p, int cluster_, int grid_clusters, int k_rank = 0) {
    stream_k = p.stream_k;
    k_blocks = p.k_blocks;
    slice_kb0 = p.cluster_k > 1 ? p.k_blocks * k_rank / p.cluster_k : 0;
    slice_kb1 = p.cluster_k > 1 ? p.k_blocks * (k_rank + 1) / p.cluster_k : p.k_blocks;
    step = grid_clusters;
    clusters = stream_k ? p.sk_clusters : grid_clusters;
    cluster = cluster_;
    tile = cluster_;
    static_tiles = stream_k ? (p.num_tiles / grid_clusters) * grid_clusters : p.num_tiles;
    total = 0, u = 0, u_end = 0;
    if (stream_k) {  // 64-bit divisions: kept off the static schedule's start-up path
      total = (long long)(p.num_tiles - static_tiles) * p.k_blocks;
      const bool shares = cluster_ < clusters;
      u = shares ? total * cluster_ / clusters : 0;
      u_end = shares ? total * (cluster_ + 1) / clusters : 0;
    }
    use_clc = 0;
    answered = -1;
  }
  __device__ __forceinline__ void enable_clc(const ClcState& state, int cta_group_) {
    use_clc = 1;
    cta_group = cta_group_;
    clc = state;
  }
  // Leader's producer, at the start of the tile it is about to load: ask for
  // the tile after it.  `answered` answers have been consumed so far, so
  // this is request number `answered`.
  __device__ __forceinline__ bool clc_request() {
    const int n = answered;
    const int slot = n % CLC_SLOTS;
    const uint32_t phase = (n / CLC_SLOTS) & 1;
    if (!mbar_wait(clc.empty_leader + 8 * slot, phase ^ 1, *clc.ctx, SITE_CLC)) return false;
    mbar_expect_tx(clc.full + 8 * slot, 16);
    clc_try_cancel(clc.answers + 16 * slot, clc.full + 8 * slot);
    return true;
  }
  __device__ __forceinline__ bool next_clc(Work& w) {
    if (answered < 0) {  // the tile this cluster was launched for
      answered = 0;
      w = {cluster, 0, k_blocks};
      return true;
    }
    const int n = answered;
    const int slot = n % CLC_SLOTS;
    const uint32_t phase = (n / CLC_SLOTS) & 1;
    if (!mbar_wait(clc.full + 8 * slot, phase, *clc.ctx, SITE_CLC)) return false;
    const uint4 answer = ld_shared_v4(clc.answers + 16 * slot);
    if (clc.forwards && cta_group == 2) {
      st_cluster_v4(map_to_cta(clc.answers + 16 * slot, 1), answer);
      mbar_arrive_cluster(map_to_cta(clc.full + 8 * slot, 1));
    }
    fence_async_smem();  // the slot's next answer arrives through the async proxy
    if (clc.arrives) {
      if (cta_group == 2) mbar_arrive_cluster(clc.empty_leader + 8 * slot);
      else mbar_arrive(clc.empty_leader + 8 * slot);
    }
    answered = n + 1;
    const int first_cta = clc_decode(answer);
    if (first_cta < 0) return false;
    w = {first_cta / cta_group, 0, k_blocks};
    return true;
  }
  __device__ __forceinline__ bool next(Work& w) {
    if (use_clc) return next_clc(w);
    if (tile < static_tiles) {
      w = {tile, slice_kb0, slice_kb1};
      tile += step;
      return true;
    }
    if (u >= u_end) return false;
    const int t = int(u / k_blocks);
    const int kb0 = int(u - (long long)t * k_blocks);
    const long long left = u_end - u;
    const int kb1 = left < k_blocks - kb0 ? kb0 + int(left) : k_blocks;
    w = {static_tiles + t, kb0, kb1};
    u += kb1 - kb0;
    return true;
  }
  // For the finisher of `w` (kb0 == 0, kb1 < k_blocks): the last cluster
  // after this one whose range starts inside the same tile.  Clusters in
  // between may hold an empty range (fewer units than clusters); has_work
  // tells which ones actually contribute.
  __device__ __forceinline__ int last_sharer(const Work& w) const {
    const long long tile_end = (long long)(w.tile - static_tiles + 1) * k_blocks;
    int last = cluster;
    for (int j = cluster + 1; j < clusters && total * j / clusters < tile_end; ++j) last = j;
    return last;
  }
  __device__ __forceinline__ bool has_work(int j) const {
    return total * (j + 1) / clusters > total * j / clusters;
  }
};

#ifndef OG_FIXED_PLAN
// Overwrite, in a local copy of the launch parameters, everything that
// follows from the tile shape alone with compile-time values (the same
// tile_shape() the host plans with), and switch off the options a kernel
// compiled for one shape does not serve: the compiler then folds loop bounds
// and address arithmetic and drops the unused paths.  The host launches such
// a kernel only for a plan whose fields equal these (kernels_fixed.cu).
template <int KIND, int CTA_GROUP, int OUT_BYTES, int FIXED_N, int FIXED_EPI>
struct FoldedShape {
  static constexpr int SMEM_BITS = KIND == KIND_F16 ? 16 : KIND == KIND_TF32 ? 32 : (KIND == KIND_MXF4 || KIND == KIND_NVF4) ? 4 : 8;
  static constexpr int SF_BLOCK = KIND == KIND_NVF4 ? 16 : kind_scaled(KIND) ? 32 : 0;
#define OG_FOLDED(field) \
  static constexpr int field = tile_shape(SMEM_BITS, SF_BLOCK, CTA_GROUP, OUT_BYTES, FIXED_N, FIXED_EPI).field
  OG_FOLDED(tile_n); OG_FOLDED(block_k); OG_FOLDED(mma_k); OG_FOLDED(stages);
  OG_FOLDED(x_bytes); OG_FOLDED(y_bytes); OG_FOLDED(stage_bytes);
  OG_FOLDED(acc_slots); OG_FOLDED(acc_stride); OG_FOLDED(sf_col); OG_FOLDED(sf_slots); OG_FOLDED(sf_cols);
  OG_FOLDED(tmem_cols); OG_FOLDED(sf_atoms); OG_FOLDED(sf_yblocks); OG_FOLDED(epi_staged); OG_FOLDED(epi_tma);
#undef OG_FOLDED
};

template <int KIND, int CTA_GROUP, int OUT_BYTES, int FIXED_N, int FIXED_EPI>
__device__ __forceinline__ void fold_tile_shape(GemmParams& p) {
  using T = FoldedShape<KIND, CTA_GROUP, OUT_BYTES, FIXED_N, FIXED_EPI>;
  p.tile_n = T::tile_n, p.block_k = T::block_k, p.mma_k = T::mma_k, p.stages = T::stages;
  p.x_bytes = T::x_bytes, p.y_bytes = T::y_bytes, p.stage_bytes = T::stage_bytes;
  p.acc_slots = T::acc_slots, p.acc_stride = T::acc_stride;
  p.sf_col = T::sf_col, p.sf_slots = T::sf_slots, p.sf_cols = T::sf_cols, p.tmem_cols = T::tmem_cols;
  p.sf_atoms = T::sf_atoms, p.sf_yblocks = T::sf_yblocks;
  p.epi_staged = T::epi_staged, p.epi_tma = T::epi_tma;
  p.transpose_out = 0, p.vec_ok = 1, p.walk = 0;
  p.use_clc = 0, p.stream_k = 0, p.scale_out = 0, p.out_f16 = 0, p.out_quant = 0, p.cluster_k = 1;
  p.bias = nullptr;
}

// What a launch without any optional feature leaves unused: folding these to
// constants removes the stream-K, cluster launch control, cluster-K, bias,
// scaling, half and block-scaled output code and all tile walks but the
// default from the kernel.  The tile shape stays a run-time value.
__device__ __forceinline__ void fold_features_off(GemmParams& p) {
  p.walk = 0, p.use_clc = 0, p.stream_k = 0, p.scale_out = 0, p.out_f16 = 0, p.out_quant = 0, p.cluster_k = 1;
  p.bias = nullptr;
}
#endif

// FIXED_N == 0: every tile-plan value is read from `params` at run time.
// FIXED_N != 0: the kernel is compiled for tiles FIXED_N wide with epilogue
// path FIXED_EPI (0 each thread its own row, 1 staged rows, 2 TMA stores).
// PLAIN: compiled without the optional features (fold_features_off).  A GEMM
// of one or two tiles per CTA executes most of its instructions once, straight
// from a cold instruction cache, so its time follows the amount of code on
// the path it takes: bf16 128^3 spends 2.2 us between the previous grid's
// completion and its own in the full kernel, 1.5 us in the plain one and
// 1.0 us in one compiled for its tile shape.
template <int KIND, int CTA_GROUP, int OUT_BYTES, int FIXED_N = 0, int FIXED_EPI = 0, bool PLAIN = false>
__global__ void __launch_bounds__(THREADS, 1) gemm_kernel(const __grid_constant__ GemmParams params, const LaunchPad) {
  // `p` is the scalar view of the launch parameters.  A standalone kernel
  // emitted for one shape defines OG_FIXED_PLAN to overwrite the plan fields
  // of a local copy with literals, which lets the compiler fold them; tensor
  // maps are always addressed in `params`, where TMA needs them.
#ifdef OG_FIXED_PLAN
  GemmParams p = params;
  OG_FIXED_PLAN(p);
#else
  GemmParams folded;
  const GemmParams* view = &params;
  if constexpr (FIXED_N != 0) {
    folded = params;
    fold_tile_shape<KIND, CTA_GROUP, OUT_BYTES, FIXED_N, FIXED_EPI>(folded);
    view = &folded;
  } else if constexpr (PLAIN) {
    folded = params;
    fold_features_off(folded);
    view = &folded;
  }
  const GemmParams& p = *view;
#endif
  constexpr bool SCALED = kind_scaled(KIND);
  constexpr int TILE_M = 128 * CTA_GROUP;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 4 + 2 * CLC_SLOTS + 1 + 8];
  __shared__ __align__(16) uint4 clc_answers[CLC_SLOTS];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (CTA_GROUP == 2) ? cluster_cta_rank() : 0u;
  // Cluster-K: `cluster_k` one-CTA MMAs form a cluster that shares each tile along K.
  const int cluster_k = (CTA_GROUP == 1 && p.cluster_k > 1) ? p.cluster_k : 1;
  const int k_rank = cluster_k > 1 ? int(cluster_cta_rank()) : 0;
  const int cluster_id = blockIdx.x / (CTA_GROUP * cluster_k);
  const int num_clusters = gridDim.x / (CTA_GROUP * cluster_k);

  const uint32_t ring = (smem_u32(dyn_smem) + SWIZZLE_ALIGN - 1) & ~uint32_t(SWIZZLE_ALIGN - 1);
  const uint32_t epi_base = ring + p.stages * p.stage_bytes;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * MAX_STAGES;
  const uint32_t bar_acc_full = bar_empty + 8 * MAX_STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  const uint32_t bar_clc_full = bar_acc_empty + 16;
  const uint32_t bar_clc_empty = bar_clc_full + 8 * CLC_SLOTS;
  const uint32_t bar_tmem = bar_clc_empty + 8 * CLC_SLOTS;  // tensor memory of every CTA of the pair is allocated
  const uint32_t bar_ck_partial = bar_tmem + 8;    // rank 0, per epilogue warp: the other ranks' partial sums have arrived
  const uint32_t bar_ck_free = bar_ck_partial + 32;  // ranks above 0, per epilogue warp: rank 0 has consumed them
  // Rank 0's landing zone for the other ranks' accumulators, behind the epilogue's staging buffers.
  const uint32_t ck_buffer = epi_base + (p.epi_staged ? 4 * (p.epi_tma ? 2 : 1) * EPI_BUF_BYTES : 0);

  const WaitCtx ctx{&abort_flag, p.status, p.wait_limit_ns};

  // Set-up is ordered for a short critical path: the tensor maps are requested
  // first (their fetch overlaps the rest), only the barriers are synchronised
  // on, and the producer starts loading while warp 1 is still allocating
  // tensor memory - its users wait for that on a barrier of its own.
  if (threadIdx.x == 0) {
    prefetch_tmap(&params.map_x);
    prefetch_tmap(&params.map_y);
    if constexpr (SCALED) {
      prefetch_tmap(&params.map_sfx);
      prefetch_tmap(&params.map_sfy);
    }
    if (p.epi_tma) prefetch_tmap(&params.map_d);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 4 * CTA_GROUP);
    }
    if (p.use_clc) {
      for (int s = 0; s < CLC_SLOTS; ++s) {
        mbar_init(bar_clc_full + 8 * s, 1);  // leader: the answer's 16 bytes; peer: the leader's forward
        mbar_init(bar_clc_empty + 8 * s, CLC_READERS * CTA_GROUP);
      }
    }
    mbar_init(bar_tmem, CTA_GROUP);
    if (cluster_k > 1) {
      for (int q = 0; q < 4; ++q) {
        mbar_init(bar_ck_partial + 8 * q, cluster_k - 1);
        mbar_init(bar_ck_free + 8 * q, 1);
      }
    }
    abort_flag = 0;
    mbar_init_fence();
  }
  __syncthreads();
  if (CTA_GROUP == 2 || cluster_k > 1) cluster_sync_all();
  if (warp == 1) {
    tmem_alloc<CTA_GROUP>(smem_u32(&tmem_slot), p.tmem_cols);
    tmem_relinquish<CTA_GROUP>();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {  // tell this CTA and, in a pair, the other one
      mbar_arrive(bar_tmem);
      if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(map_to_cta(bar_tmem, rank ^ 1u));
    }
  }
  // Programmatic dependent launch: from here on the next kernel in the stream
  // may start its own set-up on SMs this grid leaves free.  Every thread of
  // this grid that touches global memory first waits for the previous grid.
  if (p.pdl && threadIdx.x == 0) pdl_launch_dependents();
  const uint32_t clc_empty_leader = (CTA_GROUP == 2) ? map_to_cta(bar_clc_empty, 0) : bar_clc_empty;
  auto clc_state = [&](bool forwards, bool arrives) {
    return ClcState{bar_clc_full, clc_empty_leader, smem_u32(clc_answers), rank, forwards, arrives, &ctx};
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // One thread; the loop body is kept to a handful of instructions per
    // stage (ring position and phase advance by increment, never by division).
    if (elect_one()) {
      if (p.pdl == 1) pdl_wait_prior_grids();
      // Plan values used every stage live in registers: the inline PTX below
      // clobbers memory, which would otherwise force a constant-bank reload
      // of each p.field per iteration.
      const int stages = p.stages, block_k = p.block_k;
      const uint32_t stage_bytes = p.stage_bytes, x_bytes = p.x_bytes, tx_bytes = p.tx_bytes;
      const bool two_sfy = p.sf_yblocks == 2;
      const int y_rows = p.tile_n / CTA_GROUP;
      const uint32_t sfx_off = p.x_bytes + p.y_bytes;
      const uint32_t sf_block_bytes = p.sf_atoms * 512;
      const int sf_step = 2 * p.sf_atoms;       // tensor-map rows of scales per stage
      const int sf_block_step = 2 * p.k_groups; // rows between consecutive 128-row blocks
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      WorkIter work(p, cluster_id, num_clusters, k_rank);
      if (p.use_clc) work.enable_clc(clc_state(rank == 0, true), CTA_GROUP);
      Work w;
      while (ok && work.next(w)) {
        if (p.use_clc && rank == 0 && !work.clc_request()) break;
        const TileCoord t = tile_coord(p, w.tile);
        const int row_x = t.mi * TILE_M + int(rank) * 128;
        const int row_y = t.ni * p.tile_n + int(rank) * y_rows;
        int sfx_row = 2 * (row_x >> 7) * p.k_groups + w.kb0 * sf_step;
        int sfy_row = 2 * ((t.ni * p.tile_n) >> 7) * p.k_groups + w.kb0 * sf_step;
        int kx = w.kb0 * block_k;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, ctx, SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full_local = bar_full + 8 * stage;
          const uint32_t full = (CTA_GROUP == 2) ? map_to_cta(full_local, 0) : full_local;
          if (rank == 0) mbar_expect_tx(full_local, tx_bytes);
          const uint32_t sx = ring + stage * stage_bytes;
          tma_load_2d<CTA_GROUP>(sx, &params.map_x, kx, row_x, full);
          tma_load_2d<CTA_GROUP>(sx + x_bytes, &params.map_y, kx, row_y, full);
          if constexpr (SCALED) {
            const uint32_t ssfx = sx + sfx_off;
            tma_load_2d<CTA_GROUP>(ssfx, &params.map_sfx, 0, sfx_row, full);
            tma_load_2d<CTA_GROUP>(ssfx + sf_block_bytes, &params.map_sfy, 0, sfy_row, full);
            if (two_sfy)
              tma_load_2d<CTA_GROUP>(ssfx + 2 * sf_block_bytes, &params.map_sfy, 0,
                                     sfy_row + sf_block_step, full);
            sfx_row += sf_step;
            sfy_row += sf_step;
          }
          kx += block_k;
          ++issued;
          if (++stage == stages) stage = 0, phase ^= 1;
        }
      }
      if (!ok && rank == 0) {
        // Loads already issued still land in this CTA's stages: give each
        // armed barrier a bounded chance to complete before teardown.
        int s = stage;
        uint32_t ph = phase;
        const uint32_t pending = issued < uint32_t(p.stages) ? issued : uint32_t(p.stages);
        for (uint32_t back = 0; back < pending; ++back) {
          if (--s < 0) s = p.stages - 1, ph ^= 1;
          const uint64_t start = global_timer_ns();
          while (!mbar_try_wait(bar_full + 8 * s, ph) && global_timer_ns() - start < 1000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // One thread of the pair's leader.  Descriptors advance by addition; the
    // scale copies and the four MMAs of a stage are fully unrolled.
    if (rank != 0) {
      if (p.use_clc && elect_one()) {  // the peer's idle warp still reads every answer
        WorkIter work(p, cluster_id, num_clusters, k_rank);
        work.enable_clc(clc_state(false, true), CTA_GROUP);
        Work w;
        while (work.next(w)) {
        }
      }
    } else if (elect_one()) {
      constexpr int SF_ATOMS = KIND == KIND_NVF4 ? 4 : KIND == KIND_MXF4 ? 2 : 1;
      const uint64_t desc_stage = uint64_t(p.stage_bytes >> 4);
      const uint64_t dx0 = operand_desc(ring);
      const uint64_t dy0 = operand_desc(ring + p.x_bytes);
      const uint64_t dsf0 = scale_desc(ring + p.x_bytes + p.y_bytes);
      const bool two_yblocks = p.sf_yblocks == 2;
      const int yb = p.sf_yblocks;
      const int stages = p.stages, block_k = p.block_k, mma_k = p.mma_k, k_total = p.k;
      const uint32_t idesc = p.idesc, acc_stride = p.acc_stride, sf_cols = p.sf_cols;
      const bool two_acc = p.acc_slots == 2, two_sf = p.sf_slots == 2;
      int stage = 0;
      uint32_t phase = 0;
      uint64_t stage_off = 0;  // stage * (stage_bytes >> 4)
      uint32_t sf_slot = 0;
      int tile_idx = 0;
      bool ok = mbar_wait(bar_tmem, 0, ctx, SITE_TMEM_READY);  // both CTAs' allocations
      tc_fence_after_sync();
      const uint32_t tmem_base = tmem_slot;
      const uint32_t sf_base = tmem_base + p.sf_col;
      WorkIter work(p, cluster_id, num_clusters, k_rank);
      if (p.use_clc) work.enable_clc(clc_state(false, true), CTA_GROUP);
      Work w;
      for (; ok && work.next(w); ++tile_idx) {
        const int slot = two_acc ? (tile_idx & 1) : 0;
        const uint32_t use = two_acc ? (tile_idx >> 1) : tile_idx;
        if (!mbar_wait(bar_acc_empty + 8 * slot, (use & 1) ^ 1, ctx, SITE_MMA_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + slot * acc_stride;
        uint32_t sfy_shift = 0;
        if constexpr (SCALED) {
          const TileCoord t = tile_coord(p, w.tile);
          sfy_shift = ((t.ni * p.tile_n) & 127) >> 5;  // tile origin inside its 128-row scale block
        }
        uint32_t accumulate = 0;
        int k_left = k_total - w.kb0 * block_k;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, ctx, SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          // No tcgen05 fence here: the stage was written by TMA (async proxy)
          // and is read by tcgen05.mma / cp through the same proxy, ordered by
          // the barrier's completion.
          uint32_t sfx_tmem = 0, sfy_tmem = 0;
          if constexpr (SCALED) {
            sfx_tmem = sf_base + sf_slot * sf_cols;
            sfy_tmem = sfx_tmem + 4 * SF_ATOMS;
            const uint64_t dsf = dsf0 + stage_off;
#pragma unroll
            for (int w = 0; w < SF_ATOMS; ++w) {
              scale_copy<CTA_GROUP>(sfx_tmem + 4 * w, dsf + 32 * w);
              scale_copy<CTA_GROUP>(sfy_tmem + 4 * w * yb, dsf + 32 * (SF_ATOMS + w));
              if (two_yblocks)
                scale_copy<CTA_GROUP>(sfy_tmem + 4 * w * yb + 4, dsf + 32 * (2 * SF_ATOMS + w));
            }
            sf_slot = two_sf ? (sf_slot ^ 1) : 0;
          }
          const uint64_t dx = dx0 + stage_off;
          const uint64_t dy = dy0 + stage_off;
#pragma unroll
          for (int ki = 0; ki < 4; ++ki) {
            // Past the end of K a stage holds TMA's zero fill; an MMA that
            // would read only that is skipped.  Each MMA covers 32 bytes of
            // every row, two 16-byte units of the descriptor's start field.
            if (ki == 0 || ki * mma_k < k_left) {
              if constexpr (SCALED) {
                constexpr int NVF4 = KIND == KIND_NVF4, MXF4 = KIND == KIND_MXF4;
                const int atom = NVF4 ? ki : MXF4 ? (ki >> 1) : 0;
                const uint32_t id = NVF4 ? 0u : MXF4 ? uint32_t((ki & 1) * 2) : uint32_t(ki);
                mma_scaled<KIND, CTA_GROUP>(d_tmem, dx + 2 * ki, dy + 2 * ki,
                                            idesc | (id << 29) | (id << 4), sfx_tmem + 4 * atom,
                                            sfy_tmem + 4 * atom * yb + sfy_shift, accumulate);
              } else {
                mma_dense<KIND, CTA_GROUP>(d_tmem, dx + 2 * ki, dy + 2 * ki, idesc, accumulate);
              }
              accumulate = 1;
            }
          }
          mma_commit<CTA_GROUP>(bar_empty + 8 * stage);
          k_left -= block_k;
          stage_off += desc_stage;
          if (++stage == stages) stage = 0, phase ^= 1, stage_off = 0;
        }
        if (ok) mma_commit<CTA_GROUP>(bar_acc_full + 8 * slot);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t acc_empty_leader =
        (CTA_GROUP == 2) ? map_to_cta(bar_acc_empty, 0) : bar_acc_empty;
    // One staging buffer per warp; two when they drain by TMA store, which
    // reads a buffer asynchronously while the next one is filled.
    const bool tma_out = p.epi_tma != 0;
    const uint32_t my_buf = epi_base + (warp - 2) * (tma_out ? 2 : 1) * EPI_BUF_BYTES;
    int buf_use = 0;
    constexpr int CHUNK = (OUT_BYTES == 2) ? 64 : 32;  // columns per 128-byte staging row
    constexpr int UNIT = 16 / OUT_BYTES;               // columns per 16-byte unit of a row
    // A store instruction of the staged path writes four rows x 128 contiguous
    // bytes: this lane's row of the four and its 16-byte unit of the eight.
    const int sub_row = lane >> 3, unit = lane & 7;
    bool touched_memory = false;
    const int tile_n = p.tile_n, rows_m = p.rows_m, rows_n = p.rows_n, ldd = p.ldd;
    const bool staged = p.epi_staged != 0, transpose_out = p.transpose_out != 0, vec_ok = p.vec_ok != 0;
    uint8_t* const out = static_cast<uint8_t*>(p.d);
    const bool scale_out = p.scale_out != 0;  // scaled or biased output takes the general loop below
    const float alpha = p.alpha;
    const float* const bias = p.bias;
    const bool out_f16 = p.out_f16 != 0;
    auto pack2 = [&](uint32_t lo, uint32_t hi) {
      return out_f16 ? pack_f16x2(__uint_as_float(lo), __uint_as_float(hi))
                     : pack_bf16x2(__uint_as_float(lo), __uint_as_float(hi));
    };
    int tile_idx = 0;
    const bool allocated = mbar_wait(bar_tmem, 0, ctx, SITE_TMEM_READY);
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    // Stream-K bookkeeping: this warp's region of the partial-sum workspace
    // and its neighbour's (the same warp of the next cluster).
    const int my_region = (cluster_id * CTA_GROUP + int(rank)) * 4 + quarter;
    int last_sharer = 0;  // last cluster after this one that shares the tile being finished
    WorkIter work(p, cluster_id, num_clusters, k_rank);
    if (p.use_clc) work.enable_clc(clc_state(false, lane == 0), CTA_GROUP);
    Work w;
    for (; __all_sync(0xFFFFFFFFu, allocated) && work.next(w); ++tile_idx) {
      const TileCoord t = tile_coord(p, w.tile);
      // Stream-K roles (a cluster-K rank also holds a K slice, but exchanges it through shared memory below).
      const bool contributes = p.stream_k && w.kb0 > 0;          // publish partial sums instead of output
      const bool finishes = p.stream_k && w.kb0 == 0 && w.kb1 < p.k_blocks;  // add the sharers' partials before storing
      const int slot = (p.acc_slots == 2) ? (tile_idx & 1) : 0;
      const uint32_t use = (p.acc_slots == 2) ? (tile_idx >> 1) : tile_idx;
      const bool ready = mbar_wait(bar_acc_full + 8 * slot, use & 1, ctx, SITE_EPI_ACC_FULL);
      if (!__all_sync(0xFFFFFFFFu, ready)) break;
      tc_fence_after_sync();
      // The previous grid is waited for as late as possible: by whichever path
      // below first touches global memory, with its accumulators already in
      // registers where it can.
      auto before_global_memory = [&] {
        if (p.pdl && !touched_memory) pdl_wait_prior_grids();
        touched_memory = true;
      };

      const int row0 = t.mi * TILE_M + int(rank) * 128 + quarter * 32;  // first row of this warp
      const int row = row0 + lane;
      const int col0 = t.ni * tile_n;
      const uint32_t acc_tmem = tmem_base + lane_base + slot * p.acc_stride;

      // Staged output: each lane writes its row's 128 bytes (32 words `w`, the
      // first `width` columns valid) into the warp's buffer with the 16-byte
      // units XOR-swizzled by row, then the warp reads the buffer back four
      // rows at a time and stores whole 128-byte segments, clipped at the
      // edges of D.  Plain st.global: nothing to wait for before the buffer
      // is reused but the warp's own reads.
      auto store_staged = [&](const uint32_t* w, int c, int width) {
        const uint32_t rowaddr = my_buf + lane * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (u * UNIT < width)
            st_shared_v4(rowaddr + ((u ^ (lane & 7)) << 4), w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
        __syncwarp();
        const int gcol = col0 + c + unit * UNIT;
        if (unit * UNIT < width && gcol < rows_n) {
          uint8_t* dst = out + (size_t(row0 + sub_row) * ldd + gcol) * OUT_BYTES;
          const size_t step = size_t(4) * ldd * OUT_BYTES;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + sub_row;
            if (row0 + r < rows_m)
              *reinterpret_cast<uint4*>(dst + i * step) = ld_shared_v4(my_buf + r * 128 + ((unit ^ (r & 7)) << 4));
          }
        }
        __syncwarp();
      };

      // The same staged block handed to a TMA store, which clips it at the edges
      // of D: the fewest instructions, the least power on a capped part, and
      // more bytes in flight per SM than its own stores manage.  Two buffers
      // alternate; a buffer is refilled once the store issued from it two
      // blocks ago has read it.
      auto store_rows = [&](const uint32_t* w, int c, int width) {
        if (!tma_out || width != CHUNK) {
          if (tma_out) {  // the plain path reuses the first buffer
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          store_staged(w, c, width);
          return;
        }
        const uint32_t buf = my_buf + (buf_use & 1) * EPI_BUF_BYTES;
        if (buf_use >= 2) {
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
        ++buf_use;
        const uint32_t rowaddr = buf + lane * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          st_shared_v4(rowaddr + ((u ^ (lane & 7)) << 4), w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&params.map_d, buf, col0 + c, row0);
          tma_store_commit();
        }
      };

      // A 256-wide block-scaled tile leaves tensor memory no room for a second
      // accumulator, so the MMA warp idles until this one is handed back.  The
      // hand-back therefore comes as early as possible: the first two 64-column
      // chunks are stored while the loads of the next chunk are in flight, the
      // last two are packed to bf16 and held in registers, the accumulator is
      // released, and only then are the held chunks stored.
      bool handed_back = false, handed_back_late = false;
      if constexpr (OUT_BYTES == 2) {
        if (p.acc_slots == 1 && staged && tile_n == 256 && !contributes && !finishes && !scale_out && !bias && !out_f16 &&
            !p.out_quant && cluster_k == 1 && row0 < rows_m) {
          auto pack64 = [](const uint32_t* f, uint32_t* w) {
#pragma unroll
            for (int u = 0; u < 32; ++u)
              w[u] = pack_bf16x2(__uint_as_float(f[2 * u]), __uint_as_float(f[2 * u + 1]));
          };
          uint32_t va[64], vb[64], held[64];
          tmem_ld_32(acc_tmem, va), tmem_ld_32(acc_tmem + 32, va + 32);
          tmem_ld_wait();
          tmem_ld_settle_32(va), tmem_ld_settle_32(va + 32);
          tmem_ld_32(acc_tmem + 64, vb), tmem_ld_32(acc_tmem + 96, vb + 32);
          pack64(va, held);
          before_global_memory();
          store_rows(held, 0, 64);
          tmem_ld_wait();
          tmem_ld_settle_32(vb), tmem_ld_settle_32(vb + 32);
          tmem_ld_32(acc_tmem + 128, va), tmem_ld_32(acc_tmem + 160, va + 32);
          pack64(vb, held);
          store_rows(held, 64, 64);
          tmem_ld_wait();
          tmem_ld_settle_32(va), tmem_ld_settle_32(va + 32);
          tmem_ld_32(acc_tmem + 192, vb), tmem_ld_32(acc_tmem + 224, vb + 32);
          pack64(va, held);
          tmem_ld_wait();
          tmem_ld_settle_32(vb), tmem_ld_settle_32(vb + 32);
          pack64(vb, held + 32);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(acc_empty_leader + 8 * slot);
            else mbar_arrive(bar_acc_empty + 8 * slot);
          }
          handed_back = true;
          store_rows(held, 128, 64);
          store_rows(held + 32, 192, 64);
        }
      }

      // A finisher first makes sure every sharer's partial sums are published,
      // then keeps the loads of the first sharer's next chunk in flight while
      // it works on the current one (32-bit output; two sharers is the common
      // cut), so the tile costs one L2 round trip rather than one per chunk.
      constexpr bool AHEAD = OUT_BYTES == 4;
      int first_sharer = 0;
      bool sharers_ready = true;
      if (finishes) {
        before_global_memory();
        last_sharer = work.last_sharer(w);
        for (int j = cluster_id + 1; j <= last_sharer && sharers_ready; ++j)
          if (work.has_work(j)) {
            if (!first_sharer) first_sharer = j;
            sharers_ready = wait_flag(p.flags + my_region + (j - cluster_id) * CTA_GROUP * 4, p.epoch, ctx);
          }
      }
      // Cluster-K hand-shake for this tile: a rank above 0 may overwrite its part
      // of rank 0's landing zone once rank 0 has consumed the previous tile's;
      // rank 0 may read once every other rank's partial sums have arrived.
      const bool ck_contributes = k_rank > 0, ck_finishes = cluster_k > 1 && k_rank == 0;
      const bool ck_live = row0 < rows_m;  // warps whose rows lie past the matrix exchange no data
      bool ck_ready = true;
      if (ck_contributes && tile_idx > 0)
        ck_ready = mbar_wait(bar_ck_free + 8 * quarter, (tile_idx - 1) & 1, ctx, SITE_CLUSTER_K);
      if (ck_finishes) ck_ready = mbar_wait(bar_ck_partial + 8 * quarter, tile_idx & 1, ctx, SITE_CLUSTER_K);
      if (!__all_sync(0xFFFFFFFFu, ck_ready)) sharers_ready = false;
      auto ck_slot = [&](int peer, int c) {  // 16-byte vector g of row `lane` sits at (g * 32 + lane)
        return ck_buffer + uint32_t((((peer * 4 + quarter) * (tile_n >> 2) + (c >> 2)) * 32 + lane) * 16);
      };
      auto partial_of = [&](int j, int c) {
        return reinterpret_cast<const uint4*>(p.partial) +
               (size_t(my_region + (j - cluster_id) * CTA_GROUP * 4) * 64 + (c >> 2)) * 32 + lane;
      };
      uint4 ahead[AHEAD ? CHUNK / 4 : 1];
      if (AHEAD && finishes && sharers_ready && first_sharer) {
        const uint4* src = partial_of(first_sharer, 0);
#pragma unroll
        for (int u = 0; u < CHUNK / 4; ++u) ahead[AHEAD ? u : 0] = (4 * u < tile_n) ? __ldcg(src + u * 32) : make_uint4(0u, 0u, 0u, 0u);
      }

      // 32-bit output: the loads of the next chunk are in flight while this
      // one is converted and stored (one chunk of registers ahead), so a tile's
      // drain costs the stores rather than stores plus tensor-memory latency -
      // which is what a launch-bound GEMM's tail, and every last tile, is made of.
      constexpr bool PIPELINED = OUT_BYTES == 4;
      auto chunk_live = [&](int c) { return c < tile_n && col0 + c < rows_n; };
      auto issue_loads = [&](int c, uint32_t* v) {
        const int width = min(CHUNK, tile_n - c);
        if (width >= 32) tmem_ld_32(acc_tmem + c, v);
        else tmem_ld_16(acc_tmem + c, v);
        if constexpr (CHUNK == 64) {
          if (width > 32) {
            if (width >= 64) tmem_ld_32(acc_tmem + c + 32, v + 32);
            else tmem_ld_16(acc_tmem + c + 32, v + 32);
          }
        }
      };
      const bool drains = !handed_back && sharers_ready;
      uint32_t coming[PIPELINED ? CHUNK : 1];
      if constexpr (PIPELINED) {
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) coming[j] = 0u;
        if (drains && chunk_live(0)) issue_loads(0, coming);
      }
      for (int c = 0; drains && chunk_live(c); c += CHUNK) {
        const int width = min(CHUNK, tile_n - c);
        const bool last_chunk = !chunk_live(c + CHUNK);
        uint32_t v[CHUNK];
        if constexpr (PIPELINED) {
          tmem_ld_wait();
          tmem_ld_settle_32(coming);
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) v[j] = coming[PIPELINED ? j : 0];
          if (!last_chunk) issue_loads(c + CHUNK, coming);
        } else {
          issue_loads(c, v);
          tmem_ld_wait();
        }
        if (last_chunk) {
          // The last columns are in registers: the accumulator goes back to
          // the MMA warp before they are converted and stored.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(acc_empty_leader + 8 * slot);
            else mbar_arrive(bar_acc_empty + 8 * slot);
          }
          handed_back_late = true;
        }
        before_global_memory();

        if (finishes) {
          // Partial sums of every cluster that shares this tile.
          for (int j = cluster_id + 1; j <= last_sharer; ++j) {
            if (!work.has_work(j)) continue;
            uint4 q[CHUNK / 4];
            if (AHEAD && j == first_sharer) {
#pragma unroll
              for (int u = 0; u < CHUNK / 4; ++u) q[u] = ahead[AHEAD ? u : 0];
              const int next = c + CHUNK;
              if (next < tile_n && col0 + next < rows_n) {  // the next chunk's loads go out before this one's sums are used
                const uint4* src = partial_of(j, next);
#pragma unroll
                for (int u = 0; u < CHUNK / 4; ++u)
                  ahead[AHEAD ? u : 0] = (4 * u < tile_n - next) ? __ldcg(src + u * 32) : make_uint4(0u, 0u, 0u, 0u);
              }
            } else {
              const uint4* src = partial_of(j, c);
#pragma unroll
              for (int u = 0; u < CHUNK / 4; ++u)
                q[u] = (4 * u < width) ? __ldcg(src + u * 32) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (p.acc_int) {
#pragma unroll
              for (int u = 0; u < CHUNK / 4; ++u)
                v[4 * u] += q[u].x, v[4 * u + 1] += q[u].y, v[4 * u + 2] += q[u].z, v[4 * u + 3] += q[u].w;
            } else {
#pragma unroll
              for (int u = 0; u < CHUNK / 4; ++u) {
                v[4 * u] = __float_as_uint(__uint_as_float(v[4 * u]) + __uint_as_float(q[u].x));
                v[4 * u + 1] = __float_as_uint(__uint_as_float(v[4 * u + 1]) + __uint_as_float(q[u].y));
                v[4 * u + 2] = __float_as_uint(__uint_as_float(v[4 * u + 2]) + __uint_as_float(q[u].z));
                v[4 * u + 3] = __float_as_uint(__uint_as_float(v[4 * u + 3]) + __uint_as_float(q[u].w));
              }
            }
          }
        }
        if (ck_finishes && ck_live) {
          for (int peer = 0; peer < cluster_k - 1; ++peer) {
            const uint32_t src = ck_slot(peer, c);
#pragma unroll
            for (int u = 0; u < CHUNK / 4; ++u) {
              if (4 * u >= width) continue;
              const uint4 q = ld_shared_v4(src + u * 512);
              if (p.acc_int) {
                v[4 * u] += q.x, v[4 * u + 1] += q.y, v[4 * u + 2] += q.z, v[4 * u + 3] += q.w;
              } else {
                v[4 * u] = __float_as_uint(__uint_as_float(v[4 * u]) + __uint_as_float(q.x));
                v[4 * u + 1] = __float_as_uint(__uint_as_float(v[4 * u + 1]) + __uint_as_float(q.y));
                v[4 * u + 2] = __float_as_uint(__uint_as_float(v[4 * u + 2]) + __uint_as_float(q.z));
                v[4 * u + 3] = __float_as_uint(__uint_as_float(v[4 * u + 3]) + __uint_as_float(q.w));
              }
            }
          }
        }
        if (ck_contributes) {
          if (ck_live) {
            const uint32_t dst = map_to_cta(ck_slot(k_rank - 1, c), 0);
#pragma unroll
            for (int u = 0; u < CHUNK / 4; ++u)
              if (4 * u < width) st_cluster_v4(dst + u * 512, make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]));
          }
          continue;
        }
        if (scale_out && !contributes) {  // the finished sum, scaled once; partial sums travel unscaled
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
        }
        if (bias && !contributes) {
          // One bias value per column of C: along this thread's registers, or
          // (operands swapped, C written transposed) one value for its whole row.
          if (!transpose_out) {
#pragma unroll
            for (int j = 0; j < CHUNK; ++j)
              v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(bias + min(col0 + c + j, rows_n - 1)));
          } else {
            const float mine = __ldg(bias + min(row, rows_m - 1));
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + mine);
          }
        }
        if constexpr (OUT_BYTES == 2) {
          if (p.out_quant && !contributes) {
            // Block-scaled C: this thread quantises its row's 64 columns - four
            // nvfp4 blocks or two mx blocks - from the accumulator rounded to
            // bfloat16 (so the bytes equal those of quantising a bfloat16 C), and
            // stores the packed codes and its scale bytes in the blocked layout.
            if (row < rows_m) {
              float x[64];
#pragma unroll
              for (int u = 0; u < 32; ++u) {
                const uint32_t both = pack_bf16x2(__uint_as_float(v[2 * u]), __uint_as_float(v[2 * u + 1]));
                x[2 * u] = __uint_as_float(both << 16);
                x[2 * u + 1] = __uint_as_float(both & 0xFFFF0000u);
              }
              const int gc = col0 + c;
              uint8_t* const atom_row = p.out_scales + (size_t(row >> 7) * p.out_k_groups) * 512 +
                                        (row & 31) * 16 + ((row >> 5) & 3) * 4;
              if (p.out_quant == 1 + Q_NVFP4) {
                uint32_t words[8], scales = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  uint32_t stored;
                  quantize_block<Q_NVFP4>(x + 16 * b, words + 2 * b, stored);
                  scales |= (stored & 0xFFu) << (8 * b);
                }
                uint4* dst = reinterpret_cast<uint4*>(out + size_t(row) * (rows_n >> 1) + (gc >> 1));
                dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
                dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
                *reinterpret_cast<uint32_t*>(atom_row + size_t(gc >> 6) * 512) = scales;
              } else if (p.out_quant == 1 + Q_MXFP4) {
                uint32_t words[8], scales = 0;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                  uint32_t stored;
                  quantize_block<Q_MXFP4>(x + 32 * b, words + 4 * b, stored);
                  scales |= (stored & 0xFFu) << (8 * b);
                }
                uint4* dst = reinterpret_cast<uint4*>(out + size_t(row) * (rows_n >> 1) + (gc >> 1));
                dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
                dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
                *reinterpret_cast<uint16_t*>(atom_row + size_t(gc >> 7) * 512 + ((gc >> 5) & 3)) = uint16_t(scales);
              } else {
                uint32_t words[16], scales = 0;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                  uint32_t stored;
                  quantize_block<Q_MXFP8>(x + 32 * b, words + 8 * b, stored);
                  scales |= (stored & 0xFFu) << (8 * b);
                }
                uint4* dst = reinterpret_cast<uint4*>(out + size_t(row) * rows_n + gc);
#pragma unroll
                for (int u = 0; u < 4; ++u) dst[u] = make_uint4(words[4 * u], words[4 * u + 1], words[4 * u + 2], words[4 * u + 3]);
                *reinterpret_cast<uint16_t*>(atom_row + size_t(gc >> 7) * 512 + ((gc >> 5) & 3)) = uint16_t(scales);
              }
            }
            continue;
          }
        }
        if (contributes) {
          // Raw accumulators, 16 bytes per lane per vector so a warp writes 512
          // contiguous bytes: vector g of row `lane` sits at (g * 32 + lane).
          uint4* dst = reinterpret_cast<uint4*>(p.partial) +
                       (size_t(my_region) * 64 + (c >> 2)) * 32 + lane;
#pragma unroll
          for (int u = 0; u < CHUNK / 4; ++u)
            if (4 * u < width) __stcg(dst + u * 32, make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]));
          continue;
        }

        if (staged && row0 < rows_m) {
          if constexpr (OUT_BYTES == 4) {
            store_rows(v, c, width);
          } else {
            uint32_t w[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) w[u] = pack2(v[2 * u], v[2 * u + 1]);
            store_rows(w, c, width);
          }
        } else if (!transpose_out) {
          if (row < rows_m) {
            const int gc = col0 + c;
            if (vec_ok && gc + width <= rows_n) {
              if constexpr (OUT_BYTES == 4) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) +
                                                      size_t(row) * ldd + gc);
#pragma unroll
                for (int u = 0; u < CHUNK / 4; ++u)
                  if (4 * u < width) dst[u] = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
              } else {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) +
                                                      size_t(row) * ldd + gc);
#pragma unroll
                for (int u = 0; u < CHUNK / 8; ++u)
                  if (8 * u < width)
                    dst[u] = make_uint4(pack2(v[8 * u], v[8 * u + 1]), pack2(v[8 * u + 2], v[8 * u + 3]),
                                        pack2(v[8 * u + 4], v[8 * u + 5]), pack2(v[8 * u + 6], v[8 * u + 7]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < CHUNK; ++j) {
                if (j < width && gc + j < rows_n) {
                  const size_t at = size_t(row) * ldd + gc + j;
                  if constexpr (OUT_BYTES == 4)
                    reinterpret_cast<uint32_t*>(out)[at] = v[j];
                  else
                    reinterpret_cast<uint16_t*>(out)[at] =
                        uint16_t(pack2(v[j], 0u) & 0xFFFFu);
                }
              }
            }
          }
        } else {
          // Transposed output: this thread's MMA row is an output column, so
          // the lanes of a warp write consecutive elements of one output row.
          if (row < rows_m) {
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) {
              const int orow = col0 + c + j;
              if (j < width && orow < rows_n) {
                const size_t at = size_t(orow) * ldd + row;
                if constexpr (OUT_BYTES == 4)
                  reinterpret_cast<uint32_t*>(out)[at] = v[j];
                else
                  reinterpret_cast<uint16_t*>(out)[at] =
                      uint16_t(pack2(v[j], 0u) & 0xFFFFu);
              }
            }
          }
        }
      }
      if (contributes) {
        __syncwarp();
        if (lane == 0) flag_release(p.flags + my_region, p.epoch);
      }
      if (cluster_k > 1 && sharers_ready) {
        // The arrive carries release semantics at cluster scope and follows the
        // warp's synchronisation, so the partial sums written above (or, on rank
        // 0, its reads of the landing zone) are ordered before it.
        __syncwarp();
        if (lane == 0) {
          if (ck_contributes) mbar_arrive_cluster(map_to_cta(bar_ck_partial + 8 * quarter, 0));
          else
            for (int peer = 1; peer < cluster_k; ++peer) mbar_arrive_cluster(map_to_cta(bar_ck_free + 8 * quarter, peer));
        }
      }
      // A tile that left its loop early (nothing to store, or a give-up) still
      // hands the accumulator back.
      if (!handed_back && !handed_back_late) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(acc_empty_leader + 8 * slot);
          else mbar_arrive(bar_acc_empty + 8 * slot);
        }
      }
    }
    // Shared memory may be released once the last TMA stores have read it.
    if (tma_out && lane == 0) tma_store_wait_read<0>();
    // Every grid waits for its predecessor before it ends, so that completion
    // stays transitive along the stream even for a warp that stored nothing.
    if (p.pdl && !touched_memory) pdl_wait_prior_grids();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (CTA_GROUP == 2 || cluster_k > 1) cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<CTA_GROUP>(tmem_slot, p.tmem_cols);
  }
}

}  // namespace og
