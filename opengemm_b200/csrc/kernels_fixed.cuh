// Kernels compiled for one tile shape each: the plans the large, tensor-bound
// shapes run (pairs of CTAs on 256-row tiles), where the run-time plan's
// address arithmetic and untaken branches cost a few per cent of tensor-pipe
// time under the board's power limit.  The run-time kernel remains the
// fallback for every other plan.  The reference compiles every kernel for one
// tile shape (opengemm/src/mm/registry.cuh:43-118, opengemm/src/smm/registry.cuh:39-114);
// here only the hot ones are.
#pragma once

#include "kernels_common.cuh"

namespace og {

// One compiled shape: which run-time variant it stands in for, the tile
// width and the epilogue path (0 own row, 1 staged rows, 2 TMA stores).
struct FixedKernel {
  int variant, tile_n, epi;
  cudaError_t (*configure)(int smem_bytes);
  cudaError_t (*launch)(const GemmParams& params, int grid, int smem_bytes, cudaStream_t stream, bool pdl);
};

#define OG_FIXED_KERNEL(VARIANT, KIND, GROUP, OUT, N, EPI) \
  FixedKernel { VARIANT, N, EPI, configure_one<KIND, GROUP, OUT, N, EPI>, launch_one<KIND, GROUP, OUT, N, EPI> }

// The run-time-shaped kernel of a variant compiled without the optional
// features (tile_n and epi are unused in these rows): what every launch that
// asks for none of them runs, unless a fixed-shape kernel serves its plan.
#define OG_PLAIN_KERNEL(VARIANT, KIND, GROUP, OUT) \
  FixedKernel { VARIANT, 0, 0, configure_one<KIND, GROUP, OUT, 0, 0, true>, launch_one<KIND, GROUP, OUT, 0, 0, true> }

}  // namespace og
