// Instantiations of gemm_kernel for the dense MMA kinds (f16, tf32, i8,
// f8f6f4), one CTA or a pair per MMA: 32-bit output (variants 0-7) and, for
// the float kinds, bfloat16 output (variants 14-19).
#include "kernels_common.cuh"

namespace og {

cudaError_t configure_dense(int variant, int smem_bytes) {
  switch (variant) {
    case 0: return configure_one<KIND_F16, 1, 4>(smem_bytes);
    case 1: return configure_one<KIND_F16, 2, 4>(smem_bytes);
    case 2: return configure_one<KIND_TF32, 1, 4>(smem_bytes);
    case 3: return configure_one<KIND_TF32, 2, 4>(smem_bytes);
    case 4: return configure_one<KIND_I8, 1, 4>(smem_bytes);
    case 5: return configure_one<KIND_I8, 2, 4>(smem_bytes);
    case 6: return configure_one<KIND_F8F6F4, 1, 4>(smem_bytes);
    case 7: return configure_one<KIND_F8F6F4, 2, 4>(smem_bytes);
    case 14: return configure_one<KIND_F16, 1, 2>(smem_bytes);
    case 15: return configure_one<KIND_F16, 2, 2>(smem_bytes);
    case 16: return configure_one<KIND_TF32, 1, 2>(smem_bytes);
    case 17: return configure_one<KIND_TF32, 2, 2>(smem_bytes);
    case 18: return configure_one<KIND_F8F6F4, 1, 2>(smem_bytes);
    case 19: return configure_one<KIND_F8F6F4, 2, 2>(smem_bytes);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_dense(int variant, const GemmParams& params, int grid, int smem_bytes,
                         cudaStream_t stream, bool pdl) {
  switch (variant) {
    case 0: return launch_one<KIND_F16, 1, 4>(params, grid, smem_bytes, stream, pdl);
    case 1: return launch_one<KIND_F16, 2, 4>(params, grid, smem_bytes, stream, pdl);
    case 2: return launch_one<KIND_TF32, 1, 4>(params, grid, smem_bytes, stream, pdl);
    case 3: return launch_one<KIND_TF32, 2, 4>(params, grid, smem_bytes, stream, pdl);
    case 4: return launch_one<KIND_I8, 1, 4>(params, grid, smem_bytes, stream, pdl);
    case 5: return launch_one<KIND_I8, 2, 4>(params, grid, smem_bytes, stream, pdl);
    case 6: return launch_one<KIND_F8F6F4, 1, 4>(params, grid, smem_bytes, stream, pdl);
    case 7: return launch_one<KIND_F8F6F4, 2, 4>(params, grid, smem_bytes, stream, pdl);
    case 14: return launch_one<KIND_F16, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 15: return launch_one<KIND_F16, 2, 2>(params, grid, smem_bytes, stream, pdl);
    case 16: return launch_one<KIND_TF32, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 17: return launch_one<KIND_TF32, 2, 2>(params, grid, smem_bytes, stream, pdl);
    case 18: return launch_one<KIND_F8F6F4, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 19: return launch_one<KIND_F8F6F4, 2, 2>(params, grid, smem_bytes, stream, pdl);
  }
  return cudaErrorInvalidValue;
}

}  // namespace og
