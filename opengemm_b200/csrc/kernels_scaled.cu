// Instantiations of gemm_kernel for the block-scaled MMA kinds (mxf8f6f4,
// mxf4, mxf4nvf4), one CTA or a pair per MMA, bfloat16 output.
#include "kernels_common.cuh"

namespace og {

cudaError_t configure_scaled(int variant, int smem_bytes) {
  switch (variant) {
    case 8: return configure_one<KIND_MXF8F6F4, 1, 2>(smem_bytes);
    case 9: return configure_one<KIND_MXF8F6F4, 2, 2>(smem_bytes);
    case 10: return configure_one<KIND_MXF4, 1, 2>(smem_bytes);
    case 11: return configure_one<KIND_MXF4, 2, 2>(smem_bytes);
    case 12: return configure_one<KIND_NVF4, 1, 2>(smem_bytes);
    case 13: return configure_one<KIND_NVF4, 2, 2>(smem_bytes);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_scaled(int variant, const GemmParams& params, int grid, int smem_bytes,
                          cudaStream_t stream, bool pdl) {
  switch (variant) {
    case 8: return launch_one<KIND_MXF8F6F4, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 9: return launch_one<KIND_MXF8F6F4, 2, 2>(params, grid, smem_bytes, stream, pdl);
    case 10: return launch_one<KIND_MXF4, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 11: return launch_one<KIND_MXF4, 2, 2>(params, grid, smem_bytes, stream, pdl);
    case 12: return launch_one<KIND_NVF4, 1, 2>(params, grid, smem_bytes, stream, pdl);
    case 13: return launch_one<KIND_NVF4, 2, 2>(params, grid, smem_bytes, stream, pdl);
  }
  return cudaErrorInvalidValue;
}

}  // namespace og
