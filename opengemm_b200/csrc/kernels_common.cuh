// Shared by the two translation units that instantiate gemm_kernel: one
// launch through cudaLaunchKernelEx with the pair's cluster shape and, when
// asked, programmatic dependent launch.
#pragma once

#include "kernel.cuh"

namespace og {

template <int KIND, int CTA_GROUP, int OUT_BYTES, int FIXED_N = 0, int FIXED_EPI = 0, bool PLAIN = false>
cudaError_t launch_one(const GemmParams& params, int grid, int smem_bytes, cudaStream_t stream,
                       bool pdl) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3(THREADS, 1, 1);
  config.dynamicSmemBytes = size_t(smem_bytes);
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  int count = 0;
  const int cluster = CTA_GROUP * (params.cluster_k > 1 ? params.cluster_k : 1);  // the pair, or the CTAs sharing K
  if (cluster > 1) {  // a single CTA needs no cluster launch
    attrs[count].id = cudaLaunchAttributeClusterDimension;
    attrs[count].val.clusterDim.x = cluster;
    attrs[count].val.clusterDim.y = 1;
    attrs[count].val.clusterDim.z = 1;
    ++count;
  }
  if (pdl) {
    attrs[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attrs;
  config.numAttrs = count;
  return cudaLaunchKernelEx(&config, gemm_kernel<KIND, CTA_GROUP, OUT_BYTES, FIXED_N, FIXED_EPI, PLAIN>, params,
                            LaunchPad{});
}

template <int KIND, int CTA_GROUP, int OUT_BYTES, int FIXED_N = 0, int FIXED_EPI = 0, bool PLAIN = false>
cudaError_t configure_one(int smem_bytes) {
  return cudaFuncSetAttribute(gemm_kernel<KIND, CTA_GROUP, OUT_BYTES, FIXED_N, FIXED_EPI, PLAIN>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
}

}  // namespace og
