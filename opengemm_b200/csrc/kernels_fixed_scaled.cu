// Fixed-shape instantiations for the block-scaled kinds (see kernels_fixed.cuh).
#include "kernels_fixed.cuh"

namespace og {

extern const FixedKernel FIXED_SCALED[] = {
    OG_FIXED_KERNEL(13, KIND_NVF4, 2, 2, 192, 1),     // nvfp4, pair, 256 x 192, two accumulators
    OG_FIXED_KERNEL(13, KIND_NVF4, 2, 2, 256, 1),     // nvfp4, pair, 256 x 256, one accumulator
    OG_FIXED_KERNEL(11, KIND_MXF4, 2, 2, 256, 1),
    OG_FIXED_KERNEL(10, KIND_MXF4, 1, 2, 256, 1),     // the decode shapes: one CTA, 128 x 256
    OG_FIXED_KERNEL(9, KIND_MXF8F6F4, 2, 2, 256, 1),
    OG_FIXED_KERNEL(9, KIND_MXF8F6F4, 2, 2, 192, 1),
};
extern const int FIXED_SCALED_COUNT = sizeof(FIXED_SCALED) / sizeof(FIXED_SCALED[0]);

}  // namespace og
