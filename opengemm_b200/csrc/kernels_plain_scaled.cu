// Feature-free instantiations of the run-time-shaped kernel for the
// block-scaled kinds (see kernels_fixed.cuh), in the order of their variant numbers.
#include "kernels_fixed.cuh"

namespace og {

extern const FixedKernel PLAIN_SCALED[] = {
    OG_PLAIN_KERNEL(8, KIND_MXF8F6F4, 1, 2), OG_PLAIN_KERNEL(9, KIND_MXF8F6F4, 2, 2),
    OG_PLAIN_KERNEL(10, KIND_MXF4, 1, 2),    OG_PLAIN_KERNEL(11, KIND_MXF4, 2, 2),
    OG_PLAIN_KERNEL(12, KIND_NVF4, 1, 2),    OG_PLAIN_KERNEL(13, KIND_NVF4, 2, 2),
};
extern const int PLAIN_SCALED_COUNT = sizeof(PLAIN_SCALED) / sizeof(PLAIN_SCALED[0]);

}  // namespace og
