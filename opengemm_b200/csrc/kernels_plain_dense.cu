// Feature-free instantiations of the run-time-shaped kernel for the dense
// kinds (see kernels_fixed.cuh), in the order of their variant numbers.
#include "kernels_fixed.cuh"

namespace og {

extern const FixedKernel PLAIN_DENSE[] = {
    OG_PLAIN_KERNEL(0, KIND_F16, 1, 4),     OG_PLAIN_KERNEL(1, KIND_F16, 2, 4),
    OG_PLAIN_KERNEL(2, KIND_TF32, 1, 4),    OG_PLAIN_KERNEL(3, KIND_TF32, 2, 4),
    OG_PLAIN_KERNEL(4, KIND_I8, 1, 4),      OG_PLAIN_KERNEL(5, KIND_I8, 2, 4),
    OG_PLAIN_KERNEL(6, KIND_F8F6F4, 1, 4),  OG_PLAIN_KERNEL(7, KIND_F8F6F4, 2, 4),
    OG_PLAIN_KERNEL(14, KIND_F16, 1, 2),    OG_PLAIN_KERNEL(15, KIND_F16, 2, 2),
    OG_PLAIN_KERNEL(16, KIND_TF32, 1, 2),   OG_PLAIN_KERNEL(17, KIND_TF32, 2, 2),
    OG_PLAIN_KERNEL(18, KIND_F8F6F4, 1, 2), OG_PLAIN_KERNEL(19, KIND_F8F6F4, 2, 2),
};
extern const int PLAIN_DENSE_COUNT = sizeof(PLAIN_DENSE) / sizeof(PLAIN_DENSE[0]);

}  // namespace og
