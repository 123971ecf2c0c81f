// Fixed-shape instantiations for the dense kinds (see kernels_fixed.cuh).
#include "kernels_fixed.cuh"

namespace og {

extern const FixedKernel FIXED_DENSE[] = {
    OG_FIXED_KERNEL(1, KIND_F16, 2, 4, 256, 2),      // bf16 / f16 -> f32, pair, 256 x 256, TMA stores
    OG_FIXED_KERNEL(1, KIND_F16, 2, 4, 128, 2),      // ... 256 x 128
    OG_FIXED_KERNEL(3, KIND_TF32, 2, 4, 256, 2),
    OG_FIXED_KERNEL(5, KIND_I8, 2, 4, 256, 2),       // s8 / u8 -> s32
    OG_FIXED_KERNEL(7, KIND_F8F6F4, 2, 4, 256, 2),   // fp8 / fp6 / fp4 -> f32
    OG_FIXED_KERNEL(19, KIND_F8F6F4, 2, 2, 256, 1),  // fp8 -> bfloat16, staged rows
};
extern const int FIXED_DENSE_COUNT = sizeof(FIXED_DENSE) / sizeof(FIXED_DENSE[0]);

}  // namespace og
