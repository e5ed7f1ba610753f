#include <cuda_bf16.h>
#define PSDEV_DENSE_GT float
#define PSDEV_DENSE_OT float
#define PSDEV_DENSE_FN dense_dispatch_f32_f32
#define PSDEV_DENSE_LL_FN dense_ll_dispatch_f32_f32
#include "kernels/dense_inst.inl"
