#include <cuda_bf16.h>
#define PSDEV_DENSE_GT __nv_bfloat16
#define PSDEV_DENSE_OT __nv_bfloat16
#define PSDEV_DENSE_FN dense_dispatch_bf16_bf16
#define PSDEV_DENSE_LL_FN dense_ll_dispatch_bf16_bf16
#include "kernels/dense_inst.inl"
