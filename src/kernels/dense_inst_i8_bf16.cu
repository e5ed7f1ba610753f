#include <cuda_bf16.h>
#define PSDEV_DENSE_GT signed char
#define PSDEV_DENSE_OT __nv_bfloat16
#define PSDEV_DENSE_FN dense_dispatch_i8_bf16
#include "kernels/dense_inst.inl"
