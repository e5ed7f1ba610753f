#include <cuda_bf16.h>
#define PSDEV_DENSE_GT signed char
#define PSDEV_DENSE_OT float
#define PSDEV_DENSE_FN dense_dispatch_i8_f32
#include "kernels/dense_inst.inl"
