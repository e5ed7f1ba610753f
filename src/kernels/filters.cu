// Communication filters: transforms applied to a value buffer before it is pushed and after
// it is pulled.  The reference advertises "user-defined filters for communication
// compression" (README.md:24-25) but ships no filter code; these are the two this package
// provides on the device:
//   * cast / scale  fp32 <-> bf16 with a scale factor (the dense push kernel also applies the
//     same cast and scale while it loads, so this standalone form is for custom pipelines);
//   * int8 block-scale  groups of 256 values share one fp32 scale = max|x| / 127; values are
//     rounded to int8.  4x smaller than fp32 on the wire plus 1.6 % for the scales.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/psdev.h"

namespace psdev {
extern std::atomic<uint64_t> g_launches;
namespace filt {
constexpr int kGroup = 256;

__global__ void cast_scale_f32_to_bf16(const float* in, __nv_bfloat16* out, long long n, float s) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i] * s);
}
__global__ void cast_scale_bf16_to_f32(const __nv_bfloat16* in, float* out, long long n, float s) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]) * s;
}

// one warp per group of 256 values (8 per lane)
__global__ void int8_pack(const float* in, signed char* q, float* scales, long long n) {
  const long long ngroups = (n + kGroup - 1) / kGroup;
  const int lane = threadIdx.x & 31;
  for (long long g = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; g < ngroups;
       g += ((long long)gridDim.x * blockDim.x) >> 5) {
    float v[8];
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = g * kGroup + j * 32 + lane;
      v[j] = i < n ? in[i] : 0.f;
      m = fmaxf(m, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = m > 0.f ? m / 127.f : 1.f;
    const float inv = 1.f / scale;
    if (lane == 0) scales[g] = scale;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = g * kGroup + j * 32 + lane;
      if (i < n) q[i] = (signed char)__float2int_rn(fminf(fmaxf(v[j] * inv, -127.f), 127.f));
    }
  }
}
__global__ void int8_unpack(const signed char* q, const float* scales, float* out, long long n,
                            int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = (float)q[i] * scales[i / kGroup];
    out[i] = accumulate ? out[i] + v : v;
  }
}
}  // namespace filt
}  // namespace psdev

using namespace psdev;

extern "C" {
// dir 0: fp32 -> bf16, dir 1: bf16 -> fp32; out[i] = cast(in[i] * scale)
int psdev_filter_cast(const void* in, void* out, int64_t n, float scale, int dir, void* stream) {
  if (n < 0 || (dir != 0 && dir != 1)) return PSDEV_ERR_ARG;
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dir == 0)
    filt::cast_scale_f32_to_bf16<<<592, 256, 0, s>>>((const float*)in, (__nv_bfloat16*)out, n,
                                                     scale);
  else
    filt::cast_scale_bf16_to_f32<<<592, 256, 0, s>>>((const __nv_bfloat16*)in, (float*)out, n,
                                                     scale);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}
// fp32 -> int8 values + one fp32 scale per 256 values (scales has ceil(n/256) entries)
int psdev_filter_int8_pack(const float* in, int8_t* q, float* scales, int64_t n, void* stream) {
  if (n < 0) return PSDEV_ERR_ARG;
  if (n == 0) return 0;
  filt::int8_pack<<<592, 256, 0, (cudaStream_t)stream>>>(in, (signed char*)q, scales, n);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}
// out[i] = (accumulate ? out[i] : 0) + q[i] * scales[i / 256]
int psdev_filter_int8_unpack(const int8_t* q, const float* scales, float* out, int64_t n,
                             int accumulate, void* stream) {
  if (n < 0) return PSDEV_ERR_ARG;
  if (n == 0) return 0;
  filt::int8_unpack<<<592, 256, 0, (cudaStream_t)stream>>>((const signed char*)q, scales, out, n,
                                                           accumulate);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}
}  // extern "C"
