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

// Eight values per thread and trip (two 16-byte loads, one 16-byte store, or the reverse) when
// both arrays are 16-byte aligned; scalar accesses for the tail and for unaligned arrays.
__global__ void cast_scale_f32_to_bf16(const float* in, __nv_bfloat16* out, long long n, float s) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long vec = 0;
  if ((((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    vec = n / 8;
    for (long long v = tid; v < vec; v += nthreads) {
      const float4 a = reinterpret_cast<const float4*>(in)[2 * v];
      const float4 b = reinterpret_cast<const float4*>(in)[2 * v + 1];
      __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x * s, a.y * s);
      __nv_bfloat162 p1 = __floats2bfloat162_rn(a.z * s, a.w * s);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x * s, b.y * s);
      __nv_bfloat162 p3 = __floats2bfloat162_rn(b.z * s, b.w * s);
      uint4 u;
      u.x = *reinterpret_cast<unsigned int*>(&p0);
      u.y = *reinterpret_cast<unsigned int*>(&p1);
      u.z = *reinterpret_cast<unsigned int*>(&p2);
      u.w = *reinterpret_cast<unsigned int*>(&p3);
      reinterpret_cast<uint4*>(out)[v] = u;
    }
  }
  for (long long i = vec * 8 + tid; i < n; i += nthreads) out[i] = __float2bfloat16_rn(in[i] * s);
}
__global__ void cast_scale_bf16_to_f32(const __nv_bfloat16* in, float* out, long long n, float s) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long vec = 0;
  if ((((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    vec = n / 8;
    for (long long v = tid; v < vec; v += nthreads) {
      const uint4 u = reinterpret_cast<const uint4*>(in)[v];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.z));
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.w));
      reinterpret_cast<float4*>(out)[2 * v] = make_float4(a.x * s, a.y * s, b.x * s, b.y * s);
      reinterpret_cast<float4*>(out)[2 * v + 1] = make_float4(c.x * s, c.y * s, d.x * s, d.y * s);
    }
  }
  for (long long i = vec * 8 + tid; i < n; i += nthreads) out[i] = __bfloat162float(in[i]) * s;
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
  // sixteen values per thread and trip (one 16-byte load, four 16-byte stores) when aligned; a
  // vector of 16 never straddles a group of 256
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long vec = 0;
  if ((((uintptr_t)q | (uintptr_t)out) & 15) == 0) {
    vec = n / 16;
    for (long long v = tid; v < vec; v += nthreads) {
      const uint4 u = reinterpret_cast<const uint4*>(q)[v];
      const float sc = scales[(v * 16) / kGroup];
      const unsigned int w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 o = make_float4((float)(signed char)(w[j] & 0xff) * sc,
                               (float)(signed char)((w[j] >> 8) & 0xff) * sc,
                               (float)(signed char)((w[j] >> 16) & 0xff) * sc,
                               (float)(signed char)((w[j] >> 24) & 0xff) * sc);
        float4* dst = reinterpret_cast<float4*>(out) + 4 * v + j;
        if (accumulate) {
          const float4 p = *dst;
          o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
        }
        *dst = o;
      }
    }
  }
  for (long long i = vec * 16 + tid; i < n; i += nthreads) {
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
