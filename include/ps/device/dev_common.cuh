// Device-side building blocks shared by every kernel of the data plane:
// the layout of the control region at the start of each symmetric heap, system-scope
// flag accessors, and bounded waits.  No wait in this library spins without a deadline.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ps/device/ctrl_layout.h"
#include "ps/device/psdev.h"

namespace psdev {

// Control region: first PSDEV_CTRL_BYTES of every heap (layout in ctrl_layout.h).
using Ctrl = psdev_ctrl_t;
static_assert(sizeof(Ctrl) <= PSDEV_CTRL_BYTES, "control region too small");

__device__ __forceinline__ Ctrl* ctrl_of(void* base) { return reinterpret_cast<Ctrl*>(base); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 16-byte load that always goes to the memory system (peer data may have been
// rewritten by its owner since this SM last touched the line).
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_v2(void* p, uint2 v) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ---- NVLS (NVSwitch multicast) accesses ------------------------------------------------------
// `mc` is an address inside the multicast alias of the symmetric heap: a load-reduce returns
// the element-wise sum over every rank's copy, computed in the switch; a store is replicated
// into every rank's copy.
__device__ __forceinline__ uint4 multimem_ld_reduce_f32x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// Eight bf16 values per rank, summed with fp32 accumulation, returned rounded to bf16.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_v2(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x),
               "r"(v.y)
               : "memory");
}

// Spin until *flag >= want or the deadline passes.  Returns true on success.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag,
                                             unsigned long long want,
                                             unsigned long long timeout_ns) {
  // the common case is a peer that is a few microseconds away: poll without pausing first,
  // then back off so that a long wait does not hammer the memory system
  for (int i = 0; i < 64; ++i)
    if (ld_acquire_sys(flag) >= want) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int backoff = 32;
  for (;;) {
    if (ld_acquire_sys(flag) >= want) return true;
    if (globaltimer_ns() - t0 > timeout_ns) return false;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
}

// bf16 <-> fp32 pack helpers on raw 32-bit lanes
__device__ __forceinline__ float2 bf16x2_to_f2(unsigned int u) {
  __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(h);
}
__device__ __forceinline__ unsigned int f2_to_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned int*>(&h);
}

}  // namespace psdev
