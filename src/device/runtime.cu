// Thin C entry points over the CUDA runtime, for the host runtime's device plane.
//
// The host library (libpsb200_core.so: Postoffice, vans, KVWorker) does not link against CUDA:
// it must load and run on machines without a GPU.  Its device plane (src/van/nvl_van.cc)
// binds this library at run time and reaches streams, events, copies and allocations through
// the functions below, next to the psdev_* kernels.  Every function returns 0 or a
// cudaError_t value.
#include <cuda_runtime.h>

#include "ps/device/psdev.h"

extern "C" {

int psdev_rt_device_count(int* n) { return (int)cudaGetDeviceCount(n); }
int psdev_rt_set_device(int device) { return (int)cudaSetDevice(device); }
int psdev_rt_get_device(int* device) { return (int)cudaGetDevice(device); }

int psdev_rt_malloc(void** p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*p, 0, bytes);
}
int psdev_rt_free(void* p) { return (int)cudaFree(p); }
int psdev_rt_memset_async(void* p, int value, size_t bytes, void* stream) {
  return (int)cudaMemsetAsync(p, value, bytes, (cudaStream_t)stream);
}

// priority: 0 = default, 1 = highest priority the device offers
int psdev_rt_stream_create(void** stream, int priority) {
  cudaStream_t s;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  cudaError_t e = cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority ? hi : lo);
  *stream = s;
  return (int)e;
}
int psdev_rt_stream_destroy(void* stream) { return (int)cudaStreamDestroy((cudaStream_t)stream); }
int psdev_rt_stream_sync(void* stream) { return (int)cudaStreamSynchronize((cudaStream_t)stream); }

int psdev_rt_event_create(void** event) {
  cudaEvent_t e;
  cudaError_t rc = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  *event = e;
  return (int)rc;
}
int psdev_rt_event_destroy(void* event) { return (int)cudaEventDestroy((cudaEvent_t)event); }
int psdev_rt_event_record(void* event, void* stream) {
  return (int)cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream);
}
int psdev_rt_event_sync(void* event) { return (int)cudaEventSynchronize((cudaEvent_t)event); }
int psdev_rt_stream_wait_event(void* stream, void* event) {
  return (int)cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0);
}

// One asynchronous copy; the direction is inferred from the pointers (unified addressing).
int psdev_rt_memcpy_async(void* dst, const void* src, size_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream);
}

// 1 if `p` is device memory, 0 if it is host memory (pinned or pageable).
int psdev_rt_is_device_pointer(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}
// 1 if `p` is page-locked host memory that the device can copy from without staging.
int psdev_rt_is_pinned_host(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return a.type == cudaMemoryTypeHost;
}
int psdev_rt_host_alloc(void** p, size_t bytes) {
  return (int)cudaHostAlloc(p, bytes, cudaHostAllocDefault);
}
int psdev_rt_host_free(void* p) { return (int)cudaFreeHost(p); }

}  // extern "C"
