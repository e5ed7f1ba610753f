// Symmetric heap arenas from the CUDA virtual-memory-management API.
//
// Second implementation of the arena behind the symmetric heap (the first, heap.cu, uses
// cudaMalloc + CUDA IPC handles): physical memory from cuMemCreate, exported as a POSIX file
// descriptor, mapped into every rank's address space with cuMemMap + cuMemSetAccess.  What it
// buys over CUDA IPC: the handle is an ordinary descriptor (it travels over a Unix socket like
// the shared-memory frames of the host runtime, and the kernel keeps the memory alive while
// anybody holds it), the mapping does not depend on peer-access state of the runtime, and the
// same allocation could later be bound to an NVSwitch multicast object.  That binding is NOT
// done here: a rank that dies while its memory is bound to a multicast object can take the
// fabric down for its peers, so the multicast alias keeps coming from torch's symmetric memory
// (ps_lite_b200/parallel/heap.py), which owns that life cycle.
//
// Role in the design: the analogue of the reference's registered-memory pool for its RDMA
// transport (src/ibverbs_van.h:86-214) -- memory is registered once, peers address it directly.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the library does not link
// against libcuda and still loads on a machine without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <map>
#include <mutex>

#include "ps/device/dev_common.cuh"

namespace {

template <typename Fn>
Fn Entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

struct Api {
  CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                     unsigned long long);
  CUresult (*Release)(CUmemGenericAllocationHandle);
  CUresult (*Export)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                     unsigned long long);
  CUresult (*Import)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*Reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*AddressFree)(CUdeviceptr, size_t);
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*Unmap)(CUdeviceptr, size_t);
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  bool ok;
};

const Api& api() {
  static const Api a = [] {
    Api x{};
    cudaFree(nullptr);  // make sure the runtime has a context
    x.GetGranularity = Entry<decltype(x.GetGranularity)>("cuMemGetAllocationGranularity");
    x.Create = Entry<decltype(x.Create)>("cuMemCreate");
    x.Release = Entry<decltype(x.Release)>("cuMemRelease");
    x.Export = Entry<decltype(x.Export)>("cuMemExportToShareableHandle");
    x.Import = Entry<decltype(x.Import)>("cuMemImportFromShareableHandle");
    x.Reserve = Entry<decltype(x.Reserve)>("cuMemAddressReserve");
    x.AddressFree = Entry<decltype(x.AddressFree)>("cuMemAddressFree");
    x.Map = Entry<decltype(x.Map)>("cuMemMap");
    x.Unmap = Entry<decltype(x.Unmap)>("cuMemUnmap");
    x.SetAccess = Entry<decltype(x.SetAccess)>("cuMemSetAccess");
    x.ok = x.GetGranularity && x.Create && x.Release && x.Export && x.Import && x.Reserve &&
           x.AddressFree && x.Map && x.Unmap && x.SetAccess;
    return x;
  }();
  return a;
}

struct Mapping {
  CUmemGenericAllocationHandle handle;
  size_t bytes;
};
std::mutex g_mu;
std::map<CUdeviceptr, Mapping> g_maps;

CUmemAllocationProp PropFor(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// Reserves a range, maps `h` there and opens it for loads and stores of the current device.
int MapHere(CUmemGenericAllocationHandle h, size_t bytes, size_t gran, CUdeviceptr* out) {
  const Api& a = api();
  int dev = 0;
  cudaGetDevice(&dev);
  CUdeviceptr ptr = 0;
  if (a.Reserve(&ptr, bytes, gran, 0, 0) != CUDA_SUCCESS) return PSDEV_ERR_UNSUPPORTED;
  if (a.Map(ptr, bytes, 0, h, 0) != CUDA_SUCCESS) {
    a.AddressFree(ptr, bytes);
    return PSDEV_ERR_UNSUPPORTED;
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (a.SetAccess(ptr, bytes, &acc, 1) != CUDA_SUCCESS) {
    a.Unmap(ptr, bytes);
    a.AddressFree(ptr, bytes);
    return PSDEV_ERR_UNSUPPORTED;
  }
  *out = ptr;
  return 0;
}

}  // namespace

// 1 when the current device can export allocations as file descriptors, else 0.
extern "C" int psdev_vmm_supported(void) {
  if (!api().ok) return 0;
  int dev = 0, vmm = 0, fd = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  auto get = Entry<CUresult (*)(int*, CUdevice_attribute, CUdevice)>("cuDeviceGetAttribute");
  if (!get) return 0;
  get(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  get(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  return vmm && fd;
}

// Allocates an arena of at least `bytes` on the current device.  *mapped_bytes is the size
// after rounding up to the allocation granularity (peers must import with that size), *fd a
// descriptor of the allocation that the caller owns (send it to the peers, then close it).
// The control region at the start of the arena is cleared.
extern "C" int psdev_vmm_create(size_t bytes, void** base, int* fd, size_t* mapped_bytes) {
  if (!base || !fd || !mapped_bytes || bytes < PSDEV_CTRL_BYTES) return PSDEV_ERR_ARG;
  const Api& a = api();
  if (!a.ok) return PSDEV_ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUmemAllocationProp prop = PropFor(dev);
  size_t gran = 0;
  if (a.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS ||
      gran == 0)
    return PSDEV_ERR_UNSUPPORTED;
  const size_t size = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  CUresult r = a.Create(&h, size, &prop, 0);
  if (r != CUDA_SUCCESS) return r == CUDA_ERROR_OUT_OF_MEMORY ? (int)cudaErrorMemoryAllocation
                                                             : PSDEV_ERR_UNSUPPORTED;
  int out_fd = -1;
  if (a.Export(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    a.Release(h);
    return PSDEV_ERR_UNSUPPORTED;
  }
  CUdeviceptr ptr = 0;
  int rc = MapHere(h, size, gran, &ptr);
  if (rc) {
    ::close(out_fd);
    a.Release(h);
    return rc;
  }
  cudaError_t e = cudaMemset(reinterpret_cast<void*>(ptr), 0, PSDEV_CTRL_BYTES);
  if (e != cudaSuccess) {
    a.Unmap(ptr, size);
    a.AddressFree(ptr, size);
    ::close(out_fd);
    a.Release(h);
    return (int)e;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_maps[ptr] = Mapping{h, size};
  }
  *base = reinterpret_cast<void*>(ptr);
  *fd = out_fd;
  *mapped_bytes = size;
  return 0;
}

// Maps a peer's arena, received as descriptor `fd` (stays owned by the caller), of the size
// that the peer's psdev_vmm_create reported, for the current device.
extern "C" int psdev_vmm_import(int fd, size_t mapped_bytes, void** base) {
  if (fd < 0 || !base || mapped_bytes == 0) return PSDEV_ERR_ARG;
  const Api& a = api();
  if (!a.ok) return PSDEV_ERR_UNSUPPORTED;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUmemAllocationProp prop = PropFor(dev);
  size_t gran = 0;
  if (a.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS ||
      gran == 0)
    return PSDEV_ERR_UNSUPPORTED;
  CUmemGenericAllocationHandle h;
  if (a.Import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return PSDEV_ERR_UNSUPPORTED;
  CUdeviceptr ptr = 0;
  int rc = MapHere(h, mapped_bytes, gran, &ptr);
  if (rc) {
    a.Release(h);
    return rc;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_maps[ptr] = Mapping{h, mapped_bytes};
  }
  *base = reinterpret_cast<void*>(ptr);
  return 0;
}

// Unmaps an arena obtained from psdev_vmm_create or psdev_vmm_import and drops this
// process's reference to the physical memory (it is freed when the last holder is gone).
extern "C" int psdev_vmm_release(void* base) {
  const Api& a = api();
  if (!a.ok) return PSDEV_ERR_UNSUPPORTED;
  Mapping m;
  const CUdeviceptr ptr = reinterpret_cast<CUdeviceptr>(base);
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(ptr);
    if (it == g_maps.end()) return PSDEV_ERR_ARG;
    m = it->second;
    g_maps.erase(it);
  }
  cudaDeviceSynchronize();
  a.Unmap(ptr, m.bytes);
  a.AddressFree(ptr, m.bytes);
  a.Release(m.handle);
  return 0;
}
