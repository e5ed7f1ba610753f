// Symmetric heap arenas from the CUDA virtual-memory-management API.
//
// Second implementation of the arena behind the symmetric heap (the first, heap.cu, uses
// cudaMalloc + CUDA IPC handles): physical memory from cuMemCreate, exported as a POSIX file
// descriptor, mapped into every rank's address space with cuMemMap + cuMemSetAccess.  What it
// buys over CUDA IPC: the handle is an ordinary descriptor (it travels over a Unix socket like
// the shared-memory frames of the host runtime, and the kernel keeps the memory alive while
// anybody holds it), the mapping does not depend on peer-access state of the runtime, and the
// same allocation can be bound to an NVSwitch multicast object (psdev_mc_* below): one address
// range whose loads reduce over, and whose stores replicate into, every rank's arena.
//
// Life cycle of the multicast binding, which every rank follows in lock step (the host-side
// barriers are the caller's: src/van/nvl_van.cc): rank 0 creates the object and hands its
// descriptor round; every rank adds its device; barrier; every rank binds its arena; barrier;
// every rank maps the object.  Teardown is the mirror image after a barrier that follows the
// last kernel: unmap, unbind, release.  A rank must not leave while peers may still issue
// multimem accesses; failure tests therefore run with the binding off (PSB200_NVLS=0).
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
  // multicast objects (optional: absent on drivers or fabrics without NVLS)
  CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                        size_t, size_t, unsigned long long);
  CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*McGetGranularity)(size_t*, const CUmulticastObjectProp*,
                               CUmulticastGranularity_flags);
  bool ok, mc_ok;
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
    x.McCreate = Entry<decltype(x.McCreate)>("cuMulticastCreate");
    x.McAddDevice = Entry<decltype(x.McAddDevice)>("cuMulticastAddDevice");
    x.McBindMem = Entry<decltype(x.McBindMem)>("cuMulticastBindMem");
    x.McUnbind = Entry<decltype(x.McUnbind)>("cuMulticastUnbind");
    x.McGetGranularity = Entry<decltype(x.McGetGranularity)>("cuMulticastGetGranularity");
    x.mc_ok = x.McCreate && x.McAddDevice && x.McBindMem && x.McUnbind && x.McGetGranularity;
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
  return psdev_vmm_create_aligned(bytes, 0, base, fd, mapped_bytes);
}

// Same, with the size also rounded up to a multiple of `align` (0: none), which a later
// multicast binding of the whole arena needs (psdev_mc_granularity).
extern "C" int psdev_vmm_create_aligned(size_t bytes, size_t align, void** base, int* fd,
                                        size_t* mapped_bytes) {
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
  size_t size = (bytes + gran - 1) / gran * gran;
  if (align > gran) {
    if (align % gran) return PSDEV_ERR_ARG;
    size = (bytes + align - 1) / align * align;
  }
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

// ---- NVSwitch multicast object over the arenas --------------------------------------------
namespace {
struct McObject {
  CUmemGenericAllocationHandle handle;
  size_t bytes;
  CUdeviceptr mapped = 0;
  bool bound = false;
  size_t gran = 0;
};

CUmulticastObjectProp McProp(int num_devices, size_t bytes) {
  CUmulticastObjectProp p{};
  p.numDevices = static_cast<unsigned int>(num_devices);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  p.flags = 0;
  return p;
}
}  // namespace

// 1 when the current device can take part in a multicast object, else 0.
extern "C" int psdev_mc_supported(void) {
  if (!api().ok || !api().mc_ok) return 0;
  int dev = 0, mc = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  auto get = Entry<CUresult (*)(int*, CUdevice_attribute, CUdevice)>("cuDeviceGetAttribute");
  if (!get) return 0;
  if (get(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return mc ? 1 : 0;
}

// Size granularity of a multicast object over `num_devices` devices holding `bytes` each:
// the recommended one when the arena is at least that large, else the minimum.
extern "C" int psdev_mc_granularity(int num_devices, size_t bytes, size_t* gran) {
  const Api& a = api();
  if (!a.ok || !a.mc_ok || !gran || num_devices < 2) return PSDEV_ERR_UNSUPPORTED;
  CUmulticastObjectProp p = McProp(num_devices, bytes);
  size_t rec = 0, min = 0;
  if (a.McGetGranularity(&min, &p, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS || !min)
    return PSDEV_ERR_UNSUPPORTED;
  if (a.McGetGranularity(&rec, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) rec = 0;
  *gran = (rec && bytes >= rec) ? rec : min;
  return 0;
}

// Rank 0: creates the object for `num_devices` arenas of `bytes` (a multiple of the
// granularity) and exports it; *fd belongs to the caller.
extern "C" int psdev_mc_create(size_t bytes, int num_devices, int* fd, void** mc) {
  const Api& a = api();
  if (!a.ok || !a.mc_ok) return PSDEV_ERR_UNSUPPORTED;
  if (!fd || !mc || num_devices < 2) return PSDEV_ERR_ARG;
  CUmulticastObjectProp p = McProp(num_devices, bytes);
  CUmemGenericAllocationHandle h;
  if (a.McCreate(&h, &p) != CUDA_SUCCESS) return PSDEV_ERR_UNSUPPORTED;
  int out_fd = -1;
  if (a.Export(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    a.Release(h);
    return PSDEV_ERR_UNSUPPORTED;
  }
  auto* o = new McObject{h, bytes};
  *fd = out_fd;
  *mc = o;
  return 0;
}

// Other ranks: the object from rank 0's descriptor (which stays the caller's).
extern "C" int psdev_mc_import(int fd, size_t bytes, void** mc) {
  const Api& a = api();
  if (!a.ok || !a.mc_ok) return PSDEV_ERR_UNSUPPORTED;
  if (fd < 0 || !mc) return PSDEV_ERR_ARG;
  CUmemGenericAllocationHandle h;
  if (a.Import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return PSDEV_ERR_UNSUPPORTED;
  *mc = new McObject{h, bytes};
  return 0;
}

// Every rank, before anybody binds: adds the current device to the object.
extern "C" int psdev_mc_add_device(void* mc) {
  const Api& a = api();
  auto* o = static_cast<McObject*>(mc);
  if (!o) return PSDEV_ERR_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  return a.McAddDevice(o->handle, dev) == CUDA_SUCCESS ? 0 : PSDEV_ERR_UNSUPPORTED;
}

// Every rank, after all devices were added: binds its arena (from psdev_vmm_create*, of
// exactly the object's size) at offset 0.
extern "C" int psdev_mc_bind(void* mc, void* arena_base) {
  const Api& a = api();
  auto* o = static_cast<McObject*>(mc);
  if (!o || !arena_base) return PSDEV_ERR_ARG;
  Mapping m;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(reinterpret_cast<CUdeviceptr>(arena_base));
    if (it == g_maps.end()) return PSDEV_ERR_ARG;
    m = it->second;
  }
  if (m.bytes != o->bytes) return PSDEV_ERR_ARG;
  if (a.McBindMem(o->handle, 0, m.handle, 0, m.bytes, 0) != CUDA_SUCCESS)
    return PSDEV_ERR_UNSUPPORTED;
  o->bound = true;
  return 0;
}

// Every rank, after all arenas were bound: maps the object; *mc_base is the multicast alias.
extern "C" int psdev_mc_map(void* mc, void** mc_base) {
  const Api& a = api();
  auto* o = static_cast<McObject*>(mc);
  if (!o || !mc_base) return PSDEV_ERR_ARG;
  size_t gran = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUmemAllocationProp prop = PropFor(dev);
  if (a.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS)
    return PSDEV_ERR_UNSUPPORTED;
  CUdeviceptr ptr = 0;
  int rc = MapHere(o->handle, o->bytes, gran, &ptr);
  if (rc) return rc;
  o->mapped = ptr;
  *mc_base = reinterpret_cast<void*>(ptr);
  return 0;
}

// Every rank, after a barrier that follows the last kernel using the alias: unmaps the alias,
// unbinds this device's arena and drops the object.
extern "C" int psdev_mc_release(void* mc) {
  const Api& a = api();
  auto* o = static_cast<McObject*>(mc);
  if (!o) return PSDEV_ERR_ARG;
  cudaDeviceSynchronize();
  if (o->mapped) {
    a.Unmap(o->mapped, o->bytes);
    a.AddressFree(o->mapped, o->bytes);
  }
  if (o->bound) {
    int dev = 0;
    cudaGetDevice(&dev);
    a.McUnbind(o->handle, dev, 0, o->bytes);
  }
  a.Release(o->handle);
  delete o;
  return 0;
}
