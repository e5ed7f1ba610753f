// Symmetric device heap: one arena per rank, exported to the other processes of the box.
//
// Role in the design: the analogue of the reference's registered-memory machinery for its
// RDMA transport (SimpleMempool over ibv_reg_mr regions, src/ibverbs_van.h:86-214, and the
// rkey exchange of its rendezvous protocol, :632-724).  A buffer placed in the arena is
// "registered" once; afterwards any rank's kernel can load and store it directly, and no
// per-message address exchange is needed because offsets are identical on every rank.
#include <cuda_runtime.h>
#include <string.h>

#include <map>
#include <mutex>

#include "ps/device/dev_common.cuh"

extern "C" int psdev_heap_create(size_t bytes, void** base, unsigned char* ipc_handle) {
  if (!base || bytes < PSDEV_CTRL_BYTES) return PSDEV_ERR_ARG;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, PSDEV_CTRL_BYTES);
  if (e != cudaSuccess) return (int)e;
  if (ipc_handle) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
      cudaFree(p);
      return (int)e;
    }
    static_assert(sizeof(h) == PSDEV_IPC_HANDLE_BYTES, "ipc handle size");
    memcpy(ipc_handle, &h, sizeof(h));
  }
  *base = p;
  return 0;
}

extern "C" int psdev_heap_open(const unsigned char* ipc_handle, void** peer_base) {
  if (!ipc_handle || !peer_base) return PSDEV_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(peer_base, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int psdev_heap_close(void* peer_base) { return (int)cudaIpcCloseMemHandle(peer_base); }

extern "C" int psdev_heap_destroy(void* base) { return (int)cudaFree(base); }

extern "C" int psdev_enable_peer(int peer_device) {
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur == peer_device) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
  if (e != cudaSuccess) return (int)e;
  if (!can) return PSDEV_ERR_UNSUPPORTED;
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

// ---- first-fit sub-allocator -------------------------------------------------------------
namespace {
struct SubAlloc {
  std::mutex mu;
  size_t heap_bytes;
  std::map<size_t, size_t> free_;  // offset -> length, coalesced
  std::map<size_t, size_t> used_;  // offset -> length
  size_t in_use = 0;
};
}  // namespace

extern "C" void* psdev_suballoc_new(size_t heap_bytes) {
  auto* sa = new SubAlloc;
  sa->heap_bytes = heap_bytes;
  if (heap_bytes > PSDEV_CTRL_BYTES) sa->free_[PSDEV_CTRL_BYTES] = heap_bytes - PSDEV_CTRL_BYTES;
  return sa;
}
extern "C" void psdev_suballoc_delete(void* p) { delete static_cast<SubAlloc*>(p); }

extern "C" int64_t psdev_suballoc_alloc(void* p, size_t bytes, size_t align) {
  auto* sa = static_cast<SubAlloc*>(p);
  if (!sa || bytes == 0) return PSDEV_ERR_ARG;
  if (align < 256) align = 256;
  if (align & (align - 1)) return PSDEV_ERR_ARG;
  bytes = (bytes + 255) & ~size_t(255);
  std::lock_guard<std::mutex> lk(sa->mu);
  for (auto it = sa->free_.begin(); it != sa->free_.end(); ++it) {
    const size_t off = it->first, len = it->second;
    const size_t a = (off + align - 1) & ~(align - 1);
    if (a + bytes > off + len) continue;
    sa->free_.erase(it);
    if (a > off) sa->free_[off] = a - off;
    if (a + bytes < off + len) sa->free_[a + bytes] = off + len - (a + bytes);
    sa->used_[a] = bytes;
    sa->in_use += bytes;
    return (int64_t)a;
  }
  return PSDEV_ERR_NOMEM;
}

extern "C" int psdev_suballoc_free(void* p, int64_t offset) {
  auto* sa = static_cast<SubAlloc*>(p);
  if (!sa) return PSDEV_ERR_ARG;
  std::lock_guard<std::mutex> lk(sa->mu);
  auto u = sa->used_.find((size_t)offset);
  if (u == sa->used_.end()) return PSDEV_ERR_ARG;
  size_t off = u->first, len = u->second;
  sa->used_.erase(u);
  sa->in_use -= len;
  auto nx = sa->free_.lower_bound(off);
  if (nx != sa->free_.end() && off + len == nx->first) {
    len += nx->second;
    nx = sa->free_.erase(nx);
  }
  if (nx != sa->free_.begin()) {
    auto pv = std::prev(nx);
    if (pv->first + pv->second == off) {
      pv->second += len;
      return 0;
    }
  }
  sa->free_[off] = len;
  return 0;
}

extern "C" size_t psdev_suballoc_in_use(void* p) {
  auto* sa = static_cast<SubAlloc*>(p);
  std::lock_guard<std::mutex> lk(sa->mu);
  return sa->in_use;
}

// ---- channel state -----------------------------------------------------------------------
extern "C" int psdev_channel_status(void* local_base, int channel, int32_t* status,
                                    uint64_t* epoch) {
  if (!local_base || channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  auto* c = static_cast<psdev::Ctrl*>(local_base);
  cudaError_t e;
  if (status) {
    e = cudaMemcpy(status, &c->status[channel], sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
  }
  if (epoch) {
    e = cudaMemcpy(epoch, &c->epoch[channel], sizeof(uint64_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// Same read on a stream of the caller's (a non-blocking one: the plain form above copies on the
// default stream, which waits for every blocking stream of the process).
extern "C" int psdev_channel_status_on(void* local_base, int channel, void* stream,
                                       int32_t* status, uint64_t* epoch) {
  if (!local_base || channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  auto* c = static_cast<psdev::Ctrl*>(local_base);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (status) {
    e = cudaMemcpyAsync(status, &c->status[channel], sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return (int)e;
  }
  if (epoch) {
    e = cudaMemcpyAsync(epoch, &c->epoch[channel], sizeof(uint64_t), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaStreamSynchronize(s);
}

extern "C" int psdev_channel_clear(void* local_base, int channel) {
  if (!local_base || channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  auto* c = static_cast<psdev::Ctrl*>(local_base);
  cudaError_t e = cudaMemset(&c->status[channel], 0, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(&c->late_mask[channel], 0, sizeof(unsigned));
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(&c->done[channel], 0, sizeof(unsigned));
}
