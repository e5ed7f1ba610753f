// Sparse (keyed) push and pull on the device data plane.
//
// Keys are 64-bit, sorted and unique per request (the contract of KVWorker::Push,
// include/ps/kv_app.h:17,106); server s owns the contiguous key range
// [s*range, (s+1)*range) (src/postoffice.cc:169-180) and keeps its values in a direct-index
// table.  One step is three kernels per rank, separated by rendezvous of the ranks:
//
//   lookup+scatter (worker role)  K1: binary search of the S+1 range boundaries in the sorted
//        key list (what DefaultSlicer does on the CPU, kv_app.h:517-572); K3: every (key, grad)
//        is added into the owner's accumulator with a reduction sent over NVLink
//        (red.global.add.f32 on peer memory) -- no message, no per-server buffer;
//   apply (server role)  for each worker r the server walks r's key segment (read from r's
//        memory), takes the accumulated gradient with an atomic exchange (so a key pushed by
//        several workers is updated once) and applies the handle: sum, SGD or FTRL-proximal;
//   respond (server role)  writes the new value of every requested key straight into the
//        requesting worker's output array at the key's position: the pull needs neither a
//        response message nor the worker-side sort and concatenation (kv_app.h:681-708).
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/dev_common.cuh"

namespace psdev {
extern std::atomic<uint64_t> g_launches;

struct SparseArgs {
  void* base[PSDEV_MAX_RANKS];
  int rank, world;
  unsigned long long range;      // keys per shard
  unsigned long long keys_off;   // heap: u64[max_n]   worker's request keys
  unsigned long long grads_off;  // heap: f32[max_n]   worker's gradients
  unsigned long long out_off;    // heap: f32[max_n]   worker's pulled values
  unsigned long long pos_off;    // heap: i64[world+2] cut points, [world+1] = n
  unsigned long long acc_off;    // heap: f32[range]   server's gradient accumulator
  float* w;                      // server state, local: values
  float* z;                      // FTRL z (or NULL)
  float* nacc;                   // FTRL n (or NULL)
  long long n;                   // keys in this worker's request
  // hash store (capacity != 0): slots are found by open addressing in a key table that lives
  // in the owner's heap, so that workers can claim slots with remote compare-and-swap
  unsigned long long hkeys_off;  // heap: u64[capacity], all ones = empty
  unsigned long long capacity;   // power of two, or 0 for the direct-index store
  int* overflow;                 // local: set to 1 if a table ran out of slots
  int kind;                      // 0 sum, 1 sgd, 2 ftrl
  float lr, alpha, beta, l1, l2;
};

__device__ __forceinline__ char* heap(const SparseArgs& a, int r) {
  return reinterpret_cast<char*>(a.base[r]);
}

constexpr unsigned long long kEmptyKey = ~0ull;

__device__ __forceinline__ unsigned long long mix64(unsigned long long k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}
// Slot of `key` in the owner's table, claiming an empty slot if the key is new.  `tab` may be
// peer memory: the claim is a system-scope compare-and-swap.  -1 if the table is full.
__device__ __forceinline__ long long slot_find_or_insert(unsigned long long* tab,
                                                         unsigned long long cap,
                                                         unsigned long long key) {
  unsigned long long h = mix64(key) & (cap - 1);
  for (unsigned long long probes = 0; probes < cap; ++probes) {
    unsigned long long cur;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(cur) : "l"(tab + h) : "memory");
    if (cur == key) return (long long)h;
    if (cur == kEmptyKey) {
      cur = atomicCAS_system(tab + h, kEmptyKey, key);
      if (cur == kEmptyKey || cur == key) return (long long)h;
    }
    h = (h + 1) & (cap - 1);
  }
  return -1;
}
__device__ __forceinline__ long long slot_find(const unsigned long long* tab,
                                               unsigned long long cap, unsigned long long key) {
  unsigned long long h = mix64(key) & (cap - 1);
  for (unsigned long long probes = 0; probes < cap; ++probes) {
    unsigned long long cur;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(cur) : "l"(tab + h) : "memory");
    if (cur == key) return (long long)h;
    if (cur == kEmptyKey) return -1;
    h = (h + 1) & (cap - 1);
  }
  return -1;
}
// Index of `key` in the state arrays of server `rank`.
__device__ __forceinline__ long long state_index(const SparseArgs& a, int rank,
                                                 unsigned long long key, bool insert) {
  if (a.capacity == 0) return (long long)(key - (unsigned long long)rank * a.range);
  unsigned long long* tab =
      reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(a.base[rank]) + a.hkeys_off);
  return insert ? slot_find_or_insert(tab, a.capacity, key) : slot_find(tab, a.capacity, key);
}

// K1: pos[s] = first index whose key >= s*range, for s = 0..world; pos[world+1] = n.
__global__ void key_shard_lookup_kernel(const unsigned long long* keys, long long n,
                                        unsigned long long range, int world, long long* pos) {
  const int s = threadIdx.x;
  if (s > world) return;
  long long lo = 0, hi = n;
  if (s == world) {
    lo = n;
    // keys at or beyond world*range belong to nobody: report them through pos[world] < n
    const unsigned long long bound = range * (unsigned long long)world;
    long long l = 0, h = n;
    while (l < h) {
      long long m = (l + h) >> 1;
      if (keys[m] < bound) l = m + 1; else h = m;
    }
    lo = l;
  } else {
    const unsigned long long bound = range * (unsigned long long)s;
    while (lo < hi) {
      long long m = (lo + hi) >> 1;
      if (keys[m] < bound) lo = m + 1; else hi = m;
    }
  }
  pos[s] = lo;
  if (s == 0) pos[world + 1] = n;
}

// K3: scatter-add this worker's gradients into the owners' accumulators.
__global__ void sparse_scatter_kernel(const __grid_constant__ SparseArgs a) {
  const unsigned long long* keys =
      reinterpret_cast<const unsigned long long*>(heap(a, a.rank) + a.keys_off);
  const float* grads = reinterpret_cast<const float*>(heap(a, a.rank) + a.grads_off);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long k = keys[i];
    const unsigned long long s = k / a.range;
    if (s >= (unsigned long long)a.world) continue;  // outside every range: dropped
    const long long idx = state_index(a, (int)s, k, true);
    if (idx < 0) {
      *a.overflow = 1;
      continue;
    }
    float* acc = reinterpret_cast<float*>(heap(a, (int)s) + a.acc_off) + idx;
    asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(acc), "f"(grads[i]) : "memory");
  }
}

__device__ __forceinline__ float ftrl_weight(float z, float n, const SparseArgs& a) {
  if (fabsf(z) <= a.l1) return 0.f;
  const float sgn = z > 0.f ? 1.f : -1.f;
  return -(z - sgn * a.l1) / ((a.beta + sqrtf(n)) / a.alpha + a.l2);
}

// Server: apply the handle to every key that any worker pushed.
__global__ void sparse_apply_kernel(const __grid_constant__ SparseArgs a) {
  float* acc = reinterpret_cast<float*>(heap(a, a.rank) + a.acc_off);
  for (int r = 0; r < a.world; ++r) {
    const long long* pos = reinterpret_cast<const long long*>(heap(a, r) + a.pos_off);
    const long long lo = pos[a.rank], hi = pos[a.rank + 1];
    const unsigned long long* keys =
        reinterpret_cast<const unsigned long long*>(heap(a, r) + a.keys_off);
    for (long long i = lo + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hi;
         i += (long long)gridDim.x * blockDim.x) {
      unsigned long long k;
      asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(k) : "l"(keys + i) : "memory");
      const long long idx = state_index(a, a.rank, k, false);
      if (idx < 0) continue;  // the key found no slot (table full): reported by the scatter
      const float g = atomicExch(acc + idx, 0.f);
      if (g == 0.f) continue;  // already applied for another worker, or nothing to add
      if (a.kind == 0) {
        a.w[idx] += g;
      } else if (a.kind == 1) {
        a.w[idx] -= a.lr * g;
      } else {
        const float w = a.w[idx], n = a.nacc[idx];
        const float n2 = n + g * g;
        const float sigma = (sqrtf(n2) - sqrtf(n)) / a.alpha;
        const float z = a.z[idx] + g - sigma * w;
        a.z[idx] = z;
        a.nacc[idx] = n2;
        a.w[idx] = ftrl_weight(z, n2, a);
      }
    }
  }
}

// Server: write the value of every requested key into the requester's output array.
__global__ void sparse_respond_kernel(const __grid_constant__ SparseArgs a) {
  for (int rr = 0; rr < a.world; ++rr) {
    int r = a.rank + rr;
    if (r >= a.world) r -= a.world;
    const long long* pos = reinterpret_cast<const long long*>(heap(a, r) + a.pos_off);
    const long long lo = pos[a.rank], hi = pos[a.rank + 1];
    const unsigned long long* keys =
        reinterpret_cast<const unsigned long long*>(heap(a, r) + a.keys_off);
    float* out = reinterpret_cast<float*>(heap(a, r) + a.out_off);
    for (long long i = lo + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hi;
         i += (long long)gridDim.x * blockDim.x) {
      unsigned long long k;
      asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(k) : "l"(keys + i) : "memory");
      const long long idx = state_index(a, a.rank, k, false);
      out[i] = idx >= 0 ? a.w[idx] : 0.f;
    }
  }
}

}  // namespace psdev

using namespace psdev;

extern "C" {

typedef struct {
  uint64_t range;
  uint64_t keys_off, grads_off, out_off, pos_off, acc_off;
  float* w;
  float* z;
  float* n;
  int32_t kind;
  float lr, alpha, beta, l1, l2;
  uint64_t hkeys_off; /* hash store: heap offset of the u64 key table (filled with 0xff) */
  uint64_t capacity;  /* hash store: slots per server, power of two; 0 = direct index   */
  int32_t* overflow;  /* hash store: device int set to 1 when a table is full           */
} psdev_sparse_t;

static int fill(SparseArgs* a, const psdev_world_t* w, const psdev_sparse_t* t, int64_t n) {
  if (!w || !t || w->world < 1 || w->world > PSDEV_MAX_RANKS || t->range == 0) return PSDEV_ERR_ARG;
  if (!t->w || (t->kind == 2 && (!t->z || !t->n))) return PSDEV_ERR_ARG;
  for (int p = 0; p < w->world; ++p) a->base[p] = w->peer_base[p];
  a->rank = w->rank; a->world = w->world;
  a->range = t->range;
  a->keys_off = t->keys_off; a->grads_off = t->grads_off; a->out_off = t->out_off;
  a->pos_off = t->pos_off; a->acc_off = t->acc_off;
  a->w = t->w; a->z = t->z; a->nacc = t->n;
  a->n = n; a->kind = t->kind;
  a->lr = t->lr; a->alpha = t->alpha; a->beta = t->beta; a->l1 = t->l1; a->l2 = t->l2;
  a->hkeys_off = t->hkeys_off;
  a->capacity = t->capacity;
  a->overflow = t->overflow;
  if (t->capacity && ((t->capacity & (t->capacity - 1)) || !t->overflow)) return PSDEV_ERR_ARG;
  if (w->heap_bytes) {
    // what can be said without the buffers' capacities: the n staged pairs, their answers and
    // the W+1 cut points lie inside the arena, behind the control region
    const uint64_t un = n > 0 ? static_cast<uint64_t>(n) : 0;
    auto inside = [&](uint64_t off, uint64_t bytes) {
      return off >= PSDEV_CTRL_BYTES && off <= w->heap_bytes && bytes <= w->heap_bytes - off;
    };
    if (!inside(t->keys_off, un * 8) || !inside(t->grads_off, un * 4) ||
        !inside(t->out_off, un * 4) || !inside(t->pos_off, (w->world + 1) * 8ull) ||
        !inside(t->acc_off, 0) || (t->capacity && !inside(t->hkeys_off, t->capacity * 8)))
      return PSDEV_ERR_BOUNDS;
  }
  return 0;
}

// Cut points of a sorted key list at the shard boundaries (device pointers).
int psdev_key_shard_lookup(const uint64_t* keys, int64_t n, uint64_t range, int world,
                           int64_t* pos, void* stream) {
  if (world < 1 || world > PSDEV_MAX_RANKS || range == 0) return PSDEV_ERR_ARG;
  key_shard_lookup_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const unsigned long long*>(keys), n, range, world,
      reinterpret_cast<long long*>(pos));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Worker role: lookup + scatter-add of the n (key, grad) pairs stored in this rank's heap.
int psdev_sparse_scatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n,
                         int num_ctas, void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, n);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  char* mine = static_cast<char*>(w->peer_base[w->rank]);
  key_shard_lookup_kernel<<<1, 32, 0, s>>>(
      reinterpret_cast<const unsigned long long*>(mine + t->keys_off), n, t->range, w->world,
      reinterpret_cast<long long*>(mine + t->pos_off));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (n > 0) {
    sparse_scatter_kernel<<<num_ctas > 0 ? num_ctas : 592, 256, 0, s>>>(a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return (int)cudaGetLastError();
}

// Server role, after every rank's scatter has completed.
int psdev_sparse_apply(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas,
                       void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, 0);
  if (rc) return rc;
  sparse_apply_kernel<<<num_ctas > 0 ? num_ctas : 592, 256, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Server role: answer every worker's pull of the keys it pushed.
int psdev_sparse_respond(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas,
                         void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, 0);
  if (rc) return rc;
  sparse_respond_kernel<<<num_ctas > 0 ? num_ctas : 592, 256, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

}  // extern "C"
