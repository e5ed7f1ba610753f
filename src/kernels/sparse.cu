// Sparse (keyed) push and pull on the device data plane.
//
// Keys are 64-bit, sorted and unique per request (the contract of KVWorker::Push,
// include/ps/kv_app.h:17,106).  A value is a short fp32 vector: every key has `width` elements,
// or -- with per-key lengths, the reference's dynamic-length values (kv_app.h:24-31) --
// lens[i] <= width elements packed back to back, value i starting at the prefix sum of the
// lengths (what DefaultSlicer computes on the CPU, kv_app.h:547-567).  Server s owns the
// contiguous key range [s*range, (s+1)*range) (src/postoffice.cc:169-180) and keeps its values
// in a direct-index table or, for huge key spaces, an open-addressing hash table.
//
// One step is three kernels per rank and no message:
//
//   scatter (worker role)  cut points of the sorted key list at the W+1 range boundaries (K1)
//        and, with lengths, their prefix sum; every element of every (key, gradient) is added
//        into the owner's accumulator with a reduction sent over NVLink
//        (red.global.add.f32 on peer memory);
//   apply (server role)  starts with a rendezvous of the ranks (everybody's scatter has
//        completed); for each worker r the server walks r's key segment (read from r's memory),
//        takes the accumulated gradient with an atomic exchange (so a key pushed by several
//        workers is updated once) and applies the handle: sum, SGD or FTRL-proximal;
//   respond (server role)  writes the new value of every requested key straight into the
//        requesting worker's output array at the value's offset -- the pull needs neither a
//        response message nor the worker-side sort and concatenation (kv_app.h:681-708) --
//        and ends with a rendezvous (everybody's answers have landed).
//
// Every wait is bounded; the checks build (-DPSDEV_CHECKS) verifies every slot index against
// the table's capacity and every value offset against the request buffers before it is used,
// records PSDEV_ERR_BOUNDS in the channel's status word and skips the access.
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/push_pull.cuh"

namespace psdev {
extern std::atomic<uint64_t> g_launches;

struct SparseArgs {
  void* base[PSDEV_MAX_RANKS];
  int rank, world;
  unsigned long long range;      // keys per shard
  unsigned long long keys_off;   // heap: u64[max_n]        worker's request keys
  unsigned long long grads_off;  // heap: f32[max_vals]     worker's gradients
  unsigned long long out_off;    // heap: f32[max_vals]     worker's pulled values
  unsigned long long pos_off;    // heap: i64[world+2]      cut points, [world+1] = n
  unsigned long long lens_off;   // heap: i32[max_n] per-key lengths, or 0 (all = width)
  unsigned long long offs_off;   // heap: i64[max_n+1] value offsets (with lengths only)
  unsigned long long acc_off;    // heap: f32[slots*width]  server's gradient accumulator
  float* w;                      // server state, local: values [slots*width]
  float* z;                      // FTRL z (or NULL)
  float* nacc;                   // FTRL n (or NULL)
  int* klen;                     // server state: stored length per slot (with lengths), or NULL
  long long n;                   // keys in this worker's request
  long long max_n, max_vals;     // capacities of the request buffers
  long long slots;               // slots of the server's store (range, or hash capacity)
  int width;
  int sstride;                   // floats between consecutive values in w, z, nacc
  // hash store (capacity != 0): slots are found by open addressing in a key table that lives
  // in the owner's heap, so that workers can claim slots with remote compare-and-swap
  unsigned long long hkeys_off;  // heap: u64[capacity], all ones = empty
  unsigned long long capacity;   // power of two, or 0 for the direct-index store
  int* overflow;                 // local: set to 1 if a table ran out of slots
  int kind;                      // 0 sum, 1 sgd, 2 ftrl
  float lr, alpha, beta, l1, l2;
  int channel, sync;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ char* heap(const SparseArgs& a, int r) {
  return reinterpret_cast<char*>(a.base[r]);
}
__device__ __forceinline__ long long ld_volatile_s64(const long long* p) {
  long long v;
  asm volatile("ld.volatile.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void note_bounds(const SparseArgs& a) {
  atomicMin(&ctrl_of(a.base[a.rank])->status[a.channel], (int)PSDEV_ERR_BOUNDS);
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
// Index of `key` in the state arrays of server `rank`, or -1.
__device__ __forceinline__ long long state_index(const SparseArgs& a, int rank,
                                                 unsigned long long key, bool insert) {
  long long idx;
  if (a.capacity == 0) {
    idx = (long long)(key - (unsigned long long)rank * a.range);
  } else {
    unsigned long long* tab = reinterpret_cast<unsigned long long*>(
        reinterpret_cast<char*>(a.base[rank]) + a.hkeys_off);
    idx = insert ? slot_find_or_insert(tab, a.capacity, key) : slot_find(tab, a.capacity, key);
  }
#ifdef PSDEV_CHECKS
  if (idx >= a.slots) {
    note_bounds(a);
    return -1;
  }
#endif
  return idx;
}

// K1: pos[s] = first index whose key >= s*range, for s = 0..world; pos[world+1] = n.
__device__ __forceinline__ void shard_lookup(const unsigned long long* keys, long long n,
                                             unsigned long long range, int world,
                                             long long* pos, int s) {
  if (s > world) return;
  // keys at or beyond world*range belong to nobody: reported through pos[world] < n
  const unsigned long long bound = range * (unsigned long long)s;
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long m = (lo + hi) >> 1;
    if (keys[m] < bound) lo = m + 1; else hi = m;
  }
  pos[s] = lo;
  if (s == 0) pos[world + 1] = n;
}
__global__ void key_shard_lookup_kernel(const unsigned long long* keys, long long n,
                                        unsigned long long range, int world, long long* pos) {
  shard_lookup(keys, n, range, world, pos, threadIdx.x);
}

// Exclusive prefix sum of the per-key lengths into offs[0..n] (offs[n] = number of values).
// One block of 1024 threads: each thread sums a contiguous chunk, the chunk sums are scanned
// in shared memory, each thread then writes its chunk's offsets.
__global__ void __launch_bounds__(1024) lens_scan_kernel(const int* lens, long long n,
                                                         long long* offs) {
  __shared__ long long part[1024];
  const int t = threadIdx.x;
  const long long chunk = (n + 1023) / 1024;
  const long long lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
  long long s = 0;
  for (long long i = lo; i < hi; ++i) s += lens[i] > 0 ? lens[i] : 0;
  part[t] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const long long v = t >= off ? part[t - off] : 0;
    __syncthreads();
    part[t] += v;
    __syncthreads();
  }
  long long run = part[t] - s;
  for (long long i = lo; i < hi; ++i) {
    offs[i] = run;
    run += lens[i] > 0 ? lens[i] : 0;
  }
  if (t == 1023) offs[n] = part[1023];
}

// Length and value offset of request entry i of worker r.
__device__ __forceinline__ void value_span(const SparseArgs& a, int r, long long i, long long* off,
                                           int* len) {
  if (a.lens_off == 0) {
    *off = i * a.width;
    *len = a.width;
    return;
  }
  const int* lens = reinterpret_cast<const int*>(heap(a, r) + a.lens_off);
  const long long* offs = reinterpret_cast<const long long*>(heap(a, r) + a.offs_off);
  int l;
  long long o;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(l) : "l"(lens + i) : "memory");
  asm volatile("ld.volatile.global.s64 %0, [%1];" : "=l"(o) : "l"(offs + i) : "memory");
  if (l < 0) l = 0;
  if (l > a.width) l = a.width;  // a value never exceeds its slot
  *off = o;
  *len = l;
}

// K1 + K3: cut points, then scatter-add this worker's gradients into the owners' accumulators.
__global__ void __launch_bounds__(256, 8)
    sparse_scatter_kernel(const __grid_constant__ SparseArgs a) {
  const unsigned long long* keys =
      reinterpret_cast<const unsigned long long*>(heap(a, a.rank) + a.keys_off);
  if (blockIdx.x == 0 && threadIdx.x <= a.world)
    shard_lookup(keys, a.n, a.range, a.world,
                 reinterpret_cast<long long*>(heap(a, a.rank) + a.pos_off), threadIdx.x);
  const float* grads = reinterpret_cast<const float*>(heap(a, a.rank) + a.grads_off);
  // one thread per (key, element) when every value has `width` elements; one per key otherwise
  const bool per_elem = a.lens_off == 0;
  const long long work = per_elem ? a.n * a.width : a.n;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < work;
       t += (long long)gridDim.x * blockDim.x) {
    const long long i = per_elem ? t / a.width : t;
    const int j0 = per_elem ? (int)(t - i * a.width) : 0;
    const unsigned long long k = keys[i];
    const unsigned long long s = k / a.range;
    if (s >= (unsigned long long)a.world) continue;  // outside every range: dropped
    const long long idx = state_index(a, (int)s, k, true);
    if (idx < 0) {
      if (a.capacity) *a.overflow = 1;
      continue;
    }
    long long off;
    int len;
    value_span(a, a.rank, i, &off, &len);
#ifdef PSDEV_CHECKS
    if (off < 0 || off + len > a.max_vals) {
      note_bounds(a);
      continue;
    }
#endif
    float* acc = reinterpret_cast<float*>(heap(a, (int)s) + a.acc_off) + idx * a.width;
    if (per_elem) {
      asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(acc + j0),
                   "f"(grads[off + j0])
                   : "memory");
    } else {
      for (int j = 0; j < len; ++j)
        asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(acc + j),
                     "f"(grads[off + j])
                     : "memory");
    }
  }
}

__device__ __forceinline__ float ftrl_weight(float z, float n, const SparseArgs& a) {
  if (fabsf(z) <= a.l1) return 0.f;
  const float sgn = z > 0.f ? 1.f : -1.f;
  return -(z - sgn * a.l1) / ((a.beta + sqrtf(n)) / a.alpha + a.l2);
}

__device__ __forceinline__ void apply_one(const SparseArgs& a, long long e, float g) {
  const long long s = e * a.sstride;  // the value's place in the state arrays
  if (a.kind == 0) {
    a.w[s] += g;
  } else if (a.kind == 1) {
    a.w[s] -= a.lr * g;
  } else {
    const float w = a.w[s], n = a.nacc[s];
    const float n2 = n + g * g;
    const float sigma = (sqrtf(n2) - sqrtf(n)) / a.alpha;
    const float z = a.z[s] + g - sigma * w;
    a.z[s] = z;
    a.nacc[s] = n2;
    a.w[s] = ftrl_weight(z, n2, a);
  }
}

// Server: after every rank's scatter has completed, apply the handle to every key that any
// worker pushed.
__global__ void __launch_bounds__(256, 8)
    sparse_apply_kernel(const __grid_constant__ SparseArgs a) {
  __shared__ unsigned long long s_epoch;
  __shared__ int s_err;
  unsigned long long e = 1;
  if (a.sync)
    e = channel_enter(a.base, a.rank, a.world, a.channel, a.timeout_ns, &s_epoch, &s_err);
  if (e != 0ull) {
    float* acc = reinterpret_cast<float*>(heap(a, a.rank) + a.acc_off);
    for (int r = 0; r < a.world; ++r) {
      const long long* pos = reinterpret_cast<const long long*>(heap(a, r) + a.pos_off);
      const long long lo = ld_volatile_s64(pos + a.rank), hi = ld_volatile_s64(pos + a.rank + 1);
#ifdef PSDEV_CHECKS
      if (lo < 0 || hi < lo || hi > a.max_n) {
        if (threadIdx.x == 0 && blockIdx.x == 0) note_bounds(a);
        continue;
      }
#endif
      const unsigned long long* keys =
          reinterpret_cast<const unsigned long long*>(heap(a, r) + a.keys_off);
      const long long work = (hi - lo) * a.width;
      for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < work;
           t += (long long)gridDim.x * blockDim.x) {
        const long long i = lo + t / a.width;
        const int j = (int)(t % a.width);
        unsigned long long k;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(k) : "l"(keys + i) : "memory");
        const long long idx = state_index(a, a.rank, k, false);
        if (idx < 0) continue;  // the key found no slot (table full): reported by the scatter
        if (a.klen && a.lens_off && j == 0) {
          // the owner remembers how long the value of this key is (every pusher says the same)
          long long off;
          int len;
          value_span(a, r, i, &off, &len);
          if (len > 0) a.klen[idx] = len;  // a pull (length 0) leaves the stored length alone
        }
        const long long el = idx * a.width + j;
        const float g = atomicExch(acc + el, 0.f);
        if (g == 0.f) continue;  // already applied for another worker, or nothing to add
        apply_one(a, el, g);
      }
    }
  }
  // the round that this rendezvous opened is closed by the respond kernel, which follows on
  // the same stream
}

// Server: store the length of the value of every requested key into the requester's array of
// lengths (a pull whose caller does not know the lengths).  Keys that own no slot get 0.
__global__ void sparse_lens_kernel(const __grid_constant__ SparseArgs a) {
  for (int rr = 0; rr < a.world; ++rr) {
    int r = a.rank + rr;
    if (r >= a.world) r -= a.world;
    const long long* pos = reinterpret_cast<const long long*>(heap(a, r) + a.pos_off);
    const long long lo = ld_volatile_s64(pos + a.rank), hi = ld_volatile_s64(pos + a.rank + 1);
#ifdef PSDEV_CHECKS
    if (lo < 0 || hi < lo || hi > a.max_n) {
      if (threadIdx.x == 0 && blockIdx.x == 0) note_bounds(a);
      continue;
    }
#endif
    const unsigned long long* keys =
        reinterpret_cast<const unsigned long long*>(heap(a, r) + a.keys_off);
    int* lens = reinterpret_cast<int*>(heap(a, r) + a.lens_off);
    for (long long i = lo + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hi;
         i += (long long)gridDim.x * blockDim.x) {
      unsigned long long k;
      asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(k) : "l"(keys + i) : "memory");
      const long long idx = state_index(a, a.rank, k, false);
      lens[i] = idx >= 0 ? a.klen[idx] : 0;
    }
  }
}

// Server: write the value of every requested key into the requester's output array, then wait
// until every server has done so.
__global__ void __launch_bounds__(256, 8)
    sparse_respond_kernel(const __grid_constant__ SparseArgs a) {
  __shared__ int s_last;
  Ctrl* my = ctrl_of(a.base[a.rank]);
  const bool healthy = !a.sync || *(volatile int*)&my->status[a.channel] == 0;
  if (healthy) {
    for (int rr = 0; rr < a.world; ++rr) {
      int r = a.rank + rr;
      if (r >= a.world) r -= a.world;
      const long long* pos = reinterpret_cast<const long long*>(heap(a, r) + a.pos_off);
      const long long lo = ld_volatile_s64(pos + a.rank), hi = ld_volatile_s64(pos + a.rank + 1);
#ifdef PSDEV_CHECKS
      if (lo < 0 || hi < lo || hi > a.max_n) {
        if (threadIdx.x == 0 && blockIdx.x == 0) note_bounds(a);
        continue;
      }
#endif
      const unsigned long long* keys =
          reinterpret_cast<const unsigned long long*>(heap(a, r) + a.keys_off);
      float* out = reinterpret_cast<float*>(heap(a, r) + a.out_off);
      const long long work = (hi - lo) * a.width;
      for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < work;
           t += (long long)gridDim.x * blockDim.x) {
        const long long i = lo + t / a.width;
        const int j = (int)(t % a.width);
        unsigned long long k;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(k) : "l"(keys + i) : "memory");
        long long off;
        int len;
        value_span(a, r, i, &off, &len);
        if (j >= len) continue;
#ifdef PSDEV_CHECKS
        if (off < 0 || off + len > a.max_vals) {
          note_bounds(a);
          continue;
        }
#endif
        const long long idx = state_index(a, a.rank, k, false);
        out[off + j] = idx >= 0 ? a.w[(idx * a.width + j) * a.sstride] : 0.f;
      }
    }
  }
  if (a.sync) {
    // the epoch that the apply kernel entered with: one ahead of the last completed one
    const unsigned long long e = healthy ? ld_volatile_u64(&my->epoch[a.channel]) + 1ull : 0ull;
    channel_leave(a.base, a.rank, a.world, a.channel, e, a.timeout_ns, &s_last);
  }
}

}  // namespace psdev

using namespace psdev;

extern "C" {

// Grid of the keyed kernels: 4 CTAs of 256 threads per SM.  On one GPU 592, 1184 and 2368 CTAs
// take the same time within 2 % (the kernels are bound by the rate of random 64-byte DRAM
// accesses, accumulator and state group of every key, not by occupancy); across GPUs more CTAs
// cost more, because every CTA ends the rendezvous with a system-scope fence (2 GPUs: 0.279 ms
// per step with 592 CTAs, 0.311 with 1184).  PSB200_SPARSE_CTAS overrides.
static int default_ctas() {
  static const int n = [] {
    const char* e = getenv("PSB200_SPARSE_CTAS");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 148 * 4;
  }();
  return n;
}

static int fill(SparseArgs* a, const psdev_world_t* w, const psdev_sparse_t* t, int64_t n) {
  if (!w || !t || w->world < 1 || w->world > PSDEV_MAX_RANKS || t->range == 0) return PSDEV_ERR_ARG;
  if (!t->w || (t->kind == 2 && (!t->z || !t->n))) return PSDEV_ERR_ARG;
  if (t->width < 1 || t->max_n < 1 || t->max_vals < t->max_n || t->slots < 1) return PSDEV_ERR_ARG;
  if (n < 0 || n > t->max_n) return PSDEV_ERR_ARG;
  if (t->lens_off != 0 && (t->offs_off == 0 || !t->klen)) return PSDEV_ERR_ARG;
  if (t->lens_off == 0 && n * t->width > t->max_vals) return PSDEV_ERR_ARG;
  if (t->channel < 0 || t->channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  for (int p = 0; p < w->world; ++p) a->base[p] = w->peer_base[p];
  a->rank = w->rank; a->world = w->world;
  a->range = t->range;
  a->keys_off = t->keys_off; a->grads_off = t->grads_off; a->out_off = t->out_off;
  a->pos_off = t->pos_off; a->acc_off = t->acc_off;
  a->lens_off = t->lens_off; a->offs_off = t->offs_off;
  a->w = t->w; a->z = t->z; a->nacc = t->n; a->klen = t->klen;
  a->sstride = t->state_stride > 1 ? t->state_stride : 1;
  a->n = n; a->kind = t->kind;
  a->max_n = t->max_n; a->max_vals = t->max_vals; a->slots = t->slots; a->width = t->width;
  a->lr = t->lr; a->alpha = t->alpha; a->beta = t->beta; a->l1 = t->l1; a->l2 = t->l2;
  a->hkeys_off = t->hkeys_off;
  a->capacity = t->capacity;
  a->overflow = t->overflow;
  a->channel = t->channel;
  a->timeout_ns = t->timeout_ns ? t->timeout_ns : 20000000000ull;
  if (t->capacity && ((t->capacity & (t->capacity - 1)) || !t->overflow ||
                      t->capacity != (uint64_t)t->slots))
    return PSDEV_ERR_ARG;
  if (w->heap_bytes) {
    // every buffer of the table, at its full capacity, lies inside the arena behind the
    // control region
    auto inside = [&](uint64_t off, uint64_t bytes) {
      return off >= PSDEV_CTRL_BYTES && off <= w->heap_bytes && bytes <= w->heap_bytes - off;
    };
    const uint64_t mn = (uint64_t)t->max_n, mv = (uint64_t)t->max_vals;
    if (!inside(t->keys_off, mn * 8) || !inside(t->grads_off, mv * 4) ||
        !inside(t->out_off, mv * 4) || !inside(t->pos_off, (w->world + 2) * 8ull) ||
        !inside(t->acc_off, (uint64_t)t->slots * t->width * 4) ||
        (t->lens_off && (!inside(t->lens_off, mn * 4) || !inside(t->offs_off, (mn + 1) * 8))) ||
        (t->capacity && !inside(t->hkeys_off, t->capacity * 8)))
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

// Value offsets of a request with per-key lengths: offs[i] = lens[0] + ... + lens[i-1],
// offs[n] = number of values (device pointers).
int psdev_lens_to_offsets(const int32_t* lens, int64_t n, int64_t* offs, void* stream) {
  if (!lens || !offs || n < 0) return PSDEV_ERR_ARG;
  lens_scan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(lens, n,
                                                         reinterpret_cast<long long*>(offs));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Worker role: lookup + scatter-add of the n (key, gradient) pairs stored in this rank's heap
// (with per-key lengths: the offsets are computed first).
int psdev_sparse_scatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n,
                         int num_ctas, void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, n);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  char* mine = static_cast<char*>(w->peer_base[w->rank]);
  if (t->lens_off) {
    lens_scan_kernel<<<1, 1024, 0, s>>>(reinterpret_cast<const int*>(mine + t->lens_off), n,
                                        reinterpret_cast<long long*>(mine + t->offs_off));
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  // (an empty request still publishes its cut points: the servers read them)
  sparse_scatter_kernel<<<num_ctas > 0 ? num_ctas : default_ctas(), 256, 0, s>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Server role.  `sync` != 0: the kernel first waits until every rank has entered it, i.e.
// until every rank's scatter (which precedes it on that rank's stream) has completed.
int psdev_sparse_apply(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas, int sync,
                       void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, 0);
  if (rc) return rc;
  a.sync = sync ? 1 : 0;
  const int ctas = num_ctas > 0 ? num_ctas : default_ctas();
  sparse_apply_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Server role: answer every worker's pull of the keys it pushed.  `sync` != 0: the kernel ends
// by waiting until every rank's answers have been stored (closing the round that the apply
// kernel opened).
int psdev_sparse_respond(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas, int sync,
                         void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, 0);
  if (rc) return rc;
  a.sync = sync ? 1 : 0;
  const int ctas = num_ctas > 0 ? num_ctas : default_ctas();
  sparse_respond_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

// Server role: the stored length of every key that a worker staged (keys and cut points, see
// psdev_key_shard_lookup) goes into that worker's array of lengths.  The caller orders it after
// every rank's staging and before anybody reads the lengths (psdev_device_barrier on both sides).
int psdev_sparse_lens(const psdev_world_t* w, const psdev_sparse_t* t, int num_ctas,
                      void* stream) {
  SparseArgs a{};
  int rc = fill(&a, w, t, 0);
  if (rc) return rc;
  if (!t->lens_off || !t->klen) return PSDEV_ERR_ARG;
  sparse_lens_kernel<<<num_ctas > 0 ? num_ctas : 296, 256, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

}  // extern "C"
