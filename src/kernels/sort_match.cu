// Utility kernels for key lists: radix sort of 64-bit keys, 8 bits per pass (with an
// optional payload of 32-bit indices) and ordered match (merge-join) of two sorted key lists
// with an assignment operator applied to the values of the keys present in both.
//
// They are the device form of helpers the reference ships as headers that nothing includes
// and that do not compile as written: ParallelSort (include/ps/internal/parallel_sort.h:23-55,
// recursive std::thread split + inplace_merge), ParallelOrderedMatch
// (include/ps/internal/parallel_kv_match.h:29-120, recursive merge-join applying
// `dst op= src` per matched key with value width k) and the AssignOp enum
// (include/ps/internal/assign_op.h:12-21).  Users need them to turn unsorted, possibly
// repeated keys into the sorted unique lists Push/Pull require, and servers to match request
// keys against stored keys.
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/psdev.h"

namespace psdev {
extern std::atomic<uint64_t> g_launches;

namespace sortk {
// Least-significant-digit radix sort with 8-bit digits, one sweep per pass:
//   digit_hist   reads the keys once and counts the digits of EVERY pass (shared-memory atomics,
//                then one global add per digit and CTA);
//   digit_scan   exclusive prefix of each pass's 256 totals -> where each digit's run starts;
//   sweep        one launch per pass.  A CTA takes the next tile of 4096 keys from a counter (so
//                every earlier tile belongs to a CTA that is already running), ranks each key
//                among the keys of the same digit in the tile, in input order (the sort is
//                stable), publishes the tile's 256 digit counts, and finds how many keys of each
//                digit precede the tile by looking back over the earlier tiles' published words:
//                a tile's own counts ("aggregate") until one is met whose word already holds the
//                whole prefix ("inclusive").  Keys (and payloads) are then put in sorted order
//                inside the tile in shared memory and stored, runs of equal digits to consecutive
//                addresses.
// ceil(key_bits / 8) passes: a caller that knows its keys are below 2^30 pays four passes,
// not eight.  Per pass every key is read once and written once.
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kItems = 16;                 // keys per thread
constexpr int kTile = kThreads * kItems;   // keys per CTA
constexpr int kRadixBits = 8;
constexpr int kDigits = 1 << kRadixBits;
constexpr int kMaxPasses = 64 / kRadixBits;

// one word per (tile, digit): 2 flag bits and a 30-bit count
constexpr unsigned int kFlagAggregate = 1u << 30;
constexpr unsigned int kFlagInclusive = 2u << 30;
constexpr unsigned int kCountMask = (1u << 30) - 1;
constexpr unsigned long long kLookbackNs = 2000000000ull;  // bound of one look-back wait

// Head of the scratch memory, cleared before every sort.
struct SortHead {
  int error;                                   // 1: a look-back wait ran out
  unsigned int next_tile[kMaxPasses];          // tile counter of each pass
  unsigned int pad[23];
  unsigned int hist[kMaxPasses * kDigits];     // digit totals, then (digit_scan) run starts
};

__device__ __forceinline__ unsigned int digit_of(unsigned long long k, int shift) {
  return (unsigned int)((k >> shift) & (kDigits - 1));
}
__device__ __forceinline__ unsigned int lanemask_lt() {
  unsigned int m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}
__device__ __forceinline__ unsigned int ld_relaxed(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Lanes of the warp whose (valid, digit) equal this lane's: one ballot per digit bit.
__device__ __forceinline__ unsigned int peers_of(unsigned int d, bool valid) {
  unsigned int m = __ballot_sync(0xffffffffu, valid);
  if (!valid) m = ~m;
#pragma unroll
  for (int b = 0; b < kRadixBits; ++b) {
    const bool bit = (d >> b) & 1u;
    const unsigned int v = __ballot_sync(0xffffffffu, bit);
    m &= bit ? v : ~v;
  }
  return m;
}

// hist[pass * 256 + d] += keys whose digit of that pass is d
__global__ void __launch_bounds__(kThreads)
    digit_hist_kernel(const unsigned long long* keys, long long n, int passes, unsigned int* hist) {
  __shared__ unsigned int s[kMaxPasses * kDigits];
  for (int i = threadIdx.x; i < passes * kDigits; i += kThreads) s[i] = 0;
  __syncthreads();
  // four independent loads in flight per thread
  const long long stride = (long long)gridDim.x * kThreads;
  for (long long i0 = blockIdx.x * (long long)kThreads + threadIdx.x; i0 < n; i0 += 4 * stride) {
    unsigned long long k[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) k[u] = i0 + u * stride < n ? keys[i0 + u * stride] : 0ull;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < n)
        for (int p = 0; p < passes; ++p)
          atomicAdd(&s[p * kDigits + digit_of(k[u], p * kRadixBits)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kDigits; i += kThreads)
    if (s[i]) atomicAdd(&hist[i], s[i]);
}

// One CTA per pass: totals -> exclusive prefix (the output index where each digit's run starts).
__global__ void __launch_bounds__(kDigits) digit_scan_kernel(unsigned int* hist) {
  __shared__ unsigned int s[kDigits];
  unsigned int* row = hist + blockIdx.x * kDigits;
  const unsigned int mine = row[threadIdx.x];
  s[threadIdx.x] = mine;
  __syncthreads();
  unsigned int incl = mine;
  for (int off = 1; off < kDigits; off <<= 1) {
    const unsigned int v = threadIdx.x >= off ? s[threadIdx.x - off] : 0u;
    __syncthreads();
    incl += v;
    s[threadIdx.x] = incl;
    __syncthreads();
  }
  row[threadIdx.x] = incl - mine;
}

// One pass.  Shared memory: the tile's keys and payloads in sorted order, per-warp digit
// counters, and two 256-entry tables.
constexpr int kSweepSmem = kTile * 8 + kTile * 4 + kWarps * kDigits * 2 + 2 * kDigits * 4;

__global__ void __launch_bounds__(kThreads, 4)
    sweep_kernel(const unsigned long long* keys_in, unsigned long long* keys_out,
                 const unsigned int* pay_in, unsigned int* pay_out, long long n, int shift,
                 const unsigned int* run_start, unsigned int* status, unsigned int* next_tile,
                 int* error) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* skeys = reinterpret_cast<unsigned long long*>(smem_raw);
  unsigned int* spay = reinterpret_cast<unsigned int*>(smem_raw + kTile * 8);
  // cnt[w][d]: first the number of keys with digit d seen so far by warp w, afterwards the
  // position inside the tile's digit-d run of that warp's first key with digit d
  // (16 bits are enough: a warp holds 512 keys, a tile 4096)
  unsigned short (*cnt)[kDigits] =
      reinterpret_cast<unsigned short (*)[kDigits]>(smem_raw + kTile * 12);
  unsigned int* tile_start = reinterpret_cast<unsigned int*>(smem_raw + kTile * 12 +
                                                             kWarps * kDigits * 2);
  unsigned int* goff = tile_start + kDigits;  // output index of sorted position q: goff[d] + q
  __shared__ unsigned int s_tile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_tile = atomicAdd(next_tile, 1u);
#pragma unroll
  for (int w = 0; w < kWarps; ++w) cnt[w][threadIdx.x] = 0;
  __syncthreads();
  const unsigned int tile = s_tile;
  const long long tile_base = (long long)tile * kTile;
  const long long base = tile_base + (long long)warp * (32 * kItems) + lane;
  const int tile_n = (int)(n - tile_base < kTile ? n - tile_base : kTile);
  unsigned long long k[kItems];
  unsigned short rank[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const long long i = base + j * 32;
    k[j] = i < n ? keys_in[i] : ~0ull;
  }
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const bool valid = base + j * 32 < n;
    const unsigned int d = digit_of(k[j], shift);
    const unsigned int same = peers_of(d, valid);
    const unsigned int before = __popc(same & lanemask_lt());
    unsigned int seen = 0;
    if (valid) seen = cnt[warp][d];
    __syncwarp();
    if (valid && before == 0) cnt[warp][d] = (unsigned short)(seen + __popc(same));
    __syncwarp();
    rank[j] = (unsigned short)(seen + before);
  }
  __syncthreads();
  // digit threadIdx.x: each warp's start inside the digit's run, and the run's length
  unsigned int run = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const unsigned int c = cnt[w][threadIdx.x];
    cnt[w][threadIdx.x] = (unsigned short)run;
    run += c;
  }
  tile_start[threadIdx.x] = run;
  // publish this tile's count of the digit, then add up the earlier tiles' counts
  unsigned int* mine = status + (size_t)tile * kDigits + threadIdx.x;
  unsigned int before_tile = 0;
  if (tile == 0) {
    st_relaxed(mine, kFlagInclusive | run);
  } else {
    st_relaxed(mine, kFlagAggregate | run);
    const unsigned int* look = mine - kDigits;
    unsigned long long t0 = 0;
    for (unsigned int left = tile; left > 0; --left, look -= kDigits) {
      unsigned int v = ld_relaxed(look);
      unsigned int polls = 0;
      while ((v >> 30) == 0) {
        // the earlier tile's CTA is running (it took its tile before this one did) but has not
        // ranked its keys yet
        if ((++polls & 63u) == 0) {
          const unsigned long long t = now_ns();
          if (t0 == 0) t0 = t;
          if (t - t0 > kLookbackNs) break;
        }
        v = ld_relaxed(look);
      }
      if ((v >> 30) == 0) {
        *error = 1;  // the output of this sort is not valid
        break;
      }
      before_tile += v & kCountMask;
      if (v & kFlagInclusive) break;
    }
    st_relaxed(mine, kFlagInclusive | ((before_tile + run) & kCountMask));
  }
  __syncthreads();
  // exclusive prefix of the run lengths over the digits (256 values, one per thread)
  {
    unsigned int incl = run;
    for (int off = 1; off < kDigits; off <<= 1) {
      const unsigned int v = threadIdx.x >= off ? tile_start[threadIdx.x - off] : 0u;
      __syncthreads();
      incl += v;
      tile_start[threadIdx.x] = incl;
      __syncthreads();
    }
    const unsigned int excl = incl - run;
    __syncthreads();
    tile_start[threadIdx.x] = excl;
    goff[threadIdx.x] = run_start[threadIdx.x] + before_tile - excl;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const long long i = base + j * 32;
    if (i < n) {
      const unsigned int d = digit_of(k[j], shift);
      const unsigned int q = tile_start[d] + cnt[warp][d] + rank[j];
      skeys[q] = k[j];
      if (pay_out) spay[q] = pay_in ? pay_in[i] : (unsigned int)i;
    }
  }
  __syncthreads();
#pragma unroll 4
  for (int j = 0; j < kItems; ++j) {
    const int q = threadIdx.x + j * kThreads;
    if (q < tile_n) {
      const unsigned long long key = skeys[q];
      const unsigned int p = goff[digit_of(key, shift)] + (unsigned int)q;
      keys_out[p] = key;
      if (pay_out) pay_out[p] = spay[q];
    }
  }
}

// ---- ordered match -------------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ V apply_op(int op, V dst, V src) {
  switch (op) {
    case 0: return src;        // ASSIGN
    case 1: return dst + src;  // PLUS
    case 2: return dst - src;  // MINUS
    case 3: return dst * src;  // TIMES
    case 4: return dst / src;  // DIVIDE
    default: return dst;
  }
}
__device__ __forceinline__ int apply_bitop(int op, int dst, int src) {
  switch (op) {
    case 5: return dst & src;  // AND
    case 6: return dst | src;  // OR
    case 7: return dst ^ src;  // XOR
    default: return apply_op<int>(op, dst, src);
  }
}

// For every src key: binary search among the dst keys; on a hit, dst_val[j*k..] op= src_val[i*k..]
template <typename V, bool INT>
__global__ void ordered_match_kernel(const unsigned long long* src_keys, const V* src_vals,
                                     long long n_src, const unsigned long long* dst_keys,
                                     V* dst_vals, long long n_dst, int k, int op,
                                     unsigned long long* matched) {
  unsigned long long local = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_src;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long key = src_keys[i];
    long long lo = 0, hi = n_dst;
    while (lo < hi) {
      const long long m = (lo + hi) >> 1;
      if (dst_keys[m] < key) lo = m + 1; else hi = m;
    }
    if (lo < n_dst && dst_keys[lo] == key) {
      ++local;
      for (int j = 0; j < k; ++j) {
        V* d = dst_vals + lo * k + j;
        const V s = src_vals[i * k + j];
        if constexpr (INT) *d = (V)apply_bitop(op, (int)*d, (int)s);
        else *d = apply_op<V>(op, *d, s);
      }
    }
  }
  if (local) atomicAdd(matched, local);
}

}  // namespace sortk
}  // namespace psdev

using namespace psdev;
using namespace psdev::sortk;

extern "C" {

static size_t round256(size_t b) { return (b + 255) & ~size_t(255); }

// Bytes of scratch psdev_sort_keys needs for n keys (with or without a payload).
size_t psdev_sort_scratch_bytes(int64_t n, int with_payload) {
  const size_t ntiles = (size_t)((n + kTile - 1) / kTile);
  size_t b = round256(sizeof(SortHead));
  b += round256(ntiles * kDigits * 4 * kMaxPasses);   // one word per (pass, tile, digit)
  b += round256((size_t)n * 8);                        // second key buffer
  if (with_payload) b += round256((size_t)n * 4);      // second payload buffer
  return b + 256;
}

// Sorts `n` 64-bit keys ascending by their low `key_bits` bits (64 for full keys; fewer bits
// = fewer passes).  `keys` is sorted in place.  If `perm` is not NULL it receives, for every
// output position, the index the key had in the input (a stable sort permutation).
// `scratch` is device memory of psdev_sort_scratch_bytes(n, perm != NULL) bytes; n < 2^30.
// psdev_sort_status(scratch) tells afterwards whether a wait inside the sort ran out.
int psdev_sort_keys(uint64_t* keys, uint32_t* perm, int64_t n, int key_bits, void* scratch,
                    size_t scratch_bytes, void* stream) {
  if (n < 0 || key_bits < 1 || key_bits > 64 || !keys) return PSDEV_ERR_ARG;
  if (n == 0) return 0;
  if (n >= (int64_t)1 << 30) return PSDEV_ERR_UNSUPPORTED;
  if (!scratch || scratch_bytes < psdev_sort_scratch_bytes(n, perm != nullptr))
    return PSDEV_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int ntiles = (int)((n + kTile - 1) / kTile);
  const int passes = (key_bits + kRadixBits - 1) / kRadixBits;
  char* p = static_cast<char*>(scratch);
  p = reinterpret_cast<char*>(((uintptr_t)p + 255) & ~uintptr_t(255));
  SortHead* head = reinterpret_cast<SortHead*>(p);
  p += round256(sizeof(SortHead));
  unsigned int* status = reinterpret_cast<unsigned int*>(p);
  const size_t status_pass = (size_t)ntiles * kDigits;
  // head and the status words of the passes that run are cleared together
  const size_t clear = round256(sizeof(SortHead)) + status_pass * 4 * passes;
  p += round256(status_pass * 4 * kMaxPasses);
  unsigned long long* alt = reinterpret_cast<unsigned long long*>(p);
  p += round256((size_t)n * 8);
  unsigned int* alt_pay = nullptr;
  if (perm) alt_pay = reinterpret_cast<unsigned int*>(p);
  {
    // the sweep kernel's tile buffers exceed the default limit of dynamic shared memory
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(sweep_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kSweepSmem);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev & 63].store(true, std::memory_order_release);
    }
  }
  cudaMemsetAsync(head, 0, clear, s);
  unsigned long long* in = reinterpret_cast<unsigned long long*>(keys);
  unsigned long long* out = alt;
  unsigned int* pin = perm;
  unsigned int* pout = alt_pay;
  const int hist_ctas = ntiles < 592 ? ntiles : 592;
  digit_hist_kernel<<<hist_ctas, kThreads, 0, s>>>(in, n, passes, head->hist);
  digit_scan_kernel<<<passes, kDigits, 0, s>>>(head->hist);
  g_launches.fetch_add(2, std::memory_order_relaxed);
  for (int pass = 0; pass < passes; ++pass) {
    // the first pass makes the payload: the index of every key in the input
    sweep_kernel<<<ntiles, kThreads, kSweepSmem, s>>>(
        in, out, pass == 0 ? nullptr : pin, pout, n, pass * kRadixBits,
        head->hist + pass * kDigits,
        status + status_pass * pass, &head->next_tile[pass], &head->error);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    unsigned long long* t = in; in = out; out = t;
    unsigned int* tp = pin; pin = pout; pout = tp;
  }
  if (passes & 1) {
    // an odd number of passes leaves the result in the scratch buffers
    cudaMemcpyAsync(keys, in, (size_t)n * 8, cudaMemcpyDeviceToDevice, s);
    if (perm) cudaMemcpyAsync(perm, pin, (size_t)n * 4, cudaMemcpyDeviceToDevice, s);
  }
  return (int)cudaGetLastError();
}

// 0 when the last sort that used `scratch` completed every look-back, PSDEV_ERR_TIMEOUT_ENTRY
// when one ran out (the output of that sort is not valid).  Waits for `stream`.
int psdev_sort_status(const void* scratch, void* stream) {
  if (!scratch) return PSDEV_ERR_ARG;
  const char* p = reinterpret_cast<const char*>(((uintptr_t)scratch + 255) & ~uintptr_t(255));
  int err = 0;
  cudaError_t e = cudaMemcpyAsync(&err, p, sizeof(int), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return err ? PSDEV_ERR_TIMEOUT_ENTRY : 0;
}

// dst_vals[j] op= src_vals[i] for every key present in both sorted unique lists; values have
// `k` elements per key.  op: 0 assign, 1 plus, 2 minus, 3 times, 4 divide, and for int32
// values also 5 and, 6 or, 7 xor.  dtype: 0 = float32, 1 = int32.  `*matched` (device, 8
// bytes, must be zeroed by the caller) receives the number of matched keys.
int psdev_ordered_match(const uint64_t* src_keys, const void* src_vals, int64_t n_src,
                        const uint64_t* dst_keys, void* dst_vals, int64_t n_dst, int k, int op,
                        int dtype, uint64_t* matched, void* stream) {
  if (k < 1 || op < 0 || op > 7 || (dtype == 0 && op > 4) || !matched) return PSDEV_ERR_ARG;
  if (n_src == 0 || n_dst == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned long long* sk = reinterpret_cast<const unsigned long long*>(src_keys);
  const unsigned long long* dk = reinterpret_cast<const unsigned long long*>(dst_keys);
  unsigned long long* m = reinterpret_cast<unsigned long long*>(matched);
  if (dtype == 0)
    ordered_match_kernel<float, false><<<592, 256, 0, s>>>(sk, static_cast<const float*>(src_vals),
                                                           n_src, dk, static_cast<float*>(dst_vals),
                                                           n_dst, k, op, m);
  else if (dtype == 1)
    ordered_match_kernel<int, true><<<592, 256, 0, s>>>(sk, static_cast<const int*>(src_vals),
                                                        n_src, dk, static_cast<int*>(dst_vals),
                                                        n_dst, k, op, m);
  else
    return PSDEV_ERR_UNSUPPORTED;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

}  // extern "C"
