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
// Least-significant-digit radix sort with 8-bit digits.  One pass = three kernels:
//   tile_count  every CTA counts the digits of its tile of 4096 keys (warp-aggregated shared
//               atomics) into hist[digit][tile] and adds them to the pass's 256 digit totals;
//   tile_scan   one CTA per digit: exclusive prefix of that digit's row over the tiles, plus
//               the number of keys with smaller digits -> where each (digit, tile) group starts;
//   scatter     every CTA re-reads its tile, ranks each key among the keys of the same digit
//               in the tile, in input order (the sort is stable), and stores key and payload at
//               group start + rank.
// ceil(key_bits / 8) passes: a caller that knows its keys are below 2^30 pays four passes,
// not eight.
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kItems = 16;                 // keys per thread
constexpr int kTile = kThreads * kItems;   // keys per CTA
constexpr int kRadixBits = 8;
constexpr int kDigits = 1 << kRadixBits;

__device__ __forceinline__ unsigned int digit_of(unsigned long long k, int shift) {
  return (unsigned int)((k >> shift) & (kDigits - 1));
}
__device__ __forceinline__ unsigned int lanemask_lt() {
  unsigned int m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// hist[d * ntiles + tile] = keys of the tile with digit d; totals[d] += the same
__global__ void __launch_bounds__(kThreads)
    tile_count_kernel(const unsigned long long* keys, long long n, int shift, unsigned int* hist,
                      unsigned int* totals, int ntiles) {
  __shared__ unsigned int s[kDigits];
  s[threadIdx.x] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long base = (long long)blockIdx.x * kTile + (long long)warp * (32 * kItems) + lane;
#pragma unroll 4
  for (int j = 0; j < kItems; ++j) {
    const long long i = base + j * 32;
    const bool valid = i < n;
    // lanes past the end vote with a digit no key can have
    const unsigned int d = valid ? digit_of(keys[i], shift) : (unsigned int)kDigits;
    const unsigned int same = __match_any_sync(0xffffffffu, d);
    if (valid && (same & lanemask_lt()) == 0) atomicAdd(&s[d], (unsigned int)__popc(same));
  }
  __syncthreads();
  const unsigned int c = s[threadIdx.x];
  hist[(size_t)threadIdx.x * ntiles + blockIdx.x] = c;
  if (c) atomicAdd(&totals[threadIdx.x], c);
}

// One CTA per digit: hist row -> exclusive prefix over the tiles + keys with smaller digits.
__global__ void __launch_bounds__(1024)
    tile_scan_kernel(unsigned int* hist, const unsigned int* totals, int ntiles) {
  __shared__ unsigned int s[1024];
  __shared__ unsigned int carry;
  const int d = blockIdx.x;
  // keys with a smaller digit
  unsigned int below = 0;
  for (int j = threadIdx.x; j < d; j += 1024) below += totals[j];
  s[threadIdx.x] = below;
  __syncthreads();
  for (int off = 512; off > 0; off >>= 1) {
    if (threadIdx.x < off) s[threadIdx.x] += s[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) carry = s[0];
  __syncthreads();
  unsigned int* row = hist + (size_t)d * ntiles;
  for (int base = 0; base < ntiles; base += 1024) {
    const int i = base + threadIdx.x;
    const unsigned int v = i < ntiles ? row[i] : 0u;
    __syncthreads();
    s[threadIdx.x] = v;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const unsigned int t = threadIdx.x >= off ? s[threadIdx.x - off] : 0u;
      __syncthreads();
      s[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < ntiles) row[i] = carry + s[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry += s[1023];
  }
}

// Stable scatter of one 8-bit digit.  Keys (and payloads) are first put in sorted order inside
// the tile in shared memory, then stored: consecutive threads store consecutive keys of one
// digit, i.e. consecutive addresses.
constexpr int kScatterSmem = kTile * 8 + kTile * 4 + kWarps * kDigits * 4 + 2 * kDigits * 4;

__global__ void __launch_bounds__(kThreads)
    scatter_kernel(const unsigned long long* keys_in, unsigned long long* keys_out,
                   const unsigned int* pay_in, unsigned int* pay_out, long long n, int shift,
                   const unsigned int* offsets, int ntiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* skeys = reinterpret_cast<unsigned long long*>(smem_raw);
  unsigned int* spay = reinterpret_cast<unsigned int*>(smem_raw + kTile * 8);
  // cnt[w][d]: first the number of keys with digit d seen so far by warp w, afterwards the
  // position inside the tile's digit-d run of that warp's first key with digit d
  unsigned int (*cnt)[kDigits] =
      reinterpret_cast<unsigned int (*)[kDigits]>(smem_raw + kTile * 12);
  unsigned int* tile_start = reinterpret_cast<unsigned int*>(smem_raw + kTile * 12 +
                                                             kWarps * kDigits * 4);
  unsigned int* goff = tile_start + kDigits;  // output index of sorted position q: goff[d] + q
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) cnt[w][threadIdx.x] = 0;
  __syncthreads();
  const long long tile_base = (long long)blockIdx.x * kTile;
  const long long base = tile_base + (long long)warp * (32 * kItems) + lane;
  const int tile_n = (int)(n - tile_base < kTile ? n - tile_base : kTile);
  unsigned long long k[kItems];
  unsigned short rank[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const long long i = base + j * 32;
    const bool valid = i < n;
    k[j] = valid ? keys_in[i] : ~0ull;
    const unsigned int d = valid ? digit_of(k[j], shift) : (unsigned int)kDigits;
    const unsigned int same = __match_any_sync(0xffffffffu, d);
    const unsigned int before = __popc(same & lanemask_lt());
    unsigned int seen = 0;
    if (valid) seen = cnt[warp][d];
    __syncwarp();
    if (valid && before == 0) cnt[warp][d] = seen + __popc(same);
    __syncwarp();
    rank[j] = (unsigned short)(seen + before);
  }
  __syncthreads();
  {
    // digit threadIdx.x: each warp's start inside the digit's run, and the run's length
    unsigned int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned int c = cnt[w][threadIdx.x];
      cnt[w][threadIdx.x] = run;
      run += c;
    }
    tile_start[threadIdx.x] = run;
  }
  __syncthreads();
  // exclusive prefix of the run lengths over the digits (256 values, one per thread)
  {
    const unsigned int mine = tile_start[threadIdx.x];
    unsigned int incl = mine;
    for (int off = 1; off < kDigits; off <<= 1) {
      const unsigned int v = threadIdx.x >= off ? tile_start[threadIdx.x - off] : 0u;
      __syncthreads();
      incl += v;
      tile_start[threadIdx.x] = incl;
      __syncthreads();
    }
    const unsigned int excl = incl - mine;
    __syncthreads();
    tile_start[threadIdx.x] = excl;
    goff[threadIdx.x] = offsets[(size_t)threadIdx.x * ntiles + blockIdx.x] - excl;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const long long i = base + j * 32;
    if (i < n) {
      const unsigned int d = digit_of(k[j], shift);
      const unsigned int q = tile_start[d] + cnt[warp][d] + rank[j];
      skeys[q] = k[j];
      if (pay_in) spay[q] = pay_in[i];
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
      if (pay_in) pay_out[p] = spay[q];
    }
  }
}

__global__ void iota_kernel(unsigned int* p, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    p[i] = (unsigned int)i;
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

// Bytes of scratch psdev_sort_keys needs for n keys (with or without a payload).
size_t psdev_sort_scratch_bytes(int64_t n, int with_payload) {
  const int64_t ntiles = (n + kTile - 1) / kTile;
  size_t b = ((size_t)n * 8 + 255) & ~size_t(255);                 // second key buffer
  if (with_payload) b += (((size_t)n * 4 + 255) & ~size_t(255));   // second payload buffer
  b += (((size_t)ntiles * kDigits * 4 + 255) & ~size_t(255));      // digit counts per tile
  b += 8 * kDigits * 4;                                            // digit totals per pass
  return b + 256;
}

// Sorts `n` 64-bit keys ascending by their low `key_bits` bits (64 for full keys; fewer bits
// = fewer passes).  `keys` is sorted in place.  If `perm` is not NULL it receives, for every
// output position, the index the key had in the input (a stable sort permutation).
// `scratch` is device memory of psdev_sort_scratch_bytes(n, perm != NULL) bytes.
int psdev_sort_keys(uint64_t* keys, uint32_t* perm, int64_t n, int key_bits, void* scratch,
                    size_t scratch_bytes, void* stream) {
  if (n < 0 || key_bits < 1 || key_bits > 64 || !keys) return PSDEV_ERR_ARG;
  if (n == 0) return 0;
  if (n >= (int64_t)1 << 32) return PSDEV_ERR_UNSUPPORTED;
  if (!scratch || scratch_bytes < psdev_sort_scratch_bytes(n, perm != nullptr))
    return PSDEV_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int ntiles = (int)((n + kTile - 1) / kTile);
  char* p = static_cast<char*>(scratch);
  p = reinterpret_cast<char*>(((uintptr_t)p + 255) & ~uintptr_t(255));
  unsigned long long* alt = reinterpret_cast<unsigned long long*>(p);
  p += ((size_t)n * 8 + 255) & ~size_t(255);
  unsigned int* alt_pay = nullptr;
  if (perm) {
    alt_pay = reinterpret_cast<unsigned int*>(p);
    p += ((size_t)n * 4 + 255) & ~size_t(255);
    iota_kernel<<<296, 256, 0, s>>>(perm, n);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  unsigned int* hist = reinterpret_cast<unsigned int*>(p);
  p += ((size_t)ntiles * kDigits * 4 + 255) & ~size_t(255);
  unsigned int* totals = reinterpret_cast<unsigned int*>(p);
  const int passes = (key_bits + kRadixBits - 1) / kRadixBits;
  {
    // the scatter kernel's tile buffers exceed the default limit of dynamic shared memory
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(scatter_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kScatterSmem);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev & 63].store(true, std::memory_order_release);
    }
  }
  cudaMemsetAsync(totals, 0, (size_t)passes * kDigits * 4, s);
  unsigned long long* in = reinterpret_cast<unsigned long long*>(keys);
  unsigned long long* out = alt;
  unsigned int* pin = perm;
  unsigned int* pout = alt_pay;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * kRadixBits;
    unsigned int* tot = totals + pass * kDigits;
    tile_count_kernel<<<ntiles, kThreads, 0, s>>>(in, n, shift, hist, tot, ntiles);
    tile_scan_kernel<<<kDigits, 1024, 0, s>>>(hist, tot, ntiles);
    scatter_kernel<<<ntiles, kThreads, kScatterSmem, s>>>(in, out, pin, pout, n, shift, hist,
                                                         ntiles);
    g_launches.fetch_add(3, std::memory_order_relaxed);
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
