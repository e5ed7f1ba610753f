// Utility kernels for key lists: radix sort of 64-bit keys (with an optional payload of
// 32-bit indices) and ordered match (merge-join) of two sorted key lists with an assignment
// operator applied to the values of the keys present in both.
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
constexpr int kThreads = 256;
constexpr int kItems = 8;                  // keys per thread, contiguous
constexpr int kTile = kThreads * kItems;   // keys per block
constexpr int kRadixBits = 4;
constexpr int kDigits = 1 << kRadixBits;

__device__ __forceinline__ int digit_of(unsigned long long k, int shift) {
  return (int)((k >> shift) & (kDigits - 1));
}

// counts[d * nblocks + b] = number of keys of block b whose digit is d
__global__ void histogram_kernel(const unsigned long long* keys, long long n, int shift,
                                 unsigned int* counts, int nblocks) {
  __shared__ unsigned int s[kDigits];
  if (threadIdx.x < kDigits) s[threadIdx.x] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * kTile + (long long)threadIdx.x * kItems;
#pragma unroll
  for (int i = 0; i < kItems; ++i)
    if (base + i < n) atomicAdd(&s[digit_of(keys[base + i], shift)], 1u);
  __syncthreads();
  if (threadIdx.x < kDigits) counts[threadIdx.x * nblocks + blockIdx.x] = s[threadIdx.x];
}

// exclusive prefix sum over `len` counters, in place (one block; len = 16 * nblocks)
__global__ void scan_kernel(unsigned int* counts, int len) {
  __shared__ unsigned int s[1024];
  __shared__ unsigned int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < len; base += 1024) {
    const int i = base + threadIdx.x;
    const unsigned int v = i < len ? counts[i] : 0u;
    s[threadIdx.x] = v;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      unsigned int t = threadIdx.x >= off ? s[threadIdx.x - off] : 0u;
      __syncthreads();
      s[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < len) counts[i] = carry + s[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry += s[1023];
    __syncthreads();
  }
}

// stable scatter of one 4-bit digit
__global__ void scatter_kernel(const unsigned long long* keys_in, unsigned long long* keys_out,
                               const unsigned int* pay_in, unsigned int* pay_out, long long n,
                               int shift, const unsigned int* offsets, int nblocks) {
  // per-thread digit counts, then an exclusive scan over threads for every digit
  __shared__ unsigned short cnt[kDigits][kThreads + 1];
  const long long base = (long long)blockIdx.x * kTile + (long long)threadIdx.x * kItems;
  unsigned long long k[kItems];
  int d[kItems];
  unsigned short mine[kDigits];
#pragma unroll
  for (int j = 0; j < kDigits; ++j) mine[j] = 0;
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    d[i] = -1;
    if (base + i < n) {
      k[i] = keys_in[base + i];
      d[i] = digit_of(k[i], shift);
      ++mine[d[i]];
    }
  }
#pragma unroll
  for (int j = 0; j < kDigits; ++j) cnt[j][threadIdx.x] = mine[j];
  __syncthreads();
  // 16 warps-worth of work: thread t < 16 scans digit t over the 256 threads
  if (threadIdx.x < kDigits) {
    unsigned short run = 0;
    for (int t = 0; t < kThreads; ++t) {
      const unsigned short c = cnt[threadIdx.x][t];
      cnt[threadIdx.x][t] = run;
      run += c;
    }
  }
  __syncthreads();
  unsigned int pos[kDigits];
#pragma unroll
  for (int j = 0; j < kDigits; ++j)
    pos[j] = offsets[j * nblocks + blockIdx.x] + cnt[j][threadIdx.x];
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    if (d[i] >= 0) {
      unsigned int p = 0;
#pragma unroll
      for (int j = 0; j < kDigits; ++j)
        if (j == d[i]) p = pos[j]++;
      keys_out[p] = k[i];
      if (pay_in) pay_out[p] = pay_in[base + i];
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
  const int64_t nblocks = (n + kTile - 1) / kTile;
  size_t b = ((size_t)n * 8 + 255) & ~size_t(255);                 // second key buffer
  if (with_payload) b += (((size_t)n * 4 + 255) & ~size_t(255));   // second payload buffer
  b += (((size_t)nblocks * kDigits * 4 + 255) & ~size_t(255));     // digit counters
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
  const int nblocks = (int)((n + kTile - 1) / kTile);
  char* p = static_cast<char*>(scratch);
  p = reinterpret_cast<char*>(((uintptr_t)p + 255) & ~uintptr_t(255));
  unsigned long long* alt = reinterpret_cast<unsigned long long*>(p);
  p += ((size_t)n * 8 + 255) & ~size_t(255);
  unsigned int* alt_pay = nullptr;
  if (perm) {
    alt_pay = reinterpret_cast<unsigned int*>(p);
    p += ((size_t)n * 4 + 255) & ~size_t(255);
    iota_kernel<<<296, 256, 0, s>>>(perm, n);
  }
  unsigned int* counts = reinterpret_cast<unsigned int*>(p);
  unsigned long long* in = reinterpret_cast<unsigned long long*>(keys);
  unsigned long long* out = alt;
  unsigned int* pin = perm;
  unsigned int* pout = alt_pay;
  int passes = (key_bits + kRadixBits - 1) / kRadixBits;
  if (passes & 1) ++passes;  // an even number of passes leaves the result in `keys`
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * kRadixBits;
    if (shift >= 64) {
      // padding pass beyond the key width: plain copy back
      cudaMemcpyAsync(out, in, (size_t)n * 8, cudaMemcpyDeviceToDevice, s);
      if (perm) cudaMemcpyAsync(pout, pin, (size_t)n * 4, cudaMemcpyDeviceToDevice, s);
    } else {
      histogram_kernel<<<nblocks, kThreads, 0, s>>>(in, n, shift, counts, nblocks);
      scan_kernel<<<1, 1024, 0, s>>>(counts, nblocks * kDigits);
      scatter_kernel<<<nblocks, kThreads, 0, s>>>(in, out, pin, pout, n, shift, counts, nblocks);
      g_launches.fetch_add(3, std::memory_order_relaxed);
    }
    unsigned long long* t = in; in = out; out = t;
    unsigned int* tp = pin; pin = pout; pout = tp;
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
