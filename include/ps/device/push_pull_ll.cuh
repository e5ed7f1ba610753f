// Low-latency form of the fused push+pull for small requests.
//
// The general kernel (push_pull.cuh) brackets its work with two flag rendezvous: "everybody's
// gradients are in place" before, "everybody's stores have landed" after.  Each costs a system
// fence and a flag round; below a few hundred kilobytes those two rounds ARE the cost of the
// request.  Here no separate flag exists: every 4-byte value travels in an 8-byte word next to
// the 32-bit sequence number of the round, written with one 8-byte store (single-copy atomic),
// and the receiver polls the word itself -- a value is known to have arrived when its
// sequence number matches.  One round is then
//     A  every worker stores (gradient, seq) into the OWNER's receive slots   [one NVLink hop]
//     B  the owner polls its W slots per value, sums in rank order, applies the server
//        handle to its fp32 master and stores (new weight, seq) into EVERY worker's receive
//        buffer                                                               [one NVLink hop]
//     C  every worker polls its receive buffer and writes its weight buffer.
// No fence, no second round.  The price is twice the bytes on the wire, which is why the host
// dispatch uses this kernel only up to `ll_cap` values per request.
//
// Buffers (symmetric heap, per table, zero-initialised; `ll_off` = offset of the region):
//     header   256 bytes: [0] sequence number of the last completed round, [1] CTA counter
//     push     W slots x ll_cap words: slot p, word k = rank p's contribution for value begin+k
//     pull     ll_cap words: word k = new weight of value begin+k
// Reuse across rounds is safe without double buffering because a worker starts round i+1 only
// after it has received every weight of round i, which an owner sends only after it has
// consumed every contribution of round i.
//
// Every poll is bounded by the timeout; on expiry the channel's status word receives
// PSDEV_ERR_TIMEOUT_ENTRY and the kernel returns without touching master or weights further.
//
// The reference moves a small push as one message per server through its van
// (include/ps/kv_app.h:574-613) and pays a socket round trip; this is the device-plane answer
// to its "priority send of small slices" use (src/p3_van.h:40-50).
#pragma once
#include "ps/device/push_pull.cuh"

namespace psdev {

constexpr int kLLThreads = 512;
constexpr int kLLHeaderBytes = 256;

struct LLArgs {
  void* base[PSDEV_MAX_RANKS];
  int rank, world;
  unsigned long long grad_off, weight_off, ll_off;
  long long ll_cap;      // words per slot
  long long blk, begin, end;
  float* master;
  float* s1;
  float* s2;
  psdev_opt_t opt;
  int channel;
  unsigned long long timeout_ns;
  long long n_total, local_len;  // extents for the checks build
};

struct LLHeader {
  unsigned int seq;   // last completed round
  unsigned int done;  // CTAs that have finished the current round
};

__device__ __forceinline__ void ll_store(unsigned long long* p, unsigned int data,
                                         unsigned int seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(seq)
               : "memory");
}
// Polls one word until its sequence number is `seq`; false after the deadline.
__device__ __forceinline__ bool ll_wait(const unsigned long long* p, unsigned int seq,
                                        unsigned long long timeout_ns, unsigned int* data) {
  unsigned int d, s;
  for (int i = 0; i < 256; ++i) {
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(d), "=r"(s) : "l"(p) : "memory");
    if (s == seq) {
      *data = d;
      return true;
    }
  }
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(d), "=r"(s) : "l"(p) : "memory");
    if (s == seq) {
      *data = d;
      return true;
    }
    if (globaltimer_ns() - t0 > timeout_ns) return false;
    __nanosleep(64);
  }
}

template <typename GT>
__device__ __forceinline__ unsigned int ll_pack(const GT* g, long long i);
template <>
__device__ __forceinline__ unsigned int ll_pack<float>(const float* g, long long i) {
  return __float_as_uint(g[i]);
}
template <>
__device__ __forceinline__ unsigned int ll_pack<__nv_bfloat16>(const __nv_bfloat16* g,
                                                               long long i) {
  return (unsigned int)__bfloat16_as_ushort(g[i]);
}
template <typename GT>
__device__ __forceinline__ float ll_unpack(unsigned int u);
template <>
__device__ __forceinline__ float ll_unpack<float>(unsigned int u) {
  return __uint_as_float(u);
}
template <>
__device__ __forceinline__ float ll_unpack<__nv_bfloat16>(unsigned int u) {
  return __bfloat162float(__ushort_as_bfloat16((unsigned short)u));
}

// One word per value (a bf16 gradient occupies the low half of its word): requests are small,
// what counts is the number of hops, not the bytes.
template <typename GT, typename OT, class Opt>
__global__ void __launch_bounds__(kLLThreads) dense_ll_kernel(const __grid_constant__ LLArgs a) {
  __shared__ unsigned int s_seq;
  __shared__ int s_err;
  const int W = a.world, R = a.rank;
  Ctrl* ctrl = ctrl_of(a.base[R]);
  char* mine = static_cast<char*>(a.base[R]);
  LLHeader* hdr = reinterpret_cast<LLHeader*>(mine + a.ll_off);
  if (threadIdx.x == 0) {
    unsigned int seq = *(volatile unsigned int*)&hdr->seq + 1u;
    if (seq == 0u) seq = 1u;  // zero marks a word that was never written
    s_seq = seq;
    s_err = (*(volatile int*)&ctrl->status[a.channel] != 0);
  }
  __syncthreads();
  const unsigned int seq = s_seq;
  bool ok = !s_err;
  const long long m = a.end - a.begin;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long push_off = a.ll_off + kLLHeaderBytes;
  const unsigned long long pull_off = push_off + (unsigned long long)W * a.ll_cap * 8ull;

  if (ok) {
    // A: my contribution for value begin+k goes into slot R of its owner
    const GT* grad = reinterpret_cast<const GT*>(mine + a.grad_off);
    for (long long k = t0; k < m; k += stride) {
      const long long i = a.begin + k;
      const int o = (int)((i / a.blk) % W);
      unsigned long long* dst =
          reinterpret_cast<unsigned long long*>(static_cast<char*>(a.base[o]) + push_off) +
          (long long)R * a.ll_cap + k;
      ll_store(dst, ll_pack<GT>(grad, i), seq);
    }
    // B: values I own -- wait for every worker's word, reduce, update, send the new weight out
    const unsigned long long* slots = reinterpret_cast<const unsigned long long*>(mine + push_off);
    for (long long k = t0; k < m && ok; k += stride) {
      const long long i = a.begin + k;
      const long long j = i / a.blk;
      if ((int)(j % W) != R) continue;
      const long long si = (j / W) * a.blk + (i - j * a.blk);
#ifdef PSDEV_CHECKS
      if (i < 0 || i >= a.n_total || si < 0 || si >= a.local_len) {
        atomicMin(&ctrl->status[a.channel], (int)PSDEV_ERR_BOUNDS);
        ok = false;
        break;
      }
#endif
      float g = 0.f;
      for (int p = 0; p < W; ++p) {
        unsigned int u;
        if (!ll_wait(slots + (long long)p * a.ll_cap + k, seq, a.timeout_ns, &u)) {
          atomicOr(&ctrl->late_mask[a.channel], 1u << p);
          atomicMin(&ctrl->status[a.channel], (int)PSDEV_ERR_TIMEOUT_ENTRY);
          ok = false;
          break;
        }
        g += ll_unpack<GT>(u);
      }
      if (!ok) break;
      float w = a.master[si];
      float mm = Opt::kStates >= 1 ? a.s1[si] : 0.f;
      float vv = Opt::kStates >= 2 ? a.s2[si] : 0.f;
      Opt::apply(w, g * a.opt.scale, mm, vv, a.opt);
      a.master[si] = w;
      if (Opt::kStates >= 1) a.s1[si] = mm;
      if (Opt::kStates >= 2) a.s2[si] = vv;
      // what the workers receive is the value as their weight buffer will hold it
      unsigned int out;
      if constexpr (sizeof(OT) == 4) out = __float_as_uint(w);
      else out = (unsigned int)__bfloat16_as_ushort(__float2bfloat16_rn(w));
      for (int pp = 0; pp < W; ++pp) {
        int p = R + pp;
        if (p >= W) p -= W;
        unsigned long long* dst =
            reinterpret_cast<unsigned long long*>(static_cast<char*>(a.base[p]) + pull_off) + k;
        ll_store(dst, out, seq);
      }
    }
    // C: my copy of every value of the request
    const unsigned long long* in = reinterpret_cast<const unsigned long long*>(mine + pull_off);
    OT* weight = reinterpret_cast<OT*>(mine + a.weight_off);
    for (long long k = t0; k < m && ok; k += stride) {
      unsigned int u;
      if (!ll_wait(in + k, seq, a.timeout_ns, &u)) {
        atomicOr(&ctrl->late_mask[a.channel], 1u << (int)(((a.begin + k) / a.blk) % W));
        atomicMin(&ctrl->status[a.channel], (int)PSDEV_ERR_TIMEOUT_EXIT);
        ok = false;
        break;
      }
      if constexpr (sizeof(OT) == 4) weight[a.begin + k] = __uint_as_float(u);
      else weight[a.begin + k] = __ushort_as_bfloat16((unsigned short)u);
    }
  }
  // the last CTA to finish closes the round: the next launch uses the next sequence number
  // (also after a failure, so that stale words of this round are never mistaken for new ones)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&hdr->done, 1u) == gridDim.x - 1) {
      hdr->done = 0;
      hdr->seq = seq;
      __threadfence();
    }
  }
}

}  // namespace psdev
