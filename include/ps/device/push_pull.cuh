// Fused dense push / pull kernel template.
//
// One launch per rank.  The rank acts as the server of the key blocks it owns inside the
// requested element range: for each 16-byte vector it
//   (push)  loads the vector from every worker's gradient buffer (its own HBM and up to
//           seven peers over NVLink), sums in fp32 in rank order, scales, and applies the
//           server handle `Opt` to its fp32 master weights and optimizer state;
//   (pull)  casts the new weights and stores them into every worker's weight buffer.
// The summed gradient is never written to memory, and there is no message, no staging
// buffer and no library collective: the reduce-scatter and the all-gather are the loads
// and stores of this kernel.
//
// This replaces the reference's push path (KVWorker::Send slicing + van transfer,
// include/ps/kv_app.h:574-613, and the CPU server handle, :440-463) and its pull path
// (server response + worker-side sort/memcpy reassembly, :616-717).
//
// A user-defined server handle is any struct with the static interface of the Opt*
// structs below; instantiate `dense_kernel<GT, OT, MyOpt, true, true>` in your own .cu.
#pragma once
#include "ps/device/dev_common.cuh"

namespace psdev {

constexpr int kDenseThreads = 512;

// One slice of a multi-slice launch, in the order the CTAs consume them (highest priority
// first).  Entry [nseg] is a sentinel whose tile_begin is the total number of tiles.
struct SchedEntry {
  long long begin, end;    // element range of the slice
  long long first_owned;   // first block of the slice owned by this rank
  long long n_owned;       // owned blocks that meet the slice
  long long tile_begin;    // index of the slice's first tile in the launch-wide tile order
};

struct DenseArgs {
  void* base[PSDEV_MAX_RANKS];
  void* mc_base;  // multicast alias of the heap (used by the MC kernel variant only)
  int rank, world;
  unsigned long long grad_off, weight_off;
  unsigned long long gscale_off;  // int8 gradients: heap offset of the fp32 scales (one per 256)
  long long blk, begin, end;
  long long first_owned;  // first block index owned by this rank that meets [begin,end)
  long long n_owned;      // how many owned blocks meet the range
  long long tiles_per_blk;
  float* master;
  float* s1;
  float* s2;
  psdev_opt_t opt;
  int channel, sync;
  int self_only;  // broadcast stores go to this rank's own weight buffer only (publish)
  const SchedEntry* sched;  // multi-slice launch: nseg+1 entries written by the schedule kernel
  int nseg;                 // 0: single range [begin, end)
  const long long* segs_in; // multi-slice launch: nseg x (begin, end, priority), device memory
  unsigned long long timeout_ns;
  // extents, used by the checks build (-DPSDEV_CHECKS): arena size (0 = unknown), elements of
  // the table, elements of this rank's master/state arrays
  unsigned long long heap_bytes;
  long long n_total, local_len;
};

#ifdef PSDEV_CHECKS
// Checks build: may the vector of VEC elements at table index i (state index si) be touched?
template <typename GT, typename OT, int VEC>
__device__ __forceinline__ bool dense_index_ok(const DenseArgs& a, long long i, long long si) {
  if (i < 0 || i + VEC > a.n_total || si < 0 || si + VEC > a.local_len) return false;
  if (a.heap_bytes) {
    if (a.grad_off + (unsigned long long)(i + VEC) * sizeof(GT) > a.heap_bytes) return false;
    if (a.weight_off + (unsigned long long)(i + VEC) * sizeof(OT) > a.heap_bytes) return false;
  }
  return true;
}
#endif

// ---- server handles ---------------------------------------------------------------
// apply(w, g, s1, s2, o): g is the scaled sum over workers; w, s1, s2 are updated in place.
struct OptSum {
  static constexpr int kStates = 0;
  __device__ static __forceinline__ void apply(float& w, float g, float&, float&,
                                               const psdev_opt_t&) {
    w += g;
  }
};
struct OptAssign {
  static constexpr int kStates = 0;
  __device__ static __forceinline__ void apply(float& w, float g, float&, float&,
                                               const psdev_opt_t&) {
    w = g;
  }
};
struct OptSgd {
  static constexpr int kStates = 0;
  __device__ static __forceinline__ void apply(float& w, float g, float&, float&,
                                               const psdev_opt_t& o) {
    g = fmaf(o.weight_decay, w, g);
    w = fmaf(-o.lr, g, w);
  }
};
struct OptMomentum {
  static constexpr int kStates = 1;
  __device__ static __forceinline__ void apply(float& w, float g, float& m, float&,
                                               const psdev_opt_t& o) {
    g = fmaf(o.weight_decay, w, g);
    m = fmaf(o.momentum, m, g);
    w = fmaf(-o.lr, m, w);
  }
};
struct OptAdam {
  static constexpr int kStates = 2;
  __device__ static __forceinline__ void apply(float& w, float g, float& m, float& v,
                                               const psdev_opt_t& o) {
    if (o.decoupled_wd) {
      w *= (1.f - o.lr * o.weight_decay);
    } else {
      g = fmaf(o.weight_decay, w, g);
    }
    m = fmaf(o.beta1, m, (1.f - o.beta1) * g);
    v = fmaf(o.beta2, v, (1.f - o.beta2) * g * g);
    const float denom = sqrtf(v) / o.bias2 + o.eps;
    w -= (o.lr / o.bias1) * (m / denom);
  }
};

// ---- vector helpers -----------------------------------------------------------------
template <typename T>
struct VecOf;
template <>
struct VecOf<float> {
  static constexpr int kPer16 = 4;
  __device__ static __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
};
template <>
struct VecOf<__nv_bfloat16> {
  static constexpr int kPer16 = 8;
  __device__ static __forceinline__ void unpack(const uint4& u, float* f) {
    float2 a = bf16x2_to_f2(u.x), b = bf16x2_to_f2(u.y), c = bf16x2_to_f2(u.z),
           d = bf16x2_to_f2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
};

// Stores VEC weights as OT at dst.  MC: dst is a multicast address (one store reaches every
// rank's buffer); otherwise an ordinary (local or peer) address.
// int8 gradients with one fp32 scale per 256 values (the block-scale filter): sixteen values
// per 16-byte load; the scale is applied when the vector is added to the sum.
template <>
struct VecOf<signed char> {
  static constexpr int kPer16 = 16;
  __device__ static __forceinline__ void unpack(const uint4& u, float* f) {
    const unsigned int w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int b = 0; b < 4; ++b) f[4 * j + b] = (float)(signed char)((w[j] >> (8 * b)) & 0xff);
    }
  }
};
constexpr int kInt8Group = 256;

template <typename OT, int VEC, bool MC = false>
__device__ __forceinline__ void store_out(OT* dst, const float* w) {
  if constexpr (sizeof(OT) == 4) {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      uint4 u = make_uint4(__float_as_uint(w[4 * q]), __float_as_uint(w[4 * q + 1]),
                           __float_as_uint(w[4 * q + 2]), __float_as_uint(w[4 * q + 3]));
      if constexpr (MC) multimem_st_v4(dst + 4 * q, u); else st_v4(dst + 4 * q, u);
    }
  } else {
    if constexpr (VEC == 16) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float* x = w + 8 * h;
        uint4 u = make_uint4(f2_to_bf16x2(x[0], x[1]), f2_to_bf16x2(x[2], x[3]),
                             f2_to_bf16x2(x[4], x[5]), f2_to_bf16x2(x[6], x[7]));
        if constexpr (MC) multimem_st_v4(dst + 8 * h, u); else st_v4(dst + 8 * h, u);
      }
    } else if constexpr (VEC == 8) {
      uint4 u = make_uint4(f2_to_bf16x2(w[0], w[1]), f2_to_bf16x2(w[2], w[3]),
                           f2_to_bf16x2(w[4], w[5]), f2_to_bf16x2(w[6], w[7]));
      if constexpr (MC) multimem_st_v4(dst, u); else st_v4(dst, u);
    } else {
      uint2 u = make_uint2(f2_to_bf16x2(w[0], w[1]), f2_to_bf16x2(w[2], w[3]));
      if constexpr (MC) multimem_st_v2(dst, u); else st_v2(dst, u);
    }
  }
}

template <int VEC>
__device__ __forceinline__ void load_f32(const float* p, float* f) {
#pragma unroll
  for (int q = 0; q < VEC / 4; ++q) {
    float4 v = *reinterpret_cast<const float4*>(p + 4 * q);
    f[4 * q] = v.x; f[4 * q + 1] = v.y; f[4 * q + 2] = v.z; f[4 * q + 3] = v.w;
  }
}
template <int VEC>
__device__ __forceinline__ void store_f32(float* p, const float* f) {
#pragma unroll
  for (int q = 0; q < VEC / 4; ++q)
    *reinterpret_cast<float4*>(p + 4 * q) =
        make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
}

// ---- rendezvous ---------------------------------------------------------------------
// Entry: announce "my gradients of this epoch are in place and my weight buffer may be
// overwritten", then wait for the same announcement from every rank.  Returns the epoch,
// or 0 after a timeout (the channel status then holds the error).
__device__ __forceinline__ unsigned long long channel_enter(void* const* base, int rank,
                                                            int world, int channel,
                                                            unsigned long long timeout_ns,
                                                            unsigned long long* s_epoch,
                                                            int* s_err) {
  Ctrl* my = ctrl_of(base[rank]);
  const int tid = threadIdx.x;
  if (tid == 0) {
    *s_epoch = ld_volatile_u64(&my->epoch[channel]) + 1ull;
    // a channel whose last wait ran out stays out of service until the host has cleared its
    // status: later launches return at once instead of waiting the deadline out again
    *s_err = (*(volatile int*)&my->status[channel] != 0);
  }
  __syncthreads();
  if (*s_err) return 0ull;
  const unsigned long long e = *s_epoch;
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    st_release_sys(&ctrl_of(base[tid])->flag_in[channel][rank], e);
  }
  if (tid < world) {
    if (!wait_flag_ge(&my->flag_in[channel][tid], e, timeout_ns)) {
      atomicOr(&my->late_mask[channel], 1u << tid);
      atomicMin(&my->status[channel], (int)PSDEV_ERR_TIMEOUT_ENTRY);
      *s_err = 1;
    }
  }
  __syncthreads();
  return *s_err ? 0ull : e;
}

// Exit: the last CTA of the grid tells every rank "I no longer read your gradients and
// my stores into your weight buffer are complete", waits for the same from everyone, and
// advances the local epoch.
__device__ __forceinline__ void channel_leave(void* const* base, int rank, int world,
                                              int channel, unsigned long long e,
                                              unsigned long long timeout_ns, int* s_last) {
  Ctrl* my = ctrl_of(base[rank]);
  const int tid = threadIdx.x;
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    *s_last = (atomicAdd(&my->done[channel], 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  const bool healthy = (e != 0ull) && (*(volatile int*)&my->status[channel] == 0);
  if (healthy && tid < world) {
    st_release_sys(&ctrl_of(base[tid])->flag_out[channel][rank], e);
    if (!wait_flag_ge(&my->flag_out[channel][tid], e, timeout_ns)) {
      atomicOr(&my->late_mask[channel], 1u << tid);
      atomicMin(&my->status[channel], (int)PSDEV_ERR_TIMEOUT_EXIT);
    }
  }
  __syncthreads();
  if (tid == 0) {
    my->done[channel] = 0;
    if (e != 0ull) my->epoch[channel] = e;
    __threadfence();
  }
}

// ---- the kernel -----------------------------------------------------------------------
// WMAX: compile-time bound on the number of ranks (1, 2, 4 or 8); the peer loops are fully
// unrolled to WMAX and predicated on the runtime world size.  Each thread handles
// U = max(1, 4 / ... ) vectors per trip so that about 128 bytes of gradient loads per
// thread are in flight whatever the world size.
template <int WMAX>
struct DenseShape {
  static constexpr int kUnroll = WMAX >= 8 ? 1 : (WMAX == 4 ? 2 : 4);
};
template <typename GT, typename OT, bool REDUCE>
struct DenseVec {
  static constexpr int kVec = REDUCE ? VecOf<GT>::kPer16 : (sizeof(OT) == 2 ? 8 : 4);
};
template <typename GT, typename OT, bool REDUCE, int WMAX>
struct DenseTile {
  static constexpr int kVec = DenseVec<GT, OT, REDUCE>::kVec;
  static constexpr int kBase = DenseShape<WMAX>::kUnroll;
  static constexpr int kUnroll = kVec == 16 ? 1 : ((kVec == 8 && kBase > 2) ? 2 : kBase);
  static constexpr int kElems = kDenseThreads * kVec * kUnroll;
};

// MC: reduce with one multimem.ld_reduce and broadcast with one multimem.st per vector (the
// NVSwitch does the fan-in and fan-out); instantiate with WMAX = 1 so that four vectors per
// thread are in flight.  Otherwise plain loads from and stores to each peer.
template <typename GT, typename OT, class Opt, bool REDUCE, bool BCAST, int WMAX, bool MC = false>
__global__ void __launch_bounds__(kDenseThreads)
    dense_kernel(const __grid_constant__ DenseArgs a) {
  constexpr int VEC = DenseVec<GT, OT, REDUCE>::kVec;
  constexpr int U = DenseTile<GT, OT, REDUCE, WMAX>::kUnroll;
  constexpr int TILE = kDenseThreads * VEC * U;
  __shared__ unsigned long long s_epoch;
  __shared__ int s_err, s_last;
  const int W = a.world, R = a.rank;
  unsigned long long e = 1;
  if (a.sync) {
    e = channel_enter(a.base, R, W, a.channel, a.timeout_ns, &s_epoch, &s_err);
  }
  const long long ntiles_all =
      a.nseg > 0 ? a.sched[a.nseg].tile_begin : a.n_owned * a.tiles_per_blk;
  if (e != 0ull && ntiles_all > 0) {
    const long long ntiles = ntiles_all;
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
      long long seg_begin = a.begin, seg_end = a.end, first_owned = a.first_owned, tl = t;
      if (a.nseg > 0) {
        // tiles are numbered slice after slice in priority order: find this tile's slice
        int slo = 0, shi = a.nseg - 1;
        while (slo < shi) {
          const int mid = (slo + shi + 1) >> 1;
          if (a.sched[mid].tile_begin <= t) slo = mid; else shi = mid - 1;
        }
        const SchedEntry se = a.sched[slo];
        seg_begin = se.begin; seg_end = se.end; first_owned = se.first_owned;
        tl = t - se.tile_begin;
      }
      const long long k = tl / a.tiles_per_blk;
      const long long sub = tl - k * a.tiles_per_blk;
      const long long j = first_owned + k * W;  // global block index
      const long long blk_lo = j * a.blk;
      long long lo = blk_lo + sub * TILE;
      long long hi = lo + TILE;
      const long long blk_hi = blk_lo + a.blk;
      if (hi > blk_hi) hi = blk_hi;
      if (hi > seg_end) hi = seg_end;
      // `lo` is not clamped to a.begin: lanes keep their alignment and skip i < begin
      const long long st_base = (j / W) * a.blk - blk_lo;  // state index = st_base + i
      const long long i0 = lo + (long long)threadIdx.x * VEC;
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * kDenseThreads * VEC;
        live[u] = (i < hi) && (i >= seg_begin);
#ifdef PSDEV_CHECKS
        // an index outside the table, the owner's state arrays or the arena is recorded in
        // the channel's status word and skipped, never dereferenced
        if (live[u] && !dense_index_ok<GT, OT, VEC>(a, i, st_base + i)) {
          atomicMin(&ctrl_of(a.base[R])->status[a.channel], (int)PSDEV_ERR_BOUNDS);
          live[u] = false;
        }
#endif
      }
      float w[U][VEC], m[U][VEC], v[U][VEC];
      if constexpr (REDUCE) {
        uint4 gv[U][WMAX];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * kDenseThreads * VEC;
          if constexpr (MC) {
            if (live[u]) {
              const GT* src = reinterpret_cast<const GT*>(
                                  reinterpret_cast<const char*>(a.mc_base) + a.grad_off) + i;
              if constexpr (sizeof(GT) == 4) gv[u][0] = multimem_ld_reduce_f32x4(src);
              else if constexpr (sizeof(GT) == 2) gv[u][0] = multimem_ld_reduce_bf16x8(src);
            }
          } else {
#pragma unroll
            for (int p = 0; p < WMAX; ++p) {
              if (p < W && live[u]) {
                const GT* src = reinterpret_cast<const GT*>(
                                    reinterpret_cast<const char*>(a.base[p]) + a.grad_off) + i;
                gv[u][p] = ld_sys_v4(src);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long si = st_base + i0 + (long long)u * kDenseThreads * VEC;
          if (live[u]) {
            load_f32<VEC>(a.master + si, w[u]);
            if constexpr (Opt::kStates >= 1) load_f32<VEC>(a.s1 + si, m[u]);
            if constexpr (Opt::kStates >= 2) load_f32<VEC>(a.s2 + si, v[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (!live[u]) continue;
          const long long si = st_base + i0 + (long long)u * kDenseThreads * VEC;
          float g[VEC];
#pragma unroll
          for (int q = 0; q < VEC; ++q) g[q] = 0.f;
#pragma unroll
          for (int p = 0; p < WMAX; ++p) {
            if (MC || p < W) {
              float f[VEC];
              VecOf<GT>::unpack(gv[u][p], f);
              float sc = 1.f;
              if constexpr (sizeof(GT) == 1) {
                // a vector of 16 never straddles a group of 256
                const long long gi = (i0 + (long long)u * kDenseThreads * VEC) / kInt8Group;
                sc = *(reinterpret_cast<const volatile float*>(
                           reinterpret_cast<const char*>(a.base[p]) + a.gscale_off) + gi);
              }
#pragma unroll
              for (int q = 0; q < VEC; ++q) g[q] = fmaf(f[q], sc, g[q]);
            }
          }
#pragma unroll
          for (int q = 0; q < VEC; ++q) {
            float mm = Opt::kStates >= 1 ? m[u][q] : 0.f;
            float vv = Opt::kStates >= 2 ? v[u][q] : 0.f;
            Opt::apply(w[u][q], g[q] * a.opt.scale, mm, vv, a.opt);
            if (Opt::kStates >= 1) m[u][q] = mm;
            if (Opt::kStates >= 2) v[u][q] = vv;
          }
          store_f32<VEC>(a.master + si, w[u]);
          if constexpr (Opt::kStates >= 1) store_f32<VEC>(a.s1 + si, m[u]);
          if constexpr (Opt::kStates >= 2) store_f32<VEC>(a.s2 + si, v[u]);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long si = st_base + i0 + (long long)u * kDenseThreads * VEC;
          if (live[u]) load_f32<VEC>(a.master + si, w[u]);
        }
      }
      if constexpr (BCAST && MC) {
        OT* dst0 = reinterpret_cast<OT*>(reinterpret_cast<char*>(a.mc_base) + a.weight_off);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * kDenseThreads * VEC;
          if (live[u]) store_out<OT, VEC, true>(dst0 + i, w[u]);
        }
      } else if constexpr (BCAST) {
#pragma unroll
        for (int pp = 0; pp < WMAX; ++pp) {
          if (pp < W && (pp == 0 || !a.self_only)) {
            int p = R + pp;
            if (p >= W) p -= W;
            OT* dst0 = reinterpret_cast<OT*>(reinterpret_cast<char*>(a.base[p]) + a.weight_off);
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const long long i = i0 + (long long)u * kDenseThreads * VEC;
              if (live[u]) store_out<OT, VEC>(dst0 + i, w[u]);
            }
          }
        }
      }
    }
  }
  if (a.sync) channel_leave(a.base, R, W, a.channel, e, a.timeout_ns, &s_last);
}

}  // namespace psdev
