// Launch helpers of the fused dense kernel: pick the kernel variant for the world size and the
// path (peer accesses or NVSwitch multicast), size the grid, run the device-side slice schedule
// when the launch carries several slices.  Shared by the library's own instantiations
// (src/kernels/dense_inst.inl) and by user-defined server handles (user_handle.cuh).
#pragma once
#include <cuda_runtime.h>

#include "ps/device/push_pull_ll.cuh"

extern "C" void psdev_count_launch(void);

namespace psdev {
void launch_p3_schedule(const long long* segs, int nseg, long long blk, int world, int rank,
                        long long tiles_per_blk, SchedEntry* out, cudaStream_t s);

template <typename GT, typename OT, class Opt, bool RED, bool BC, int WMAX>
inline int launch_w(DenseArgs a, int num_ctas, cudaStream_t s) {
  constexpr int tile = DenseTile<GT, OT, RED, WMAX>::kElems;
  a.tiles_per_blk = (a.blk + tile - 1) / tile;
  const long long ntiles = a.n_owned * a.tiles_per_blk;
  int ctas = num_ctas > 0 ? num_ctas : 2 * 148;
  if (a.nseg > 0) {
    // device-side schedule: slices ordered by priority, tiles numbered across slices
    launch_p3_schedule(a.segs_in, a.nseg, a.blk, a.world, a.rank, a.tiles_per_blk,
                       const_cast<SchedEntry*>(a.sched), s);
  } else if (ntiles < ctas) {
    ctas = ntiles > 0 ? (int)ntiles : 1;
  }
  dense_kernel<GT, OT, Opt, RED, BC, WMAX><<<ctas, kDenseThreads, 0, s>>>(a);
  psdev_count_launch();
  return (int)cudaGetLastError();
}

template <typename GT, typename OT, class Opt, bool RED, bool BC>
inline int launch_mc(DenseArgs a, int num_ctas, cudaStream_t s) {
  constexpr int tile = DenseTile<GT, OT, RED, 1>::kElems;
  a.tiles_per_blk = (a.blk + tile - 1) / tile;
  const long long ntiles = a.n_owned * a.tiles_per_blk;
  int ctas = num_ctas > 0 ? num_ctas : 2 * 148;
  if (a.nseg > 0) {
    launch_p3_schedule(a.segs_in, a.nseg, a.blk, a.world, a.rank, a.tiles_per_blk,
                       const_cast<SchedEntry*>(a.sched), s);
  } else if (ntiles < ctas) {
    ctas = ntiles > 0 ? (int)ntiles : 1;
  }
  dense_kernel<GT, OT, Opt, RED, BC, 1, true><<<ctas, kDenseThreads, 0, s>>>(a);
  psdev_count_launch();
  return (int)cudaGetLastError();
}

template <typename GT, typename OT, class Opt, bool RED, bool BC>
inline int launch(const DenseArgs& a, int ctas, cudaStream_t s) {
  if (a.mc_base && a.world > 1) return launch_mc<GT, OT, Opt, RED, BC>(a, ctas, s);
  if (a.world == 1) return launch_w<GT, OT, Opt, RED, BC, 1>(a, ctas, s);
  if (a.world == 2) return launch_w<GT, OT, Opt, RED, BC, 2>(a, ctas, s);
  if (a.world <= 4) return launch_w<GT, OT, Opt, RED, BC, 4>(a, ctas, s);
  return launch_w<GT, OT, Opt, RED, BC, 8>(a, ctas, s);
}


template <typename GT, typename OT, class Opt>
inline int launch_ll(const LLArgs& a, cudaStream_t s) {
  const long long m = a.end - a.begin;
  long long ctas = (m + kLLThreads - 1) / kLLThreads;
  if (ctas > 148) ctas = 148;  // every CTA of every rank must get to run: stay within one wave
  if (ctas < 1) ctas = 1;
  dense_ll_kernel<GT, OT, Opt><<<(int)ctas, kLLThreads, 0, s>>>(a);
  psdev_count_launch();
  return (int)cudaGetLastError();
}

}  // namespace psdev
